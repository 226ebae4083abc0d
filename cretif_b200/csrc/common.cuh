// Shared device helpers: element types, conversions, reductions, the status word.
//
// Every kernel file of the library includes this header.  Kernels are compiled for
// sm_100a only and are called through the extern "C" launchers declared in api.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cretif {

// Element type codes used across the C interface.
enum DType : int { kF32 = 0, kBF16 = 1 };

// Error codes returned by launchers (0 = launched; >0 = a cudaError_t).
enum Status : int {
  kOk = 0,
  kBadArgument = -1,      // a size or combination the kernel does not take
  kBadDType = -2,
  kMisaligned = -3,
};

// Bits of the device status word that kernels set instead of trapping.
enum DeviceFault : unsigned int {
  kFaultTokenRange = 1u,      // a token id outside [0, vocab)
  kFaultWaitExpired = 2u,     // a bounded wait on a barrier gave up
  kFaultBlockTable = 4u,      // a position mapped to no cache block
};

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// silu(g) = g / (1 + e^-g) for the bfloat16 kernels: exponential and quotient on the
// special-function unit (relative error about 2^-21, far below the 2^-9 of the bfloat16 the
// result is rounded to).  The float32 path divides and calls expf.
__device__ __forceinline__ float silu_bf16_path(float g) {
  return __fdividef(g, 1.0f + __expf(-g));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();                 // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// 8 consecutive elements as floats (16-byte load for bf16, two for f32).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = u;
}

// Phase timestamps inside the kernels (%globaltimer written to a buffer) are a tuning aid.
// They are compiled only with -DCRETIF_STAMPS; in the ordinary build the constant below is
// false and the compiler drops every trace of them.
#ifdef CRETIF_STAMPS
constexpr bool kStamps = true;
#else
constexpr bool kStamps = false;
#endif

// Which variant of a kernel a launch took, counted on the host at launch time (a replayed
// CUDA graph counts nothing).  Tests read the counts to know that the path they mean to check
// is the one that ran; nothing in the library depends on them.
enum Variant : int {
  kVarFusedRegisters = 0,   // fused projection, weights through registers, one row group
  kVarFusedRowGroups,       // ... more than 32 rows as groups along gridDim.y
  kVarFusedCluster2,        // ... norm prologue shared by clusters of two CTAs
  kVarFusedCluster4,        // ... of four
  kVarStream,               // fused projection, weights through a shared-memory ring
  kVarStreamRowGroups,      // ... more than 16 rows as groups of 16
  kVarDecodeCluster,        // decode attention merged inside a cluster
  kVarDecodeSplit,          // decode attention merged through global scratch
  kVarPrefillAttn,          // tcgen05 prefill attention
  kVarTc64, kVarTc128, kVarTc256,   // tcgen05 product by tile width
  kVarTcSeveralTiles,       // ... whose persistent CTAs walk more than one tile
  kVarTc192,                // ... 192 columns wide
  kVarPrefillAttnPair,      // tcgen05 prefill attention, a thread per row, two query tiles per CTA
  kVarPrefillAttnSplit,     // ... one tile per CTA, its key steps split between two slots
  kVarTcBulkAdd,            // tcgen05 product added into a float32 matrix through TMA
  kVarTcPair,               // tcgen05 product with two CTAs on a tile (cta_group::2)
  kVarCount
};
void count_variant(int v);

// Whether kernels that support it are launched as programmatic dependents of the kernel
// before them (decode_fused.cu owns the switch).
int dependent_launch_enabled();

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace cretif
