// Row-wise and element-wise kernels: embedding rows, residual + RMSNorm, SiLU·mul,
// rotary position encoding fused with the write into the block cache, decode bookkeeping.
//
// Formulas follow the reference (embedding gather src/embedding.cu:39-60; RMSNorm
// src/kernels/elementwise.cu:30-72; residual + RMSNorm :463-506; SiLU :93-99 and
// multiply :300-306; rotary :232-258; cache append src/kv_cache.cu:176-199), but each
// kernel takes all tokens of a step in one launch and the residual stream stays in
// 32-bit whatever the storage type of the activations is.
#include "api.h"
#include "common.cuh"

namespace cretif {

// ---------------------------------------------------------------- embedding rows
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ out, int H, int V,
                                  unsigned int* __restrict__ fault) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* row = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultTokenRange);
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = to_float(src[i]);
}

// ---------------------------------------------------------------- residual + RMSNorm
// v = h[src] (+ delta[src]);  optionally h[src] = v;  out[r] = v * w * rsqrt(mean(v^2) + eps)
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, int write_h) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* hrow = h + (size_t)src * H;
  const TD* drow = delta ? delta + (size_t)src * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hrow[i];
    if (drow) v += to_float(drow[i]);
    if (write_h) hrow[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  TO* orow = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hrow[i];
    if (drow && !write_h) v += to_float(drow[i]);
    orow[i] = from_float<TO>(v * weight[i] * inv);
  }
}

// The same with 16-byte accesses: H % 4 == 0 and 16-byte aligned rows.  A thread keeps up to
// four float4 of its row in registers, so a row makes one trip through memory.
__device__ __forceinline__ float4 load4f(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4f(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void store4f(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4f(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TD, typename TO>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const float* __restrict__ weight, TO* __restrict__ out,
                                       const int* __restrict__ rows, int H, float eps,
                                       int write_h) {
  __shared__ float scratch[33];
  constexpr int kKeep = 4;
  // (a no-op pair unless the launch was a programmatic dependent one)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* hrow = h + (size_t)src * H;
  const TD* drow = delta ? delta + (size_t)src * H : nullptr;
  const int n4 = H >> 2;
  float4 keep[kKeep];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kKeep; ++it) {
    const int i = it * blockDim.x + threadIdx.x;
    if (i < n4) {
      float4 v = load4f(hrow + 4 * i);
      if (drow) {
        const float4 d = load4f(drow + 4 * i);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
      }
      if (write_h) store4f(hrow + 4 * i, v);
      keep[it] = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  for (int i = kKeep * blockDim.x + threadIdx.x; i < n4; i += blockDim.x) {   // very wide rows
    float4 v = load4f(hrow + 4 * i);
    if (drow) {
      const float4 d = load4f(drow + 4 * i);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    if (write_h) store4f(hrow + 4 * i, v);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  TO* orow = out + (size_t)r * H;
#pragma unroll
  for (int it = 0; it < kKeep; ++it) {
    const int i = it * blockDim.x + threadIdx.x;
    if (i < n4) {
      const float4 w = load4f(weight + 4 * i), v = keep[it];
      store4f(orow + 4 * i, make_float4(v.x * w.x * inv, v.y * w.y * inv, v.z * w.z * inv,
                                        v.w * w.w * inv));
    }
  }
  for (int i = kKeep * blockDim.x + threadIdx.x; i < n4; i += blockDim.x) {
    float4 v = load4f(hrow + 4 * i);
    if (drow && !write_h) {
      const float4 d = load4f(drow + 4 * i);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    const float4 w = load4f(weight + 4 * i);
    store4f(orow + 4 * i, make_float4(v.x * w.x * inv, v.y * w.y * inv, v.z * w.z * inv,
                                      v.w * w.w * inv));
  }
}

// Many rows: a warp per row, eight rows per block, no block-wide barrier.  A lane keeps its
// REGS float4 of the row between the sum of squares and the scaling, so a row makes one trip
// from memory.  Lanes, order of the sums and the arithmetic are those of the fused decode
// prologue (decode_fused.cuh), so a row gets the same numbers from either.
template <int REGS, typename TD, typename TO>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                        const float* __restrict__ weight, TO* __restrict__ out,
                        const int* __restrict__ rows, int R, int H, float eps, int write_h) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  const int n4 = H >> 2;
  float4 w[REGS];                       // the weight does not wait for the kernel before
#pragma unroll
  for (int u = 0; u < REGS; ++u) {
    const int i = u * 32 + lane;
    w[u] = i < n4 ? load4f(weight + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (r >= R) return;
  const int src = rows ? rows[r] : r;
  float* hrow = h + (size_t)src * H;
  const TD* drow = delta ? delta + (size_t)src * H : nullptr;
  float4 v[REGS];
#pragma unroll
  for (int u = 0; u < REGS; ++u) {
    const int i = u * 32 + lane;
    v[u] = i < n4 ? load4f(hrow + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (drow) {
#pragma unroll
    for (int u = 0; u < REGS; ++u) {
      const int i = u * 32 + lane;
      if (i < n4) {
        const float4 d = load4f(drow + 4 * i);
        v[u].x += d.x; v[u].y += d.y; v[u].z += d.z; v[u].w += d.w;
        if (write_h) store4f(hrow + 4 * i, v[u]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < REGS; ++u)
    ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)H + eps);
  TO* orow = out + (size_t)r * H;
#pragma unroll
  for (int u = 0; u < REGS; ++u) {
    const int i = u * 32 + lane;
    if (i < n4)
      store4f(orow + 4 * i, make_float4(v[u].x * w[u].x * inv, v[u].y * w[u].y * inv,
                                        v[u].z * w[u].z * inv, v[u].w * w[u].w * inv));
  }
}

// ---------------------------------------------------------------- SiLU(gate) * up
// `block` = 0: gu row = [gate (I) | up (I)]; block = b > 0: gate and up alternate in groups of b
// columns (b gate columns, then the b up columns that belong to them).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, int I, int block,
                                size_t total) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  const int gcol = block ? (i / block) * 2 * block + i % block : i;
  const int ucol = block ? gcol + block : I + i;
  const float g = to_float(gu[t * 2 * (size_t)I + gcol]);
  const float u = to_float(gu[t * 2 * (size_t)I + ucol]);
  // float32: the reference's x / (1 + expf(-x)) (src/kernels/elementwise.cu:93-99);
  // bfloat16: the same on the special-function unit, as in the fused epilogues
  const float s = sizeof(T) == 4 ? g / (1.0f + expf(-g)) : silu_bf16_path(g);
  act[idx] = from_float<T>(s * u);
}

// ---------------------------------------------------------------- rotary + cache write
// One block per token.  qkv row = [q heads | k heads | v heads]; q is rotated in place.
// write_cache bit 0: rotated k and v go to the cache; bit 1: k is rotated in place as well
// (position encoding alone, for a caller that stores the keys itself).
template <typename T>
__global__ void rope_kv_append_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int pairing, int rot_dim,
                                      int nh, int nkv, int hd, const int* __restrict__ tok_pos,
                                      const int* __restrict__ tok_seq,
                                      const int* __restrict__ seq_slot,
                                      const int* __restrict__ table, int table_stride,
                                      T* __restrict__ kc, T* __restrict__ vc, int bt,
                                      int write_cache, unsigned int* __restrict__ fault) {
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  T* row = qkv + (size_t)t * ld;
  const int half = rot_dim >> 1;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;

  size_t cache_row = 0;
  bool cache_ok = false;
  if (write_cache & 1) {
    const int slot = seq_slot[tok_seq[t]];
    const int blk = table[(size_t)slot * table_stride + pos / bt];
    if (blk < 0) {
      if (threadIdx.x == 0) atomicOr(fault, kFaultBlockTable);
    } else {
      cache_ok = true;
      cache_row = (size_t)blk * nkv * bt + (pos % bt);   // + kvh * bt, then * hd
    }
  }
  // rotary pairs of q and k heads
  const int n_rot_heads = nh + nkv;
  for (int idx = threadIdx.x; idx < n_rot_heads * half; idx += blockDim.x) {
    const int head = idx / half, j = idx - head * half;
    const int i0 = pairing ? 2 * j : j;
    const int i1 = pairing ? 2 * j + 1 : j + half;
    T* hp = row + (size_t)head * hd;          // q heads then k heads are contiguous
    const float x0 = to_float(hp[i0]), x1 = to_float(hp[i1]);
    const float y0 = x0 * c[j] - x1 * s[j];
    const float y1 = x0 * s[j] + x1 * c[j];
    if (head < nh) {
      hp[i0] = from_float<T>(y0);
      hp[i1] = from_float<T>(y1);
    } else {
      if (cache_ok) {
        T* kp = kc + (cache_row + (size_t)(head - nh) * bt) * hd;
        kp[i0] = from_float<T>(y0);
        kp[i1] = from_float<T>(y1);
      }
      if (write_cache & 2) {
        hp[i0] = from_float<T>(y0);
        hp[i1] = from_float<T>(y1);
      }
    }
  }
  if (!cache_ok) return;
  // the part of k beyond rot_dim (not rotated) and all of v
  const int tail = hd - rot_dim;
  for (int idx = threadIdx.x; idx < nkv * tail; idx += blockDim.x) {
    const int kvh = idx / tail, i = rot_dim + (idx - kvh * tail);
    kc[(cache_row + (size_t)kvh * bt) * hd + i] = row[(size_t)(nh + kvh) * hd + i];
  }
  const T* vrow = row + (size_t)(nh + nkv) * hd;
  for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
    const int kvh = idx / hd, i = idx - kvh * hd;
    vc[(cache_row + (size_t)kvh * bt) * hd + i] = vrow[idx];
  }
}

// ---------------------------------------------------------------- decode bookkeeping
__global__ void advance_decode_kernel(int* __restrict__ tok_ids, int* __restrict__ tok_pos,
                                      int* __restrict__ seq_start,
                                      const int* __restrict__ sampled, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (sampled) tok_ids[b] = sampled[b];
  tok_pos[b] += 1;
  seq_start[b] += 1;
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_embed_rows(const void* table, int table_dt, const int* ids, float* out,
                                 int T, int H, int V, unsigned int* fault, void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || V <= 0) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = H >= 256 ? 256 : 64;
  if (table_dt == kF32)
    embed_rows_kernel<float><<<T, threads, 0, st>>>((const float*)table, ids, out, H, V, fault);
  else if (table_dt == kBF16)
    embed_rows_kernel<__nv_bfloat16><<<T, threads, 0, st>>>((const __nv_bfloat16*)table, ids, out,
                                                          H, V, fault);
  else
    return kBadDType;
  return launch_status();
}

template <typename TD>
static int add_rmsnorm_out(float* h, const TD* delta, const float* w, void* out, int out_dt,
                           const int* rows, int R, int H, float eps, int write_h,
                           cudaStream_t st) {
  const bool aligned = H % 4 == 0 && (((uintptr_t)h | (uintptr_t)delta | (uintptr_t)w |
                                       (uintptr_t)out) & 15) == 0;
  if (aligned && R >= 64 && H / 4 <= 32 * 16) {
    // many rows (a prompt): a warp per row
    const int n4 = H / 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((R + 7) / 8);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
#define CRETIF_ROWS(REGS, TO)                                                                  \
  e = cudaLaunchKernelEx(&cfg, add_rmsnorm_rows_kernel<REGS, TD, TO>, h, delta, w, (TO*)out,   \
                         rows, R, H, eps, write_h)
    if (out_dt == kF32) {
      if (n4 <= 32 * 8) CRETIF_ROWS(8, float); else CRETIF_ROWS(16, float);
    } else if (out_dt == kBF16) {
      if (n4 <= 32 * 8) CRETIF_ROWS(8, __nv_bfloat16); else CRETIF_ROWS(16, __nv_bfloat16);
    } else {
      return kBadDType;
    }
#undef CRETIF_ROWS
    return e == cudaSuccess ? launch_status() : (int)e;
  }
  if (aligned) {
    const int n4 = H / 4;
    const int vthreads = n4 >= 512 ? 256 : (n4 >= 128 ? 128 : (n4 >= 64 ? 64 : 32));
    // as a programmatic dependent of the kernel before it: its launch runs under that tail
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(R);
    cfg.blockDim = dim3(vthreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
    if (out_dt == kF32)
      e = cudaLaunchKernelEx(&cfg, add_rmsnorm_vec_kernel<TD, float>, h, delta, w, (float*)out,
                             rows, H, eps, write_h);
    else if (out_dt == kBF16)
      e = cudaLaunchKernelEx(&cfg, add_rmsnorm_vec_kernel<TD, __nv_bfloat16>, h, delta, w,
                             (__nv_bfloat16*)out, rows, H, eps, write_h);
    else
      return kBadDType;
    return e == cudaSuccess ? launch_status() : (int)e;
  }
  const int threads = H >= 2048 ? 512 : (H >= 256 ? 256 : 64);
  if (out_dt == kF32)
    add_rmsnorm_kernel<TD, float><<<R, threads, 0, st>>>(h, delta, w, (float*)out, rows, H, eps,
                                                        write_h);
  else if (out_dt == kBF16)
    add_rmsnorm_kernel<TD, __nv_bfloat16><<<R, threads, 0, st>>>(h, delta, w, (__nv_bfloat16*)out,
                                                                rows, H, eps, write_h);
  else
    return kBadDType;
  return launch_status();
}

extern "C" int cretif_add_rmsnorm(float* h, const void* delta, int delta_dt, const float* weight,
                                  void* out, int out_dt, const int* rows, int R, int H, float eps,
                                  int write_h, void* stream) {
  if (R <= 0) return kOk;
  if (H <= 0) return kBadArgument;
  if (rows && write_h) return kBadArgument;   // gathered rows never update the stream
  cudaStream_t st = (cudaStream_t)stream;
  if (!delta || delta_dt == kF32)
    return add_rmsnorm_out<float>(h, (const float*)delta, weight, out, out_dt, rows, R, H, eps,
                                  write_h, st);
  if (delta_dt == kBF16)
    return add_rmsnorm_out<__nv_bfloat16>(h, (const __nv_bfloat16*)delta, weight, out, out_dt,
                                          rows, R, H, eps, write_h, st);
  return kBadDType;
}

extern "C" int cretif_silu_mul(const void* gu, void* act, int dt, int T, int I, int block,
                               void* stream) {
  if (T <= 0) return kOk;
  if (I <= 0 || block < 0 || (block > 0 && I % block)) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)T * I;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dt == kF32)
    silu_mul_kernel<float><<<blocks, 256, 0, st>>>((const float*)gu, (float*)act, I, block, total);
  else if (dt == kBF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)gu,
                                                          (__nv_bfloat16*)act, I, block, total);
  else
    return kBadDType;
  return launch_status();
}

extern "C" int cretif_rope_kv_append(void* qkv, int ld, int dt, const float* cos_t,
                                     const float* sin_t, int pairing, int rot_dim, int nh, int nkv,
                                     int hd, const int* tok_pos, const int* tok_seq,
                                     const int* seq_slot, const int* table, int table_stride,
                                     void* kc, void* vc, int bt, int write_cache, int T,
                                     unsigned int* fault, void* stream) {
  if (T <= 0) return kOk;
  if (nh <= 0 || nkv <= 0 || hd <= 0 || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || bt <= 0 ||
      ld < (nh + 2 * nkv) * hd)
    return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = 128;
  if (dt == kF32)
    rope_kv_append_kernel<float><<<T, threads, 0, st>>>(
        (float*)qkv, ld, cos_t, sin_t, pairing, rot_dim, nh, nkv, hd, tok_pos, tok_seq, seq_slot,
        table, table_stride, (float*)kc, (float*)vc, bt, write_cache, fault);
  else if (dt == kBF16)
    rope_kv_append_kernel<__nv_bfloat16><<<T, threads, 0, st>>>(
        (__nv_bfloat16*)qkv, ld, cos_t, sin_t, pairing, rot_dim, nh, nkv, hd, tok_pos, tok_seq,
        seq_slot, table, table_stride, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, bt, write_cache,
        fault);
  else
    return kBadDType;
  return launch_status();
}

extern "C" int cretif_advance_decode(int* tok_ids, int* tok_pos, int* seq_start,
                                     const int* sampled, int B, void* stream) {
  if (B <= 0) return kOk;
  advance_decode_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(tok_ids, tok_pos,
                                                                          seq_start, sampled, B);
  return launch_status();
}
