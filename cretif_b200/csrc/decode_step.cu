// One decode step of the whole model in one launch (bfloat16, few tokens).
//
// A decode step of a small model is hundreds of tiny dependent kernels; even as a CUDA graph
// each costs several microseconds of launch, ramp and drain, far more than its memory
// traffic.  Here one persistent grid (one CTA per SM) walks the scheduled layers itself:
//
//   embed rows -> for every scheduled layer
//     A  norm -> q|k|v product -> rotary -> cache write        (decode_fused.cuh)
//     B  attention over the block cache, ranges merged by the last CTA (attn_decode_mma.cuh)
//     C  output projection added into the residual stream
//     D  norm -> gate|up product -> SiLU·mul
//     E  down projection added into the residual stream
//   -> final norm -> head product at the wanted rows.
//
// Phases are separated by a grid-wide barrier (a counter in global memory; arrivals release,
// the spin acquires, and the wait is bounded like every other wait in this library).  Data
// that one phase writes and the next reads crosses CTAs, so such reads bypass L1.  The device
// code of the phases is the same code the separate kernels run.
//
// The reference has no counterpart (it launches ~16 kernels per layer and token,
// src/model.cu:887-1022).
#include <cuda.h>
#include <cuda_runtime.h>

#include "api.h"
#include "attn_decode_mma.cuh"
#include "decode_fused.cuh"

namespace cretif {

struct alignas(64) StepLayer {
  CUtensorMap map_k, map_v;          // 2-d maps of this visit's key and value cache
  const __nv_bfloat16* w_qkv;
  const __nv_bfloat16* w_o;
  const __nv_bfloat16* w_gu;
  const __nv_bfloat16* w_down;
  const float* norm1;
  const float* norm2;
  __nv_bfloat16* kc;
  __nv_bfloat16* vc;
  const int* table;
  int table_stride;
  int write_cache;
  float eps1, eps2;
};

struct StepParams {
  int n_layers, B, H, I, nh, nkv, hd, gu_block, pairing, bt, window, n_splits, V, n_want;
  float eps_final, scale_log2;
  const StepLayer* layers;
  float* h;                           // [B, H] residual stream
  __nv_bfloat16* q;                   // [B, nh*hd]
  __nv_bfloat16* attn;                // [B, nh*hd]
  __nv_bfloat16* act;                 // [B, I]
  float* part_o;
  float* part_ml;
  int* counters;
  const int* tok_ids;
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const float* cos_t;
  const float* sin_t;
  const __nv_bfloat16* embed;         // [V, H]
  const float* final_norm;
  const __nv_bfloat16* head;          // [V, H]
  const int* want_rows;               // [n_want] or null (all rows)
  float* logits;                      // [n_want, V]
  unsigned int* barrier;              // [2]: arrivals, leavers; zero before the first launch
  unsigned int* fault;
  unsigned long long* stamps;         // optional: CTA 0 notes the time (ns) after every barrier
};

constexpr unsigned kGridSpinLimit = 1u << 22;

// Ask L2 for a matrix the grid will read soon (one 128-byte line per thread and pass), so
// that the phase that needs it finds it on the chip: weights of the next layer travel while
// this layer computes and waits at its barriers.
__device__ __forceinline__ void prefetch_l2(const void* base, size_t bytes, int cta, int P) {
  const char* p = static_cast<const char*>(base);
  const size_t lines = (bytes + 127) >> 7;
  for (size_t i = (size_t)cta * blockDim.x + threadIdx.x; i < lines; i += (size_t)P * blockDim.x)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p + (i << 7)));
}

// All CTAs of the grid meet here; `target` = number of arrivals that completes this barrier.
__device__ __forceinline__ void grid_barrier(unsigned int* arrivals, unsigned int target,
                                             unsigned int* fault, bool before_tma = false) {
  // stores that a later phase reads with TMA (the cache rows) must cross to the async proxy
  if (before_tma) asm volatile("fence.proxy.async;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(arrivals, 1u);
    unsigned spins = 0;
    while (true) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(arrivals) : "memory");
      if (v >= target) break;
      if ((++spins & 1023u) == 0u) {
        unsigned f;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(f) : "l"(fault) : "memory");
        if ((f & kFaultWaitExpired) || spins >= kGridSpinLimit) {
          atomicOr(fault, kFaultWaitExpired);
          break;
        }
      }
    }
    __threadfence();
  }
  __syncthreads();
}

template <int NT, int HD16>
__global__ void __launch_bounds__(kFuWarps * 32, 1)
decode_step_kernel(const StepParams p) {
  extern __shared__ unsigned char step_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(step_smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* attn_smem = smem;                                           // tiles, barriers
  unsigned char* gemv_smem = smem + ((dm_smem_core<HD16>() + 1023) & ~size_t(1023));
  const int P = gridDim.x, cta = blockIdx.x;
  unsigned int done = 0;            // barriers passed so far
  auto stamp = [&]() {
    if (p.stamps && cta == 0 && threadIdx.x == 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      p.stamps[done] = t;
    }
  };
  stamp();
  dm_init<HD16>(attn_smem);
  uint32_t it_base = 0;

  // ---- token embeddings into the residual stream
  for (int row = cta; row < p.B; row += P) {
    const int id = p.tok_ids[row];
    const bool ok = id >= 0 && id < p.V;
    if (!ok && threadIdx.x == 0) atomicOr(p.fault, kFaultTokenRange);
    const __nv_bfloat16* src = p.embed + (size_t)(ok ? id : 0) * p.H;
    for (int i = threadIdx.x; i < p.H; i += blockDim.x)
      p.h[(size_t)row * p.H + i] = ok ? __bfloat162float(src[i]) : 0.f;
  }
  const int q_dim = p.nh * p.hd, qkv_rows = (p.nh + 2 * p.nkv) * p.hd;
  const int n_items = p.B * p.nkv * p.n_splits;
  const size_t qkv_bytes = (size_t)qkv_rows * p.H * 2, o_bytes = (size_t)p.H * q_dim * 2;
  const size_t gu_bytes = (size_t)2 * p.I * p.H * 2, down_bytes = (size_t)p.H * p.I * 2;
  const size_t head_bytes = (size_t)p.V * p.H * 2;
  const int head_layers = p.n_layers < 8 ? p.n_layers : 8;     // the head travels in 8 parts
  {
    const StepLayer& L0 = p.layers[0];
    prefetch_l2(L0.w_qkv, qkv_bytes, cta, P);
    prefetch_l2(L0.w_o, o_bytes, cta, P);
    prefetch_l2(L0.w_gu, gu_bytes, cta, P);
    prefetch_l2(L0.w_down, down_bytes, cta, P);
  }
  grid_barrier(p.barrier, ++done * P, p.fault);
  stamp();

  for (int l = 0; l < p.n_layers; ++l) {
    const StepLayer& L = p.layers[l];
    if (l + 1 < p.n_layers) {                 // next layer's first two matrices
      prefetch_l2(p.layers[l + 1].w_qkv, qkv_bytes, cta, P);
      prefetch_l2(p.layers[l + 1].w_o, o_bytes, cta, P);
    }
    if (l >= p.n_layers - head_layers) {      // a slice of the head's matrix
      const int part = l - (p.n_layers - head_layers);
      const size_t chunk = (head_bytes / head_layers + 127) & ~size_t(127);
      const size_t off = chunk * part;
      if (off < head_bytes)
        prefetch_l2(reinterpret_cast<const char*>(p.head) + off,
                    off + chunk <= head_bytes ? chunk : head_bytes - off, cta, P);
    }
    {   // A: norm -> q|k|v -> rotary -> cache
      FusedParams f = {};
      f.W = L.w_qkv; f.M = p.B; f.N = qkv_rows; f.K = p.H; f.ldw = p.H;
      f.H = p.h; f.norm_w = L.norm1; f.eps = L.eps1;
      f.Q = p.q; f.ldq = q_dim; f.cos_t = p.cos_t; f.sin_t = p.sin_t; f.pairing = p.pairing;
      f.nh = p.nh; f.nkv = p.nkv; f.hd = p.hd; f.tok_pos = p.tok_pos; f.tok_seq = p.tok_seq;
      f.seq_slot = p.seq_slot; f.table = L.table; f.table_stride = L.table_stride;
      f.kc = L.kc; f.vc = L.vc; f.bt = p.bt; f.write_cache = L.write_cache; f.fault = p.fault;
      derive_fields(f);
      skinny_fused_tiles<NT, kProNorm, kEpiRope>(f, qkv_rows / kFuRows, gemv_smem, cta, P, false);
    }
    grid_barrier(p.barrier, ++done * P, p.fault, true);
    stamp();
    // B: attention
    for (int item = cta; item < n_items; item += P) {
      const int split = item % p.n_splits, rest = item / p.n_splits;
      attn_decode_mma_item<HD16>(attn_smem, &L.map_k, &L.map_v, p.q, q_dim, L.table,
                                 L.table_stride, p.tok_pos, p.tok_seq, p.seq_slot, p.nh, p.nkv,
                                 p.scale_log2, p.window, p.part_o, p.part_ml, p.attn, q_dim,
                                 p.counters, p.fault, split, p.n_splits, rest % p.nkv,
                                 rest / p.nkv, it_base);
    }
    grid_barrier(p.barrier, ++done * P, p.fault);
    stamp();
    if (l + 1 < p.n_layers) {                 // next layer's feed-forward matrices
      prefetch_l2(p.layers[l + 1].w_gu, gu_bytes, cta, P);
      prefetch_l2(p.layers[l + 1].w_down, down_bytes, cta, P);
    }
    {   // C: h += attn · Wo^T
      FusedParams f = {};
      f.W = L.w_o; f.M = p.B; f.N = p.H; f.K = q_dim; f.ldw = q_dim;
      f.X = p.attn; f.ldx = q_dim; f.C = p.h; f.ldc = p.H; f.c_dt = kF32; f.accumulate = 1;
      derive_fields(f);
      skinny_fused_tiles<NT, kProPlain, kEpiPlain>(f, (p.H + kFuRows - 1) / kFuRows, gemv_smem,
                                                   cta, P, false);
    }
    grid_barrier(p.barrier, ++done * P, p.fault);
    stamp();
    {   // D: norm -> gate|up -> SiLU·mul
      FusedParams f = {};
      f.W = L.w_gu; f.M = p.B; f.N = 2 * p.I; f.K = p.H; f.ldw = p.H;
      f.H = p.h; f.norm_w = L.norm2; f.eps = L.eps2; f.act = p.act; f.I = p.I;
      f.gu_block = p.gu_block;
      derive_fields(f);
      skinny_fused_tiles<NT, kProNorm, kEpiSilu>(f, (p.I + 7) / 8, gemv_smem, cta, P, false);
    }
    grid_barrier(p.barrier, ++done * P, p.fault);
    stamp();
    {   // E: h += act · Wdown^T
      FusedParams f = {};
      f.W = L.w_down; f.M = p.B; f.N = p.H; f.K = p.I; f.ldw = p.I;
      f.X = p.act; f.ldx = p.I; f.C = p.h; f.ldc = p.H; f.c_dt = kF32; f.accumulate = 1;
      derive_fields(f);
      skinny_fused_tiles<NT, kProPlain, kEpiPlain>(f, (p.H + kFuRows - 1) / kFuRows, gemv_smem,
                                                   cta, P, false);
    }
    grid_barrier(p.barrier, ++done * P, p.fault);
    stamp();
  }
  {   // final norm -> head at the wanted rows
    FusedParams f = {};
    f.W = p.head; f.M = p.n_want; f.N = p.V; f.K = p.H; f.ldw = p.H;
    f.H = p.h; f.norm_w = p.final_norm; f.rows = p.want_rows; f.eps = p.eps_final;
    f.C = p.logits; f.ldc = p.V; f.c_dt = kF32; f.accumulate = 0;
    derive_fields(f);
    skinny_fused_tiles<NT, kProNorm, kEpiPlain>(f, (p.V + kFuRows - 1) / kFuRows, gemv_smem, cta,
                                                P, false);
  }
  ++done;
  stamp();
  // ---- the last CTA to leave resets the barrier for the next launch (every CTA has passed the
  // last barrier before it gets here, so nobody still reads the arrival counter)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned left = atomicAdd(p.barrier + 1, 1u);
    if (left == (unsigned)P - 1u) {
      p.barrier[0] = 0u;
      p.barrier[1] = 0u;
      __threadfence();
    }
  }
}

template <int NT, int HD16>
static size_t step_smem_bytes(int B, int H) {
  const size_t attn = (dm_smem_core<HD16>() + 1023) & ~size_t(1023);
  return attn + fused_smem(NT, kProNorm, B, H) + 1024;
}

template <int NT, int HD16>
static int launch_step(const StepParams& p, int ctas, cudaStream_t st) {
  const size_t smem = step_smem_bytes<NT, HD16>(p.B, p.H);
  if (smem > 200 * 1024) return kBadArgument;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel<NT, HD16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  // every CTA must be resident at once: ask for a cooperative launch, which checks that
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kFuWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_step_kernel<NT, HD16>, p);
  return e == cudaSuccess ? launch_status() : (int)e;
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_step_layer_bytes(void) { return (int)sizeof(StepLayer); }

extern "C" int cretif_decode_step_supported(int B, int hd) {
  return B > 0 && B <= 32 && (hd == 16 || hd == 32 || hd == 48 || hd == 64 || hd == 128);
}

// Fill one StepLayer record in host memory (the caller copies the array to the device).
extern "C" int cretif_step_layer_fill(void* dst, const void* w_qkv, const void* w_o,
                                      const void* w_gu, const void* w_down, const float* norm1,
                                      const float* norm2, float eps1, float eps2, void* kc,
                                      void* vc, long long n_blocks, int nkv, int hd,
                                      const int* table, int table_stride, int write_cache) {
  StepLayer L = {};
  const long long rows = n_blocks * nkv * kDmTile;
  if (rows <= 0 || rows > 0x7fffffffLL || hd % 16 || hd < 16 || hd > 128) return kBadArgument;
  if (make_tile_map_bf16(&L.map_k, kc, (int)rows, hd, hd, kDmTile)) return kBadArgument;
  if (make_tile_map_bf16(&L.map_v, vc, (int)rows, hd, hd, kDmTile)) return kBadArgument;
  L.w_qkv = (const __nv_bfloat16*)w_qkv; L.w_o = (const __nv_bfloat16*)w_o;
  L.w_gu = (const __nv_bfloat16*)w_gu; L.w_down = (const __nv_bfloat16*)w_down;
  L.norm1 = norm1; L.norm2 = norm2; L.eps1 = eps1; L.eps2 = eps2;
  L.kc = (__nv_bfloat16*)kc; L.vc = (__nv_bfloat16*)vc;
  L.table = table; L.table_stride = table_stride; L.write_cache = write_cache;
  memcpy(dst, &L, sizeof(L));
  return kOk;
}

// ints: n_layers, B, H, I, nh, nkv, hd, gu_block, pairing, bt, window, n_splits, V, n_want
// ptrs: layers, h, q, attn, act, part_o, part_ml, counters, tok_ids, tok_pos, tok_seq, seq_slot,
//       cos, sin, embed, final_norm, head, want_rows, logits, barrier, fault, stamps (or null)
extern "C" int cretif_decode_step(const int* ints, const float* floats, void* const* ptrs,
                                  int ctas, void* stream) {
  StepParams p = {};
  p.n_layers = ints[0]; p.B = ints[1]; p.H = ints[2]; p.I = ints[3]; p.nh = ints[4];
  p.nkv = ints[5]; p.hd = ints[6]; p.gu_block = ints[7]; p.pairing = ints[8]; p.bt = ints[9];
  p.window = ints[10]; p.n_splits = ints[11]; p.V = ints[12]; p.n_want = ints[13];
  p.eps_final = floats[0]; p.scale_log2 = floats[1] * 1.4426950408889634f;
  p.layers = (const StepLayer*)ptrs[0]; p.h = (float*)ptrs[1]; p.q = (__nv_bfloat16*)ptrs[2];
  p.attn = (__nv_bfloat16*)ptrs[3]; p.act = (__nv_bfloat16*)ptrs[4]; p.part_o = (float*)ptrs[5];
  p.part_ml = (float*)ptrs[6]; p.counters = (int*)ptrs[7]; p.tok_ids = (const int*)ptrs[8];
  p.tok_pos = (const int*)ptrs[9]; p.tok_seq = (const int*)ptrs[10];
  p.seq_slot = (const int*)ptrs[11]; p.cos_t = (const float*)ptrs[12];
  p.sin_t = (const float*)ptrs[13]; p.embed = (const __nv_bfloat16*)ptrs[14];
  p.final_norm = (const float*)ptrs[15]; p.head = (const __nv_bfloat16*)ptrs[16];
  p.want_rows = (const int*)ptrs[17]; p.logits = (float*)ptrs[18];
  p.barrier = (unsigned int*)ptrs[19]; p.fault = (unsigned int*)ptrs[20];
  p.stamps = (unsigned long long*)ptrs[21];
  if (p.n_layers <= 0 || p.B <= 0 || p.B > 32 || p.n_want <= 0 || p.n_want > p.B ||
      p.H % 8 || p.I % 8 || p.H <= 0 || p.I <= 0 || p.nh <= 0 || p.nkv <= 0 || p.nh % p.nkv ||
      p.nh / p.nkv > 8 || p.hd % 16 || p.hd < 16 || p.hd > 128 || p.bt != kDmTile ||
      p.n_splits <= 0 || p.n_splits > kDmTile || p.V <= 0 || ctas <= 0 || p.window < 0 ||
      !(floats[1] > 0.f) || (p.gu_block && (p.I % p.gu_block || p.gu_block % 8)))
    return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const int nt = p.B <= 8 ? 1 : (p.B <= 16 ? 2 : 4);
#define CRETIF_STEP(NT, HD16) return launch_step<NT, HD16>(p, ctas, st)
#define CRETIF_STEP_HD(HD16)                 \
  case HD16:                                 \
    if (nt == 1) CRETIF_STEP(1, HD16);       \
    if (nt == 2) CRETIF_STEP(2, HD16);       \
    CRETIF_STEP(4, HD16)
  switch (p.hd / 16) {          // the head sizes in use; others take the separate kernels
    CRETIF_STEP_HD(1); CRETIF_STEP_HD(2); CRETIF_STEP_HD(3); CRETIF_STEP_HD(4);
    CRETIF_STEP_HD(8);
  }
#undef CRETIF_STEP_HD
#undef CRETIF_STEP
  return kBadArgument;
}
