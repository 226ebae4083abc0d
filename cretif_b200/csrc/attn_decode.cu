// Decode attention over the block cache: one new query token per sequence, bfloat16.
//
// The reference walks the cached positions of one sequence serially with one block per
// query head (src/attention.cu:410-494).  Here the keys of every (sequence, key/value
// head) are cut into `n_splits` ranges of whole cache blocks so that a batch of one still
// fills the GPU; one CTA streams its range's K and V tiles once (bulk asynchronous copies
// of the contiguous block_tokens x head_dim tiles into shared memory, two stages deep) and
// serves all query heads that share the key/value head.  Scores, running maximum and sum
// are 32-bit.  The CTA that finishes last for a (sequence, key/value head) — found with a
// counter in global memory that it resets for the next launch — merges the ranges' partial
// results in a fixed order and writes the output, so there is no second launch.
//
// Scratch, provided by the caller: part_o [tokens, heads, n_splits, head_dim] and part_ml
// [tokens, heads, n_splits, 2] in float32, and `counters` [tokens * kv_heads] int32 that must
// be zero before the first launch (every launch leaves them zero).
#include "api.h"
#include "common.cuh"

namespace cretif {

constexpr int kDecThreads = 128;
constexpr int kDecTile = 64;          // keys per tile = tokens per cache block
constexpr int kDecStages = 2;
constexpr int kDecMaxGroup = 8;       // query heads per key/value head
constexpr unsigned kSpinLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// Bounded wait: false if the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// grid (n_splits, nkv, B); GMAX >= heads per key/value head, fixed at compile time so that
// the per-head accumulators stay in registers.
template <int GMAX>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                   const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                   const int* __restrict__ table, int table_stride,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                   const int* __restrict__ seq_slot, int nh, int nkv, int hd, float scale,
                   int window, float* __restrict__ part_o, float* __restrict__ part_ml,
                   __nv_bfloat16* __restrict__ out, int ldo, int* __restrict__ counters,
                   unsigned int* __restrict__ fault) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int is_last;
  // A kernel launched behind this one with programmatic serialization may start its
  // prologue now; it still waits for this grid to finish before it reads the output.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int g = nh / nkv;
  const int split = blockIdx.x, n_splits = gridDim.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int pos = tok_pos[b];
  const int slot = seq_slot[tok_seq[b]];
  const int* tab = table + (size_t)slot * table_stride;
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int first_tile = first_key / kDecTile, n_tiles = pos / kDecTile + 1;
  const int per = (n_tiles - first_tile + n_splits - 1) / n_splits;
  const int t_begin = first_tile + split * per, t_end = min(n_tiles, t_begin + per);

  // shared memory carve-up
  const int tile_elems = kDecTile * hd;
  __nv_bfloat16* ktile = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [stages][tile]
  __nv_bfloat16* vtile = ktile + (size_t)kDecStages * tile_elems;                 // [stages][tile]
  float* qs = reinterpret_cast<float*>(vtile + (size_t)kDecStages * tile_elems);  // [g][hd]
  float* ps = qs + g * hd;                                                        // [g][tile]
  float* alpha = ps + g * kDecTile;                                               // [g]
  uint64_t* bars = reinterpret_cast<uint64_t*>(alpha + kDecMaxGroup);              // [stages]
  float* red = reinterpret_cast<float*>(bars + kDecStages);       // [groups][chunks][8]

  float* po = part_o + (((size_t)b * nh + (size_t)kvh * g) * n_splits + split) * hd;
  float* pml = part_ml + (((size_t)b * nh + (size_t)kvh * g) * n_splits + split) * 2;
  const bool empty_range = t_begin >= t_end;
  if (empty_range) {                   // nothing in this range: an empty partial
    for (int j = 0; j < g; ++j) {
      if (tid == 0) { pml[(size_t)j * n_splits * 2] = -INFINITY; pml[(size_t)j * n_splits * 2 + 1] = 0.f; }
      for (int d = tid; d < hd; d += kDecThreads) po[(size_t)j * n_splits * hd + d] = 0.f;
    }
  }

  // Thread 0 sets up the barriers and asks for the first tiles at once; the others fill the
  // query buffer meanwhile.
  const uint32_t tile_bytes = (uint32_t)tile_elems * 2u;
  auto issue = [&](int tile, int stage) {
    const int blk = tab[tile];
    if (blk < 0) { atomicOr(fault, kFaultBlockTable); }
    const size_t off = ((size_t)max(blk, 0) * nkv + kvh) * tile_elems;
    mbar_expect_tx(&bars[stage], 2u * tile_bytes);
    bulk_load(ktile + (size_t)stage * tile_elems, kc + off, tile_bytes, &bars[stage]);
    bulk_load(vtile + (size_t)stage * tile_elems, vc + off, tile_bytes, &bars[stage]);
  };
  if (tid == 0 && !empty_range) {
    for (int s = 0; s < kDecStages; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    issue(t_begin, 0);
    if (t_begin + 1 < t_end) issue(t_begin + 1, 1);
  }
  for (int i = tid; i < g * hd; i += kDecThreads) {
    const int j = i / hd, d = i - j * hd;
    qs[i] = __bfloat162float(q[(size_t)b * ldq + (size_t)(kvh * g + j) * hd + d]);
  }
  __syncthreads();

  // thread roles
  const int key_r = tid >> 1, half = tid & 1;            // QK: 2 threads per key
  const int half_dims = hd >> 1, half_chunks = half_dims >> 3;
  const int n_chunks = hd >> 3;                          // PV: 8-dim chunks
  const int n_groups = kDecThreads / n_chunks;
  const int pv_chunk = tid % n_chunks, pv_group = tid / n_chunks;
  const bool pv_active = pv_group < n_groups;

  float acc[GMAX][8];
#pragma unroll
  for (int j = 0; j < GMAX; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  // Heads are owned by warps: warp w owns heads w, w+4, ...; the running maximum and sum
  // of a warp's heads live in registers of all its lanes (same value), indexed by j / 4.
  constexpr int kOwn = (GMAX + 3) / 4;
  float m_own[kOwn], l_own[kOwn];
#pragma unroll
  for (int i = 0; i < kOwn; ++i) { m_own[i] = -INFINITY; l_own[i] = 0.f; }
  const int warp = tid >> 5, lane = tid & 31;
  bool ok = true;

  for (int tile = t_begin; tile < t_end; ++tile) {
    const int it = tile - t_begin, stage = it & 1;
    const bool got = mbar_wait(&bars[stage], (uint32_t)((it >> 1) & 1));
    if (!__syncthreads_and(got)) { ok = false; break; }      // the same decision for all
    const __nv_bfloat16* kt = ktile + (size_t)stage * tile_elems;
    const __nv_bfloat16* vt = vtile + (size_t)stage * tile_elems;
    const int key0 = tile * kDecTile;

    // ---- scores: s[j][r] = (q_j . k_r) * scale
    {
      float dot[GMAX];
#pragma unroll
      for (int j = 0; j < GMAX; ++j) dot[j] = 0.f;
      const __nv_bfloat16* krow = kt + (size_t)key_r * hd + half * half_dims;
      for (int i = 0; i < half_chunks; ++i) {
        const int c = (i + key_r) % half_chunks;          // rotate: spreads banks across rows
        float kv[8];
        load8(krow + c * 8, kv);
        const float* qp = qs + half * half_dims + c * 8;
#pragma unroll
        for (int j = 0; j < GMAX; ++j) {
          if (j < g) {
            const float4 q0 = *reinterpret_cast<const float4*>(qp + j * hd);
            const float4 q1 = *reinterpret_cast<const float4*>(qp + j * hd + 4);
            dot[j] = fmaf(q0.x, kv[0], dot[j]); dot[j] = fmaf(q0.y, kv[1], dot[j]);
            dot[j] = fmaf(q0.z, kv[2], dot[j]); dot[j] = fmaf(q0.w, kv[3], dot[j]);
            dot[j] = fmaf(q1.x, kv[4], dot[j]); dot[j] = fmaf(q1.y, kv[5], dot[j]);
            dot[j] = fmaf(q1.z, kv[6], dot[j]); dot[j] = fmaf(q1.w, kv[7], dot[j]);
          }
        }
      }
      const int key = key0 + key_r;
      const bool valid = key <= pos && key >= first_key;
#pragma unroll
      for (int j = 0; j < GMAX; ++j) {
        if (j < g) {
          const float full = dot[j] + __shfl_xor_sync(0xffffffffu, dot[j], 1);
          if (half == 0) ps[j * kDecTile + key_r] = valid ? full * scale : -INFINITY;
        }
      }
    }
    __syncthreads();

    // ---- running maximum and sum per head; p = exp(s - m) back into ps
#pragma unroll
    for (int o = 0; o < kOwn; ++o) {
      const int j = warp + 4 * o;
      if (j >= g) break;
      const float s0 = ps[j * kDecTile + lane], s1 = ps[j * kDecTile + 32 + lane];
      const float m_new = fmaxf(m_own[o], warp_max(fmaxf(s0, s1)));
      // a tile can be fully masked only at a window's edge; then m_new stays -inf
      const float p0 = (s0 == -INFINITY) ? 0.f : expf(s0 - m_new);
      const float p1 = (s1 == -INFINITY) ? 0.f : expf(s1 - m_new);
      const float corr = (m_own[o] == -INFINITY) ? 0.f : expf(m_own[o] - m_new);
      l_own[o] = l_own[o] * corr + warp_sum(p0 + p1);
      m_own[o] = m_new;
      ps[j * kDecTile + lane] = p0;
      ps[j * kDecTile + 32 + lane] = p1;
      if (lane == 0) alpha[j] = corr;
    }
    __syncthreads();

    // ---- o_j = o_j * alpha_j + sum_r p[j][r] * v[r]
    if (pv_active) {
#pragma unroll
      for (int j = 0; j < GMAX; ++j) {
        if (j < g) {
          const float a = alpha[j];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[j][e] *= a;
        }
      }
      for (int r = pv_group; r < kDecTile; r += n_groups) {
        float vv[8];
        load8(vt + (size_t)r * hd + pv_chunk * 8, vv);
#pragma unroll
        for (int j = 0; j < GMAX; ++j) {
          if (j < g) {
            const float p = ps[j * kDecTile + r];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(p, vv[e], acc[j][e]);
          }
        }
      }
    }
    __syncthreads();                    // the stage's tiles and ps are free again
    if (tid == 0 && tile + 2 < t_end) issue(tile + 2, stage);
  }

  if (!ok) {
    // A copy never arrived.  Flag it, give copies still in flight one more bounded chance to
    // land before this CTA's shared memory is handed to another, and write what was summed.
    if (tid == 0) {
      atomicOr(fault, kFaultWaitExpired);
      for (int s = 0; s < kDecStages; ++s) mbar_wait(&bars[s], 0u);
    }
    __syncthreads();
  }

  // ---- reduce the key groups' accumulators and write the partial
#pragma unroll
  for (int j = 0; j < GMAX; ++j) {
    if (j >= g || empty_range) break;
    __syncthreads();
    if (pv_active) {
#pragma unroll
      for (int e = 0; e < 8; ++e) red[(pv_group * n_chunks + pv_chunk) * 8 + e] = acc[j][e];
    }
    __syncthreads();
    for (int d = tid; d < hd; d += kDecThreads) {
      const int c = d >> 3, e = d & 7;
      float sum = 0.f;
      for (int grp = 0; grp < n_groups; ++grp) sum += red[(grp * n_chunks + c) * 8 + e];
      po[(size_t)j * n_splits * hd + d] = sum;
    }
    if ((j & 3) == warp && lane == 0) {
      float mj = -INFINITY, lj = 0.f;
#pragma unroll
      for (int o = 0; o < kOwn; ++o)
        if (o == (j >> 2)) { mj = m_own[o]; lj = l_own[o]; }
      pml[(size_t)j * n_splits * 2] = mj;
      pml[(size_t)j * n_splits * 2 + 1] = lj;
    }
  }

  // ---- the CTA that finishes last for this (sequence, kv head) merges the ranges
  __syncthreads();                       // the CTA's partial is written ...
  if (tid == 0) {
    __threadfence();                     // ... and made visible to the device by one fence
    int* ctr = counters + (size_t)b * nkv + kvh;
    const int prev = atomicAdd(ctr, 1);
    is_last = prev == n_splits - 1;
    if (is_last) {
      *ctr = 0;                          // ready for the next launch
      __threadfence();                   // the other CTAs' partials are read after this
    }
  }
  __syncthreads();
  if (!is_last) return;
  float* wts = ps;                       // [g][n_splits] weights, reusing the score buffer
  float* inv_den = alpha;                // [g]
  const float* ml_base = part_ml + ((size_t)b * nh + (size_t)kvh * g) * n_splits * 2;
  const float* po_base = part_o + ((size_t)b * nh + (size_t)kvh * g) * n_splits * hd;
  for (int j = warp; j < g; j += 4) {
    float mx = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) mx = fmaxf(mx, __ldcg(ml_base + ((size_t)j * n_splits + s) * 2));
    mx = warp_max(mx);
    float den = 0.f;
    for (int s = lane; s < n_splits; s += 32) {
      const float ms = __ldcg(ml_base + ((size_t)j * n_splits + s) * 2);
      const float ls = __ldcg(ml_base + ((size_t)j * n_splits + s) * 2 + 1);
      const float w = (ms == -INFINITY) ? 0.f : expf(ms - mx);
      if (j * n_splits + s < GMAX * kDecTile) wts[j * n_splits + s] = w;
      den += w * ls;
    }
    den = warp_sum(den);
    if (lane == 0) inv_den[j] = 1.0f / den;
  }
  __syncthreads();
  for (int i = tid; i < g * hd; i += kDecThreads) {
    const int j = i / hd, d = i - j * hd;
    float acc_o = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 16) {       // 16 loads in flight, summed in order
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        v[u] = s0 + u < n_splits ? __ldcg(po_base + ((size_t)j * n_splits + s0 + u) * hd + d) : 0.f;
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (s0 + u < n_splits) acc_o = fmaf(wts[j * n_splits + s0 + u], v[u], acc_o);
    }
    out[(size_t)b * ldo + (size_t)(kvh * g + j) * hd + d] = __float2bfloat16_rn(acc_o * inv_den[j]);
  }
}

static size_t decode_smem_bytes(int g, int hd) {
  const int n_chunks = hd / 8, n_groups = kDecThreads / n_chunks;
  size_t bytes = (size_t)2 * kDecStages * kDecTile * hd * 2;        // K and V tiles
  bytes += (size_t)(g * hd + g * kDecTile + kDecMaxGroup) * 4;      // q, p, alpha
  bytes += kDecStages * 8;                                          // barriers
  bytes += (size_t)n_groups * n_chunks * 8 * 4;                     // reduction
  return bytes;
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_attn_decode_scratch_floats(int B, int nh, int hd, int n_splits,
                                                 long long* part_o, long long* part_ml) {
  *part_o = (long long)B * nh * n_splits * hd;
  *part_ml = (long long)B * nh * n_splits * 2;
  return kOk;
}

extern "C" int cretif_attn_decode(const void* q, int ldq, void* out, int ldo, const void* kc,
                                  const void* vc, const int* table, int table_stride,
                                  const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                  int nh, int nkv, int hd, float scale, int window, int bt, int B,
                                  int n_splits, float* part_o, float* part_ml, int* counters,
                                  unsigned int* fault, void* stream) {
  if (B <= 0) return kOk;
  if (nh <= 0 || nkv <= 0 || nh % nkv || nh / nkv > kDecMaxGroup || hd % 16 || hd < 16 ||
      hd > 256 || bt != kDecTile || n_splits <= 0 || n_splits > kDecTile || nkv > 65535 ||
      B > 65535 || window < 0)
    return kBadArgument;
  if (((uintptr_t)kc | (uintptr_t)vc) & 15) return kMisaligned;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = nh / nkv;
  const size_t smem = decode_smem_bytes(g, hd);
  dim3 grid(n_splits, nkv, B);
  int rc;
#define CRETIF_DECODE(GMAX)                                                                     \
  do {                                                                                          \
    static size_t configured = 0;                                                               \
    if (smem > configured) {                                                                    \
      cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<GMAX>,                            \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                           (int)smem);                                          \
      if (e != cudaSuccess) return (int)e;                                                      \
      configured = smem;                                                                        \
    }                                                                                           \
    attn_decode_kernel<GMAX><<<grid, kDecThreads, smem, st>>>(                                  \
        (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, table, \
        table_stride, tok_pos, tok_seq, seq_slot, nh, nkv, hd, scale, window, part_o, part_ml,  \
        (__nv_bfloat16*)out, ldo, counters, fault);                                             \
    rc = launch_status();                                                                       \
  } while (0)
  if (g == 1) CRETIF_DECODE(1);
  else if (g == 2) CRETIF_DECODE(2);
  else if (g <= 4) CRETIF_DECODE(4);
  else CRETIF_DECODE(8);
#undef CRETIF_DECODE
  return rc;
}
