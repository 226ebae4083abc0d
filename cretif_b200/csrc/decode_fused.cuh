// Fused decode projections: the weight-streaming product of gemm_skinny.cu with the work
// that surrounds it in a decode step folded into its prologue and epilogue, so that a
// layer needs five launches instead of ten:
//
//   prologue NORM   x = bf16(h * w_norm * rsqrt(mean(h^2) + eps)) computed by every CTA from the
//                   32-bit residual stream (a few KB for a decode batch) into shared memory,
//                   optionally from gathered rows (the rows whose logits are wanted); with
//                   more than 8 rows the CTAs of a thread-block cluster share that work;
//   epilogue ROPE   the stacked q|k|v product: rotary pairs of q and k are rotated in 32-bit,
//                   q goes to the query buffer, rotated k and v go straight into the block
//                   cache at each token's position;
//   epilogue SILU   the stacked gate|up product: act = silu(gate) * up;
//   epilogue PLAIN  store (bfloat16 / float32) or add into the 32-bit residual stream.
//
// To make the epilogues local, a CTA's 16 weight rows are not consecutive: for ROPE they are
// the two halves of 8 rotary pairs, for SILU 8 gate rows and the 8 up rows below them.  The
// 8-row distance is exactly the distance between the two accumulator rows a lane of the
// m16n8k16 product holds, and after the warps' partial sums have met in shared memory one
// thread finishes one pair.
//
// Arithmetic is the unfused kernels' (elementwise.cu), so a token gets the same numbers
// whichever path ran it.  The reference fuses only residual + norm
// (src/kernels/elementwise.cu:463-506).
#pragma once

#include "api.h"
#include "common.cuh"

namespace cretif {

constexpr int kFuWarps = 8;
constexpr int kFuRows = 16;
enum Prologue : int { kProPlain = 0, kProNorm = 1 };
enum Epilogue : int { kEpiPlain = 0, kEpiRope = 1, kEpiSilu = 2 };

// n / d for 0 <= n < 65536 without a division instruction (an integer division in the short
// dependent chains of these kernels costs about 0.1 us): a shift for powers of two, else a
// multiplication by ceil(2^32 / d), exact for n, d < 65536.
struct FastDiv {
  int d, shift;
  uint32_t magic;
};
__host__ __device__ inline FastDiv make_fast_div(int d) {
  FastDiv f = {d > 0 ? d : 1, -1, 0u};
  if ((f.d & (f.d - 1)) == 0) {
    f.shift = 0;
    while ((1 << f.shift) < f.d) ++f.shift;
  } else {
    f.magic = 0xffffffffu / (uint32_t)f.d + 1u;
  }
  return f;
}
__device__ __forceinline__ int fast_div(const FastDiv& f, int n) {
  return f.shift >= 0 ? n >> f.shift : (int)__umulhi((uint32_t)n, f.magic);
}

struct FusedParams {
  // product
  const __nv_bfloat16* W;   // [N, K]
  int M, N, K, ldw;
  // prologue
  const __nv_bfloat16* X;   // plain: [M, K] bf16
  int ldx;
  const float* H;           // norm: residual stream [*, K]
  const float* norm_w;      // [K]
  const int* rows;          // optional gather: x row m comes from H[rows[m]]
  float eps;
  // epilogue plain
  void* C;
  int ldc, c_dt, accumulate;
  // epilogue rope
  __nv_bfloat16* Q;         // [M, nh*hd]
  int ldq;
  const float* cos_t;
  const float* sin_t;
  int pairing, nh, nkv, hd;
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const int* table;
  int table_stride;
  __nv_bfloat16* kc;
  __nv_bfloat16* vc;
  int bt, write_cache;
  unsigned int* fault;
  // epilogue silu
  __nv_bfloat16* act;       // [M, I]
  int I, gu_block;          // gu_block > 0: gate/up rows interleaved in groups of that size
  // set by the launcher from the above
  FastDiv gu_div, tph_div;  // by gu_block; by tiles per head (hd / 16)
  int bt_shift;             // log2 of bt (a power of two)
};

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Fills the derived fields; false if a size is outside what they can express.
__host__ __device__ inline bool derive_fields(FusedParams& p) {
  p.gu_div = make_fast_div(p.gu_block > 0 ? p.gu_block : 1);
  p.tph_div = make_fast_div(p.hd >= 16 ? p.hd >> 4 : 1);
  p.bt_shift = 0;
  if (p.bt > 0) {
    if (p.bt & (p.bt - 1)) return false;                 // cache blocks are powers of two
    while ((1 << p.bt_shift) < p.bt) ++p.bt_shift;
  }
  // the multiplication that stands for a division is exact below 65536
  if (p.gu_div.shift < 0 && (p.I >= 65536 || p.gu_block >= 65536)) return false;
  return true;
}

// Weight row of tile row r (0..15) of CTA `tile`; -1 if beyond the matrix.
template <int EPI>
__device__ __forceinline__ int tile_row(const FusedParams& p, int tile, int r) {
  if (EPI == kEpiPlain) {
    const int n = tile * kFuRows + r;
    return n < p.N ? n : -1;
  } else if (EPI == kEpiSilu) {
    const int i = tile * 8 + (r & 7);
    if (i >= p.I) return -1;
    if (p.gu_block) {
      const int blk = fast_div(p.gu_div, i);        // i = blk * gu_block + rest
      const int g = i + blk * p.gu_block;           // = blk * 2 gu_block + rest
      return r < 8 ? g : g + p.gu_block;
    }
    return r < 8 ? i : p.I + i;
  } else {
    const int tiles_per_head = p.hd >> 4;
    const int head = fast_div(p.tph_div, tile), t = tile - head * tiles_per_head;
    if (head >= p.nh + p.nkv) return head * p.hd + t * 16 + r;        // v: plain rows
    const int j = t * 8 + (r & 7);                                    // rotary pair index
    if (p.pairing) return head * p.hd + 2 * j + (r >> 3);
    return head * p.hd + j + (r >> 3) * (p.hd >> 1);
  }
}

// What a tile's epilogue reads from memory besides the accumulator — the token's position,
// its cache block and rotation, or the value it adds to — does not depend on the product.
// It is asked for before the product runs, so that the epilogue does not wait for it.
// (A tile has 16 weight rows and up to 8 NT tokens: the plain epilogue makes ceil(NT / 2)
// passes of the block's 256 threads over its 128 NT outputs, the pair epilogues ceil(NT / 4)
// over its 64 NT pairs.)
template <int NT>
struct EpiAhead {
  static constexpr int kPlainPasses = NT >= 2 ? NT / 2 : 1;
  static constexpr int kPairPasses = NT >= 4 ? NT / 4 : 1;
  float old[kPlainPasses];        // plain, accumulate: the values to add to
  int pos[kPairPasses], blk[kPairPasses];        // rope
  float cs[kPairPasses], sn[kPairPasses];
};

template <int NT, int EPI>
__device__ __forceinline__ void epi_prefetch(const FusedParams& p, int tile, EpiAhead<NT>& a) {
  if (EPI == kEpiPlain) {
    if (p.c_dt == kF32 && p.accumulate) {
#pragma unroll
      for (int it = 0; it < EpiAhead<NT>::kPlainPasses; ++it) {
        const int i = threadIdx.x + it * kFuWarps * 32;
        const int m = i / kFuRows, n = tile * kFuRows + (i - m * kFuRows);
        a.old[it] = (m < p.M && n < p.N)
                        ? __ldcg(reinterpret_cast<const float*>(p.C) + (size_t)m * p.ldc + n)
                        : 0.f;
      }
    }
  } else if (EPI == kEpiRope) {
#pragma unroll
    for (int it = 0; it < EpiAhead<NT>::kPairPasses; ++it) {
      const int i = threadIdx.x + it * kFuWarps * 32;
      a.pos[it] = 0; a.blk[it] = -1; a.cs[it] = 1.f; a.sn[it] = 0.f;
      if (i < 8 * p.M) {
        const int m = i >> 3, pr = i & 7;
        const int tiles_per_head = p.hd >> 4;
        const int head = fast_div(p.tph_div, tile), t = tile - head * tiles_per_head;
        a.pos[it] = p.tok_pos[m];
        if (head >= p.nh && p.write_cache)
          a.blk[it] = p.table[(size_t)p.seq_slot[p.tok_seq[m]] * p.table_stride +
                              (a.pos[it] >> p.bt_shift)];
        if (head < p.nh + p.nkv) {
          const int j = t * 8 + pr;
          a.cs[it] = p.cos_t[(size_t)a.pos[it] * (p.hd >> 1) + j];
          a.sn[it] = p.sin_t[(size_t)a.pos[it] * (p.hd >> 1) + j];
        }
      }
    }
  }
}

template <int NT, int EPI>
__device__ __forceinline__ void finish_tile(const FusedParams& p, int tile,
                                            float (*red)[kFuRows][8 * NT + 1],
                                            const EpiAhead<NT>& ahead) {
  if (EPI == kEpiPlain) {
#pragma unroll
    for (int it = 0; it < EpiAhead<NT>::kPlainPasses; ++it) {
      const int i = threadIdx.x + it * kFuWarps * 32;
      if (i >= kFuRows * p.M) break;
      const int m = i / kFuRows, rr = i - m * kFuRows;
      const int n = tile * kFuRows + rr;
      if (n >= p.N) continue;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kFuWarps; ++w) sum += red[w][rr][m];
      if (p.c_dt == kF32) {
        float* out = reinterpret_cast<float*>(p.C) + (size_t)m * p.ldc + n;
        if (p.accumulate) sum += ahead.old[it];
        *out = sum;
      } else {
        reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(sum);
      }
    }
  } else {
    // one thread per (token, pair): rows pr and pr + 8 of the tile
#pragma unroll
    for (int it = 0; it < EpiAhead<NT>::kPairPasses; ++it) {
      const int i = threadIdx.x + it * kFuWarps * 32;
      if (i >= 8 * p.M) break;
      const int m = i >> 3, pr = i & 7;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int w = 0; w < kFuWarps; ++w) { s0 += red[w][pr][m]; s1 += red[w][pr + 8][m]; }
      if (EPI == kEpiSilu) {
        const int col = tile * 8 + pr;
        if (col >= p.I) continue;
        // the unfused path stores gate and up as bfloat16 before the activation
        const float g = __bfloat162float(__float2bfloat16_rn(s0));
        const float u = __bfloat162float(__float2bfloat16_rn(s1));
        p.act[(size_t)m * p.I + col] = __float2bfloat16_rn(silu_bf16_path(g) * u);
      } else {
        const int tiles_per_head = p.hd >> 4;
        const int head = fast_div(p.tph_div, tile), t = tile - head * tiles_per_head;
        const int pos = ahead.pos[it];
        size_t cache_row = 0;
        bool cache_ok = false;
        if (head >= p.nh && p.write_cache) {
          const int blk = ahead.blk[it];
          if (blk < 0) atomicOr(p.fault, kFaultBlockTable);
          else {
            cache_ok = true;
            const int kvh = head < p.nh + p.nkv ? head - p.nh : head - p.nh - p.nkv;
            cache_row = (((size_t)blk * p.nkv + kvh) * p.bt + (pos & (p.bt - 1))) * p.hd;
          }
        }
        if (head >= p.nh + p.nkv) {                      // v: rows t*16 + pr and + 8, no rotation
          if (cache_ok) {
            p.vc[cache_row + t * 16 + pr] = __float2bfloat16_rn(s0);
            p.vc[cache_row + t * 16 + pr + 8] = __float2bfloat16_rn(s1);
          }
          continue;
        }
        const int j = t * 8 + pr;
        const int i0 = p.pairing ? 2 * j : j, i1 = p.pairing ? 2 * j + 1 : j + (p.hd >> 1);
        // the unfused path stores q and k as bfloat16 before rotating them
        const float x0 = __bfloat162float(__float2bfloat16_rn(s0));
        const float x1 = __bfloat162float(__float2bfloat16_rn(s1));
        const float cs = ahead.cs[it], sn = ahead.sn[it];
        const __nv_bfloat16 y0 = __float2bfloat16_rn(x0 * cs - x1 * sn);
        const __nv_bfloat16 y1 = __float2bfloat16_rn(x0 * sn + x1 * cs);
        if (head < p.nh) {
          __nv_bfloat16* q = p.Q + (size_t)m * p.ldq + (size_t)head * p.hd;
          q[i0] = y0;
          q[i1] = y1;
        } else if (cache_ok) {
          p.kc[cache_row + i0] = y0;
          p.kc[cache_row + i1] = y1;
        }
      }
    }
  }
}

// The norm prologue: x[m] = bf16(h[row m] * w * rsqrt(mean(h^2) + eps)) into shared memory, a
// warp per token.  A row of up to 128 * REGS columns makes one trip from memory: the lane
// keeps its REGS float4 in registers between the sum of squares and the scaling.
//
// The norm's weight depends on nothing that runs before the kernel.  For K <= 1024 N the
// CTA's threads fetch it (N float4 each) before the kernel waits for the one before it
// (norm_weight_fetch), and put it into shared memory (`nws`) once the first residual rows
// have been asked for, so that its latency and theirs do not add up.
template <int N>
struct NormStash {
  static constexpr int kMaxK = N * kFuWarps * 32 * 4;
  float4 w[N];
};

template <int N>
__device__ __forceinline__ void norm_weight_fetch(const FusedParams& p, NormStash<N>& st) {
  const int n4 = p.K >> 2;
  const float4* w4 = reinterpret_cast<const float4*>(p.norm_w);
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const int i = threadIdx.x + u * kFuWarps * 32;
    st.w[u] = (p.K <= NormStash<N>::kMaxK && i < n4) ? __ldg(w4 + i)
                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Called by the kFuWarps * 32 threads that also called norm_weight_fetch; `sync` is the
// barrier among exactly those threads, run once by each after its first loads are issued.
template <int REGS, int N, typename Sync>
__device__ __forceinline__ void norm_rows_to_smem(const FusedParams& p, unsigned char* xs,
                                                  int xs_stride, int warp, int lane, float4* nws,
                                                  const NormStash<N>& st, Sync sync) {
  const int n4 = p.K >> 2;
  const bool stash = p.K <= NormStash<N>::kMaxK;
  const float4* w4 = reinterpret_cast<const float4*>(p.norm_w);
  bool first = true;
  for (int m = warp; m < p.M || first; m += kFuWarps) {
    const bool row = m < p.M;
    const float4* h4 = reinterpret_cast<const float4*>(
        p.H + (size_t)(row ? (p.rows ? p.rows[m] : m) : 0) * p.K);
    __nv_bfloat16* xr = reinterpret_cast<__nv_bfloat16*>(xs + (size_t)m * xs_stride);
    const bool fits = n4 <= 32 * REGS;
    float4 v[REGS];
    if (row && fits) {
#pragma unroll
      for (int u = 0; u < REGS; ++u) {
        const int i = u * 32 + lane;
        v[u] = i < n4 ? __ldcg(h4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (first) {
      first = false;
      if (stash) {
#pragma unroll
        for (int u = 0; u < N; ++u) {
          const int i = warp * 32 + lane + u * kFuWarps * 32;
          if (i < n4) nws[i] = st.w[u];
        }
      }
      sync();                 // always, and by every warp: the caller may count on it
    }
    if (!row) break;
    auto weight = [&](int i) { return stash ? nws[i] : __ldg(w4 + i); };
    auto put = [&](int i, const float4& t, float inv) {
      const float4 w = weight(i);
      __nv_bfloat162 lo = __floats2bfloat162_rn(t.x * w.x * inv, t.y * w.y * inv);
      __nv_bfloat162 hi = __floats2bfloat162_rn(t.z * w.z * inv, t.w * w.w * inv);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(xr + 4 * i) = pk;
    };
    float ss = 0.f;
    if (fits) {
#pragma unroll
      for (int u = 0; u < REGS; ++u)
        ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)p.K + p.eps);
#pragma unroll
      for (int u = 0; u < REGS; ++u) {
        const int i = u * 32 + lane;
        if (i < n4) put(i, v[u], inv);
      }
    } else {
#pragma unroll 8
      for (int i = lane; i < n4; i += 32) {
        const float4 t = __ldcg(h4 + i);
        ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
      }
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)p.K + p.eps);
#pragma unroll 4
      for (int i = lane; i < n4; i += 32) put(i, __ldcg(h4 + i), inv);
    }
  }
}

// The same prologue shared by the CTAs of a thread-block cluster (all of one group of rows):
// every CTA needs every row, and 192 CTAs that each pull 32 rows of float32 through L2 spend
// more time on that than on their weights.  Here the cluster's warps take one row each
// (row = rank * 8 + warp, then on by the cluster's warps), and store the normed row into
// the shared memory of every CTA of the cluster; a cluster barrier ends the prologue.
constexpr int kFuClusterMax = 4;

template <int REGS, int N>
__device__ __forceinline__ void norm_rows_to_cluster(const FusedParams& p, unsigned char* xs,
                                                     int xs_stride, int warp, int lane,
                                                     float4* nws, const NormStash<N>& st,
                                                     uint32_t csize) {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int n4 = p.K >> 2;
  const bool stash = p.K <= NormStash<N>::kMaxK;
  const float4* w4 = reinterpret_cast<const float4*>(p.norm_w);
  const bool fits = n4 <= 32 * REGS;
  const uint32_t local = (uint32_t)__cvta_generic_to_shared(xs);
  uint32_t base[kFuClusterMax];
#pragma unroll
  for (uint32_t t = 0; t < (uint32_t)kFuClusterMax; ++t) {
    base[t] = local;
    if (t < csize)
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(base[t]) : "r"(local), "r"(t));
  }
  bool first = true;
  for (int m = (int)rank * kFuWarps + warp; m < p.M || first; m += (int)csize * kFuWarps) {
    const bool row = m < p.M;
    const float4* h4 = reinterpret_cast<const float4*>(
        p.H + (size_t)(row ? (p.rows ? p.rows[m] : m) : 0) * p.K);
    float4 v[REGS];
    if (row && fits) {
#pragma unroll
      for (int u = 0; u < REGS; ++u) {
        const int i = u * 32 + lane;
        v[u] = i < n4 ? __ldcg(h4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (first) {
      first = false;
      if (stash) {
#pragma unroll
        for (int u = 0; u < N; ++u) {
          const int i = warp * 32 + lane + u * kFuWarps * 32;
          if (i < n4) nws[i] = st.w[u];
        }
      }
      __syncthreads();
      // every CTA of the cluster signalled at its start (skinny_fused_tiles): once all have,
      // their shared memory exists and may be written from here
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (!row) break;
    const uint32_t row_off = (uint32_t)m * (uint32_t)xs_stride;
    auto put = [&](int i, const float4& t, float inv) {
      const float4 w = stash ? nws[i] : __ldg(w4 + i);
      __nv_bfloat162 lo = __floats2bfloat162_rn(t.x * w.x * inv, t.y * w.y * inv);
      __nv_bfloat162 hi = __floats2bfloat162_rn(t.z * w.z * inv, t.w * w.w * inv);
      const uint32_t a = *reinterpret_cast<uint32_t*>(&lo), b = *reinterpret_cast<uint32_t*>(&hi);
      const uint32_t off = row_off + 8u * (uint32_t)i;
#pragma unroll
      for (uint32_t t2 = 0; t2 < (uint32_t)kFuClusterMax; ++t2)
        if (t2 < csize)
          asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(base[t2] + off), "r"(a),
                       "r"(b)
                       : "memory");
    };
    float ss = 0.f;
    if (fits) {
#pragma unroll
      for (int u = 0; u < REGS; ++u)
        ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)p.K + p.eps);
#pragma unroll
      for (int u = 0; u < REGS; ++u) {
        const int i = u * 32 + lane;
        if (i < n4) put(i, v[u], inv);
      }
    } else {
#pragma unroll 8
      for (int i = lane; i < n4; i += 32) {
        const float4 t = __ldcg(h4 + i);
        ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
      }
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)p.K + p.eps);
#pragma unroll 4
      for (int i = lane; i < n4; i += 32) put(i, __ldcg(h4 + i), inv);
    }
  }
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

constexpr int kFuPre = 3;      // weight chunks per warp fetched ahead (covers K <= 768)

template <int EPI>
__device__ __forceinline__ void fetch_weights(const FusedParams& p, int tile, int warp, int r, int c,
                                              int n_chunks, uint4 (&pa)[kFuPre], uint4 (&pb)[kFuPre]) {
  const int row_a = tile_row<EPI>(p, tile, r), row_b = tile_row<EPI>(p, tile, r + 8);
  const __nv_bfloat16* wa = p.W + (size_t)max(row_a, 0) * p.ldw + c * 8;
  const __nv_bfloat16* wb = p.W + (size_t)max(row_b, 0) * p.ldw + c * 8;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int i = 0; i < kFuPre; ++i) {
    const int ch = warp + kFuWarps * i;
    const bool in = ch < n_chunks && ch * 32 + c * 8 < p.K;
    pa[i] = in ? __ldg(reinterpret_cast<const uint4*>(wa + ch * 32)) : zero;
    pb[i] = in ? __ldg(reinterpret_cast<const uint4*>(wb + ch * 32)) : zero;
  }
}

// The body of the fused product for the CTA's share of tiles: tiles first_tile,
// first_tile + tile_stride, ...  `pdl`: signal/await the neighbouring launches
// (programmatic dependent launch).
template <int NT, int PRO, int EPI>
__device__ __forceinline__ void skinny_fused_tiles(const FusedParams& p, int n_tiles,
                                                   unsigned char* fsmem, int first_tile,
                                                   int tile_stride, bool pdl) {
  if (first_tile >= n_tiles) return;          // (the whole CTA: nothing to do in this call)
  float(*red)[kFuRows][8 * NT + 1] = reinterpret_cast<float(*)[kFuRows][8 * NT + 1]>(fsmem);
  // x tile (norm prologue) after the reduction buffer; row stride ≡ 64 (mod 128) bytes so
  // that a quarter-warp's eight 16-byte reads touch all banks once
  const int xs_stride = ((p.K * 2 + 127) / 128) * 128 + 64;
  unsigned char* xs = fsmem + sizeof(float) * kFuWarps * kFuRows * (8 * NT + 1);
  xs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(xs) + 15) & ~uintptr_t(15));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  const int n_chunks = (p.K + 31) >> 5;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  // A cluster shares the norm prologue by storing into its CTAs' shared memory, which may
  // only be touched once every CTA of the cluster runs: each says so here, at no cost, and
  // waits for the others just before its first remote store (norm_rows_to_cluster).
  if (NT > 1 && PRO == kProNorm) {
    uint32_t csize = 1;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
    if (csize > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  }
  // The first tile's weights do not depend on anything computed before this kernel: ask for
  // them first, so that their latency runs under the prologue.
  int tile = first_tile;
  uint4 pa[kFuPre], pb[kFuPre];
  if (tile < n_tiles) fetch_weights<EPI>(p, tile, warp, r, c, n_chunks, pa, pb);
  // Programmatic dependent launch: the kernel behind this one may start its own weight
  // fetch now, and this one goes on to read activations only when the kernel before it has
  // finished (a no-op when the launch was an ordinary one).
  NormStash<1> stash;
  if (PRO == kProNorm) norm_weight_fetch(p, stash);
  // Positions, the block table and the rotation table are not the work of the kernel before
  // this one either: the first tile's epilogue operands are on their way before the wait
  // (a chain of four dependent loads that the short product would not hide).
  EpiAhead<NT> ahead;
  bool have_ahead = false;
  if (EPI == kEpiRope) {
    epi_prefetch<NT, EPI>(p, tile, ahead);
    have_ahead = true;
  }
  if (pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  if (PRO == kProNorm) {
    float4* nws = reinterpret_cast<float4*>(xs + (size_t)p.M * xs_stride);
    uint32_t csize = 1;        // (launched without clusters: 1)
    if (NT > 1) asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
    if (NT > 1 && csize > 1) {
      norm_rows_to_cluster<8>(p, xs, xs_stride, warp, lane, nws, stash, csize);
    } else {
      norm_rows_to_smem<8>(p, xs, xs_stride, warp, lane, nws, stash, [] { __syncthreads(); });
      __syncthreads();
    }
  }

  for (; tile < n_tiles; tile += tile_stride) {
    if (!have_ahead) epi_prefetch<NT, EPI>(p, tile, ahead);
    have_ahead = false;
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

    auto consume = [&](const uint4& ua, const uint4& ub, int ch) {
      const int k = ch * 32 + c * 8;
      const bool in = ch < n_chunks && k < p.K;
      const uint32_t a1[4] = {ua.x, ub.x, ua.y, ub.y};
      const uint32_t a2[4] = {ua.z, ub.z, ua.w, ub.w};
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int m = t * 8 + r;
        uint4 ux = zero;
        if (in && m < p.M) {
          if (PRO == kProNorm)
            ux = *reinterpret_cast<const uint4*>(xs + (size_t)m * xs_stride + (size_t)k * 2);
          else
            ux = __ldcg(reinterpret_cast<const uint4*>(p.X + (size_t)m * p.ldx + k));
        }
        mma_16816(acc[t], a1, ux.x, ux.y);
        mma_16816(acc[t], a2, ux.z, ux.w);
      }
    };
#pragma unroll
    for (int i = 0; i < kFuPre; ++i) consume(pa[i], pb[i], warp + kFuWarps * i);
    if (n_chunks > kFuWarps * kFuPre) {
      const int row_a = tile_row<EPI>(p, tile, r), row_b = tile_row<EPI>(p, tile, r + 8);
      const __nv_bfloat16* wa = p.W + (size_t)max(row_a, 0) * p.ldw + c * 8;
      const __nv_bfloat16* wb = p.W + (size_t)max(row_b, 0) * p.ldw + c * 8;
      for (int ch = warp + kFuWarps * kFuPre; ch < n_chunks; ch += 2 * kFuWarps) {
        const int ch2 = ch + kFuWarps;
        const bool in1 = ch * 32 + c * 8 < p.K, in2 = ch2 < n_chunks && ch2 * 32 + c * 8 < p.K;
        const uint4 ua1 = in1 ? __ldg(reinterpret_cast<const uint4*>(wa + ch * 32)) : zero;
        const uint4 ub1 = in1 ? __ldg(reinterpret_cast<const uint4*>(wb + ch * 32)) : zero;
        const uint4 ua2 = in2 ? __ldg(reinterpret_cast<const uint4*>(wa + ch2 * 32)) : zero;
        const uint4 ub2 = in2 ? __ldg(reinterpret_cast<const uint4*>(wb + ch2 * 32)) : zero;
        consume(ua1, ub1, ch);
        consume(ua2, ub2, ch2);
      }
    }
    // the next tile's weights travel while this tile is reduced and finished
    if (tile + tile_stride < n_tiles)
      fetch_weights<EPI>(p, tile + tile_stride, warp, r, c, n_chunks, pa, pb);

#pragma unroll
    for (int t = 0; t < NT; ++t) {
      red[warp][r][t * 8 + 2 * c] = acc[t][0];
      red[warp][r][t * 8 + 2 * c + 1] = acc[t][1];
      red[warp][r + 8][t * 8 + 2 * c] = acc[t][2];
      red[warp][r + 8][t * 8 + 2 * c + 1] = acc[t][3];
    }
    __syncthreads();
    finish_tile<NT, EPI>(p, tile, red, ahead);
    __syncthreads();
  }
}


// The parameters of rows m0 .. m0 + n - 1 of a call as a call of their own: everything that
// is indexed by the token moves along.
__host__ __device__ inline FusedParams rows_of(const FusedParams& p, int m0, int n) {
  FusedParams q = p;
  q.M = n;
  if (p.X) q.X = p.X + (size_t)m0 * p.ldx;
  if (p.rows) q.rows = p.rows + m0;
  else if (p.H) q.H = p.H + (size_t)m0 * p.K;
  if (p.C)
    q.C = static_cast<unsigned char*>(p.C) + (size_t)m0 * p.ldc * (p.c_dt == kF32 ? 4 : 2);
  if (p.Q) q.Q = p.Q + (size_t)m0 * p.ldq;
  if (p.tok_pos) q.tok_pos = p.tok_pos + m0;
  if (p.tok_seq) q.tok_seq = p.tok_seq + m0;
  if (p.act) q.act = p.act + (size_t)m0 * p.I;
  return q;
}

// More than kFuMaxGroupRows tokens run as groups of rows along gridDim.y: every group reads
// the whole matrix (the second time from L2), which for a few dozen tokens is still far
// cheaper than a tensor-core tile of 128 tokens on a handful of CTAs.
constexpr int kFuMaxGroupRows = 32;
constexpr int kFuMaxRows = 128;

template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(kFuWarps * 32, 2)
skinny_fused_kernel(const FusedParams p, int n_tiles, int group_rows) {
  extern __shared__ __align__(16) unsigned char fsmem_k[];
  const int m0 = blockIdx.y * group_rows;            // one group: all rows from 0
  const FusedParams q = rows_of(p, m0, min(group_rows, p.M - m0));
  skinny_fused_tiles<NT, PRO, EPI>(q, n_tiles, fsmem_k, blockIdx.x, gridDim.x, true);
}

inline size_t fused_smem(int nt, int pro, int M, int K) {
  size_t bytes = sizeof(float) * kFuWarps * kFuRows * (8 * nt + 1) + 16;
  if (pro == kProNorm)     // normed x, and the norm's weight when it is kept (kNormStashK)
    bytes += (size_t)M * (((K * 2 + 127) / 128) * 128 + 64) + (K <= NormStash<1>::kMaxK ? (size_t)K * 4 : 0);
  return bytes;
}

}  // namespace cretif
