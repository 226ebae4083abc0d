// Causal grouped-query attention for whole prompts on the tcgen05 tensor cores, bfloat16.
//
// One CTA owns 128 consecutive query tokens of one sequence and one query head.  It walks
// the sequence's cache blocks up to the diagonal, two 64-key blocks (128 keys) per step:
//   warp 0     TMA producer: the Q tile once, then K and V tiles of each block straight out
//              of the block cache (a block's [64 x head_dim] tile of a key/value head is one
//              2-d box) into a ring of shared-memory stages;
//   warp 1     one thread issues S = Q K^T (tcgen05.mma, accumulator in tensor memory), and
//              after the softmax threads have written P, O_blk = P V (V is the MN-major
//              operand, exactly as it lies in the cache);
//   warps 2-9  softmax: two threads share one query row (64 of the step's keys and half of the
//              output columns each); they read S from tensor memory, keep the running
//              maximum and sum in 32-bit, write P as bfloat16 into shared memory in the
//              swizzled operand layout, then fold O_blk into their part of the output row,
//              which stays in registers.
// S, P and O_blk exist twice (for head sizes up to 64; larger heads have one P): the scores
// of step j + 1 are computed while the softmax of step j runs, and the softmax threads fold
// O_blk of step j in only after they have sent P of step j + 1, so they never wait for a
// product.  What bounds a step then is the softmax itself: 128 x 128 exponentials at the
// special-function unit's 16 a cycle.  Heavy query tiles (late queries) of all heads and
// sequences are handed out before any lighter one.
// The reference materialises [heads, S, kv_len] scores and transposes the cache for every
// call (src/attention.cu:644-728); nothing of that exists here.
//
// Queries of the next sequence that fall into a tile's 128 rows are computed and dropped.
#include <cuda.h>
#include <cuda_runtime.h>

#include "api.h"
#include "tc_common.cuh"

namespace cretif {

int make_tile_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int ld,
                       int box_rows);

constexpr int kPfThreads = 320;   // producer, MMA issuer, eight softmax warps
constexpr int kPfBQ = 128;       // queries per CTA
constexpr int kPfBlk = 64;       // tokens per cache block
constexpr int kPfBK = 128;       // keys per step: two cache blocks
constexpr int kPfMaxStages = 3;   // ring of K/V stages: 3 for head sizes up to 64, else 2

struct PfSmem {
  // byte offsets for a head size with n_sub 64-wide column groups
  int q, p, k, v, bars, xch, total, stages, p_bufs;
  __host__ __device__ explicit PfSmem(int n_sub) {
    stages = n_sub == 1 ? 3 : 2;
    p_bufs = n_sub == 1 ? 2 : 1;      // two P tiles: the softmax runs one step ahead of P V
    q = 0;
    p = q + n_sub * kPfBQ * 128;
    k = p + p_bufs * (kPfBK / 64) * kPfBQ * 128;
    v = k + stages * n_sub * kPfBK * 128;
    bars = v + stages * n_sub * kPfBK * 128;
    xch = bars + (2 * kPfMaxStages + 6) * 8 + 16;
    total = xch + 4 * kPfBQ * 4 + 1024;
  }
};

// MN-major operand tile (V): rows of 128 bytes are one key each, 8 keys form a 1024-byte
// swizzle atom; 64-wide column groups of the head are `lbo_bytes` apart.
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 2^x on the special-function unit; 2^(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The largest of three (one instruction on sm_100).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ uint64_t smem_desc_mn_sw128(const void* tile, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((tc::smem_u32(tile) & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int HDMAX>
__global__ void __launch_bounds__(kPfThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       int ldo, const int* __restrict__ table, int table_stride,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                       const int* __restrict__ seq_slot, int nh, int nkv, int hd, float scale_log2,
                       int window, unsigned int* __restrict__ fault,
                       unsigned long long* stamps) {
  extern __shared__ unsigned char smem_raw[];
  // Tuning aid: with a buffer given, the first CTA (the heaviest tile) notes the times at
  // which its MMA thread and one softmax thread pass the phases of steps 0 .. 7:
  // [step][16] nanoseconds.
  const bool stamping = kStamps && stamps && blockIdx.x + blockIdx.y + blockIdx.z == 0 && (threadIdx.x & 31) == 0;
  auto stamp = [&](int j, int i) {
    if (stamping && j < 8) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      stamps[j * 16 + i] = t;
    }
  };
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int n_sub = (hd + 63) >> 6;
  const PfSmem L(n_sub);
  const int kPfStages = L.stages;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* kv_empty = kv_full + kPfMaxStages;
  uint64_t* q_full = kv_empty + kPfMaxStages;
  uint64_t* s_full = q_full + 1;            // two: S is double-buffered in tensor memory
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 1;            // two: so is P V
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  // With two P tiles the softmax threads do not wait for a step's P V: they go on to the next
  // step's scores and fold the product in one step later.
  const bool defer = L.p_bufs == 2;
  constexpr int kPBytes = (kPfBK / 64) * kPfBQ * 128;
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, h = blockIdx.x;
  const int kvh = h / (nh / nkv);
  const int tok0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - tok0;
  // heavy tiles (late queries, many keys) first, and of all heads and sequences before any
  // lighter tile: CTAs are handed out with x fastest and z slowest
  const int q_tile = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int q0 = q_tile * kPfBQ;
  if (q0 >= n_new) return;
  const int start = seq_start[b];
  const int slot = seq_slot[b];
  const int* tab = table + (size_t)slot * table_stride;
  const int rows_here = min(kPfBQ, n_new - q0);
  const int pos_first = start + q0, pos_last = start + q0 + rows_here - 1;
  const int key_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int blk_lo = key_lo / kPfBlk, blk_hi = pos_last / kPfBlk;      // cache blocks, inclusive
  const int n_tiles = (blk_hi - blk_lo + 2) / 2;                        // steps of two blocks
  // Tensor memory: two score tiles (the product of step j + 1 runs under the softmax of
  // step j) and two tiles of P V.
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 256;      // + 128 (j & 1) each

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPfStages; ++s) { tc::mbar_init(&kv_full[s], 1); tc::mbar_init(&kv_empty[s], 1); }
    tc::mbar_init(q_full, 1);
    tc::mbar_init(&s_full[0], 1);
    tc::mbar_init(&s_full[1], 1);
    tc::mbar_init(p_full, 256);
    tc::mbar_init(&o_full[0], 1);
    tc::mbar_init(&o_full[1], 1);
    *abort = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_descriptor(&map_q);
    tc::tma_prefetch_descriptor(&map_k);
    tc::tma_prefetch_descriptor(&map_v);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // Programmatic dependent launch: the set-up above ran under the tail of the kernel before
  // this one; the queries and this prompt's keys and values are that kernel's output.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      tc::mbar_expect_tx(q_full, (uint32_t)(n_sub * kPfBQ * 128));
      for (int sub = 0; sub < n_sub; ++sub)
        tc::tma_load_2d(smem + L.q + sub * kPfBQ * 128, &map_q, h * hd + 64 * sub, tok0 + q0,
                        q_full);
      // (the ring's stage and turn are stepped, not divided: its depth is a run-time value)
      for (int j = 0, s = 0, turn = 0; j < n_tiles; ++j, s = s + 1 == kPfStages ? 0 : s + 1,
               turn += s == 0) {
        if (turn > 0 && !tc::mbar_wait(&kv_empty[s], (uint32_t)((turn - 1) & 1), abort)) break;
        tc::mbar_expect_tx(&kv_full[s], (uint32_t)(2 * n_sub * kPfBK * 128));
        for (int half = 0; half < 2; ++half) {
          // a step past the last block loads that block again: its keys are masked, and the
          // operand tile holds finite numbers instead of whatever was in shared memory
          const int blk = tab[min(blk_lo + 2 * j + half, blk_hi)];
          if (blk < 0) atomicOr(fault, kFaultBlockTable);
          const int row = (max(blk, 0) * nkv + kvh) * kPfBlk;
          for (int sub = 0; sub < n_sub; ++sub) {
            const int off = (s * n_sub + sub) * kPfBK * 128 + half * kPfBlk * 128;
            tc::tma_load_2d(smem + L.k + off, &map_k, 64 * sub, row, &kv_full[s]);
            tc::tma_load_2d(smem + L.v + off, &map_v, 64 * sub, row, &kv_full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = tc::instr_desc_bf16(kPfBQ, kPfBK);
      const uint32_t idesc_pv = tc::instr_desc_bf16(kPfBQ, hd) | (1u << 16);   // B is MN-major
      const int k_steps = hd >> 4;
      int sc_s = 0, sc_turn = 0;            // stage and turn of the next call of scores()
      auto scores = [&](int j) {            // S[j & 1] = Q K_j^T, once K_j has landed
        const int s = sc_s;
        if (!tc::mbar_wait(&kv_full[s], (uint32_t)(sc_turn & 1), abort)) return false;
        if (++sc_s == kPfStages) { sc_s = 0; ++sc_turn; }
        tc::tc_fence_after();
        for (int kk = 0; kk < k_steps; ++kk) {
          const int sub = kk >> 2, in = kk & 3;
          const uint64_t qd = tc::smem_desc_k_sw128(smem + L.q + sub * kPfBQ * 128) + 2 * in;
          const uint64_t kd =
              tc::smem_desc_k_sw128(smem + L.k + (s * n_sub + sub) * kPfBK * 128) + 2 * in;
          tc::umma_bf16(tmem + kColS + (uint32_t)(j & 1) * kPfBK, qd, kd, idesc_qk, kk != 0);
        }
        tc::umma_commit(&s_full[j & 1]);
        return true;
      };
      bool ok = tc::mbar_wait(q_full, 0u, abort);
      if (ok && n_tiles > 0) ok = scores(0);
      for (int j = 0, s = 0; j < n_tiles && ok; ++j, s = s + 1 == kPfStages ? 0 : s + 1) {
        // The next step's scores go to the other buffer, which the softmax threads left
        // before they signalled P of step j - 1 (waited for below, one step ago).
        if (j + 1 < n_tiles && !(ok = scores(j + 1))) break;
        stamp(j, 8);
        ok = tc::mbar_wait(p_full, (uint32_t)(j & 1), abort);
        if (!ok) break;
        stamp(j, 9);
        tc::tc_fence_after();
        const uint64_t vd = smem_desc_mn_sw128(smem + L.v + s * n_sub * kPfBK * 128,
                                               (uint32_t)(kPfBK * 128));
#pragma unroll
        for (int kk = 0; kk < kPfBK / 16; ++kk) {    // 16 keys = two 1024-byte atoms of V
          const uint64_t pd = tc::smem_desc_k_sw128(smem + L.p + (defer ? (j & 1) * kPBytes : 0) +
                                                    (kk >> 2) * kPfBQ * 128) +
                              2 * (kk & 3);
          tc::umma_bf16(tmem + kColO + (uint32_t)(j & 1) * 128, pd, vd + (uint64_t)(kk * 128),
                        idesc_pv, kk != 0);
        }
        tc::umma_commit(&kv_empty[s]);
        tc::umma_commit(&o_full[j & 1]);
        stamp(j, 10);
      }
    }
  } else {
    // Eight softmax warps: warps w and w + 4 share the 32 rows of TMEM lane quadrant w % 4;
    // of a row's 128 keys per step, the first of the pair takes keys 0..63 and the second
    // 64..127, and of the output's columns each keeps one half.  They meet once per step
    // (a named barrier of 64 threads) to agree on the row's maximum.
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const int q_pos = start + q0 + row;
    const bool row_valid = row < rows_here;
    const int lo_key = window > 0 ? max(0, q_pos - window + 1) : 0;
    // a step needs masks if it reaches past the first row's position or starts before the
    // last row's window
    const int lo_key_last = window > 0 ? max(0, start + q0 + kPfBQ - 1 - window + 1) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    const int ocols = hd >> 1, obase = half * ocols;     // this thread's output columns
    float o[HDMAX / 2];
#pragma unroll
    for (int d = 0; d < HDMAX / 2; ++d) o[d] = 0.f;
    float m = -INFINITY, l = 0.f;
    unsigned char* prow0 = smem + L.p + half * kPfBQ * 128 + row * 128;
    float* xch = reinterpret_cast<float*>(smem + L.xch);              // [2 buffers][2][128]
    // A wait that gives up does not leave the loop: the pair's barriers must stay matched.
    // Later waits return at once (the abort flag is up) and the result is flagged, not used.
    bool ok = true;
    // o = o * a + (P V of step jj), once that product is in tensor memory
    auto fold = [&](int jj, float a) {
      ok = tc::mbar_wait(&o_full[jj & 1], (uint32_t)((jj >> 1) & 1), abort) && ok;
      tc::tc_fence_after();
      if (warp == 2) stamp(jj, 5);
#pragma unroll
      for (int c0 = 0; c0 < HDMAX / 2; c0 += 32) {
        if (c0 < ocols) {
          uint32_t r[32];
          tc::tmem_load_32(lane_addr + kColO + (uint32_t)(jj & 1) * 128 + obase + c0, r);
          tc::tmem_load_wait();
          const float2 a2 = make_float2(a, a);
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            if (c0 + e < HDMAX / 2) {
              const float2 v = __ffma2_rn(make_float2(o[c0 + e], o[c0 + e + 1]), a2,
                                          make_float2(__uint_as_float(r[e]),
                                                      __uint_as_float(r[e + 1])));
              o[c0 + e] = v.x;
              o[c0 + e + 1] = v.y;
            }
        }
      }
      tc::tc_fence_before();
      if (warp == 2) stamp(jj, 6);
    };
    float alpha_before = 0.f;
    for (int j = 0; j < n_tiles; ++j) {
      if (warp == 2) stamp(j, 0);
      unsigned char* prow = prow0 + (defer ? (j & 1) * kPBytes : 0);
      ok = tc::mbar_wait(&s_full[j & 1], (uint32_t)((j >> 1) & 1), abort) && ok;
      tc::tc_fence_after();
      if (warp == 2) stamp(j, 1);
      uint32_t sa[32], sb[32];
      const uint32_t s_col = kColS + (uint32_t)(j & 1) * kPfBK + half * 64;
      tc::tmem_load_32(lane_addr + s_col, sa);
      tc::tmem_load_32(lane_addr + s_col + 32, sb);
      tc::tmem_load_wait();
      if (warp == 2) stamp(j, 2);
      const int key0 = (blk_lo + 2 * j) * kPfBlk + half * 64;
      // Raw scores stay in their registers; only steps that touch the diagonal, the
      // sequence's end or a window's edge pay for masking (uniform for the whole CTA).
      float t[64];
      const bool masked = key0 + 63 > pos_first || key0 < lo_key_last;
      if (masked) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = key0 + c;
          const float sv = __uint_as_float(c < 32 ? sa[c] : sb[c - 32]);
          t[c] = (key <= q_pos && key >= lo_key) ? sv : -INFINITY;
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) t[c] = __uint_as_float(c < 32 ? sa[c] : sb[c - 32]);
      }
      // (three-input maxima and two-wide float operations halve the instructions of the
      // loops below: what bounds a step is how many instructions its eight warps can issue)
      float mx4[4] = {t[0], t[1], t[2], t[3]};
#pragma unroll
      for (int c = 4; c < 60; c += 8) {
        mx4[0] = max3(mx4[0], t[c], t[c + 1]);
        mx4[1] = max3(mx4[1], t[c + 2], t[c + 3]);
        mx4[2] = max3(mx4[2], t[c + 4], t[c + 5]);
        mx4[3] = max3(mx4[3], t[c + 6], t[c + 7]);
      }
      mx4[0] = max3(mx4[0], t[60], t[61]);
      mx4[1] = max3(mx4[1], t[62], t[63]);
      // the scale is positive, so the largest raw score is the largest scaled one
      const float mine = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      float* xb = xch + (j & 1) * 256;        // double-buffered: one barrier per step
      xb[half * 128 + row] = mine;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
      if (warp == 2) stamp(j, 3);
      const float m_new = fmaxf(m, fmaxf(mine, xb[(half ^ 1) * 128 + row]));
      const float alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - m_new);
      // p = 2^(s * scale - m); a masked score (-inf) gives 0, and a row with nothing to see
      // yet (m_new = -inf) uses 0 as its reference so that no inf - inf appears
      const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
      float2 sum4[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      uint32_t packed[32];
      const float2 scale2 = make_float2(scale_log2, scale_log2), neg2 = make_float2(neg_m, neg_m);
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float2 x = __ffma2_rn(make_float2(t[c], t[c + 1]), scale2, neg2);
        const float2 pp = make_float2(fast_exp2(x.x), fast_exp2(x.y));
        sum4[(c >> 1) & 3] = __fadd2_rn(sum4[(c >> 1) & 3], pp);
        packed[c >> 1] = pack2(pp.x, pp.y);
      }
      const float2 s01 = __fadd2_rn(sum4[0], sum4[1]), s23 = __fadd2_rn(sum4[2], sum4[3]);
      const float2 s = __fadd2_rn(s01, s23);
      l = l * alpha + (s.x + s.y);
      m = m_new;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {        // 16-byte chunks, swizzled by the row
        const uint4 v4 = make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2],
                                    packed[4 * ch + 3]);
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = v4;
      }
      tc::fence_proxy_async();                // generic-proxy writes → visible to the MMA
      tc::tc_fence_before();                  // and this step's reads of S are done
      tc::mbar_arrive(p_full);
      if (warp == 2) stamp(j, 4);
      if (!defer) {
        fold(j, alpha);
      } else {
        if (j > 0) fold(j - 1, alpha_before);
        alpha_before = alpha;
      }
    }
    if (defer && n_tiles > 0) fold(n_tiles - 1, alpha_before);
    // the row's sum is the two halves' sums (the buffer of step n_tiles was last read two
    // steps ago)
    float* xb = xch + (n_tiles & 1) * 256;
    xb[half * 128 + row] = l;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
    l += xb[(half ^ 1) * 128 + row];
    if (ok && row_valid) {
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = out + (size_t)(tok0 + q0 + row) * ldo + (size_t)h * hd + obase;
#pragma unroll
      for (int d = 0; d < HDMAX / 2; d += 8) {
        if (d < ocols) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = o[d + e] * inv;
          store8(orow + d, v);
        }
      }
    }
  }
  if (*abort && threadIdx.x == 0) atomicOr(fault, kFaultWaitExpired);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// Two query tiles per CTA.
//
// In the kernel above the two softmax warps of an SM sub-partition share the same rows and
// meet at a barrier every step, so all eight warps pass through the step's phases together
// and the special-function unit (two warps x 64 ex2 x 8 cycles of a 1,280 ns step) idles for
// more than half of it.  Here a CTA owns TWO tiles of 128 queries that read the same key/value
// head — two query heads of a group, or consecutive query tiles — and a softmax thread owns a
// whole row of one of them (128 scores a step): no partner, no barrier, and the tiles' warps
// (2-5 and 6-9, one of each on every sub-partition) work side by side.  The keys and values
// of a step are loaded once for both tiles.
//   tensor memory, per tile: S (128 columns), P (64: two bfloat16 a column), O (64);
//   shared memory: Q_a, Q_b and the stages of K/V (128 keys).
// P never touches shared memory: the row's thread writes it into tensor memory, from where
// the product P V reads it as its A operand, and the product adds into O itself.  That works
// because a row's reference for the exponentials is lazy — it stays as it is until a score
// exceeds it by 2^8 — so O needs no rescaling in almost every step; when the reference does
// move, the row's thread reads O, scales it and writes it back before it hands over its P.
// A tile's chain is then: scores -> exponentials -> next scores; the product runs beside it.
//
// With `split` the CTA's two slots work on ONE tile instead: slot 0 takes the tile's steps
// 0, 2, 4, ... of 128 keys, slot 1 the steps 1, 3, 5, ..., each with a reference, a sum and an
// output of its own, and slot 0's threads merge the two at the end.  That is for grids of too
// few tiles to fill the chip as pairs (a lone prompt): as many CTAs as tiles, and the
// heaviest tile, which decides the launch, takes half as long.
// Head sizes up to 64, no sliding window; the launcher falls back to the kernel above
// otherwise.
constexpr int kPpStages = 4;       // stages of K/V in shared memory (pairs use three of them)
constexpr int kPpThreads = 352;   // producer, issuer of tile 0, 2 x 4 softmax warps, issuer of tile 1
constexpr int kPpIssuer1 = 10;

struct PpSmem {
  int q, k, v, xch, bars, total;
  __host__ __device__ PpSmem() {
    q = 0;                                   // [2][128 rows][128 B]
    k = q + 2 * kPfBQ * 128;
    v = k + kPpStages * kPfBK * 128;
    xch = v + kPpStages * kPfBK * 128;       // [128 rows] reference and sum of slot 1 (split)
    bars = xch + kPfBQ * 8;
    total = bars + (2 * kPpStages + 12) * 8 + 16 + 1024;   // barriers, two words, alignment
  }
};

__global__ void __launch_bounds__(kPpThreads, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q,
                         const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                         int ldo, const int* __restrict__ table, int table_stride,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_slot, int nh, int nkv, int hd, float scale_log2,
                         int split, unsigned int* __restrict__ fault) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const PpSmem L;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* kv_empty = kv_full + kPpStages;
  uint64_t* q_full = kv_empty + kPpStages;
  uint64_t* s_full = q_full + 1;            // [tile][half of a step's keys]
  uint64_t* p_full = s_full + 4;            // [tile][half]
  uint64_t* pv_done = p_full + 4;           // [tile]: its last product has finished
  uint64_t* xch_full = pv_done + 2;         // slot 1's references and sums are written (split)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xch_full + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int group = nh / nkv;
  const int tok0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - tok0;
  const int n_qt = (n_new + kPfBQ - 1) / kPfBQ;
  const int n_items = n_qt * group;          // (query tile, head of the group), tile-major
  // heavy pairs (late query tiles) of all sequences and key/value heads first
  const int pair = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int first = split ? pair : 2 * pair;
  if (first >= n_items) return;
  const int start = seq_start[b];
  const int* tab = table + (size_t)seq_slot[b] * table_stride;
  // The CTA's one or two items, a slot each; split: one item in both slots.  A slot's step i
  // is the ring's step i * stride + offset.
  int it_q0[2], it_head[2], it_rows[2], it_steps[2];
  const int n_mine = split ? 2 : min(2, n_items - first);
  const int stride = split ? 2 : 1;
  // split: the two slots are at ring steps g and g + 1 and ask for g + 2 and g + 3
  const int n_stages = split ? kPpStages : kPpStages - 1;
  int n_steps = 0;                           // steps of the ring of keys and values
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int idx = first + (!split && x < n_mine ? x : 0);
    const int t = idx / group;
    it_q0[x] = t * kPfBQ;
    it_head[x] = kvh * group + (idx - t * group);
    it_rows[x] = min(kPfBQ, n_new - it_q0[x]);
    const int pos_last = start + it_q0[x] + it_rows[x] - 1;
    const int all = pos_last / kPfBlk / 2 + 1;                   // steps of two cache blocks
    it_steps[x] = split ? (all - x + 1) / 2 : (x < n_mine ? all : 0);
    if (x < n_mine) n_steps = max(n_steps, all);
  }
  const int blk_hi = 2 * n_steps - 1;        // (blocks past a sequence's end are clamped below)
  const int blk_last = (start + n_new - 1) / kPfBlk;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColTile = 256, kColS = 0, kColP = 128, kColO = 192;   // per tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPpStages; ++s) { tc::mbar_init(&kv_full[s], 1); tc::mbar_init(&kv_empty[s], 2); }
    tc::mbar_init(q_full, 1);
    for (int x = 0; x < 4; ++x) {
      tc::mbar_init(&s_full[x], 1);
      tc::mbar_init(&p_full[x], 128);
    }
    tc::mbar_init(&pv_done[0], 1);
    tc::mbar_init(&pv_done[1], 1);
    tc::mbar_init(xch_full, 128);
    *abort = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_descriptor(&map_q);
    tc::tma_prefetch_descriptor(&map_k);
    tc::tma_prefetch_descriptor(&map_v);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      const int n_q = split ? 1 : n_mine;
      tc::mbar_expect_tx(q_full, (uint32_t)(n_q * kPfBQ * 128));
      for (int x = 0; x < n_q; ++x)
        tc::tma_load_2d(smem + L.q + x * kPfBQ * 128, &map_q, it_head[x] * hd, tok0 + it_q0[x],
                        q_full);
      for (int j = 0, s = 0, turn = 0; j < n_steps; ++j, s = s + 1 == n_stages ? 0 : s + 1,
               turn += s == 0) {
        if (turn > 0 && !tc::mbar_wait(&kv_empty[s], (uint32_t)((turn - 1) & 1), abort)) break;
        tc::mbar_expect_tx(&kv_full[s], (uint32_t)(2 * kPfBK * 128));
        for (int half = 0; half < 2; ++half) {
          // a block past the sequence's last loads that one again: its keys are masked
          const int blk = tab[min(min(2 * j + half, blk_hi), blk_last)];
          if (blk < 0) atomicOr(fault, kFaultBlockTable);
          const int row = (max(blk, 0) * nkv + kvh) * kPfBlk;
          const int off = s * kPfBK * 128 + half * kPfBlk * 128;
          tc::tma_load_2d(smem + L.k + off, &map_k, 0, row, &kv_full[s]);
          tc::tma_load_2d(smem + L.v + off, &map_v, 0, row, &kv_full[s]);
        }
      }
    }
  } else if (warp == 1 || warp == kPpIssuer1) {
    // ---- the products of one tile each.  (An issuing thread pays some 45 cycles a product and
    // 150-200 for every commit and barrier wait, whatever the products' sizes; one thread for
    // both tiles was busy all the time.)
    if (lane == 0) {
      const int x = warp == 1 ? 0 : 1;
      const int steps = it_steps[x];
      const uint32_t idesc_qk = tc::instr_desc_bf16(kPfBQ, kPfBK / 2);
      const uint32_t idesc_pv = tc::instr_desc_bf16(kPfBQ, hd) | (1u << 16);   // B is MN-major
      const int k_steps = hd >> 4;
      const uint32_t t_s = tmem + (uint32_t)x * kColTile + kColS;
      const uint32_t t_p = tmem + (uint32_t)x * kColTile + kColP;
      const uint32_t t_o = tmem + (uint32_t)x * kColTile + kColO;
      const int offset = split ? x : 0;
      const uint64_t qd = tc::smem_desc_k_sw128(smem + L.q + (split ? 0 : x) * kPfBQ * 128);
      const uint64_t kd0 = tc::smem_desc_k_sw128(smem + L.k);
      const uint64_t vd0 = smem_desc_mn_sw128(smem + L.v, (uint32_t)(kPfBK * 128));
      constexpr uint64_t kStage = (uint64_t)((kPfBK * 128) >> 4);    // a stage, in descriptor units
      constexpr uint64_t kHalf = (uint64_t)((kPfBlk * 128) >> 4);    // 64 keys of it
      int ready = -1;                       // highest step whose keys and values have landed
      bool ok = tc::mbar_wait(q_full, 0u, abort);
      auto landed = [&](int j) {            // wait (once) for the stage of step j
        while (ok && ready < j) {
          ++ready;
          ok = tc::mbar_wait(&kv_full[ready % n_stages], (uint32_t)((ready / n_stages) & 1), abort);
        }
        tc::tc_fence_after();
        return ok;
      };
      auto scores = [&](int g, int h) {     // S_x[:, 64 h ..] = Q_x K_g[64 h ..]^T, g a ring step
        const uint64_t kd = kd0 + (uint64_t)(g % n_stages) * kStage + (uint64_t)h * kHalf;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          if (kk < k_steps)
            tc::umma_bf16(t_s + (uint32_t)(h * kPfBlk), qd + 2 * kk, kd + 2 * kk, idesc_qk, kk != 0);
      };
      auto product = [&](int g, int i, int h) {    // O_x (+)= P_x[:, 64 h ..] V_g[64 h ..]
        const uint64_t vd = vd0 + (uint64_t)(g % n_stages) * kStage;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int kk = h * 4 + k4;
          tc::umma_bf16_a_tmem(t_o, t_p + (uint32_t)(kk * 8), vd + (uint64_t)(kk * 128), idesc_pv,
                               (i | kk) != 0);
        }
      };
      if (ok && steps > 0 && landed(offset)) {
        scores(offset, 0);
        tc::umma_commit(&s_full[2 * x]);
        scores(offset, 1);
        tc::umma_commit(&s_full[2 * x + 1]);
      }
      for (int g = 0; g < n_steps && ok; ++g) {
        const int j = (g - offset) / stride;       // the slot's own step, if the ring's is its
        if (g >= offset && j * stride + offset == g && j < steps) {
          // A step's keys go in two halves of 64.  When the tile's threads have written the P
          // of a half, its product is issued and then the same half of the next step's
          // scores (that half of S has been read for the last time); one commit tells the
          // threads both that the scores are there and that this P has been read.  The
          // threads meanwhile work on the other half and find the next scores waiting.
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            ok = tc::mbar_wait(&p_full[2 * x + h], (uint32_t)(j & 1), abort);
            if (!ok) break;
            tc::tc_fence_after();
            product(g, j, h);
            if (j + 1 < steps && landed(g + stride)) scores(g + stride, h);
            tc::umma_commit(&s_full[2 * x + h]);
          }
          if (!ok) break;
          tc::umma_commit(&kv_empty[g % n_stages]);          // this slot is done with the stage
          if (j + 1 == steps) tc::umma_commit(&pv_done[x]);
        } else if (landed(g)) {
          // a slot that has no use for the stage (the other's turn, or its tile has fewer
          // steps) says so once the stage has been filled, which keeps its arrivals in step
          // with the ring's turns
          tc::mbar_arrive(&kv_empty[g % n_stages]);
        }
      }
    }
  } else {
    // ---- softmax: warps 2-5 tile 0, warps 6-9 tile 1; a thread owns one row
    const int x = (warp - 2) >> 2, quad = warp & 3;
    const int row = quad * 32 + lane;
    const int steps = it_steps[x];
    const int q_pos = start + it_q0[x] + row;
    const int pos_first = start + it_q0[x];
    const bool row_valid = x < n_mine && row < it_rows[x];
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + (uint32_t)x * kColTile + kColS;
    const uint32_t p_addr = lane_addr + (uint32_t)x * kColTile + kColP;
    const uint32_t o_addr = lane_addr + (uint32_t)x * kColTile + kColO;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // O *= a for this thread's row (no product of the tile is in flight, see below).
    auto rescale = [&](float a) {
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        if (c0 < hd) {
          uint32_t r[32];
          tc::tmem_load_32(o_addr + (uint32_t)c0, r);
          tc::tmem_load_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * a);
          tc::tmem_store_32(o_addr + (uint32_t)c0, r);
        }
      }
    };
    const int offset = split ? x : 0;
    for (int hs = 0; hs < 2 * steps; ++hs) {
      const int j = hs >> 1, h = hs & 1;       // the slot's own step and the half of its keys
      // the scores of this half are there, and the product that read the half's last P is done
      ok = tc::mbar_wait(&s_full[2 * x + h], (uint32_t)(j & 1), abort) && ok;
      tc::tc_fence_after();
      const int key0 = ((j * stride + offset) * 2 + h) * kPfBlk;
      const bool masked = key0 + kPfBlk - 1 > pos_first;     // the half reaches the diagonal
      // One pass over the scores: p = 2^(s * scale - ref) with `ref` the reference the row
      // already has, the half's maximum found on the way.  As long as no score exceeds the
      // reference by more than 2^8 the reference stays (p <= 256 is harmless in bfloat16 and
      // in the 32-bit sums, and the output needs no rescaling: alpha = 1).  Otherwise, and at
      // the very first keys, the warp finds the maximum first and goes over the scores again.
      float alpha = 1.0f, m_new = m;
      float2 sum2[2];
      float mx4[4];
      auto pass = [&](bool want_p, float ref) {
        const float neg_m = (ref == -INFINITY) ? 0.f : -ref;
        const float2 scale2 = make_float2(scale_log2, scale_log2), neg2 = make_float2(neg_m, neg_m);
        sum2[0] = sum2[1] = make_float2(0.f, 0.f);
        mx4[0] = mx4[1] = mx4[2] = mx4[3] = -INFINITY;
        // 32 scores at a time
        auto chunk = [&](int c0, uint32_t (&r)[32]) {
          if (masked) {
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (key0 + c0 + c > q_pos) r[c] = 0xff800000u;          // -inf
          }
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            mx4[0] = max3(mx4[0], __uint_as_float(r[c]), __uint_as_float(r[c + 1]));
            mx4[1] = max3(mx4[1], __uint_as_float(r[c + 2]), __uint_as_float(r[c + 3]));
            mx4[2] = max3(mx4[2], __uint_as_float(r[c + 4]), __uint_as_float(r[c + 5]));
            mx4[3] = max3(mx4[3], __uint_as_float(r[c + 6]), __uint_as_float(r[c + 7]));
          }
          if (want_p) {
            uint32_t packed[16];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              const float2 e = __ffma2_rn(
                  make_float2(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2, neg2);
              const float2 pp = make_float2(fast_exp2(e.x), fast_exp2(e.y));
              sum2[(c >> 1) & 1] = __fadd2_rn(sum2[(c >> 1) & 1], pp);
              packed[c >> 1] = pack2(pp.x, pp.y);
            }
            tc::tmem_store_16(p_addr + (uint32_t)((h * kPfBlk + c0) >> 1), packed);
          }
        };
        // (the second 32 are on their way while the first are worked on)
        {
          uint32_t r0[32], r1[32];
          tc::tmem_load_32(s_addr + (uint32_t)(h * kPfBlk), r0);
          tc::tmem_load_wait();
          tc::tmem_load_32(s_addr + (uint32_t)(h * kPfBlk + 32), r1);
          chunk(0, r0);
          tc::tmem_load_wait();
          chunk(32, r1);
        }
        // the scale is positive, so the largest raw score is the largest scaled one
        return fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      };
      bool again = hs == 0;
      if (!again) {
        const float top = pass(true, m);
        again = __any_sync(0xffffffffu, top > m + 8.0f);
        if (again) m_new = fmaxf(m, top);
      } else {
        m_new = fmaxf(m, pass(false, m));
      }
      if (again) {
        alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - m_new);
        pass(true, m_new);
        if (hs > 0) {
          // O is scaled in place.  The product of the half before this one may still run:
          // the commit that follows it is the one the other half's scores wait for next.
          ok = tc::mbar_wait(&s_full[2 * x + (h ^ 1)], (uint32_t)((j + h) & 1), abort) && ok;
          tc::tc_fence_after();
          rescale(alpha);
        }
      }
      const float2 s2 = __fadd2_rn(sum2[0], sum2[1]);
      l = l * alpha + (s2.x + s2.y);
      m = m_new;
      tc::tmem_store_wait();                  // P (and O) are in tensor memory,
      tc::tc_fence_before();                  // this half's reads of S are done
      tc::mbar_arrive(&p_full[2 * x + h]);
    }
    if (split && x == 1) {
      // the other slot's threads read this one's output from tensor memory; they need the
      // reference and the sum that go with it
      if (steps > 0) ok = tc::mbar_wait(&pv_done[1], 0u, abort) && ok;
      reinterpret_cast<float2*>(smem + L.xch)[row] = make_float2(m, l);
      tc::tc_fence_before();
      tc::mbar_arrive(xch_full);
    } else if (steps > 0) {
      ok = tc::mbar_wait(&pv_done[x], 0u, abort) && ok;
      float w0 = 1.0f, w1 = 0.f;             // weights of the two slots' outputs (split)
      if (split) {
        ok = tc::mbar_wait(xch_full, 0u, abort) && ok;
        const float2 other = reinterpret_cast<const float2*>(smem + L.xch)[row];
        if (other.x != -INFINITY) {          // (slot 0 always has keys: its reference is finite)
          const float mm = fmaxf(m, other.x);
          w0 = fast_exp2(m - mm);
          w1 = fast_exp2(other.x - mm);
        }
        l = l * w0 + other.y * w1;
      }
      tc::tc_fence_after();
      const float inv = 1.0f / l;
      w0 *= inv;
      w1 *= inv;
      __nv_bfloat16* orow = out + (size_t)(tok0 + it_q0[x] + row) * ldo + (size_t)it_head[x] * hd;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        if (c0 < hd) {
          uint32_t r[32];
          tc::tmem_load_32(o_addr + (uint32_t)c0, r);
          tc::tmem_load_wait();
          float v32[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v32[e] = __uint_as_float(r[e]) * w0;
          if (split && __any_sync(0xffffffffu, w1 != 0.f)) {   // (a load all lanes take)
            tc::tmem_load_32(o_addr + kColTile + (uint32_t)c0, r);
            tc::tmem_load_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (w1 != 0.f) v32[e] = fmaf(__uint_as_float(r[e]), w1, v32[e]);
          }
          if (ok && row_valid) {
#pragma unroll
            for (int d = 0; d < 32; d += 8) {
              if (c0 + d < hd) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = v32[d + e];
                store8(orow + c0 + d, v);
              }
            }
          }
        }
      }
    }
  }
  if (*abort && threadIdx.x == 0) atomicOr(fault, kFaultWaitExpired);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace cretif

using namespace cretif;

// Tuning aid: a device buffer of 8 x 16 timestamps that the next launches fill (see the kernel).
static unsigned long long* g_pf_stamps = nullptr;
// Which kernel takes head sizes up to 64 without a window (for tests that run all): -1 as the
// launcher sees fit, 0 the kernel with two threads per row, 1 a thread per row and two query
// tiles per CTA, 2 a thread per row and one tile whose key steps the CTA's two slots share.
static int g_pf_pairing = -1;
extern "C" int cretif_set_prefill_pairing(int mode) {
  const int was = g_pf_pairing;
  g_pf_pairing = mode < 0 ? -1 : (mode > 2 ? 2 : mode);
  return was;
}
#ifdef CRETIF_STAMPS
extern "C" void cretif_attn_prefill_stamps(unsigned long long* device_buffer) {
  g_pf_stamps = device_buffer;
}
#endif

extern "C" int cretif_attn_prefill_tc(const void* qkv, int ldq, int T, void* out, int ldo,
                                      const void* kc, const void* vc, long long n_blocks,
                                      const int* table, int table_stride, const int* cu_seqlens,
                                      const int* seq_start, const int* seq_slot, int nh, int nkv,
                                      int hd, float scale, int window, int bt, int B, int max_new,
                                      unsigned int* fault, void* stream) {
  if (B <= 0 || T <= 0) return kOk;
  if (nh <= 0 || nkv <= 0 || nh % nkv || hd % 16 || hd < 16 || hd > 128 || bt != kPfBlk ||
      window < 0 || !(scale > 0.f) || max_new <= 0 || B > 65535 || ldq % 8 || ldo % 8 ||
      (max_new + kPfBQ - 1) / kPfBQ > 65535)
    return kBadArgument;
  if (((uintptr_t)qkv | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) & 15) return kMisaligned;
  const long long cache_rows = n_blocks * nkv * kPfBlk;
  if (cache_rows > 0x7fffffffLL) return kBadArgument;
  CUtensorMap map_q, map_k, map_v;
  if (make_tile_map_bf16(&map_q, qkv, T, ldq, ldq, kPfBQ)) return kBadArgument;
  if (make_tile_map_bf16(&map_k, kc, (int)cache_rows, hd, hd, kPfBlk)) return kBadArgument;
  if (make_tile_map_bf16(&map_v, vc, (int)cache_rows, hd, hd, kPfBlk)) return kBadArgument;
  const int n_sub = (hd + 63) / 64;
  const PfSmem L(n_sub);
  cudaStream_t st = (cudaStream_t)stream;
  const float scale_log2 = scale * 1.4426950408889634f;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nh, B, (max_new + kPfBQ - 1) / kPfBQ);
  cfg.blockDim = dim3(kPfThreads);
  cfg.dynamicSmemBytes = L.total;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  // The kernel with a thread per row (P and O in tensor memory) for head sizes up to 64 without
  // a window: two query tiles per CTA where pairs still spread over the chip, else one tile
  // per CTA with its key steps split between the CTA's two slots.
  const int group = nh / nkv;
  const long long n_qt = (max_new + kPfBQ - 1) / kPfBQ;
  const long long items = n_qt * group, pairs = (items + 1) / 2;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  const bool rows_ok = g_pf_pairing != 0 && hd <= 64 && window == 0 && items <= 65535;
  const bool paired = rows_ok && (g_pf_pairing == 1 ||
                                  (g_pf_pairing < 0 && 5 * pairs * nkv * B >= 7LL * sm_count));
  if (rows_ok) {
    const PpSmem P;
    static int configured_pair = 0;
    if (!configured_pair) {
      e = cudaFuncSetAttribute(attn_prefill_pair_kernel,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, P.total);
      if (e != cudaSuccess) return (int)e;
      configured_pair = 1;
    }
    cfg.gridDim = dim3(nkv, B, (unsigned)(paired ? pairs : items));
    cfg.blockDim = dim3(kPpThreads);
    cfg.dynamicSmemBytes = P.total;
    count_variant(paired ? kVarPrefillAttnPair : kVarPrefillAttnSplit);
    e = cudaLaunchKernelEx(&cfg, attn_prefill_pair_kernel, map_q, map_k, map_v,
                           (__nv_bfloat16*)out, ldo, table, table_stride, cu_seqlens, seq_start,
                           seq_slot, nh, nkv, hd, scale_log2, paired ? 0 : 1, fault);
    return e == cudaSuccess ? launch_status() : (int)e;
  }
  count_variant(kVarPrefillAttn);
  if (hd <= 64) {
    static int configured = 0;
    if (L.total > configured) {
      e = cudaFuncSetAttribute(attn_prefill_tc_kernel<64>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, L.total);
      if (e != cudaSuccess) return (int)e;
      configured = L.total;
    }
    e = cudaLaunchKernelEx(&cfg, attn_prefill_tc_kernel<64>, map_q, map_k, map_v,
                           (__nv_bfloat16*)out, ldo, table, table_stride, cu_seqlens, seq_start,
                           seq_slot, nh, nkv, hd, scale_log2, window, fault, g_pf_stamps);
    if (e != cudaSuccess) return (int)e;
  } else {
    static int configured = 0;
    if (L.total > configured) {
      e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, L.total);
      if (e != cudaSuccess) return (int)e;
      configured = L.total;
    }
    e = cudaLaunchKernelEx(&cfg, attn_prefill_tc_kernel<128>, map_q, map_k, map_v,
                           (__nv_bfloat16*)out, ldo, table, table_stride, cu_seqlens, seq_start,
                           seq_slot, nh, nkv, hd, scale_log2, window, fault, g_pf_stamps);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_status();
}
