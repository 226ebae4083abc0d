// Decode attention over the block cache on the tensor cores (bfloat16, head_dim <= 128).
//
// One CTA serves one (sequence, key/value head, range of cache blocks).  A producer warp moves
// the K and V tiles of each 64-key block into a ring of shared-memory stages with TMA (2-d
// boxes out of the cache, 128-byte swizzle, so that ldmatrix reads them without bank
// conflicts).  Each of the four consumer warps owns 16 of a tile's 64 keys and keeps its own
// running maximum, sum and output for all query heads of the key/value head: the heads are
// the rows of m16n8k16 products (S = Q K^T, then O += P V with P taken straight from the
// accumulator registers), so the warps never synchronise inside the loop; their four partial
// results are merged once at the end of the CTA.  Ranges of one sequence are merged in one of
// two ways.  Up to eight ranges form a thread-block cluster: every CTA owns a share of the
// (head, dim) outputs, each warp stores its partial results straight into the owners' shared
// memory (distributed shared memory), and after one cluster barrier every CTA finishes its
// share from its own memory: no trip through global memory, which costs most of the kernel's
// time at short contexts.  More ranges (a long context with few sequences) go through global
// scratch and are merged by the CTA that finishes last, as in attn_decode.cu (same scratch,
// same counters).
//
// The reference walks positions serially with one block per head (src/attention.cu:410-494).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "api.h"
#include "tc_common.cuh"

namespace cretif {

int make_tile_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int ld,
                       int box_rows);

constexpr int kDmWarps = 4;                 // consumer warps
constexpr int kDmThreads = (kDmWarps + 1) * 32;
constexpr int kDmTile = 64;
constexpr int kDmStages = 3;                // ring of K/V stages by default ...
constexpr int kDmMaxStages = 6;             // ... and at most (a launch with few CTAs goes deeper)
constexpr int kDmClusterMax = 8;            // ranges merged inside one cluster (portable size)

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816_f32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One work item (sequence b, key/value head kvh, range `split` of `n_splits`) of the decode
// attention, run by a CTA of at least 160 threads: warps 0-3 consume, warp 4 produces, further
// warps only take part in the CTA-wide synchronisation.  The mbarriers in shared memory are
// initialised once per kernel by dm_init(); `it_base` counts the tiles this CTA has pushed
// through them so far, so that stage and phase carry on from item to item.
// HD16 = head_dim / 16 (compile time: sizes the register arrays).
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Store into the shared memory of CTA `rank` of this cluster, at the address that
// `local_addr` has in this CTA's.
__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// Floats of the region in which the warps' partial results meet (later reused for the weights
// of the merge over ranges).
template <int HD16>
__host__ __device__ constexpr size_t dm_mrg_floats() {
  constexpr int hd = HD16 * 16;
  const size_t mrg = (size_t)(2 * kDmWarps * 8 + kDmWarps * 8 * hd);
  const size_t wts = (size_t)(8 * kDmTile + 8);
  return mrg > wts ? mrg : wts;
}

template <int HD16, bool CLUSTER = false>
__device__ __forceinline__ void attn_decode_mma_item(
    unsigned char* smem, const CUtensorMap* map_k, const CUtensorMap* map_v,
    const __nv_bfloat16* __restrict__ q, int ldq, const int* __restrict__ table, int table_stride,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
    const int* __restrict__ seq_slot, int nh, int nkv, float scale_log2, int window,
    float* __restrict__ part_o, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
    int ldo, int* __restrict__ counters, unsigned int* __restrict__ fault, int split,
    int n_splits, int kvh, int b, uint32_t& it_base, unsigned long long* stamps = nullptr,
    int n_stages = kDmStages) {
  constexpr int hd = HD16 * 16;
  // Tuning aid: with a buffer given, lane 0 of every warp of the first CTA notes the time at
  // which it passes each phase ([warp][16]); the CTA that merges notes its own at [8][..].
  const bool stamping = kStamps && stamps && split == 0 && kvh == 0 && b == 0;
  auto stamp = [&](int row, int i) {
    if ((threadIdx.x & 31) == 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      stamps[row * 16 + i] = t;
    }
  };
#define DM_STAMP(i) do { if (stamping) stamp(threadIdx.x >> 5, i); } while (0)
  DM_STAMP(0);
  constexpr int kSub = (hd + 63) / 64;                 // 64-wide column groups of a tile
  constexpr int kTileBytes = kSub * kDmTile * 128;     // one of K or V
  unsigned char* ktiles = smem;
  unsigned char* vtiles = smem + n_stages * kTileBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + 2 * n_stages * kTileBytes);
  uint64_t* empty = full + kDmMaxStages;
  volatile int* abort = reinterpret_cast<volatile int*>(empty + kDmMaxStages);
  int* is_last = const_cast<int*>(abort) + 1;
  float* mrg = reinterpret_cast<float*>(const_cast<int*>(abort) + 4);   // warps' partials
  // cluster merge: what the warps of all ranges send this CTA: [range][warp][8 heads]{m, l},
  // then [range][warp][share] o
  float* recv_ml = mrg + dm_mrg_floats<HD16>();
  float* recv_o = recv_ml + kDmClusterMax * kDmWarps * 8 * 2;

  const int g = nh / nkv;
  const int share = (g * hd + n_splits - 1) / n_splits;   // outputs a CTA of the cluster owns
  // n / share and n / g for n < 65536 as a multiplication: a division in the merge's short
  // dependent chains costs more than the stores it addresses
  // (floor(n / d) = umulhi(n, ceil(2^32 / d)) for n, d < 65536, d > 1; the factor of 1 does
  // not fit 32 bits)
  const uint32_t share_magic = 0xffffffffu / (uint32_t)share + 1u;
  const uint32_t g_magic = 0xffffffffu / (uint32_t)g + 1u;
  auto div_by = [](int n, int d, uint32_t magic) {
    return d == 1 ? n : (int)__umulhi((uint32_t)n, magic);
  };
  const int nthreads = blockDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = tok_pos[b];
  const int slot = seq_slot[tok_seq[b]];
  const int* tab = table + (size_t)slot * table_stride;
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int first_tile = first_key / kDmTile, n_tiles = pos / kDmTile + 1;
  // the tiles are dealt out evenly: the first (tiles % ranges) ranges take one more
  const int span = n_tiles - first_tile, per = span / n_splits, extra = span - per * n_splits;
  const int t_begin = first_tile + split * per + min(split, extra);
  const int my_tiles = per + (split < extra ? 1 : 0);
  if (stamping && my_tiles >= 0) stamp(threadIdx.x >> 5, 1);

  __syncthreads();                      // the previous item's readers of `mrg` are done

  // per-warp results for the merge: [warp][g] m, l and [warp][g][hd] o
  float* mrg_m = mrg;
  float* mrg_l = mrg + kDmWarps * 8;
  float* mrg_o = mrg + 2 * kDmWarps * 8;

  if (warp > kDmWarps) {
    if (CLUSTER) cluster_wait();          // not needed for this item
  } else if (warp == kDmWarps) {
    // ---------------- producer
    // The block table, the positions and every cache tile but the one that holds the step's
    // own token were written before this step's kernels began: the first tiles are asked for
    // before the kernel waits for the one before it (programmatic dependent launch), the
    // tile of the new token after.  Block ids are read 32 at a time.
    bool waited = false;
    // stage and turn of the ring for tile i (carried on from earlier items; stepped, not
    // divided, per tile)
    int st = (int)(it_base % (uint32_t)n_stages), turn = (int)(it_base / (uint32_t)n_stages);
    for (int i0 = 0; i0 < my_tiles; i0 += 32) {
      const int mine = i0 + lane < my_tiles ? tab[t_begin + i0 + lane] : 0;
      const int n = min(32, my_tiles - i0);
      if (stamping && mine >= -1) stamp(threadIdx.x >> 5, 2);
      bool go = true;
      for (int j = 0; j < n && go; ++j) {
        const int i = i0 + j;
        const int blk = __shfl_sync(0xffffffffu, mine, j);
        const int s = st;
        if (!waited && (i >= n_stages || t_begin + i == n_tiles - 1)) {
          asm volatile("griddepcontrol.wait;" ::: "memory");
          waited = true;
        }
        if (lane == 0) {
          if (turn > 0 && !tc::mbar_wait(&empty[s], (uint32_t)((turn - 1) & 1), abort)) {
            go = false;
          } else {
            if (blk < 0) atomicOr(fault, kFaultBlockTable);
            const int row = (max(blk, 0) * nkv + kvh) * kDmTile;
            tc::mbar_expect_tx(&full[s], 2u * kTileBytes);
#pragma unroll
            for (int sub = 0; sub < kSub; ++sub) {
              tc::tma_load_2d(ktiles + s * kTileBytes + sub * kDmTile * 128, map_k, 64 * sub, row, &full[s]);
              tc::tma_load_2d(vtiles + s * kTileBytes + sub * kDmTile * 128, map_v, 64 * sub, row, &full[s]);
            }
          }
        }
        if (++st == n_stages) { st = 0; ++turn; }
        go = __shfl_sync(0xffffffffu, go, 0);
        if (i == 0) DM_STAMP(3);
      }
      if (!go) break;
    }
    DM_STAMP(4);
    if (CLUSTER) cluster_wait();
  } else {
    // ---------------- consumers: warp w owns keys 16w .. 16w+15 of every tile
    const int r = lane >> 2, c = lane & 3;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // q comes from the kernel before
    DM_STAMP(2);
    // Q as the A operand: rows = heads of this kv head (rows >= g are zero)
    uint32_t qa[HD16][2];
    {
      const __nv_bfloat16* qrow = q + (size_t)b * ldq + (size_t)(kvh * g + r) * hd;
#pragma unroll
      for (int ks = 0; ks < HD16; ++ks) {
        qa[ks][0] = r < g ? __ldcg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * c)) : 0u;
        qa[ks][1] = r < g ? __ldcg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * c)) : 0u;
      }
    }
    if (stamping && qa[0][0] != 0x7fc07fc1u) stamp(threadIdx.x >> 5, 3);
    float o[HD16 * 2][2];                 // [8-dim tile][2 dims] of row r
#pragma unroll
    for (int i = 0; i < HD16 * 2; ++i) o[i][0] = o[i][1] = 0.f;
    float m = -INFINITY, l = 0.f;         // of row r (partial over this thread's keys for l)
    const int mat = lane >> 3, rin = lane & 7;
    bool ok = true;
    int s = (int)(it_base % (uint32_t)n_stages), turn = (int)(it_base / (uint32_t)n_stages);
    for (int i = 0; i < my_tiles; ++i) {
      if (!tc::mbar_wait(&full[s], (uint32_t)(turn & 1), abort)) { ok = false; break; }
      if (i == 0) DM_STAMP(4);
      const uint32_t kbase = tc::smem_u32(ktiles + s * kTileBytes);
      const uint32_t vbase = tc::smem_u32(vtiles + s * kTileBytes);
      // ---- S = Q K^T for this warp's 16 keys
      float sacc[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[n][e] = 0.f;
      {
        const int key = warp * 16 + (mat >> 1) * 8 + rin;          // row of the tile this lane addresses
#pragma unroll
        for (int ks = 0; ks < HD16; ++ks) {
          const int chunk = ks * 2 + (mat & 1);                    // 16-byte chunk along head_dim
          const uint32_t addr = kbase + (chunk >> 3) * (kDmTile * 128) + key * 128 +
                                (((chunk & 7) ^ (key & 7)) << 4);
          uint32_t kb[4];
          ldmatrix_x4(kb, addr);
          mma_16816_f32(sacc[0], qa[ks][0], 0u, qa[ks][1], 0u, kb[0], kb[1]);
          mma_16816_f32(sacc[1], qa[ks][0], 0u, qa[ks][1], 0u, kb[2], kb[3]);
        }
      }
      // ---- online softmax of row r over this thread's 4 keys (and the quad's 16)
      const int key0 = (t_begin + i) * kDmTile + warp * 16;
      float t4[4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + n * 8 + 2 * c + e;
          const bool valid = key <= pos && key >= first_key;
          t4[n * 2 + e] = valid ? sacc[n][e] * scale_log2 : -INFINITY;
        }
      float mx = fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m, mx);
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      float p4[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) p4[e] = (t4[e] == -INFINITY) ? 0.f : exp2f(t4[e] - m_new);
      l = l * alpha + (p4[0] + p4[1] + p4[2] + p4[3]);
      m = m_new;
#pragma unroll
      for (int i = 0; i < HD16 * 2; ++i) { o[i][0] *= alpha; o[i][1] *= alpha; }
      // ---- O += P V : P (16 x 16 keys) straight from the accumulators
      const uint32_t pa0 = pack_bf16(p4[0], p4[1]), pa2 = pack_bf16(p4[2], p4[3]);
      {
        const int key = warp * 16 + (mat & 1) * 8 + rin;
#pragma unroll
        for (int np = 0; np < HD16; ++np) {                        // pairs of 8-dim tiles
          const int chunk = np * 2 + (mat >> 1);
          const uint32_t addr = vbase + (chunk >> 3) * (kDmTile * 128) + key * 128 +
                                (((chunk & 7) ^ (key & 7)) << 4);
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, addr);
          float c0[4] = {o[2 * np][0], o[2 * np][1], 0.f, 0.f};
          float c1[4] = {o[2 * np + 1][0], o[2 * np + 1][1], 0.f, 0.f};
          mma_16816_f32(c0, pa0, 0u, pa2, 0u, vb[0], vb[1]);
          mma_16816_f32(c1, pa0, 0u, pa2, 0u, vb[2], vb[3]);
          o[2 * np][0] = c0[0]; o[2 * np][1] = c0[1];
          o[2 * np + 1][0] = c1[0]; o[2 * np + 1][1] = c1[1];
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&empty[s]);
      if (++s == n_stages) { s = 0; ++turn; }
    }
    (void)ok;
    DM_STAMP(5);
    // ---- this warp's result for the merge
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (r < g) {
      if (c == 0) { mrg_m[warp * 8 + r] = m; mrg_l[warp * 8 + r] = l; }
#pragma unroll
      for (int i = 0; i < HD16 * 2; ++i) {
        mrg_o[((size_t)warp * 8 + r) * hd + i * 8 + 2 * c] = o[i][0];
        mrg_o[((size_t)warp * 8 + r) * hd + i * 8 + 2 * c + 1] = o[i][1];
      }
    }
    if (CLUSTER) {
      // Every CTA of the cluster runs by now (they all arrived at the kernel's start): send
      // m and l to all of them and each output's partial sum to the CTA that owns it.  The
      // warp reads its results back from shared memory so that a store instruction carries
      // 32 consecutive outputs to one owner (two at a border): a remote store costs per
      // destination segment, and straight from the accumulator layout it had eight.
      DM_STAMP(10);
      cluster_wait();
      __syncwarp();
      DM_STAMP(11);
      const uint32_t a_ml = tc::smem_u32(recv_ml + (size_t)(split * kDmWarps + warp) * 8 * 2);
      const uint32_t a_o = tc::smem_u32(recv_o + (size_t)(split * kDmWarps + warp) * share);
      for (int p = lane; p < n_splits * g; p += 32) {
        const int rank = div_by(p, g, g_magic), row = p - rank * g;
        st_cluster_f32(a_ml + row * 8, rank, mrg_m[warp * 8 + row]);
        st_cluster_f32(a_ml + row * 8 + 4, rank, mrg_l[warp * 8 + row]);
      }
#pragma unroll 4
      for (int idx = lane; idx < g * hd; idx += 32) {
        const int owner = div_by(idx, share, share_magic);
        st_cluster_f32(a_o + (idx - owner * share) * 4, owner, mrg_o[(size_t)warp * 8 * hd + idx]);
      }
      DM_STAMP(12);
    }
  }
  it_base += (uint32_t)my_tiles;
  __syncthreads();
  DM_STAMP(6);
  if (*abort && threadIdx.x == 0) atomicOr(fault, kFaultWaitExpired);

  if (CLUSTER) {
    // ---- the ranges are the CTAs of one cluster; after the barrier this CTA holds what all
    // warps of all ranges sent for its share of the outputs.  (A range without tiles sent
    // m = -inf, l = 0.)  Nothing remote is touched after the barrier, so a CTA may leave
    // as soon as it is done.
    cluster_arrive();
    cluster_wait();
    DM_STAMP(7);
    // Four lanes share an output, one per source warp; they meet by shuffles.
    const int total = g * hd, w = threadIdx.x & 3;
    for (int p0 = 0; p0 < share * kDmWarps; p0 += nthreads) {
      const int t = (p0 + threadIdx.x) >> 2, i = split * share + t;
      const bool live = t < share && i < total;
      const int j = live ? i / hd : 0;
      // all loads up front (at most kDmClusterMax ranges)
      float mw[kDmClusterMax], lw[kDmClusterMax], ow[kDmClusterMax];
#pragma unroll
      for (int rank = 0; rank < kDmClusterMax; ++rank) {
        const bool in = live && rank < n_splits;
        const int sw = rank * kDmWarps + w;
        mw[rank] = in ? recv_ml[(sw * 8 + j) * 2] : -INFINITY;
        lw[rank] = in ? recv_ml[(sw * 8 + j) * 2 + 1] : 0.f;
        ow[rank] = in ? recv_o[(size_t)sw * share + t] : 0.f;
      }
      float mm = -INFINITY;
#pragma unroll
      for (int rank = 0; rank < kDmClusterMax; ++rank) mm = fmaxf(mm, mw[rank]);
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 1));
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 2));
      float acc = 0.f, ll = 0.f;
#pragma unroll
      for (int rank = 0; rank < kDmClusterMax; ++rank) {
        const float f = (mw[rank] == -INFINITY) ? 0.f : exp2f(mw[rank] - mm);
        acc = fmaf(f, ow[rank], acc);
        ll = fmaf(f, lw[rank], ll);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      ll += __shfl_xor_sync(0xffffffffu, ll, 1);
      ll += __shfl_xor_sync(0xffffffffu, ll, 2);
      if (live && w == 0)
        out[(size_t)b * ldo + (size_t)kvh * g * hd + i] = __float2bfloat16_rn(acc / ll);
    }
    DM_STAMP(8);
    return;
  }

  // ---- merge the four warps into this range's partial (unnormalised o, m, l)
  float* po = part_o + (((size_t)b * nh + (size_t)kvh * g) * n_splits + split) * hd;
  float* pml = part_ml + (((size_t)b * nh + (size_t)kvh * g) * n_splits + split) * 2;
  for (int i = threadIdx.x; i < g * hd; i += nthreads) {
    const int j = i / hd, d = i - j * hd;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDmWarps; ++w) mm = fmaxf(mm, my_tiles > 0 ? mrg_m[w * 8 + j] : -INFINITY);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < kDmWarps; ++w) {
      const float mw = my_tiles > 0 ? mrg_m[w * 8 + j] : -INFINITY;
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      acc = fmaf(f, my_tiles > 0 ? mrg_o[((size_t)w * 8 + j) * hd + d] : 0.f, acc);
      ll = fmaf(f, my_tiles > 0 ? mrg_l[w * 8 + j] : 0.f, ll);
    }
    po[(size_t)j * n_splits * hd + d] = acc;
    if (d == 0) { pml[(size_t)j * n_splits * 2] = mm; pml[(size_t)j * n_splits * 2 + 1] = ll; }
  }

  // ---- the CTA that finishes last for this (sequence, kv head) merges the ranges
  __syncthreads();
  DM_STAMP(7);
  if (threadIdx.x == 0) {
    __threadfence();
    DM_STAMP(8);
    int* ctr = counters + (size_t)b * nkv + kvh;
    const int prev = atomicAdd(ctr, 1);
    *is_last = prev == n_splits - 1;
    if (*is_last) { *ctr = 0; __threadfence(); }
  }
  __syncthreads();
  DM_STAMP(9);
  if (!*is_last) return;
  const bool stamping_last = kStamps && stamps && kvh == 0 && b == 0;
  if (stamping_last && threadIdx.x == 0) stamp(8, 0);
  float* wts = mrg;                       // [g][n_splits]
  float* inv_den = mrg + 8 * kDmTile;     // [g]
  const float* ml_base = part_ml + ((size_t)b * nh + (size_t)kvh * g) * n_splits * 2;
  const float* po_base = part_o + ((size_t)b * nh + (size_t)kvh * g) * n_splits * hd;
  for (int j = warp; j < g; j += (nthreads >> 5)) {
    float mx = -INFINITY;
    for (int s = lane; s < n_splits; s += 32)
      mx = fmaxf(mx, __ldcg(ml_base + ((size_t)j * n_splits + s) * 2));
    mx = warp_max(mx);
    float den = 0.f;
    for (int s = lane; s < n_splits; s += 32) {
      const float ms = __ldcg(ml_base + ((size_t)j * n_splits + s) * 2);
      const float ls = __ldcg(ml_base + ((size_t)j * n_splits + s) * 2 + 1);
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - mx);
      wts[j * n_splits + s] = w;
      den += w * ls;
    }
    den = warp_sum(den);
    if (lane == 0) inv_den[j] = 1.0f / den;
  }
  __syncthreads();
  if (stamping_last && threadIdx.x == 0) stamp(8, 1);
  for (int i = threadIdx.x; i < g * hd; i += nthreads) {
    const int j = i / hd, d = i - j * hd;
    float acc_o = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 16) {
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
  if (stamping_last && threadIdx.x == 0) stamp(8, 2);
#undef DM_STAMP
}


// Shared-memory bytes of one CTA (without alignment slack) and the once-per-kernel set-up.
template <int HD16>
__host__ __device__ constexpr size_t dm_smem_core(bool cluster = false, int n_stages = kDmStages) {
  constexpr int hd = HD16 * 16;
  constexpr int kSub = (hd + 63) / 64;
  size_t bytes = (size_t)2 * n_stages * kSub * kDmTile * 128;    // K and V stages
  bytes += 2 * kDmMaxStages * 8 + 16;                             // barriers, abort, is_last
  bytes += dm_mrg_floats<HD16>() * 4;
  if (cluster)     // m, l of every warp of every range; a share of the outputs from each
    bytes += (size_t)kDmClusterMax * kDmWarps * 8 * 2 * 4 +
             (size_t)kDmWarps * (8 * hd + kDmClusterMax) * 4;
  return bytes;
}

template <int HD16>
__device__ __forceinline__ void dm_init(unsigned char* smem, int n_stages = kDmStages) {
  constexpr int hd = HD16 * 16;
  constexpr int kSub = (hd + 63) / 64;
  constexpr int kTileBytes = kSub * kDmTile * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + 2 * n_stages * kTileBytes);
  uint64_t* empty = full + kDmMaxStages;
  int* abort = reinterpret_cast<int*>(empty + kDmMaxStages);
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], kDmWarps); }
    *abort = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();
}

template <int HD16, bool CLUSTER>
__global__ void __launch_bounds__(kDmThreads)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v,
                       const __nv_bfloat16* __restrict__ q, int ldq,
                       const int* __restrict__ table, int table_stride,
                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ seq_slot, int nh, int nkv, float scale_log2,
                       int window, float* __restrict__ part_o, float* __restrict__ part_ml,
                       __nv_bfloat16* __restrict__ out, int ldo, int* __restrict__ counters,
                       unsigned int* __restrict__ fault, unsigned long long* stamps,
                       int n_stages) {
  extern __shared__ unsigned char smem_raw[];
  if (kStamps && stamps && blockIdx.x + blockIdx.y + blockIdx.z == 0 && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    stamps[9 * 16] = t;
  }
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  dm_init<HD16>(smem, n_stages);
  if (CLUSTER) cluster_arrive();      // "this CTA runs": waited for before anything is sent
  uint32_t it_base = 0;
  attn_decode_mma_item<HD16, CLUSTER>(smem, &map_k, &map_v, q, ldq, table, table_stride, tok_pos,
                                      tok_seq, seq_slot, nh, nkv, scale_log2, window, part_o,
                                      part_ml, out, ldo, counters, fault, blockIdx.x, gridDim.x,
                                      blockIdx.y, blockIdx.z, it_base, stamps, n_stages);
}

}  // namespace cretif
