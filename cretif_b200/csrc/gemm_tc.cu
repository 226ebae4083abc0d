// C[M,N] (= or +=) A[M,K] · W[N,K]^T on the fifth-generation tensor cores (prefill).
//
// A CTA is persistent: it computes 128 x BN tiles one after another (as many CTAs as fit the
// chip, each taking every gridDim.x-th tile).  Warp 0 is the producer: it moves 128x64
// tiles of A and BNx64 tiles of W from global to shared memory with TMA (128-byte swizzle;
// rows and columns beyond the matrices are filled with zeros, so any M, N and K % 8 == 0
// work) through a ring of stages guarded by full/empty mbarriers, which runs on from tile to
// tile.  One thread of warp 1 issues tcgen05.mma (M=128, N=BN, K=16, bf16 in, f32
// accumulate) on shared-memory descriptors into one of two 128 x BN accumulators in tensor
// memory and commits each stage back to the producer.  Warps 2-9 read an accumulator with
// tcgen05.ld (two threads share a row, half of the columns each: with four warps a tile's
// epilogue — a read-modify-write of the residual stream, a rotation or 128 x 128 SiLUs — took
// longer than its product) while the next tile's product fills the other, and store
// it as bfloat16 or float32, add it into a float32 matrix (the residual stream), or run one
// of the fused epilogues below.  Both operands are K-major exactly as activations
// [tokens, in] and weights [out, in] lie in memory, so nothing is transposed.  The kernel is
// a programmatic dependent of the one before it: set-up and the first W tiles precede the
// wait.
//
// The reference runs every product on a 32x32-tile CUDA-core kernel
// (src/kernels/matmul.cu:74-127); this kernel has no counterpart there.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "api.h"
#include "tc_common.cuh"

namespace cretif {

constexpr int kTcBM = 128, kTcBK = 64;
// Producer warp, MMA warp, and four or eight epilogue warps (one or two per quadrant of
// tensor-memory lanes): a template parameter, chosen per launch.
constexpr int tc_threads(int epilogue_warps) { return (2 + epilogue_warps) * 32; }

// The depth of the ring is chosen per launch.  With more tiles than SMs, narrow tiles take
// three stages so that two (BN = 128) or three (BN = 64) CTAs share an SM and hide each
// other's fill and drain, and the widest tile takes four.  A grid of at most one CTA per SM
// has the SM to itself: the ring is as deep as the k-blocks or shared memory allow, so that a
// short K (9 blocks at 576) is in flight almost at once.
constexpr int kTcMaxStages = 8;
template <int BN>
struct TcSmem {
  static constexpr int kATile = kTcBM * kTcBK * 2;
  static constexpr int kBTile = BN * kTcBK * 2;
  static constexpr int kStage = kATile + kBTile;
  // Staging for the epilogue that adds its tile into a float32 matrix through TMA: each of
  // the two groups of four warps has two slabs of 128 rows x 32 columns.
  // (The SiLU epilogue stores its tile the same way: two slabs of 128 rows x 64 bfloat16.)
  static constexpr int kSlab = kTcBM * 128;
  static constexpr int total(int stages, int slabs = 0) {   // stages, staging, barriers, align slack
    return stages * kStage + slabs * kSlab + (2 * kTcMaxStages + 4) * 8 + 16 + 1024;
  }
  // Tensor memory is handed out in powers of two columns; the two accumulators lie at
  // columns 0 and BN of the allocation.
  static constexpr int kTmemCols = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);
  static int stages_for(long long ctas, int num_kb, int sm_count) {
    int stages = BN >= 256 ? 4 : (BN >= 192 ? 5 : 3);
    if (ctas <= sm_count) {
      stages = num_kb < kTcMaxStages ? (num_kb < 3 ? 3 : num_kb) : kTcMaxStages;
      while (stages > 3 && total(stages) > 200 * 1024) --stages;
    }
    return stages;
  }
  static int stages_with_staging(int stages, int slabs) {
    while (stages > 2 && total(stages, slabs) > 227 * 1024) --stages;
    return stages;
  }
};

// What the epilogue warps do with the accumulator.
//   kTcStore  store as bfloat16 / float32, or add into a float32 matrix;
//   kTcSilu   the stacked gate|up product whose weight rows are interleaved in blocks of 64
//             (64 gate rows, then the 64 up rows that belong to them): a 128-wide tile holds
//             matching gate and up columns, and act = silu(gate) * up is stored (BN = 128);
//   kTcRope   the stacked q|k|v product with one head per tile (BN = head_dim): rotary on q and
//             k, q to the query buffer, k and v into the block cache at the token's position.
enum TcEpilogue : int { kTcStore = 0, kTcSilu = 1, kTcRope = 2 };

struct TcEpi {
  void* C; int ldc, accumulate;                            // store
  int bulk;        // through TMA (map_c): the float32 add of kTcStore, the store of kTcSilu
  __nv_bfloat16* act; int I;                               // silu
  __nv_bfloat16* Q; int ldq;                               // rope
  const float* cos_t; const float* sin_t;
  int pairing, nh, nkv, hd;
  const int* tok_pos; const int* tok_seq; const int* seq_slot; const int* table;
  int table_stride;
  __nv_bfloat16* kc; __nv_bfloat16* vc;
  int bt, write_cache;
};

__device__ __forceinline__ float round_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

template <int BN, int EPI, typename TC, int EW>
__global__ void __launch_bounds__(tc_threads(EW))
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_c, const TcEpi ep, int M, int N, int K,
               unsigned int* __restrict__ fault,
               int kTcStages, unsigned long long* stamps, int n_n_tiles, int n_tiles) {
  // Tuning aid: with a buffer given, lane 0 of each warp of the first CTA notes the time at
  // which it passes the phases of its first tile: [warp][8] nanoseconds.
  const bool stamping = kStamps && stamps && blockIdx.x == 0 && (threadIdx.x & 31) == 0;
  auto stamp = [&](int i) {
    if (stamping) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      stamps[(threadIdx.x >> 5) * 8 + i] = t;
    }
  };
  stamp(0);
  TC* const C = reinterpret_cast<TC*>(ep.C);
  const int ldc = ep.ldc, accumulate = ep.accumulate;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = TcSmem<BN>;
  constexpr bool kBulk = EPI == kTcStore && sizeof(TC) == 4;
  constexpr bool kBulkSilu = EPI == kTcSilu && EW == 8 && BN == 256;
  constexpr int kSlabs = kBulk ? EW / 2 : (kBulkSilu ? 2 : 0);     // two a group of four warps
  unsigned char* staging = smem + kTcStages * L::kStage;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + (kSlabs && ep.bulk ? kSlabs * L::kSlab : 0));
  uint64_t* empty = full + kTcMaxStages;
  uint64_t* acc_full = empty + kTcMaxStages;       // two accumulators in tensor memory
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + kTcBK - 1) / kTcBK;
  // The CTA is persistent: it takes tiles blockIdx.x, + gridDim.x, ...  (n fastest, so that the
  // CTAs running at one time share rows of A).  Tile coordinates are stepped, not divided.
  struct Tile {
    int mt, nt;
  };
  const int step_m = (int)gridDim.x / n_n_tiles, step_n = (int)gridDim.x - step_m * n_n_tiles;
  const Tile first = {(int)blockIdx.x / n_n_tiles, (int)blockIdx.x % n_n_tiles};
  auto next = [&](Tile& t) {
    t.mt += step_m;
    t.nt += step_n;
    if (t.nt >= n_n_tiles) { t.nt -= n_n_tiles; ++t.mt; }
  };
  const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { tc::mbar_init(&acc_full[b], 1); tc::mbar_init(&acc_empty[b], EW * 32); }
    *abort = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_descriptor(&map_a);
    tc::tma_prefetch_descriptor(&map_w);
  }
  if (warp == 1) {                       // one warp allocates both accumulators' columns
    tc::tmem_alloc(tmem_slot, L::kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  // Programmatic dependent launch: the kernel behind this one may begin its own set-up.  The
  // weights do not depend on the kernel before this one, so the first stages' W tiles are
  // asked for before the wait; A, and everything the epilogue reads or writes, after it.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  stamp(1);

  if (warp == 0) {
    if (lane == 0 && my_tiles > 0) {
      Tile t = first;
      const int early = num_kb < kTcStages ? num_kb : kTcStages;
      for (int kb = 0; kb < early; ++kb) {
        tc::mbar_expect_tx(&full[kb], (uint32_t)L::kStage);
        tc::tma_load_2d(smem + kb * L::kStage + L::kATile, &map_w, kb * kTcBK, t.nt * BN, &full[kb]);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      stamp(2);
      for (int kb = 0; kb < early; ++kb)
        tc::tma_load_2d(smem + kb * L::kStage, &map_a, kb * kTcBK, t.mt * kTcBM, &full[kb]);
      stamp(3);
      // (stage and turn of the ring are stepped, not divided: the depth is a run-time value)
      int s = early == kTcStages ? 0 : early, turn = early == kTcStages ? 1 : 0;
      bool ok = true;
      for (int i = 0; i < my_tiles && ok; ++i, next(t)) {
        for (int kb = i == 0 ? early : 0; kb < num_kb; ++kb) {
          if (turn > 0 && !tc::mbar_wait(&empty[s], (uint32_t)((turn - 1) & 1), abort)) {
            ok = false;
            break;
          }
          unsigned char* stage = smem + s * L::kStage;
          tc::mbar_expect_tx(&full[s], (uint32_t)L::kStage);
          tc::tma_load_2d(stage, &map_a, kb * kTcBK, t.mt * kTcBM, &full[s]);
          tc::tma_load_2d(stage + L::kATile, &map_w, kb * kTcBK, t.nt * BN, &full[s]);
          if (++s == kTcStages) { s = 0; ++turn; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc_bf16(kTcBM, BN);
      bool ok = true;
      int s = 0, turn = 0;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int buf = i & 1;
        // the epilogue warps have taken this accumulator's last tile (two tiles ago) out
        if (i >= 2) ok = tc::mbar_wait(&acc_empty[buf], (uint32_t)(((i >> 1) - 1) & 1), abort);
        if (!ok) break;
        tc::tc_fence_after();
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = tc::mbar_wait(&full[s], (uint32_t)(turn & 1), abort);
          if (!ok) break;
          tc::tc_fence_after();
          if (i == 0 && kb == 0) stamp(2);
          unsigned char* stage = smem + s * L::kStage;
          const uint64_t a_desc = tc::smem_desc_k_sw128(stage);
          const uint64_t b_desc = tc::smem_desc_k_sw128(stage + L::kATile);
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k)       // 16 bf16 = 32 bytes = 2 descriptor units
            tc::umma_bf16(tmem_acc + (uint32_t)(buf * BN), a_desc + 2 * k, b_desc + 2 * k, idesc,
                          (kb | k) != 0);
          tc::umma_commit(&empty[s]);                // frees the stage when these MMAs are done
          if (++s == kTcStages) { s = 0; ++turn; }
        }
        if (ok) tc::umma_commit(&acc_full[buf]);     // accumulator complete
        if (i == 0) stamp(3);
      }
    }
  } else {
    // ---- epilogue: a thread takes one row of the tile (TMEM lanes 32*(warp%4) ..) and one
    // half of its columns (warps 2-5 the first, 6-9 the second); the eight warps work on one
    // accumulator while the next tile's product fills the other
    const int quad = warp & 3, chalf = (warp - 2) >> 2;
    constexpr int halves = EW / 4;                             // 1: a thread takes a whole row
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(2);
    Tile t = first;
    bool alive = true;
    uint32_t slabs = 0;                      // slabs this group has handed to TMA so far
    for (int i = 0; i < my_tiles; ++i, next(t)) {
      const int buf = i & 1;
      const int m0 = t.mt * kTcBM, n0 = t.nt * BN;
      const int m = m0 + quad * 32 + lane;
      // Rotary epilogue: where this thread's row goes (position → slot → cache block) is a
      // chain of dependent loads that does not need the product: it runs while the product
      // does.  A tile holds BN / head_dim heads.
      const int hd = ep.hd, half = hd >> 1;
      const int head0 = EPI == kTcRope ? n0 / hd : 0;
      const bool row_ok = EPI == kTcRope && m < M;
      int pos = 0, blk = -1;
      if (row_ok) {
        pos = ep.tok_pos[m];
        if (ep.write_cache && head0 + BN / hd > ep.nh) {       // a key or value head is here
          const int slot = ep.seq_slot[ep.tok_seq[m]];
          blk = ep.table[(size_t)slot * ep.table_stride + pos / ep.bt];
          if (blk < 0) atomicOr(fault, kFaultBlockTable);
        }
      }
      // Rotary epilogue of wide tiles (three heads of 64): the row's cosines and sines are
      // the same for every head of the tile and do not depend on the product either.
      constexpr bool kHoist = EPI == kTcRope && EW == 8 && BN >= 192;
      float cs_r[kHoist ? 32 : 1], sn_r[kHoist ? 32 : 1];
      const bool hoisted = kHoist && half == 32 && ep.pairing == 0;
      if (kHoist && hoisted && row_ok) {
        const float* cs = ep.cos_t + (size_t)pos * half;
        const float* sn = ep.sin_t + (size_t)pos * half;
#pragma unroll
        for (int j = 0; j < (kHoist ? 32 : 0); j += 8) {
          float c8[8], s8[8];
          load8(cs + j, c8);
          load8(sn + j, s8);
#pragma unroll
          for (int e = 0; e < 8; ++e) { cs_r[j + e] = c8[e]; sn_r[j + e] = s8[e]; }
        }
      }
      // Adding into a float32 matrix: the values to add to do not depend on the product, so
      // a chunk's 32 of them are asked for before the accumulator is waited for, and the next
      // chunk's while this one is added and stored.  Only where a CTA has a tile or two and a
      // short K, so that the launch is latency from end to end (2,048 tokens at SmolLM2-135M
      // sizes: o-proj 10.0 -> 7.9 us, down-proj 14.5 -> 12.4 us); where persistent CTAs walk
      // many tiles, or K is long, the early loads only get in the operands' way (8 x 2,048
      // tokens: o-proj 40 -> 52 us; K = 8192: 76 -> 84 us).
      constexpr int kCols = BN / halves;                 // this thread's columns of the tile
      const int c_first = chalf * kCols;
      const bool pre = EPI == kTcStore && sizeof(TC) == 4 && EW == 4 && accumulate && num_kb <= 24;
      float4 oldv[8];
      auto fetch_old = [&](int c0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int n = n0 + c0 + 4 * j;
          oldv[j] = (m < M && n + 4 <= N)
                        ? __ldcg(reinterpret_cast<const float4*>(
                              reinterpret_cast<const float*>(ep.C) + (size_t)m * ldc + n))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      };
      if (pre) fetch_old(c_first);
      // (a wait that gave up: later waits return at once, and nothing more is stored)
      alive = tc::mbar_wait(&acc_full[buf], (uint32_t)((i >> 1) & 1), abort) && alive;
      const bool ok = alive;
      tc::tc_fence_after();
      if (i == 0) stamp(3);
      const uint32_t lane_acc = tmem_acc + (uint32_t)(buf * BN) + ((uint32_t)(quad * 32) << 16);
      if (kBulk && ep.bulk) {
        // The tile is added into the float32 matrix by TMA: a row per thread would touch 32
        // different lines with every load and store, and the old values would pass through
        // the SM at all.  Each group of four warps (128 rows, half of the columns) writes a
        // slab of 32 columns into shared memory in the 128-byte swizzle (eight 16-byte stores
        // a thread, conflict-free), one thread hands it to the copy engine, which adds it in
        // L2 and clips it at the matrix's edges; two slabs a group, so that one is filled
        // while the other drains.
        unsigned char* mine = staging + chalf * 2 * L::kSlab;
        const bool elected = ((warp - 2) & 3) == 0 && lane == 0;
        const int row = quad * 32 + lane;
#pragma unroll 1
        for (int c0 = c_first; c0 < c_first + kCols; c0 += 32, ++slabs) {
          uint32_t r[32];
          tc::tmem_load_32(lane_acc + (uint32_t)c0, r);
          tc::tmem_load_wait();
          if (elected) tc::bulk_wait_group_read<1>();       // the slab used two slabs ago is free
          asm volatile("bar.sync %0, 128;" ::"r"(1 + chalf) : "memory");
          unsigned char* slab = mine + (slabs & 1) * L::kSlab;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(slab + row * 128 + ((j ^ (row & 7)) << 4)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          tc::fence_proxy_async();
          asm volatile("bar.sync %0, 128;" ::"r"(1 + chalf) : "memory");
          if (elected) {                   // (a group for every slab, or the count above is off)
            if (ok && n0 + c0 < N) tc::tma_reduce_add_2d(&map_c, slab, n0 + c0, m0);
            tc::bulk_commit_group();
          }
        }
      } else if (ok && EPI == kTcStore) {
#pragma unroll 1
        for (int c0 = c_first; c0 < c_first + kCols; c0 += 32) {
          uint32_t r[32];
          tc::tmem_load_32(lane_acc + (uint32_t)c0, r);
          tc::tmem_load_wait();
          float4 cur[8];
          if (pre) {
#pragma unroll
            for (int j = 0; j < 8; ++j) cur[j] = oldv[j];
            if (c0 + 32 < c_first + kCols) fetch_old(c0 + 32);
          }
          if (m < M && n0 + c0 < N) {
            TC* out = C + (size_t)m * ldc + n0 + c0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
              const int n = n0 + c0 + j;
              if (n + 8 <= N) {
                if (pre) {
                  const float4 a = cur[j >> 2], b = cur[(j >> 2) + 1];
                  v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                  v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
                } else if (accumulate) {
                  float old[8];
                  load8(out + j, old);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] += old[e];
                }
                store8(out + j, v);
              } else {
                for (int e = 0; e < 8 && n + e < N; ++e) {
                  float x = v[e];
                  if (accumulate) x += to_float(out[j + e]);
                  out[j + e] = from_float<TC>(x);
                }
              }
            }
          }
        }
      }
      if (kBulkSilu && ep.bulk) {
        // act = silu(gate) * up leaves through shared memory and TMA as well: the two groups
        // fill the halves of a slab of 128 rows x 64 columns (a thread's 32 values are four
        // 16-byte pieces of its row's 128-byte line), one thread hands it over.
        const bool elected = warp == 2 && lane == 0;
        const int row = quad * 32 + lane;
#pragma unroll 1
        for (int pair = 0; pair < BN / 128; ++pair, ++slabs) {
          const int col0 = (n0 >> 1) + pair * 64;
          const int c0 = chalf * 32;
          uint32_t g[32], u[32];
          tc::tmem_load_32(lane_acc + (uint32_t)(pair * 128 + c0), g);
          tc::tmem_load_32(lane_acc + (uint32_t)(pair * 128 + 64 + c0), u);
          tc::tmem_load_wait();
          if (elected) tc::bulk_wait_group_read<1>();
          asm volatile("bar.sync 3, 256;" ::: "memory");
          unsigned char* slab = staging + (slabs & 1) * L::kSlab;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint32_t w4[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              const float g0 = round_bf16(__uint_as_float(g[j + e]));
              const float g1 = round_bf16(__uint_as_float(g[j + e + 1]));
              const float u0 = round_bf16(__uint_as_float(u[j + e]));
              const float u1 = round_bf16(__uint_as_float(u[j + e + 1]));
              __nv_bfloat162 h2 = __floats2bfloat162_rn(silu_bf16_path(g0) * u0,
                                                        silu_bf16_path(g1) * u1);
              w4[e >> 1] = *reinterpret_cast<uint32_t*>(&h2);
            }
            const int piece = chalf * 4 + (j >> 3);
            *reinterpret_cast<uint4*>(slab + row * 128 + ((piece ^ (row & 7)) << 4)) =
                make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
          tc::fence_proxy_async();
          asm volatile("bar.sync 3, 256;" ::: "memory");
          if (elected) {
            if (ok && col0 < ep.I) tc::tma_store_2d(&map_c, slab, col0, m0);
            tc::bulk_commit_group();
          }
        }
      } else if (ok && EPI == kTcSilu) {
        // every 128 tile columns are 64 gate columns and the 64 up columns that belong to
        // them: act[:, n0/2 + 64 pair ..]
#pragma unroll 1
        for (int pair = 0; pair < BN / 128; ++pair) {
          const int col0 = (n0 >> 1) + pair * 64;
#pragma unroll 1
          for (int c0 = chalf * (64 / halves); c0 < (chalf + 1) * (64 / halves); c0 += 32) {
            uint32_t g[32], u[32];
            tc::tmem_load_32(lane_acc + (uint32_t)(pair * 128 + c0), g);
            tc::tmem_load_32(lane_acc + (uint32_t)(pair * 128 + 64 + c0), u);
            tc::tmem_load_wait();
            if (m < M && col0 + c0 < ep.I) {
              __nv_bfloat16* out = ep.act + (size_t)m * ep.I + col0 + c0;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  // gate and up pass through bfloat16 as they do when stored separately
                  const float gg = round_bf16(__uint_as_float(g[j + e]));
                  const float uu = round_bf16(__uint_as_float(u[j + e]));
                  v[e] = silu_bf16_path(gg) * uu;
                }
                if (col0 + c0 + j + 8 <= ep.I) store8(out + j, v);
              }
            }
          }
        }
      }
      if (ok && EPI == kTcRope) {
        const float* cs = ep.cos_t + (size_t)pos * half;
        const float* sn = ep.sin_t + (size_t)pos * half;
        // the heads of a tile go to the two warps of a row in turn (a tile of one head is
        // the first warp's)
        for (int hh = chalf; hh * hd < BN; hh += halves) {
          const int head = head0 + hh;                   // (the same for the whole warp)
          if (head >= ep.nh + 2 * ep.nkv) break;
          const uint32_t acc_h = lane_acc + (uint32_t)(hh * hd);
          const bool rotate = head < ep.nh + ep.nkv;
          __nv_bfloat16* dst = nullptr;                  // where this row's head goes
          if (row_ok) {
            if (head < ep.nh) {
              dst = ep.Q + (size_t)m * ep.ldq + (size_t)head * hd;
            } else if (blk >= 0) {
              const int kvh = rotate ? head - ep.nh : head - ep.nh - ep.nkv;
              dst = (rotate ? ep.kc : ep.vc) +
                    (((size_t)blk * ep.nkv + kvh) * ep.bt + (pos % ep.bt)) * hd;
            }
          }
          if (!rotate) {
#pragma unroll 1
            for (int c0 = 0; c0 < hd; c0 += 32) {
              uint32_t r[32];
              tc::tmem_load_32(acc_h + (uint32_t)c0, r);
              tc::tmem_load_wait();
              if (dst) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  float v[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
                  store8(dst + c0 + j, v);
                }
              }
            }
          } else if (kHoist && hoisted) {          // pairs (j, j + 32), table rows in registers
            uint32_t lo[32], hi[32];
            tc::tmem_load_32(acc_h, lo);
            tc::tmem_load_32(acc_h + 32u, hi);
            tc::tmem_load_wait();
            if (dst) {
#pragma unroll
              for (int j = 0; j < (kHoist ? 32 : 0); j += 8) {
                float y0[8], y1[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float x0 = round_bf16(__uint_as_float(lo[j + e]));
                  const float x1 = round_bf16(__uint_as_float(hi[j + e]));
                  y0[e] = x0 * cs_r[j + e] - x1 * sn_r[j + e];
                  y1[e] = x0 * sn_r[j + e] + x1 * cs_r[j + e];
                }
                store8(dst + j, y0);
                store8(dst + 32 + j, y1);
              }
            }
          } else if (ep.pairing == 0) {            // pairs (j, j + head_dim/2)
#pragma unroll 1
            for (int c0 = 0; c0 < half; c0 += 32) {
              uint32_t lo[32], hi[32];
              tc::tmem_load_32(acc_h + (uint32_t)c0, lo);
              tc::tmem_load_32(acc_h + (uint32_t)(half + c0), hi);
              tc::tmem_load_wait();
              if (dst) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  float c8[8], s8[8], y0[8], y1[8];
                  load8(cs + c0 + j, c8);
                  load8(sn + c0 + j, s8);
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const float x0 = round_bf16(__uint_as_float(lo[j + e]));
                    const float x1 = round_bf16(__uint_as_float(hi[j + e]));
                    y0[e] = x0 * c8[e] - x1 * s8[e];
                    y1[e] = x0 * s8[e] + x1 * c8[e];
                  }
                  store8(dst + c0 + j, y0);
                  store8(dst + half + c0 + j, y1);
                }
              }
            }
          } else {                                  // pairs (2j, 2j + 1)
#pragma unroll 1
            for (int c0 = 0; c0 < hd; c0 += 32) {
              uint32_t r[32];
              tc::tmem_load_32(acc_h + (uint32_t)c0, r);
              tc::tmem_load_wait();
              if (dst) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  float y[8];
#pragma unroll
                  for (int e = 0; e < 8; e += 2) {
                    const int jj = (c0 + j + e) >> 1;
                    const float x0 = round_bf16(__uint_as_float(r[j + e]));
                    const float x1 = round_bf16(__uint_as_float(r[j + e + 1]));
                    y[e] = x0 * cs[jj] - x1 * sn[jj];
                    y[e + 1] = x0 * sn[jj] + x1 * cs[jj];
                  }
                  store8(dst + c0 + j, y);
                }
              }
            }
          }
        }
      }
      tc::tc_fence_before();
      tc::mbar_arrive(&acc_empty[buf]);        // this accumulator may be overwritten
    }
    if (kSlabs && ep.bulk && ((warp - 2) & 3) == 0 && lane == 0) tc::bulk_wait_all();
  }
  stamp(4);
  if (*abort && threadIdx.x == 0) atomicOr(fault, kFaultWaitExpired);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_acc, L::kTmemCols);
  }
  stamp(5);
}


// ---------------------------------------------------------------------------------------
// Two CTAs on one tile of 256 rows (cta_group::2).
//
// With a tile of its own a CTA pulls (128 + BN) x 64 x 2 bytes through its SM's port to L2 per
// k-block of 4 x BN / 2 cycles of products: 96 bytes a cycle at BN = 256, more for narrower
// tiles, and the port gives some 70 (the widest product here stops at 0.76 of the tensor
// peak, gate|up at 0.65).  Here the CTAs of a cluster of two share a tile: each loads its
// 128 rows of A and its 128 of the 256 rows of W, CTA 0 issues one product of M = 256 for
// both, and each ends up with its 128 rows of the accumulator in its own tensor memory: 64
// bytes a cycle per SM.  The loads of both CTAs are counted on CTA 0's barriers; its commits
// arrive on the barriers of both.  Epilogues: the float32 add and the SiLU store through
// shared-memory slabs and TMA, as above.
constexpr int kTpThreads = 320;         // producer, issuer, eight epilogue warps
template <int kTpBN>                    // the tile's width: 256, or 192 for widths like 576 and 960
struct TpSmem {
  static constexpr int kATile = kTcBM * kTcBK * 2;       // this CTA's 128 rows of A
  static constexpr int kBTile = (kTpBN / 2) * kTcBK * 2; // its half of the tile's rows of W
  static constexpr int kStage = kATile + kBTile;
  static constexpr int kSlab = kTcBM * 128;
  static constexpr int total(int stages, int slabs) {
    return stages * kStage + slabs * kSlab + (2 * kTcMaxStages + 4) * 8 + 16 + 1024;
  }
};

template <int kTpBN, int EPI>
__global__ void __launch_bounds__(kTpThreads)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_c, const TcEpi ep, int M, int N, int K,
                    unsigned int* __restrict__ fault, int n_stages, int n_n_tiles, int n_tiles) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = TpSmem<kTpBN>;
  constexpr int kSlabs = EPI == kTcStore ? 4 : 2;
  unsigned char* staging = smem + n_stages * L::kStage;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + kSlabs * L::kSlab);   // used in CTA 0
  uint64_t* empty = full + kTcMaxStages;
  uint64_t* acc_full = empty + kTcMaxStages;
  uint64_t* acc_empty = acc_full + 2;                                          // used in CTA 0
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_rank();
  const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
  const int num_kb = (K + kTcBK - 1) / kTcBK;
  const int my_tiles = pair < n_tiles ? (n_tiles - 1 - pair) / n_pairs + 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 2 * 8);       // a warp of either CTA at a time
    }
    *abort = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_descriptor(&map_a);
    tc::tma_prefetch_descriptor(&map_w);
    tc::tma_prefetch_descriptor(&map_c);
  }
  if (warp == 1) {
    tc::tmem_alloc_pair(tmem_slot, 512);
    tc::tmem_relinquish_pair();
  }
  tc::tc_fence_before();
  tc::cluster_sync_all();                 // both CTAs' barriers exist before either touches them
  tc::tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    if (lane == 0 && my_tiles > 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      int s = 0, turn = 0;
      bool ok = true;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int tile = pair + i * n_pairs;
        const int mt = tile / n_n_tiles, nt = tile - mt * n_n_tiles;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (turn > 0 && !tc::mbar_wait(&empty[s], (uint32_t)((turn - 1) & 1), abort)) {
            ok = false;
            break;
          }
          unsigned char* stage = smem + s * L::kStage;
          if (rank == 0) tc::mbar_expect_tx(&full[s], 2u * L::kStage);    // both CTAs' bytes
          const uint32_t bar = tc::cluster_addr(&full[s], 0);
          tc::tma_load_2d_pair(stage, &map_a, kb * kTcBK, mt * 2 * kTcBM + (int)rank * kTcBM, bar);
          tc::tma_load_2d_pair(stage + L::kATile, &map_w, kb * kTcBK,
                               nt * kTpBN + (int)rank * (kTpBN / 2), bar);
          if (++s == n_stages) { s = 0; ++turn; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = tc::instr_desc_bf16(2 * kTcBM, kTpBN);
      bool ok = true;
      int s = 0, turn = 0;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int buf = i & 1;
        if (i >= 2) ok = tc::mbar_wait(&acc_empty[buf], (uint32_t)(((i >> 1) - 1) & 1), abort);
        if (!ok) break;
        tc::tc_fence_after();
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = tc::mbar_wait(&full[s], (uint32_t)(turn & 1), abort);
          if (!ok) break;
          tc::tc_fence_after();
          unsigned char* stage = smem + s * L::kStage;
          const uint64_t a_desc = tc::smem_desc_k_sw128(stage);
          const uint64_t b_desc = tc::smem_desc_k_sw128(stage + L::kATile);
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k)
            tc::umma_bf16_pair(tmem_acc + (uint32_t)(buf * kTpBN), a_desc + 2 * k, b_desc + 2 * k,
                               idesc, (kb | k) != 0);
          tc::umma_commit_pair(&empty[s], 3);          // frees the stage in both CTAs
          if (++s == n_stages) { s = 0; ++turn; }
        }
        if (ok) tc::umma_commit_pair(&acc_full[buf], 3);
      }
    }
  } else {
    // ---- epilogue (both CTAs): a thread takes one of this CTA's 128 rows and half of the
    // tile's columns; see the bulk epilogues of gemm_tc_kernel
    const int quad = warp & 3, chalf = (warp - 2) >> 2;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool alive = true;
    uint32_t slabs = 0;
    const uint32_t acc_empty_leader[2] = {tc::cluster_addr(&acc_empty[0], 0),
                                          tc::cluster_addr(&acc_empty[1], 0)};
    const int row = quad * 32 + lane;
    for (int i = 0; i < my_tiles; ++i) {
      const int buf = i & 1;
      const int tile = pair + i * n_pairs;
      const int mt = tile / n_n_tiles, nt = tile - mt * n_n_tiles;
      const int m0 = mt * 2 * kTcBM + (int)rank * kTcBM, n0 = nt * kTpBN;
      alive = tc::mbar_wait(&acc_full[buf], (uint32_t)((i >> 1) & 1), abort) && alive;
      const bool ok = alive;
      tc::tc_fence_after();
      const uint32_t lane_acc = tmem_acc + (uint32_t)(buf * kTpBN) + ((uint32_t)(quad * 32) << 16);
      if (EPI == kTcStore) {
        unsigned char* mine = staging + chalf * 2 * L::kSlab;
        const bool elected = ((warp - 2) & 3) == 0 && lane == 0;
#pragma unroll 1
        for (int c0 = chalf * (kTpBN / 2); c0 < (chalf + 1) * (kTpBN / 2); c0 += 32, ++slabs) {
          uint32_t r[32];
          tc::tmem_load_32(lane_acc + (uint32_t)c0, r);
          tc::tmem_load_wait();
          if (elected) tc::bulk_wait_group_read<1>();
          asm volatile("bar.sync %0, 128;" ::"r"(1 + chalf) : "memory");
          unsigned char* slab = mine + (slabs & 1) * L::kSlab;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(slab + row * 128 + ((j ^ (row & 7)) << 4)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          tc::fence_proxy_async();
          asm volatile("bar.sync %0, 128;" ::"r"(1 + chalf) : "memory");
          if (elected) {
            if (ok && n0 + c0 < N) tc::tma_reduce_add_2d(&map_c, slab, n0 + c0, m0);
            tc::bulk_commit_group();
          }
        }
      } else {
        const bool elected = warp == 2 && lane == 0;
#pragma unroll 1
        for (int pr = 0; pr < kTpBN / 128; ++pr, ++slabs) {
          const int col0 = (n0 >> 1) + pr * 64;
          const int c0 = chalf * 32;
          uint32_t g[32], u[32];
          tc::tmem_load_32(lane_acc + (uint32_t)(pr * 128 + c0), g);
          tc::tmem_load_32(lane_acc + (uint32_t)(pr * 128 + 64 + c0), u);
          tc::tmem_load_wait();
          if (elected) tc::bulk_wait_group_read<1>();
          asm volatile("bar.sync 3, 256;" ::: "memory");
          unsigned char* slab = staging + (slabs & 1) * L::kSlab;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint32_t w4[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              const float g0 = round_bf16(__uint_as_float(g[j + e]));
              const float g1 = round_bf16(__uint_as_float(g[j + e + 1]));
              const float u0 = round_bf16(__uint_as_float(u[j + e]));
              const float u1 = round_bf16(__uint_as_float(u[j + e + 1]));
              __nv_bfloat162 h2 = __floats2bfloat162_rn(silu_bf16_path(g0) * u0,
                                                        silu_bf16_path(g1) * u1);
              w4[e >> 1] = *reinterpret_cast<uint32_t*>(&h2);
            }
            const int piece = chalf * 4 + (j >> 3);
            *reinterpret_cast<uint4*>(slab + row * 128 + ((piece ^ (row & 7)) << 4)) =
                make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
          tc::fence_proxy_async();
          asm volatile("bar.sync 3, 256;" ::: "memory");
          if (elected) {
            if (ok && col0 < ep.I) tc::tma_store_2d(&map_c, slab, col0, m0);
            tc::bulk_commit_group();
          }
        }
      }
      // this CTA's half of the accumulator may be overwritten: CTA 0's issuer is told
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive_cluster(acc_empty_leader[buf]);
    }
    if (((EPI == kTcStore && ((warp - 2) & 3) == 0) || (EPI != kTcStore && warp == 2)) && lane == 0)
      tc::bulk_wait_all();
  }
  if (*abort && threadIdx.x == 0) atomicOr(fault, kFaultWaitExpired);
  tc::tc_fence_before();
  tc::cluster_sync_all();                 // no commit is on its way to a CTA that has left
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc_pair(tmem_acc, 512);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// A [rows, cols] bf16 matrix with row stride ld (elements), boxes of box_rows x box_cols;
// with the 128-byte swizzle a box is 64 columns wide.  Encoding a map costs a few microseconds on the host, and weights, the cache and recycled
// activation buffers come back with the same address and shape, so recent maps are kept.
struct MapKey {
  const void* base;
  int rows, cols, ld, box_rows, box_cols;
  bool swizzle, f32;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && box_cols == o.box_cols && swizzle == o.swizzle &&
           f32 == o.f32;
  }
};
constexpr int kMapCacheSize = 1024;
static MapKey g_map_keys[kMapCacheSize];
static CUtensorMap g_map_vals[kMapCacheSize];
static bool g_map_used[kMapCacheSize];
static std::mutex g_map_mutex;

static int make_box_map(CUtensorMap* map, const void* base, int rows, int cols, int ld,
                        int box_rows, int box_cols, bool swizzle, bool f32) {
  const int elem_bytes = f32 ? 4 : 2;
  if (box_rows < 1 || box_rows > 256 || box_cols < 4 || box_cols > 256 ||
      (swizzle && box_cols * elem_bytes != 128))
    return kBadArgument;
  const MapKey key = {base, rows, cols, ld, box_rows, box_cols, swizzle, f32};
  size_t hsh = (size_t)((uintptr_t)base >> 4) * 1000003u ^ (size_t)rows * 8191u ^
               (size_t)cols * 131u ^ (size_t)ld * 31u ^ (size_t)box_rows ^
               (size_t)box_cols * 524287u ^ (size_t)swizzle ^ ((size_t)f32 << 1);
  const int at = (int)(hsh % kMapCacheSize);
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (g_map_used[at] && g_map_keys[at] == key) {
      *map = g_map_vals[at];
      return 0;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return kBadArgument;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1u, 1u};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims,
                  strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return kBadArgument;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  g_map_keys[at] = key;
  g_map_vals[at] = *map;
  g_map_used[at] = true;
  return 0;
}

int make_box_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows,
                      int box_cols, bool swizzle) {
  return make_box_map(map, base, rows, cols, ld, box_rows, box_cols, swizzle, false);
}

int make_tile_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int ld,
                       int box_rows) {
  return make_box_map_bf16(map, base, rows, cols, ld, box_rows, 64, true);
}

// Tuning aid: a device buffer of 6 x 8 timestamps that the next launches fill (see the kernel).
static unsigned long long* g_tc_stamps = nullptr;
// Epilogue warps: 0 chooses per launch, 4 or 8 force (for tests that run both).
static int g_tc_epilogue_warps = 0;
// Epilogues through shared memory and TMA (the float32 add, the SiLU store) where the kernel
// can: 1 (default), 0 never (for tests that run both).
static int g_tc_bulk_add = 1;

// Two CTAs on one tile where the launch is large enough: -1 (default), 0 never, 1 wherever
// the kernel takes the product (for tests that run both).
static int g_tc_pair = -1;

// Measured at 16,384 rows (single-CTA tiles against pairs, us): 3072 x 576 47 / 55, 576 x 1536
// 33 / 33, 5120 x 960 120 / 115, 960 x 2560 80 / 77, 2048 x 2048 123 / 112, 16384 x 2048 829 / 743,
// 2048 x 8192 442 / 417: pairs pay once a tile's products outlast what two CTAs spend on
// telling each other.
static bool pair_pays(int N, int K) { return (long long)N * K >= (2LL << 20); }

template <int kTpBN, int EPI>
static int launch_tc_pair(const void* A, const void* W, TcEpi ep, int M, int N, int K, int lda,
                          int ldw, unsigned int* fault, cudaStream_t st) {
  CUtensorMap map_a, map_w, map_c;
  if (make_tile_map_bf16(&map_a, A, M, K, lda, kTcBM)) return kBadArgument;
  if (make_tile_map_bf16(&map_w, W, N, K, ldw, kTpBN / 2)) return kBadArgument;
  if (EPI == kTcStore ? make_box_map(&map_c, ep.C, M, N, ep.ldc, kTcBM, 32, true, true)
                      : make_box_map(&map_c, ep.act, M, ep.I, ep.I, kTcBM, 64, true, false))
    return kBadArgument;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  const int n_n_tiles = (N + kTpBN - 1) / kTpBN;
  const long long tiles = (long long)n_n_tiles * ((M + 2 * kTcBM - 1) / (2 * kTcBM));
  if (tiles > 0x7fffffffLL) return kBadArgument;
  constexpr int kSlabs = EPI == kTcStore ? 4 : 2;
  int stages = kTcMaxStages;
  while (stages > 2 && TpSmem<kTpBN>::total(stages, kSlabs) > 227 * 1024) --stages;
  const int smem = TpSmem<kTpBN>::total(stages, kSlabs);
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<kTpBN, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  const long long pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kTpThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  ep.bulk = 1;
  count_variant(kVarTcPair);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<kTpBN, EPI>, map_a, map_w, map_c, ep, M,
                                           N, K, fault, stages, n_n_tiles, (int)tiles);
  return e == cudaSuccess ? launch_status() : (int)e;
}

// Registers of a thread of the kernel, for the residency estimate (once per instantiation).
template <int BN, int EPI, typename TC, int EW>
static int tc_regs_per_thread() {
  static int regs = 0;
  if (!regs) {
    cudaFuncAttributes fa;
    regs = cudaFuncGetAttributes(&fa, gemm_tc_kernel<BN, EPI, TC, EW>) == cudaSuccess &&
                   fa.numRegs > 0 ? fa.numRegs : 128;
  }
  return regs;
}

template <int BN, int EPI, typename TC, int EW>
static cudaError_t launch_tc_kernel(const cudaLaunchConfig_t& cfg, int smem,
                                    const CUtensorMap& map_a, const CUtensorMap& map_w,
                                    const CUtensorMap& map_c, const TcEpi& ep, int M, int N, int K,
                                    unsigned int* fault,
                                    int stages, unsigned long long* stamps, int n_n_tiles,
                                    int tiles) {
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, TC, EW>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, EPI, TC, EW>, map_a, map_w, map_c, ep, M, N, K,
                            fault, stages, stamps, n_n_tiles, tiles);
}

template <int BN, int EPI, typename TC>
static int launch_tc(const void* A, const void* W, const TcEpi& ep_in, int M, int N, int K, int lda,
                     int ldw, unsigned int* fault, cudaStream_t st) {
  TcEpi ep = ep_in;
  CUtensorMap map_a, map_w, map_c = {};
  if (make_tile_map_bf16(&map_a, A, M, K, lda, kTcBM)) return kBadArgument;
  if (make_tile_map_bf16(&map_w, W, N, K, ldw, BN)) return kBadArgument;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  const int n_n_tiles = (N + BN - 1) / BN;
  const long long tiles = (long long)n_n_tiles * ((M + kTcBM - 1) / kTcBM);
  if (tiles > 0x7fffffffLL) return kBadArgument;
  int stages = TcSmem<BN>::stages_for(tiles, (K + kTcBK - 1) / kTcBK, sm_count);
  int smem = TcSmem<BN>::total(stages);
  // Persistent CTAs: as many as fit the chip at once (by shared memory and by the 512 columns
  // of tensor memory, of which a CTA holds two accumulators), each walking its share of tiles.
  // Eight epilogue warps where CTAs walk several tiles: a tile's epilogue (a read-modify-write
  // of the residual stream, a rotation, 128 x 128 SiLUs) then has to keep pace with the next
  // tile's product, which four warps do not (2048 x 8 tokens at SmolLM2-135M sizes: o-proj
  // 48 -> 41 us, down-proj 61 -> 53 us).  A launch of a tile or two per CTA is latency from
  // end to end and gains nothing from the larger block, and with a long K (8192: 432 -> 479
  // us) the product hides any epilogue and the larger block only costs.
  // CTAs that fit an SM at once: by shared memory, by the 512 columns of tensor memory and by
  // the register file (registers are handed out per warp in units of 256).
  auto residents = [&](int warps) {
    const int regs_per_thread = warps == 8 ? tc_regs_per_thread<BN, EPI, TC, 8>()
                                           : tc_regs_per_thread<BN, EPI, TC, 4>();
    int n = (227 * 1024) / smem;
    if (n > 512 / TcSmem<BN>::kTmemCols) n = 512 / TcSmem<BN>::kTmemCols;
    const int regs_per_warp = (regs_per_thread * 32 + 255) / 256 * 256;
    const int by_regs = 65536 / ((2 + warps) * regs_per_warp);
    if (n > by_regs) n = by_regs;
    return n < 1 ? 1 : n;
  };
  int epi_warps = g_tc_epilogue_warps;
  if (epi_warps != 4 && epi_warps != 8)
    epi_warps = tiles > 2LL * residents(4) * sm_count && K <= 4096 ? 8 : 4;
  // The float32 add through TMA needs room for its slabs (two a group of four epilogue
  // warps).  Measured against the add by the epilogue's threads, us: 4,096 x 576 x 576 24.4 ->
  // 11.4, x 1,536 29.6 -> 20.6; 2,048 x 576 x 1,536 13.7 -> 12.0; 2,048 x 960 x 2,560 22.6 -> 17.2;
  // 2,048 x 2,048 x 2,048 28.2 -> 26.1; with K = 8,192 the stages it takes away cost more than
  // it saves (69.6 -> 94.2).
  ep.bulk = 0;
  if (EPI == kTcStore && sizeof(TC) == 4 && ep.accumulate && K <= 4096 && g_tc_bulk_add && ep.ldc % 4 == 0 && ((uintptr_t)ep.C & 15) == 0 &&
      make_box_map(&map_c, ep.C, M, N, ep.ldc, kTcBM, 32, true, true) == 0) {
    ep.bulk = 1;
    stages = TcSmem<BN>::stages_with_staging(stages, epi_warps / 2);
    smem = TcSmem<BN>::total(stages, epi_warps / 2);
    count_variant(kVarTcBulkAdd);
  }
  if (EPI == kTcSilu && epi_warps == 8 && BN == 256 && g_tc_bulk_add &&
      make_box_map(&map_c, ep.act, M, ep.I, ep.I, kTcBM, 64, true, false) == 0) {
    ep.bulk = 1;
    stages = TcSmem<BN>::stages_with_staging(stages, 2);
    smem = TcSmem<BN>::total(stages, 2);
    count_variant(kVarTcBulkAdd);
  }
  const int per_sm = residents(epi_warps);
  const long long resident = (long long)per_sm * sm_count;
  const dim3 grid((unsigned)(tiles < resident ? tiles : resident));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(tc_threads(epi_warps));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  count_variant(BN == 64 ? kVarTc64 : BN == 128 ? kVarTc128 : BN == 192 ? kVarTc192 : kVarTc256);
  if (tiles > resident) count_variant(kVarTcSeveralTiles);
  const cudaError_t e =
      epi_warps == 8 ? launch_tc_kernel<BN, EPI, TC, 8>(cfg, smem, map_a, map_w, map_c, ep, M, N, K,
                                                        fault, stages, g_tc_stamps, n_n_tiles,
                                                        (int)tiles)
                     : launch_tc_kernel<BN, EPI, TC, 4>(cfg, smem, map_a, map_w, map_c, ep, M, N, K,
                                                        fault, stages, g_tc_stamps, n_n_tiles,
                                                        (int)tiles);
  return e == cudaSuccess ? launch_status() : (int)e;
}

static bool tc_operands_ok(const void* A, const void* W, int M, int K, int lda, int ldw) {
  return K > 0 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K &&
         (M + kTcBM - 1) / kTcBM <= 65535 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0;
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_set_tc_pair(int mode) {
  const int was = g_tc_pair;
  g_tc_pair = mode < 0 ? -1 : (mode > 0 ? 1 : 0);
  return was;
}

extern "C" int cretif_set_tc_bulk_add(int on) {
  const int was = g_tc_bulk_add;
  g_tc_bulk_add = on ? 1 : 0;
  return was;
}

extern "C" int cretif_set_tc_epilogue_warps(int n) {
  const int was = g_tc_epilogue_warps;
  g_tc_epilogue_warps = (n == 4 || n == 8) ? n : 0;
  return was;
}

#ifdef CRETIF_STAMPS
extern "C" void cretif_gemm_tc_stamps(unsigned long long* device_buffer) {
  g_tc_stamps = device_buffer;
}
#endif

extern "C" int cretif_gemm_tc(const void* A, const void* W, void* C, int c_dt, int M, int N, int K,
                              int lda, int ldw, int ldc, int accumulate, int bn,
                              unsigned int* fault, void* stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || K % 8 || lda % 8 || ldw % 8 || lda < K || ldw < K || ldc < N) return kBadArgument;
  if ((M + kTcBM - 1) / kTcBM > 65535) return kBadArgument;
  if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)C) & 15) return kMisaligned;
  if ((c_dt == kBF16 && ldc % 8) || (c_dt == kF32 && ldc % 4)) return kMisaligned;
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 0) {
    const long long mt = (M + kTcBM - 1) / kTcBM;
    bn = (mt * ((N + 255) / 256) >= 148) ? 256 : (mt * ((N + 127) / 128) >= 148 ? 128 : 64);
    // A width that is a multiple of 192 but not of 256 (576 = 3 x 192, 960 = 5 x 192) wastes
    // a quarter of the widest tile's columns; 192-wide tiles waste none and still pull a
    // sixth less through L2 per flop than 128-wide ones.
    if (N % 192 == 0 && N % 256 != 0 && mt * (N / 192) >= 148) bn = 192;
  }
  TcEpi ep = {};
  ep.C = C; ep.ldc = ldc; ep.accumulate = accumulate;
  // The float32 add of a large product: two CTAs a tile (see gemm_tc_pair_kernel), as wide as
  // the single-CTA tile would be.
  if (c_dt == kF32 && accumulate && g_tc_pair != 0 && g_tc_bulk_add && (bn == 256 || bn == 192) &&
      N % bn == 0 && ldc % 4 == 0 &&
      (g_tc_pair > 0 || ((long long)((M + 255) / 256) * (N / bn) >= 2 * 74 && pair_pays(N, K)))) {
    return bn == 256 ? launch_tc_pair<256, kTcStore>(A, W, ep, M, N, K, lda, ldw, fault, st)
                     : launch_tc_pair<192, kTcStore>(A, W, ep, M, N, K, lda, ldw, fault, st);
  }
#define CRETIF_TC(BN)                                                                         \
  (c_dt == kBF16 ? launch_tc<BN, kTcStore, __nv_bfloat16>(A, W, ep, M, N, K, lda, ldw, fault, \
                                                          st)                                 \
                 : launch_tc<BN, kTcStore, float>(A, W, ep, M, N, K, lda, ldw, fault, st))
  if (c_dt != kBF16 && c_dt != kF32) return kBadDType;
  if (c_dt == kBF16 && accumulate) return kBadArgument;
  switch (bn) {
    case 64: return CRETIF_TC(64);
    case 128: return CRETIF_TC(128);
    case 192: return CRETIF_TC(192);
    case 256: return CRETIF_TC(256);
    default: return kBadArgument;
  }
#undef CRETIF_TC
}

// act[M, I] = silu(A·Wg^T) * (A·Wu^T); Wgu holds gate and up rows interleaved in blocks of 64.
extern "C" int cretif_gemm_tc_silu(const void* A, const void* Wgu, void* act, int M, int I, int K,
                                   int lda, int ldw, unsigned int* fault, void* stream) {
  if (M <= 0 || I <= 0) return kOk;
  if (!tc_operands_ok(A, Wgu, M, K, lda, ldw) || I % 64) return kBadArgument;
  if (((uintptr_t)act) & 15) return kMisaligned;
  TcEpi ep = {};
  ep.act = (__nv_bfloat16*)act; ep.I = I;
  // wide tiles (two gate|up pairs, one CTA per SM) once there are four waves of them for the
  // whole chip; with fewer, the last wave's empty seats cost more than the wide tile saves
  const long long wide_tiles = (long long)((2 * I + 255) / 256) * ((M + kTcBM - 1) / kTcBM);
  if (g_tc_pair != 0 && g_tc_bulk_add && (2 * I) % 256 == 0 &&
      (g_tc_pair > 0 || (wide_tiles >= 4 * 148 && pair_pays(2 * I, K))))
    return launch_tc_pair<256, kTcSilu>(A, Wgu, ep, M, 2 * I, K, lda, ldw, fault, (cudaStream_t)stream);
  if (wide_tiles >= 4 * 148)
    return launch_tc<256, kTcSilu, __nv_bfloat16>(A, Wgu, ep, M, 2 * I, K, lda, ldw, fault,
                                                  (cudaStream_t)stream);
  return launch_tc<128, kTcSilu, __nv_bfloat16>(A, Wgu, ep, M, 2 * I, K, lda, ldw, fault,
                                                (cudaStream_t)stream);
}

// q|k|v = A·Wqkv^T with rotary on q and k; q to Q, k and v into the block cache.
extern "C" int cretif_gemm_tc_qkv_rope(const void* A, const void* Wqkv, void* Q, int ldq,
                                       const float* cos_t, const float* sin_t, int pairing, int nh,
                                       int nkv, int hd, const int* tok_pos, const int* tok_seq,
                                       const int* seq_slot, const int* table, int table_stride,
                                       void* kc, void* vc, int bt, int write_cache, int M, int K,
                                       int lda, int ldw, unsigned int* fault, void* stream) {
  if (M <= 0) return kOk;
  if (!tc_operands_ok(A, Wqkv, M, K, lda, ldw) || nh <= 0 || nkv <= 0 || (hd != 64 && hd != 128) ||
      bt <= 0 || ldq % 8 || ldq < nh * hd)
    return kBadArgument;
  if (((uintptr_t)Q | (uintptr_t)kc | (uintptr_t)vc) & 15) return kMisaligned;
  TcEpi ep = {};
  ep.Q = (__nv_bfloat16*)Q; ep.ldq = ldq; ep.cos_t = cos_t; ep.sin_t = sin_t; ep.pairing = pairing;
  ep.nh = nh; ep.nkv = nkv; ep.hd = hd; ep.tok_pos = tok_pos; ep.tok_seq = tok_seq;
  ep.seq_slot = seq_slot; ep.table = table; ep.table_stride = table_stride;
  ep.kc = (__nv_bfloat16*)kc; ep.vc = (__nv_bfloat16*)vc; ep.bt = bt; ep.write_cache = write_cache;
  const int N = (nh + 2 * nkv) * hd;
  cudaStream_t st = (cudaStream_t)stream;
  // A tile is a whole number of heads.  Small products want many narrow tiles; large ones
  // (two waves of 128-wide tiles and more) do more arithmetic per byte with wide ones.
  const long long m_tiles = (M + kTcBM - 1) / kTcBM;
  const long long wide_tiles = (long long)((N + 127) / 128) * m_tiles;
  if (hd == 64 && wide_tiles < 2 * 148)
    return launch_tc<64, kTcRope, __nv_bfloat16>(A, Wqkv, ep, M, N, K, lda, ldw, fault, st);
  // three heads of 64 per tile where that divides the matrix and 128 does not
  if (hd == 64 && N % 192 == 0 && N % 128 != 0 && m_tiles * (N / 192) >= 2 * 148)
    return launch_tc<192, kTcRope, __nv_bfloat16>(A, Wqkv, ep, M, N, K, lda, ldw, fault, st);
  return launch_tc<128, kTcRope, __nv_bfloat16>(A, Wqkv, ep, M, N, K, lda, ldw, fault, st);
}
