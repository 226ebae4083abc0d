// The fused few-token product for wide matrices: weights stream through shared memory.
//
// decode_fused.cuh moves weights global -> registers -> tensor cores, which keeps only a few
// loads per thread in flight; that is enough for the small matrices of a 135M model, whose
// launches are latency anyway, but it reaches only 1.3-2 TB/s on 2048- to 8192-wide matrices.
// Here a producer thread asks the TMA unit, for every 512-column step, for the tile's two
// groups of eight weight rows and, for the plain prologue, for the tokens' rows of x, as
// boxes of 256 columns (4 KB for a group of rows), into a ring of shared-memory stages;
// eight consumer warps take 16-byte fragments from there.  The boxes are large on purpose:
// an SM accepts a copy request only every ~64 cycles, so that a copy of one 1 KB row at a
// time held a CTA to 14 GB/s.  Rows and columns beyond the matrix arrive as zeros.
// Prologues (norm from the residual stream) and epilogues (rotary + cache, SiLU·mul,
// store / add) are the ones of decode_fused.cuh, as is the k-permutation of the m16n8k16
// operands.
#pragma once

#include <cuda.h>

#include "decode_fused.cuh"
#include "tc_common.cuh"

namespace cretif {

constexpr int kStThreads = (kFuWarps + 1) * 32;   // eight consumer warps and the producer
constexpr int kStK = 512;                          // columns per stage
constexpr int kStBoxK = 256;                       // columns per copy (the most a box may have)
constexpr int kStBoxes = kStK / kStBoxK;
constexpr int kStRowB = kStBoxK * 2;               // bytes of a box row
constexpr int kStGroup = 8 * kStRowB;              // bytes of a box of eight rows
constexpr int kStW = 2 * kStBoxes * kStGroup;      // weight bytes of a stage
constexpr int kStMaxStages = 8;                    // the ring's depth is chosen per launch (3..8)

__host__ __device__ inline size_t stream_smem(int nt, int pro, int M, int K, int stages) {
  size_t bytes = sizeof(float) * kFuWarps * kFuRows * (8 * nt + 1) + 16;        // reduction
  bytes = (bytes + 127) & ~size_t(127);
  bytes += (size_t)stages * kStW;                                                 // W stages
  if (pro == kProNorm) bytes += (size_t)M * (((K * 2 + 127) / 128) * 128 + 64) + (size_t)K * 4;
  else bytes += (size_t)stages * kStBoxes * nt * kStGroup;                        // x stages
  return bytes + (2 * kStMaxStages + 1) * 8 + 256;
}

// [rows, cols] bf16 with row stride ld, boxes of box_rows x box_cols; swizzle: 128-byte
// (box_cols must then be 64).  Recent maps are kept (gemm_tc.cu).
int make_box_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows,
                      int box_cols, bool swizzle);

// The two groups of eight consecutive weight rows that tile `tile` is made of.
template <int EPI>
__device__ __forceinline__ void tile_groups(const FusedParams& p, int tile, int& row_a, int& row_b,
                                            bool& paired) {
  paired = false;
  row_a = tile_row<EPI>(p, tile, 0);
  if (EPI == kEpiRope && p.pairing && fast_div(p.tph_div, tile) < p.nh + p.nkv) {
    row_b = row_a + 8;       // interleaved pairs: tile row r is weight row 2 (r & 7) + (r >> 3)
    paired = true;
  } else {
    row_b = tile_row<EPI>(p, tile, 8);
  }
}

template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(kStThreads, 2)
skinny_stream_kernel(const FusedParams whole, const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_x, int n_tiles, int n_stages,
                     int n_early) {
  // More than 8 NT tokens run as groups of 8 NT rows along gridDim.y (every group streams
  // the whole matrix; the groups of a tile run side by side, so the second read is L2's).
  const int m_first = blockIdx.y * 8 * NT;
  const FusedParams p = rows_of(whole, m_first, min(8 * NT, whole.M - m_first));
  extern __shared__ __align__(128) unsigned char stsmem_raw[];
  unsigned char* stsmem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(stsmem_raw) + 127) & ~uintptr_t(127));
  float(*red)[kFuRows][8 * NT + 1] = reinterpret_cast<float(*)[kFuRows][8 * NT + 1]>(stsmem);
  size_t off = (sizeof(float) * kFuWarps * kFuRows * (8 * NT + 1) + 16 + 127) & ~size_t(127);
  unsigned char* wst = stsmem + off;                      // [stages][group][box][8][512 B]
  off += (size_t)n_stages * kStW;
  const int xs_stride = ((p.K * 2 + 127) / 128) * 128 + 64;
  constexpr int kXStage = kStBoxes * NT * kStGroup;       // plain: [stages][box][8 NT][512 B]
  unsigned char* xs = stsmem + off;                       // norm: [M][xs_stride]
  off += PRO == kProNorm ? (size_t)p.M * xs_stride : (size_t)n_stages * kXStage;
  float4* nws = reinterpret_cast<float4*>(stsmem + off);  // norm: the norm's weight, float[K]
  if (PRO == kProNorm) off += (size_t)p.K * 4;
  uint64_t* full = reinterpret_cast<uint64_t*>(stsmem + ((off + 7) & ~size_t(7)));
  uint64_t* empty = full + kStMaxStages;
  volatile int* abort = reinterpret_cast<volatile int*>(empty + kStMaxStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_steps = (p.K + kStK - 1) / kStK;
  const int my_tiles = blockIdx.x < n_tiles ? (n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const int total = my_tiles * n_steps;                   // stage fills of this CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], kFuWarps); }
    *abort = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == kFuWarps) {
    // ---------------- producer: one thread issues the copies
    // An SM serves its requests in order, so what is asked for after the wait (x, or the
    // residual rows of the norm prologue) arrives behind every weight copy issued before it:
    // only n_early stages of weights go ahead, the rest follow the step's own inputs.
    // Where a fill goes is kept in a cursor that only ever steps forward (tile, step, stage,
    // turn of the ring): nothing on this thread's path divides.
    struct Cursor {
      int tile, step, s, turn, row_a, row_b;
    };
    auto rows_of_tile = [&](Cursor& c) {
      bool paired;
      if (c.tile < n_tiles) tile_groups<EPI>(p, c.tile, c.row_a, c.row_b, paired);
    };
    auto advance = [&](Cursor& c) {
      if (++c.s == n_stages) { c.s = 0; ++c.turn; }
      if (++c.step == n_steps) {
        c.step = 0;
        c.tile += gridDim.x;
        rows_of_tile(c);
      }
    };
    auto fill = [&](const Cursor& c, bool weights, bool xrows) {
      const int s = c.s, k0 = c.step * kStK;
      const int boxes = min(kStBoxes, (p.K - k0 + kStBoxK - 1) / kStBoxK);   // by a constant
      if (weights) {
        // a box is counted whole, whatever part of it lies beyond the matrix
        const int per_box = 2 * kStGroup + (PRO == kProPlain ? NT * kStGroup : 0);
        tc::mbar_expect_tx(&full[s], (uint32_t)(boxes * per_box));
        unsigned char* ws = wst + (size_t)s * kStW;
        for (int b = 0; b < boxes; ++b) {
          tc::tma_load_2d(ws + (size_t)b * kStGroup, &map_w, k0 + b * kStBoxK, c.row_a, &full[s]);
          tc::tma_load_2d(ws + (size_t)(kStBoxes + b) * kStGroup, &map_w, k0 + b * kStBoxK,
                          c.row_b, &full[s]);
        }
      }
      if (PRO == kProPlain && xrows) {
        unsigned char* xst = xs + (size_t)s * kXStage;
        for (int b = 0; b < boxes; ++b)
          tc::tma_load_2d(xst + (size_t)b * NT * kStGroup, &map_x, k0 + b * kStBoxK, m_first,
                          &full[s]);
      }
    };
    const int ahead = min(total, n_stages), early = min(ahead, n_early);
    Cursor cur = {(int)blockIdx.x, 0, 0, 0, 0, 0};
    rows_of_tile(cur);
    Cursor first = cur;
    if (lane == 0) {
      tc::tma_prefetch_descriptor(&map_w);
      if (PRO == kProPlain) tc::tma_prefetch_descriptor(&map_x);
      for (int it = 0; it < early; ++it, advance(cur)) fill(cur, true, false);   // weights need nobody
    }
    __syncwarp();
    asm volatile("griddepcontrol.wait;" ::: "memory");               // x comes from the kernel before
    if (PRO == kProNorm) asm volatile("bar.sync 2, %0;" ::"n"(kStThreads) : "memory");
    if (lane == 0) {
      cur = first;
      for (int it = 0; it < ahead; ++it, advance(cur)) fill(cur, it >= early, true);
      for (int it = ahead; it < total; ++it, advance(cur)) {
        if (!tc::mbar_wait(&empty[cur.s], (uint32_t)((cur.turn - 1) & 1), abort)) break;
        fill(cur, true, true);
      }
    }
  } else {
    // ---------------- consumer warps
    const int r = lane >> 2, c = lane & 3;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // the first tile's rotary operands (positions, block table, angles) do not wait either
    EpiAhead<NT> ahead;
    bool have_ahead = false;
    if (EPI == kEpiRope && (int)blockIdx.x < n_tiles) {
      epi_prefetch<NT, EPI>(p, blockIdx.x, ahead);
      have_ahead = true;
    }
    if (PRO == kProNorm) {
      // The norm's weight depends on nothing: it is in shared memory before the wait ends.
      // After it a warp asks for its token's whole residual row at once and tells the
      // producer, whose remaining weight copies then queue behind these loads.
      const int n4 = p.K >> 2;
      const float4* w4 = reinterpret_cast<const float4*>(p.norm_w);
      for (int i = threadIdx.x; i < n4; i += kFuWarps * 32) nws[i] = __ldg(w4 + i);
      asm volatile("bar.sync 1, 256;" ::: "memory");
      asm volatile("griddepcontrol.wait;" ::: "memory");
      constexpr int REGS = 16;
      bool told = false;
      for (int m = warp; m < p.M || !told; m += kFuWarps) {
        const bool row = m < p.M;
        const float4* h4 = reinterpret_cast<const float4*>(
            p.H + (size_t)(row ? (p.rows ? p.rows[m] : m) : 0) * p.K);
        __nv_bfloat16* xr = reinterpret_cast<__nv_bfloat16*>(xs + (size_t)m * xs_stride);
        float4 v[REGS];
        float ss = 0.f;
        const bool fits = n4 <= 32 * REGS;
        if (row && fits) {
#pragma unroll
          for (int u = 0; u < REGS; ++u) {
            const int i = u * 32 + lane;
            v[u] = i < n4 ? __ldcg(h4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        if (!told) {
          asm volatile("bar.arrive 2, %0;" ::"n"(kStThreads) : "memory");
          told = true;
        }
        if (!row) break;
        if (fits) {
#pragma unroll
          for (int u = 0; u < REGS; ++u)
            ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
        } else {
#pragma unroll 8
          for (int i = lane; i < n4; i += 32) {
            const float4 t = __ldcg(h4 + i);
            ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
          }
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)p.K + p.eps);
        auto put = [&](int i, const float4& t) {
          const float4 w = nws[i];
          __nv_bfloat162 lo = __floats2bfloat162_rn(t.x * w.x * inv, t.y * w.y * inv);
          __nv_bfloat162 hi = __floats2bfloat162_rn(t.z * w.z * inv, t.w * w.w * inv);
          uint2 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&lo);
          pk.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(xr + 4 * i) = pk;
        };
        if (fits) {
#pragma unroll
          for (int u = 0; u < REGS; ++u) {
            const int i = u * 32 + lane;
            if (i < n4) put(i, v[u]);
          }
        } else {
#pragma unroll 4
          for (int i = lane; i < n4; i += 32) put(i, __ldcg(h4 + i));
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    } else {
      asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    int s = 0, turn = 0;                         // the ring's stage and how often it has turned
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      if (!have_ahead) epi_prefetch<NT, EPI>(p, tile, ahead);
      have_ahead = false;
      // where this lane's two weight rows (tile rows r and r + 8) lie within a stage
      int off_a = r * kStRowB, off_b = kStBoxes * kStGroup + r * kStRowB;
      if (EPI == kEpiRope && p.pairing && fast_div(p.tph_div, tile) < p.nh + p.nkv) {
        const int wa = 2 * r, wb = 2 * r + 1;
        off_a = (wa >> 3) * kStBoxes * kStGroup + (wa & 7) * kStRowB;
        off_b = (wb >> 3) * kStBoxes * kStGroup + (wb & 7) * kStRowB;
      }
      float acc[NT][4];
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
      for (int step = 0; step < n_steps; ++step) {
        const int k0 = step * kStK;
        tc::mbar_wait(&full[s], (uint32_t)(turn & 1), abort);   // bounded; see abort
        const unsigned char* ws = wst + (size_t)s * kStW;
#pragma unroll
        for (int j = 0; j < kStK / (32 * kFuWarps); ++j) {   // chunks of 32 columns, two per warp
          const int kl = (warp + j * kFuWarps) * 32 + c * 8, k = k0 + kl;
          const int box = kl / kStBoxK, cb = (kl % kStBoxK) * 2;
          const bool in = k < p.K;
          const uint4 ua = in ? *reinterpret_cast<const uint4*>(ws + off_a + box * kStGroup + cb) : zero;
          const uint4 ub = in ? *reinterpret_cast<const uint4*>(ws + off_b + box * kStGroup + cb) : zero;
          const uint32_t a1[4] = {ua.x, ub.x, ua.y, ub.y};
          const uint32_t a2[4] = {ua.z, ub.z, ua.w, ub.w};
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const int m = t * 8 + r;
            uint4 ux = zero;
            if (in) {
              if (PRO == kProNorm) {
                if (m < p.M) ux = *reinterpret_cast<const uint4*>(xs + (size_t)m * xs_stride + (size_t)k * 2);
              } else {                 // rows beyond M arrived as zeros
                ux = *reinterpret_cast<const uint4*>(xs + (size_t)s * kXStage +
                                                     (size_t)box * NT * kStGroup + m * kStRowB + cb);
              }
            }
            mma_16816(acc[t], a1, ux.x, ux.y);
            mma_16816(acc[t], a2, ux.z, ux.w);
          }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&empty[s]);
        if (++s == n_stages) { s = 0; ++turn; }
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        red[warp][r][t * 8 + 2 * c] = acc[t][0];
        red[warp][r][t * 8 + 2 * c + 1] = acc[t][1];
        red[warp][r + 8][t * 8 + 2 * c] = acc[t][2];
        red[warp][r + 8][t * 8 + 2 * c + 1] = acc[t][3];
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      finish_tile<NT, EPI>(p, tile, red, ahead);
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
  }
  __syncthreads();
  if (*abort && threadIdx.x == 0 && p.fault) atomicOr(p.fault, kFaultWaitExpired);
}

}  // namespace cretif
