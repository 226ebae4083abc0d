// Host side of the fused decode projections; the kernels are in decode_fused.cuh.
#include "decode_stream.cuh"

namespace cretif {

// Launch the fused kernels with programmatic stream serialization (their weight fetch then
// overlaps the tail of the kernel before them).
static int g_dependent_launch = 1;
int dependent_launch_enabled() { return g_dependent_launch; }

static int g_variant_counts[kVarCount];
void count_variant(int v) {
  if (v >= 0 && v < kVarCount) ++g_variant_counts[v];
}

// Largest cluster that shares a norm prologue (1: none; at most kFuClusterMax).
static int g_fused_cluster = kFuClusterMax;

template <int NT, int PRO, int EPI>
static int launch_fused(const FusedParams& p, int tiles, cudaStream_t st, int groups = 1,
                        int group_rows = 0) {
  if (groups == 1) group_rows = p.M;
  const size_t smem = fused_smem(NT, PRO, group_rows, p.K);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    if (smem > 200 * 1024) return kBadArgument;
    cudaError_t e = cudaFuncSetAttribute(skinny_fused_kernel<NT, PRO, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  static int max_ctas = 0;
  if (!max_ctas) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    max_ctas = 2 * (sms > 0 ? sms : 148);      // two CTAs are resident per SM
  }
  const int per_group = max_ctas / groups > 0 ? max_ctas / groups : 1;
  // every CTA the same number of tiles, to within one
  const int waves = (tiles + per_group - 1) / per_group;
  dim3 grid((tiles + waves - 1) / waves, groups);
  // More than eight rows with the norm prologue: the CTAs of a cluster share the rows'
  // normalisation (every CTA has a tile, so the grid is cut to whole clusters).  Four CTAs
  // give 32 rows one warp each; on a grid that fills the chip, clusters of four find their
  // places more slowly than they save (64 rows: 1.38 against 1.33 ms a step with two).
  int cluster = 1;
  if (NT > 1 && PRO == kProNorm && g_fused_cluster > 1) {
    cluster = group_rows > 16 && 4 * (int)grid.x * groups <= 3 * max_ctas ? 4 : 2;
    if (cluster > g_fused_cluster) cluster = g_fused_cluster;
    if ((int)grid.x < cluster) cluster = 1;
    grid.x -= grid.x % cluster;
  }
  count_variant(groups > 1 ? kVarFusedRowGroups : kVarFusedRegisters);
  if (cluster > 1) count_variant(cluster == 4 ? kVarFusedCluster4 : kVarFusedCluster2);
  if (g_dependent_launch || cluster > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kFuWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (g_dependent_launch) {
      attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
      ++n_attr;
    }
    if (cluster > 1) {
      attr[n_attr].id = cudaLaunchAttributeClusterDimension;
      attr[n_attr].val.clusterDim.x = cluster;
      attr[n_attr].val.clusterDim.y = 1;
      attr[n_attr].val.clusterDim.z = 1;
      ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_fused_kernel<NT, PRO, EPI>, p, tiles,
                                       group_rows);
    return e == cudaSuccess ? launch_status() : (int)e;
  }
  skinny_fused_kernel<NT, PRO, EPI><<<grid, kFuWarps * 32, smem, st>>>(p, tiles, group_rows);
  return launch_status();
}

// The register variant for any number of rows up to kFuMaxRows.
template <int PRO, int EPI>
static int dispatch_registers(const FusedParams& p, int tiles, cudaStream_t st) {
  if (p.M <= 8) return launch_fused<1, PRO, EPI>(p, tiles, st);
  if (p.M <= 16) return launch_fused<2, PRO, EPI>(p, tiles, st);
  if (p.M <= kFuMaxGroupRows) return launch_fused<4, PRO, EPI>(p, tiles, st);
  // More tokens: even groups of up to 32 rows, a multiple of 8 each.  (One group of 64 rows
  // — eight token tiles per warp and k-chunk, the weights read once — was measured at
  // SmolLM2-135M sizes and lost: q|k|v 5.6 -> 8.1 us, gate|up 8.0 -> 9.7 us at 64 tokens; a
  // CTA's share of the arithmetic, not the second read of the weights from L2, is what a
  // group costs.)
  const int groups = (p.M + kFuMaxGroupRows - 1) / kFuMaxGroupRows;
  const int group_rows = (((p.M + groups - 1) / groups) + 7) & ~7;
  return launch_fused<4, PRO, EPI>(p, tiles, st, groups, group_rows);
}

// Matrices at least this wide, or this large, stream through shared memory
// (decode_stream.cuh); narrow small ones are latency and do better without the copy unit.
static int g_stream_min_k = 768;
static long long g_stream_min_bytes = 16LL << 20;
// ... and up to this many tokens (beyond 16 as groups of 16 rows that each stream the matrix)
static const int g_stream_max_rows = 64;
// Depth of the streaming ring; 0: chosen per launch.
static const int g_stream_stages = 0;
// Stages of weights asked for before the kernel waits for the kernel before it.
static const int g_stream_early = 1;

template <int NT, int PRO, int EPI>
static int launch_stream(const FusedParams& whole, int tiles, cudaStream_t st) {
  const int groups = (whole.M + 8 * NT - 1) / (8 * NT);
  FusedParams p = whole;             // sizes of one group of rows
  if (groups > 1) p.M = 8 * NT;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  // Depth of the ring.  With many tiles two CTAs share an SM if both fit (113 KB each), as
  // deep as that allows; else, or with few tiles (a narrow output and a long K), one CTA per
  // SM holds as many steps in flight as shared memory allows.
  const int steps = (p.K + kStK - 1) / kStK;
  constexpr size_t kHalfSm = 113 * 1024, kWholeSm = 200 * 1024;
  int stages = kStMaxStages, per_sm = 1;
  if (tiles > sm_count && stream_smem(NT, PRO, p.M, p.K, 3) <= kHalfSm) {
    per_sm = 2;
    while (stream_smem(NT, PRO, p.M, p.K, stages) > kHalfSm) --stages;
  } else if (tiles <= sm_count && steps < stages) {
    stages = steps < 3 ? 3 : steps;
  }
  if (g_stream_stages) stages = g_stream_stages;
  while (stages > 2 && stream_smem(NT, PRO, p.M, p.K, stages) > kWholeSm) --stages;
  const size_t smem = stream_smem(NT, PRO, p.M, p.K, stages);
  if (smem > 200 * 1024) return dispatch_registers<PRO, EPI>(whole, tiles, st);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(skinny_stream_kernel<NT, PRO, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  const int max_ctas = per_sm * sm_count / groups > 0 ? per_sm * sm_count / groups : 1;
  // every CTA the same number of tiles (to within one): 384 tiles on 296 seats run as
  // 192 CTAs of two tiles, not as 296 of which 88 work twice as long
  const int waves = (tiles + max_ctas - 1) / max_ctas;
  const int grid = (tiles + waves - 1) / waves;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, groups);
  cfg.blockDim = dim3(kStThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_dependent_launch;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int w_rows = EPI == kEpiPlain ? p.N : EPI == kEpiSilu ? 2 * p.I : (p.nh + 2 * p.nkv) * p.hd;
  CUtensorMap map_w, map_x;
  if (make_box_map_bf16(&map_w, p.W, w_rows, p.K, p.ldw, 8, kStBoxK, false))
    return dispatch_registers<PRO, EPI>(whole, tiles, st);
  if (PRO == kProPlain) {
    if (make_box_map_bf16(&map_x, whole.X, whole.M, p.K, p.ldx, 8 * NT, kStBoxK, false))
      return dispatch_registers<PRO, EPI>(whole, tiles, st);
  } else {
    map_x = map_w;
  }
  count_variant(groups > 1 ? kVarStreamRowGroups : kVarStream);
  cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_stream_kernel<NT, PRO, EPI>, whole, map_w, map_x,
                                     tiles, stages, g_stream_early);
  return e == cudaSuccess ? launch_status() : (int)e;
}

template <int PRO, int EPI>
static int dispatch_nt(const FusedParams& p, int tiles, cudaStream_t st) {
  const long long w_bytes = 2LL * tiles * kFuRows * p.K;
  if ((p.K >= g_stream_min_k || w_bytes >= g_stream_min_bytes) && p.M <= g_stream_max_rows) {
    if (p.M <= 8) return launch_stream<1, PRO, EPI>(p, tiles, st);
    return launch_stream<2, PRO, EPI>(p, tiles, st);      // groups of 16 rows beyond 16
  }
  return dispatch_registers<PRO, EPI>(p, tiles, st);
}

static bool common_ok(const FusedParams& p) {
  return p.M > 0 && p.M <= kFuMaxRows && p.K > 0 && p.K % 8 == 0 && p.ldw % 8 == 0 && p.ldw >= p.K &&
         (((uintptr_t)p.W) & 15) == 0;
}

}  // namespace cretif

using namespace cretif;

// out (+)= norm(h[rows]) · W^T  or  x · W^T, plain epilogue.
extern "C" int cretif_fused_linear(const void* X, int ldx, const float* H, const float* norm_w,
                                   const int* rows, float eps, const void* W, int ldw, void* C,
                                   int c_dt, int ldc, int accumulate, int M, int N, int K,
                                   unsigned int* fault, void* stream) {
  if (M <= 0 || N <= 0) return kOk;
  FusedParams p = {};
  p.W = (const __nv_bfloat16*)W; p.M = M; p.N = N; p.K = K; p.ldw = ldw;
  p.X = (const __nv_bfloat16*)X; p.ldx = ldx; p.H = H; p.norm_w = norm_w; p.rows = rows;
  p.eps = eps; p.C = C; p.ldc = ldc; p.c_dt = c_dt; p.accumulate = accumulate; p.fault = fault;
  if (!common_ok(p) || !derive_fields(p) || ldc < N || (c_dt != kF32 && c_dt != kBF16) ||
      (c_dt == kBF16 && accumulate))
    return kBadArgument;
  const int tiles = (N + kFuRows - 1) / kFuRows;
  cudaStream_t st = (cudaStream_t)stream;
  if (H) return dispatch_nt<kProNorm, kEpiPlain>(p, tiles, st);
  if (!X || ldx % 8 || ldx < K || (((uintptr_t)X) & 15)) return kBadArgument;
  return dispatch_nt<kProPlain, kEpiPlain>(p, tiles, st);
}

// q, k, v = norm(h) · Wqkv^T; rotary on q and k; k, v into the cache; q to Q.
extern "C" int cretif_fused_qkv_rope(const float* H, const float* norm_w, float eps,
                                     const void* Wqkv, int ldw, void* Q, int ldq,
                                     const float* cos_t, const float* sin_t, int pairing, int nh,
                                     int nkv, int hd, const int* tok_pos, const int* tok_seq,
                                     const int* seq_slot, const int* table, int table_stride,
                                     void* kc, void* vc, int bt, int write_cache, int M, int K,
                                     unsigned int* fault, void* stream) {
  if (M <= 0) return kOk;
  FusedParams p = {};
  p.W = (const __nv_bfloat16*)Wqkv; p.M = M; p.N = (nh + 2 * nkv) * hd; p.K = K; p.ldw = ldw;
  p.H = H; p.norm_w = norm_w; p.eps = eps;
  p.Q = (__nv_bfloat16*)Q; p.ldq = ldq; p.cos_t = cos_t; p.sin_t = sin_t; p.pairing = pairing;
  p.nh = nh; p.nkv = nkv; p.hd = hd; p.tok_pos = tok_pos; p.tok_seq = tok_seq;
  p.seq_slot = seq_slot; p.table = table; p.table_stride = table_stride;
  p.kc = (__nv_bfloat16*)kc; p.vc = (__nv_bfloat16*)vc; p.bt = bt; p.write_cache = write_cache;
  p.fault = fault;
  if (!common_ok(p) || !derive_fields(p) || !H || nh <= 0 || nkv <= 0 || hd % 16 || hd <= 0 ||
      bt <= 0 || ldq < nh * hd)
    return kBadArgument;
  return dispatch_nt<kProNorm, kEpiRope>(p, p.N / kFuRows, (cudaStream_t)stream);
}

// act = silu(norm(h) · Wg^T) * (norm(h) · Wu^T), Wgu = [Wg; Wu] stacked.
extern "C" int cretif_fused_gate_up_silu(const float* H, const float* norm_w, float eps,
                                         const void* Wgu, int ldw, void* act, int I, int gu_block,
                                         int M, int K, unsigned int* fault, void* stream) {
  if (M <= 0) return kOk;
  FusedParams p = {};
  p.W = (const __nv_bfloat16*)Wgu; p.M = M; p.N = 2 * I; p.K = K; p.ldw = ldw;
  p.H = H; p.norm_w = norm_w; p.eps = eps; p.act = (__nv_bfloat16*)act; p.I = I; p.gu_block = gu_block; p.fault = fault;
  if (!common_ok(p) || !derive_fields(p) || !H || I <= 0 || gu_block < 0 ||
      (gu_block && (I % gu_block || gu_block % 8)))
    return kBadArgument;
  return dispatch_nt<kProNorm, kEpiSilu>(p, (I + 7) / 8, (cudaStream_t)stream);
}

extern "C" int cretif_variant_count(int v) {
  return v >= 0 && v < kVarCount ? g_variant_counts[v] : -1;
}

extern "C" int cretif_set_stream_min_k(int k, long long min_bytes) {
  const int was = g_stream_min_k;
  g_stream_min_k = k;
  if (min_bytes >= 0) g_stream_min_bytes = min_bytes;
  return was;
}

extern "C" long long cretif_stream_min_bytes(void) { return g_stream_min_bytes; }

extern "C" int cretif_set_fused_cluster(int n) {
  const int was = g_fused_cluster;
  if (n >= 1) g_fused_cluster = n > kFuClusterMax ? kFuClusterMax : n;
  return was;
}

extern "C" int cretif_set_dependent_launch(int on) {
  const int was = g_dependent_launch;
  g_dependent_launch = on ? 1 : 0;
  return was;
}

extern "C" int cretif_fused_smem_ok(int M, int K, int norm_prologue) {
  if (M > kFuMaxRows) return 0;
  if (M > kFuMaxGroupRows) M = kFuMaxGroupRows;
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  return fused_smem(nt, norm_prologue ? kProNorm : kProPlain, M, K) <= 200 * 1024 ? 1 : 0;
}
