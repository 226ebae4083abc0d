// Host side of the tensor-core decode attention and the entry point that allocates nothing;
// the kernel is in attn_decode_mma.cuh.
#include <mutex>

#include "attn_decode_mma.cuh"
#include "attn_decode_noalloc.h"

namespace cretif {

// Tuning aid: a device buffer of 10 x 16 timestamps the next launches fill (see the kernel).
static unsigned long long* g_dm_stamps = nullptr;
// Depth of the K/V ring (3..6); 0 chooses per launch.
static const int g_dm_stages = 0;

template <int HD16>
static size_t dm_smem_bytes(bool cluster, int n_stages) {
  return dm_smem_core<HD16>(cluster, n_stages) + 1024;
}

template <int HD16, bool CLUSTER>
static int launch_dm(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int ldq,
                     const int* table, int table_stride, const int* tok_pos, const int* tok_seq,
                     const int* seq_slot, int nh, int nkv, float scale_log2, int window,
                     float* part_o, float* part_ml, void* out, int ldo, int* counters,
                     unsigned int* fault, dim3 grid, cudaStream_t st) {
  // Few CTAs (at most two per SM) walk many tiles each: a deeper ring keeps more of the cache
  // in flight per CTA, as long as two CTAs still fit an SM.
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  int n_stages = g_dm_stages ? g_dm_stages : kDmStages;
  if (!g_dm_stages && (long long)grid.x * grid.y * grid.z <= 2LL * sm_count) {
    n_stages = kDmMaxStages;
    while (n_stages > kDmStages && dm_smem_bytes<HD16>(CLUSTER, n_stages) > 112 * 1024) --n_stages;
  }
  const size_t smem = dm_smem_bytes<HD16>(CLUSTER, n_stages);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<HD16, CLUSTER>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  // Launched as a programmatic dependent of the kernel before it: set-up, the block table and
  // the first cache tiles run under that kernel's tail.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kDmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (CLUSTER) {                 // the ranges of one (sequence, kv head) are one cluster
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = grid.x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  count_variant(CLUSTER ? kVarDecodeCluster : kVarDecodeSplit);
  cudaError_t e = cudaLaunchKernelEx(
      &cfg, attn_decode_mma_kernel<HD16, CLUSTER>, mk, mv, (const __nv_bfloat16*)q, ldq, table,
      table_stride, tok_pos, tok_seq, seq_slot, nh, nkv, scale_log2, window, part_o, part_ml,
      (__nv_bfloat16*)out, ldo, counters, fault, g_dm_stamps, n_stages);
  return e == cudaSuccess ? launch_status() : (int)e;
}

}  // namespace cretif

using namespace cretif;

#ifdef CRETIF_STAMPS
extern "C" void cretif_attn_decode_stamps(unsigned long long* device_buffer) {
  g_dm_stamps = device_buffer;
}
#endif

extern "C" int cretif_attn_decode_mma(const void* q, int ldq, void* out, int ldo, const void* kc,
                                      const void* vc, long long n_blocks, const int* table,
                                      int table_stride, const int* tok_pos, const int* tok_seq,
                                      const int* seq_slot, int nh, int nkv, int hd, float scale,
                                      int window, int bt, int B, int n_splits, float* part_o,
                                      float* part_ml, int* counters, unsigned int* fault,
                                      void* stream) {
  if (B <= 0) return kOk;
  if (nh <= 0 || nkv <= 0 || nh % nkv || nh / nkv > 8 || hd % 16 || hd < 16 || hd > 128 ||
      bt != kDmTile || n_splits <= 0 || n_splits > kDmTile || nkv > 65535 || B > 65535 ||
      window < 0 || ldq % 2)
    return kBadArgument;
  if (((uintptr_t)kc | (uintptr_t)vc) & 15 || ((uintptr_t)q & 3)) return kMisaligned;
  const long long cache_rows = n_blocks * nkv * kDmTile;
  if (cache_rows > 0x7fffffffLL) return kBadArgument;
  CUtensorMap mk, mv;
  if (make_tile_map_bf16(&mk, kc, (int)cache_rows, hd, hd, kDmTile)) return kBadArgument;
  if (make_tile_map_bf16(&mv, vc, (int)cache_rows, hd, hd, kDmTile)) return kBadArgument;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_splits, nkv, B);
  cudaStream_t st = (cudaStream_t)stream;
  // Without scratch the ranges are merged inside a cluster (at most eight of them).
  const bool cluster = part_o == nullptr;
  if (cluster ? n_splits > kDmClusterMax : (!part_ml || !counters)) return kBadArgument;
#define CRETIF_DM(N)                                                                          \
  case N:                                                                                     \
    return cluster                                                                            \
               ? launch_dm<N, true>(mk, mv, q, ldq, table, table_stride, tok_pos, tok_seq,    \
                                    seq_slot, nh, nkv, scale_log2, window, part_o, part_ml,   \
                                    out, ldo, counters, fault, grid, st)                      \
               : launch_dm<N, false>(mk, mv, q, ldq, table, table_stride, tok_pos, tok_seq,   \
                                     seq_slot, nh, nkv, scale_log2, window, part_o, part_ml,  \
                                     out, ldo, counters, fault, grid, st)
  switch (hd / 16) {
    CRETIF_DM(1); CRETIF_DM(2); CRETIF_DM(3); CRETIF_DM(4);
    CRETIF_DM(5); CRETIF_DM(6); CRETIF_DM(7); CRETIF_DM(8);
  }
#undef CRETIF_DM
  return kBadArgument;
}

// ---------------------------------------------------------------- no-allocation entry point
// The scratch of the split-range kernel in a fixed array of the library (see
// attn_decode_noalloc.h).  In host code the array's name is only a stand-in for the symbol,
// not a device address: the address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CRETIF_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kNoallocMaxDevices = 64;
constexpr size_t kNoallocCounterBytes = (size_t)CRETIF_NOALLOC_MAX_COUNTERS * sizeof(int);
unsigned char* g_noalloc_ptr[kNoallocMaxDevices];     // device address of the array, per device
std::mutex g_noalloc_mutex;
}  // namespace

extern "C" unsigned int cretif_attn_decode_noalloc_capacity(void) {
  return CRETIF_NOALLOC_SCRATCH_BYTES;
}

extern "C" int cretif_attn_decode_noalloc(const void* q, int ldq, void* out, int ldo,
                                          const void* kc, const void* vc, long long n_blocks,
                                          const int* table, int table_stride, const int* tok_pos,
                                          const int* tok_seq, const int* seq_slot, int nh, int nkv,
                                          int hd, float scale, int window, int bt, int B,
                                          int n_splits, unsigned int* fault, void* stream) {
  if (B <= 0) return kOk;
  if (nh <= 0 || nkv <= 0 || hd <= 0 || n_splits <= 0) return kBadArgument;
  // sizes beyond the fixed array are refused before anything is launched
  const unsigned long long n_counters = (unsigned long long)B * nkv;
  const unsigned long long floats_o = (unsigned long long)B * nh * n_splits * hd;
  const unsigned long long floats_ml = (unsigned long long)B * nh * n_splits * 2;
  if (n_counters > CRETIF_NOALLOC_MAX_COUNTERS) return kBadArgument;
  if ((floats_o + floats_ml) * sizeof(float) > CRETIF_NOALLOC_SCRATCH_BYTES - kNoallocCounterBytes)
    return kBadArgument;

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoallocMaxDevices) return kBadArgument;
  unsigned char* base;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {                 // set-up, once per device, that device current
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess) return (int)e;
      g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    base = g_noalloc_ptr[dev];
  }
  int* counters = reinterpret_cast<int*>(base);
  float* part_o = reinterpret_cast<float*>(base + kNoallocCounterBytes);
  float* part_ml = part_o + floats_o;
  // the counters must start at zero whatever an earlier (perhaps faulted) call left there
  e = cudaMemsetAsync(counters, 0, n_counters * sizeof(int), (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return cretif_attn_decode_mma(q, ldq, out, ldo, kc, vc, n_blocks, table, table_stride, tok_pos,
                                tok_seq, seq_slot, nh, nkv, hd, scale, window, bt, B, n_splits,
                                part_o, part_ml, counters, fault, stream);
}
