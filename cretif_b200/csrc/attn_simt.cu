// Causal grouped-query attention over the block cache, one CTA per (token, query head).
//
// The plain attention kernel: it serves prefill and decode alike, in 32-bit and in
// bfloat16 storage, for any number of heads and groups, head sizes in steps of 8 up to
// 256, an optional sliding window, and it is the kernel the faster ones are checked
// against.  Maths as in the reference: s = (q·k)·scale with the scale applied after the
// dot (src/attention.cu:690-692), keys after the query's position are masked (:60-77),
// softmax with running maximum and sum in 32-bit as in the reference's decode kernel
// (:451-493), query head h reads key/value head h / (heads / kv_heads) (:421-422).
// The CTA's eight warps take the keys in blocks of 32 in turn (warp w: blocks w, w + 8, ...),
// each with its own running maximum, sum and output, and warp 0 folds the eight results
// together in the order of the warps: a decode step, whose one query per head would otherwise
// be one warp walking thousands of keys with every load's latency exposed, is eight chains
// of an eighth the length.  A (token, head) is always reduced in the same order, so its
// output does not depend on what else is in the batch or on how the tokens were cut into
// steps.
#include "api.h"
#include "common.cuh"

namespace cretif {

constexpr int kWarps = 8;
constexpr int kMaxHd = 256;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attn_simt_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo,
                 const T* __restrict__ kc, const T* __restrict__ vc,
                 const int* __restrict__ table, int table_stride,
                 const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                 const int* __restrict__ seq_slot, int nh, int nkv, int hd, float scale,
                 int window, int bt, int T_tokens) {
  __shared__ float qs[kMaxHd];
  __shared__ float part_acc[kWarps][kMaxHd];
  __shared__ float part_m[kWarps], part_l[kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = blockIdx.x;
  const int t = (int)(item / nh), h = (int)(item - (long long)t * nh);
  const int kvh = h / (nh / nkv);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int* tab = table + (size_t)slot * table_stride;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;

  const T* qrow = q + (size_t)t * ldq + (size_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += kWarps * 32) qs[d] = to_float(qrow[d]);
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[kMaxHd / 32];
#pragma unroll
  for (int i = 0; i < kMaxHd / 32; ++i) acc[i] = 0.f;

  for (int base = first + 32 * warp; base <= pos; base += 32 * kWarps) {
    const int key = base + lane;
    bool valid = key <= pos;
    float s = -INFINITY;
    unsigned long long row = 0;
    const int blk = valid ? tab[key / bt] : -1;
    valid = blk >= 0;                 // a position without a block counts as masked
    if (valid) {
      row = ((unsigned long long)blk * nkv + kvh) * bt + (key % bt);
      const T* kp = kc + row * hd;
      float dot = 0.f;
#pragma unroll 4
      for (int d = 0; d < hd; d += 8) {
        float kv[8];
        load8(kp + d, kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(qs[d + e], kv[e], dot);
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);   // nothing summed yet
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kMaxHd / 32; ++i) acc[i] *= corr;
    m = m_new;
    // Values: keys in ascending order, eight at a time so that their loads travel together
    // (a decode step has one warp per head and nothing else to hide a load behind).  A key
    // with p = 0 (masked, or underflowed) adds nothing and is not read.
    const int n_valid = min(32, pos + 1 - base);
    constexpr int kAhead = 8;
    for (int j0 = 0; j0 < n_valid; j0 += kAhead) {
      float pj[kAhead];
      const T* vp[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int j = min(j0 + u, 31);
        const float pu = __shfl_sync(0xffffffffu, p, j);
        const unsigned long long ru = __shfl_sync(0xffffffffu, row, j);
        pj[u] = j0 + u < n_valid ? pu : 0.f;
        vp[u] = vc + ru * hd;
      }
#pragma unroll
      for (int i = 0; i < kMaxHd / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) {
          float v[kAhead];
#pragma unroll
          for (int u = 0; u < kAhead; ++u) v[u] = pj[u] != 0.f ? to_float(vp[u][d]) : 0.f;
#pragma unroll
          for (int u = 0; u < kAhead; ++u)
            if (pj[u] != 0.f) acc[i] = fmaf(pj[u], v[u], acc[i]);
        }
      }
    }
  }
  // the warps' results meet in shared memory; warp 0 folds them in the warps' order
  if (lane == 0) {
    part_m[warp] = m;
    part_l[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < kMaxHd / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) part_acc[warp][d] = acc[i];
  }
  __syncthreads();
  if (warp != 0) return;
  float m_all = -INFINITY;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) m_all = fmaxf(m_all, part_m[w]);
  float l_all = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxHd / 32; ++i) acc[i] = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const float mw = part_m[w];
    if (mw == -INFINITY) continue;              // a warp without a visible key adds nothing
    const float a = expf(mw - m_all);
    l_all += part_l[w] * a;
#pragma unroll
    for (int i = 0; i < kMaxHd / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) acc[i] = fmaf(part_acc[w][d], a, acc[i]);
    }
  }
  const float inv = 1.0f / l_all;
  T* orow = out + (size_t)t * ldo + (size_t)h * hd;
#pragma unroll
  for (int i = 0; i < kMaxHd / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_attn_simt(const void* q, int ldq, void* out, int ldo, int dt, const void* kc,
                                const void* vc, const int* table, int table_stride,
                                const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                int nh, int nkv, int hd, float scale, int window, int bt, int T,
                                void* stream) {
  if (T <= 0) return kOk;
  if (nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || hd % 8 || hd > kMaxHd || bt <= 0 ||
      window < 0)
    return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const long long items = (long long)T * nh;
  if (items > 0x7fffffffLL) return kBadArgument;
  const unsigned blocks = (unsigned)items;
  if (dt == kF32)
    attn_simt_kernel<float><<<blocks, kWarps * 32, 0, st>>>(
        (const float*)q, ldq, (float*)out, ldo, (const float*)kc, (const float*)vc, table,
        table_stride, tok_pos, tok_seq, seq_slot, nh, nkv, hd, scale, window, bt, T);
  else if (dt == kBF16)
    attn_simt_kernel<__nv_bfloat16><<<blocks, kWarps * 32, 0, st>>>(
        (const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)kc,
        (const __nv_bfloat16*)vc, table, table_stride, tok_pos, tok_seq, seq_slot, nh, nkv, hd,
        scale, window, bt, T);
  else
    return kBadDType;
  return launch_status();
}
