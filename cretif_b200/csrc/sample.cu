// Sampling on the device: one block per row of 32-bit logits [rows, vocab].
//
//  * greedy: arg-max, ties go to the lowest id (reference: src/embedding.cu:155-204, a
//    single block for the one sequence it has);
//  * temperature: softmax(logits / T) over the whole vocabulary, then one uniform draw
//    walked along the cumulative sum in id order;
//  * top-k: the k largest logits, divided by T, softmax over them, the draw walked in
//    descending order of logit — the reference does this on the host after copying the
//    row back (src/embedding.cu:343-406); here the row never leaves the device.
//
// The uniform number comes from a counter-based generator keyed by (seed, request, draw
// number), so a request's tokens do not depend on which other requests share its batch.
// The reference re-seeds its generator with the same value at every step
// (src/embedding.cu:391-394, called with the default seed at src/model.cu:1075-1076),
// which repeats one uniform number for a whole generation; that is not reproduced.
#include "api.h"
#include "common.cuh"

namespace cretif {

constexpr int kSampleThreads = 512;
constexpr int kMaxTopK = 1024;

__host__ __device__ inline unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Uniform in (0, 1) from (seed, request, draw).
__host__ __device__ inline float uniform01(unsigned long long seed, long long request,
                                           int draw) {
  unsigned long long x = splitmix64(seed ^ (0xD1B54A32D192ED03ull * (unsigned long long)(request + 1)));
  x = splitmix64(x ^ (0x8CB92BA72F3D8DD7ull * (unsigned long long)(draw + 1)));
  return ((float)(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ unsigned int order_key(float v) {
  const unsigned int b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);     // larger float -> larger key
}

// Exclusive prefix sum over the block in thread order; returns the thread's prefix and
// the total through `total`.
template <typename V>
__device__ __forceinline__ V block_exclusive_scan(V v, V* warp_tot, V* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  V inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    V n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    V w = lane < nwarps ? warp_tot[lane] : V(0);
    V winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      V n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    if (lane < nwarps) warp_tot[lane] = winc - w;
    if (lane == 31) warp_tot[32] = winc;
  }
  __syncthreads();
  *total = warp_tot[32];
  return warp_tot[warp] + inc - v;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int ld, int V, float temperature, int top_k,
              unsigned long long seed, const unsigned long long* __restrict__ seed_dev,
              const long long* __restrict__ request, int* __restrict__ draw,
              int* __restrict__ out) {
  if (seed_dev) seed = *seed_dev;      // the seed of a captured launch lives in device memory
  __shared__ float scratch[33];
  __shared__ float fscan[33];
  __shared__ int iscan[33];
  __shared__ float best_v[kSampleThreads / 32];
  __shared__ int best_i[kSampleThreads / 32];
  __shared__ int hist[256];
  __shared__ float cand_v[kMaxTopK];
  __shared__ int cand_i[kMaxTopK];
  __shared__ int counter, chosen;
  __shared__ unsigned int sel_prefix;
  __shared__ int sel_need;

  const int row = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)row * ld;

  if (temperature <= 0.f) {
    // ---- greedy: arg-max with the lowest id among equals
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    auto take = [&](float v, int i) {
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    };
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {       // 16-byte loads, eight in flight
      const float4* x4 = reinterpret_cast<const float4*>(x);
      const int n4 = V >> 2;
#pragma unroll 8
      for (int i = tid; i < n4; i += kSampleThreads) {
        const float4 v = __ldg(x4 + i);
        take(v.x, 4 * i); take(v.y, 4 * i + 1); take(v.z, 4 * i + 2); take(v.w, 4 * i + 3);
      }
      done = n4 << 2;
    }
    for (int i = done + tid; i < V; i += kSampleThreads) take(x[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { best_v[tid >> 5] = bv; best_i[tid >> 5] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < kSampleThreads / 32; ++w)
        if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
      out[row] = bi == 0x7fffffff ? 0 : bi;
    }
    return;
  }

  const float u = uniform01(seed, request ? request[row] : row, draw ? draw[row] : 0);
  const float inv_t = 1.0f / temperature;
  const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
  const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);

  if (top_k <= 0 || top_k >= V) {
    // ---- the whole vocabulary, cumulative sum in id order
    float mx = -INFINITY;
    for (int i = tid; i < V; i += kSampleThreads) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, scratch);
    float local = 0.f;
    for (int i = lo; i < hi; ++i) local += expf((x[i] - mx) * inv_t);
    float total;
    const float prefix = block_exclusive_scan<float>(local, fscan, &total);
    if (tid == 0) chosen = 0x7fffffff;
    __syncthreads();
    const float target = u * total;
    if (target >= prefix && target < prefix + local) {
      float part = 0.f;               // summed exactly as `local` was
      for (int i = lo; i < hi; ++i) {
        part += expf((x[i] - mx) * inv_t);
        if (target < prefix + part) { atomicMin(&chosen, i); break; }
      }
    }
    __syncthreads();
    if (tid == 0) {
      int c = chosen;
      if (c == 0x7fffffff) {          // rounding put the target past the last step
        c = V - 1;
        while (c > 0 && expf((x[c] - mx) * inv_t) == 0.f) --c;
      }
      out[row] = c;
      if (draw) draw[row] += 1;
    }
    return;
  }

  // ---- top-k: radix-select the k-th largest key, 8 bits at a time
  const int k = top_k;
  if (tid == 0) { sel_prefix = 0u; sel_need = k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const unsigned int prefix = sel_prefix;
    const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < V; i += kSampleThreads) {
      const unsigned int key = order_key(x[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = sel_need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      sel_prefix = prefix | ((unsigned int)b << shift);
      sel_need = need;               // how many are taken from this bin
    }
    __syncthreads();
  }
  const unsigned int kth = sel_prefix;      // key of the k-th largest logit
  const int need_equal = sel_need;          // ties at that key that are kept (lowest ids)
  if (tid == 0) counter = 0;
  // ties: rank them in id order
  int ties = 0;
  for (int i = lo; i < hi; ++i) ties += order_key(x[i]) == kth;
  int total_ties;
  int tie_rank = block_exclusive_scan<int>(ties, iscan, &total_ties);
  __syncthreads();
  for (int i = lo; i < hi; ++i) {
    const unsigned int key = order_key(x[i]);
    bool take = key > kth;
    if (key == kth) { take = tie_rank < need_equal; ++tie_rank; }
    if (take) {
      const int at = atomicAdd(&counter, 1);
      if (at < kMaxTopK) { cand_v[at] = x[i]; cand_i[at] = i; }
    }
  }
  __syncthreads();
  const int n = min(counter, k);
  int np2 = 1;
  while (np2 < n) np2 <<= 1;
  for (int i = n + tid; i < np2; i += kSampleThreads) { cand_v[i] = -INFINITY; cand_i[i] = 0x7fffffff; }
  __syncthreads();
  // bitonic sort: descending logit, ascending id among equals
  for (int size = 2; size <= np2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < np2; i += kSampleThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const bool up = (i & size) == 0;
          const float vi = cand_v[i], vj = cand_v[j];
          const int ii = cand_i[i], ij = cand_i[j];
          const bool i_first = vi > vj || (vi == vj && ii < ij);   // i belongs before j
          if (i_first != up) {
            cand_v[i] = vj; cand_v[j] = vi;
            cand_i[i] = ij; cand_i[j] = ii;
          }
        }
      }
      __syncthreads();
    }
  }
  if (tid == 0) {
    const float mx = cand_v[0] * inv_t;
    float sum = 0.f;
    for (int i = 0; i < n; ++i) sum += expf(cand_v[i] * inv_t - mx);
    float run = 0.f;
    int c = cand_i[n - 1];
    for (int i = 0; i < n; ++i) {
      run += expf(cand_v[i] * inv_t - mx) / sum;
      if (u <= run) { c = cand_i[i]; break; }
    }
    out[row] = c;
    if (draw) draw[row] += 1;
  }
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_sample(const float* logits, int ld, int rows, int V, float temperature,
                             int top_k, unsigned long long seed,
                             const unsigned long long* seed_dev, const long long* request,
                             int* draw, int* out, void* stream) {
  if (rows <= 0) return kOk;
  if (V <= 0 || ld < V) return kBadArgument;
  if (temperature > 0.f && top_k > kMaxTopK && top_k < V) return kBadArgument;
  sample_kernel<<<rows, kSampleThreads, 0, (cudaStream_t)stream>>>(logits, ld, V, temperature,
                                                                  top_k, seed, seed_dev, request,
                                                                  draw, out);
  return launch_status();
}

extern "C" float cretif_uniform01(unsigned long long seed, long long request, int draw) {
  return uniform01(seed, request, draw);
}

extern "C" int cretif_max_top_k() { return kMaxTopK; }
