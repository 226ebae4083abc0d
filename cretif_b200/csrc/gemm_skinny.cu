// y[M,N] (+)= x[M,K] · W[N,K]^T for few rows of x (decode): bfloat16 in, 32-bit accumulate.
//
// A decode step reads every weight once and does little arithmetic on it, so the kernel is
// organised around streaming W: a CTA owns 16 consecutive rows of W (output features) and
// its 8 warps split K between them; every lane fetches 16 contiguous bytes of a W row per
// load and the products run on the tensor cores as mma.sync m16n8k16 with W as the 16-row
// operand and up to 64 tokens as 8-wide column tiles (the roles of the operands are swapped
// with respect to the prefill product, where tokens are the long dimension).  The k index
// inside a 32-wide chunk is permuted identically for both operands, which leaves the dot
// products unchanged and lets both fragments come from single 16-byte loads.  The warps'
// partial sums meet in shared memory.
//
// The reference has no counterpart: its decode step runs the same 32×32-tile kernel as
// prefill with one row (src/model.cu:797-825, src/kernels/matmul.cu:74-127).
#include "api.h"
#include "common.cuh"

namespace cretif {

constexpr int kSkWarps = 8;
constexpr int kSkRows = 16;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4],
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// NT = number of 8-token tiles (M <= 8 * NT)
template <int NT, typename TC>
__global__ void __launch_bounds__(kSkWarps * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                   TC* __restrict__ C, int M, int N, int K, int ldx, int ldw, int ldc,
                   int accumulate) {
  __shared__ float red[kSkWarps][kSkRows][8 * NT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * kSkRows;
  const int row_a = min(n0 + r, N - 1), row_b = min(n0 + r + 8, N - 1);
  const __nv_bfloat16* wa = W + (size_t)row_a * ldw + c * 8;
  const __nv_bfloat16* wb = W + (size_t)row_b * ldw + c * 8;

  float acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

  const int n_chunks = (K + 31) >> 5;                  // 32 k per chunk
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  // chunks are dealt to the warps round-robin so that the CTA's loads stay contiguous
  for (int ch = warp; ch < n_chunks; ch += kSkWarps) {
    const int k = ch * 32 + c * 8;
    const bool in = k < K;                              // K is a multiple of 8
    const uint4 ua = in ? __ldg(reinterpret_cast<const uint4*>(wa + ch * 32)) : zero;
    const uint4 ub = in ? __ldg(reinterpret_cast<const uint4*>(wb + ch * 32)) : zero;
    const uint32_t a1[4] = {ua.x, ub.x, ua.y, ub.y};    // first 16 (permuted) k
    const uint32_t a2[4] = {ua.z, ub.z, ua.w, ub.w};    // second 16
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int m = t * 8 + r;
      uint4 ux = zero;
      if (in && m < M) ux = __ldg(reinterpret_cast<const uint4*>(X + (size_t)m * ldx + k));
      mma_bf16_16816(acc[t], a1, ux.x, ux.y);
      mma_bf16_16816(acc[t], a2, ux.z, ux.w);
    }
  }
  // acc[t]: {row r, tokens 2c,2c+1}, {row r+8, tokens 2c,2c+1} of token tile t
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    red[warp][r][t * 8 + 2 * c] = acc[t][0];
    red[warp][r][t * 8 + 2 * c + 1] = acc[t][1];
    red[warp][r + 8][t * 8 + 2 * c] = acc[t][2];
    red[warp][r + 8][t * 8 + 2 * c + 1] = acc[t][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kSkRows * M; i += kSkWarps * 32) {
    const int m = i / kSkRows, rr = i - m * kSkRows;    // consecutive threads: consecutive n
    const int n = n0 + rr;
    if (n >= N) continue;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kSkWarps; ++w) sum += red[w][rr][m];
    TC* out = C + (size_t)m * ldc + n;
    if (accumulate) sum += to_float(*out);
    *out = from_float<TC>(sum);
  }
}

template <typename TC>
static int launch_skinny(const void* X, const void* W, void* C, int M, int N, int K, int ldx,
                         int ldw, int ldc, int accumulate, cudaStream_t st) {
  const int blocks = (N + kSkRows - 1) / kSkRows;
  const int nt = (M + 7) / 8;
#define CRETIF_SK(NT)                                                                        \
  gemm_skinny_kernel<NT, TC><<<blocks, kSkWarps * 32, 0, st>>>(                              \
      (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, (TC*)C, M, N, K, ldx, ldw, ldc,      \
      accumulate)
  switch (nt) {
    case 1: CRETIF_SK(1); break;
    case 2: CRETIF_SK(2); break;
    case 3: case 4: CRETIF_SK(4); break;
    default: CRETIF_SK(8); break;
  }
#undef CRETIF_SK
  return launch_status();
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_gemm_skinny_max_rows() { return 64; }

extern "C" int cretif_gemm_skinny(const void* X, const void* W, void* C, int c_dt, int M, int N,
                                  int K, int ldx, int ldw, int ldc, int accumulate,
                                  void* stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (M > 64 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldc < N)
    return kBadArgument;
  if (((uintptr_t)X | (uintptr_t)W) & 15) return kMisaligned;
  cudaStream_t st = (cudaStream_t)stream;
  if (c_dt == kF32) return launch_skinny<float>(X, W, C, M, N, K, ldx, ldw, ldc, accumulate, st);
  if (c_dt == kBF16)
    return launch_skinny<__nv_bfloat16>(X, W, C, M, N, K, ldx, ldw, ldc, accumulate, st);
  return kBadDType;
}
