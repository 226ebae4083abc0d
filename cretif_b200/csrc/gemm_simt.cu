// C[M,N] = A[M,K] · W[N,K]^T on the CUDA cores with 32-bit FMA accumulation.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced
// precision mode) and the plain kernel every faster product is checked against.  Both
// operands are K-major, as activations [tokens, in] and weights [out, in] are stored,
// so nothing is transposed at load (the reference transposes weights on the host for
// its 32×32 tiled kernel, src/model.cu:141-144, src/kernels/matmul.cu:74-127).
// Any M, N, K; each output sums its products in ascending k whatever M is, so a row's
// result does not depend on how many other rows are in the call.
#include "api.h"
#include "common.cuh"

namespace cretif {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M,
                 int N, int K, int lda, int ldw, int ldc, int accumulate) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4x4 outputs each
  const int lrow = tid >> 2, lk = (tid & 3) * 4;   // loader: 64 rows x 4 groups of 4 k
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // The next k-slab's operands are asked for while this one is multiplied (a product of few
  // rows is a handful of CTAs with nothing else to hide a load behind); the order of the
  // sums does not change.
  const int am = m0 + lrow, wn = n0 + lrow;
  float ra[4], rw[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      ra[e] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.f;
      rw[e] = (wn < N && k < K) ? to_float(W[(size_t)wn * ldw + k]) : 0.f;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      As[lk + e][lrow] = ra[e];
      Ws[lk + e][lrow] = rw[e];
    }
    __syncthreads();
    if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      TC* c = C + (size_t)m * ldc + n;
      float v = acc[i][j];
      if (accumulate) v += to_float(*c);
      *c = from_float<TC>(v);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw,
                  int ldc, int accumulate, cudaStream_t st) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, st>>>((const TA*)A, (const TW*)W, (TC*)C, M, N, K,
                                                     lda, ldw, ldc, accumulate);
  return launch_status();
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_gemm_simt(const void* A, int a_dt, const void* W, int w_dt, void* C,
                                int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                                int accumulate, void* stream) {
  if (M <= 0 || N <= 0) return kOk;
  if (K <= 0 || lda < K || ldw < K || ldc < N) return kBadArgument;
  if ((M + BM - 1) / BM > 65535) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  typedef __nv_bfloat16 bf16;
  if (a_dt == kF32 && w_dt == kF32 && c_dt == kF32)
    return launch<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, st);
  if (a_dt == kBF16 && w_dt == kBF16 && c_dt == kBF16)
    return launch<bf16, bf16, bf16>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, st);
  if (a_dt == kBF16 && w_dt == kBF16 && c_dt == kF32)
    return launch<bf16, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, st);
  if (a_dt == kF32 && w_dt == kBF16 && c_dt == kF32)
    return launch<float, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, st);
  return kBadDType;
}
