// C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]) with 32-bit accumulation in a fixed order.
//
// This is the matrix product of the true 32-bit path and the fallback for mixed element
// types.  Every output element sums its K products one after the other, k ascending, with
// fused multiply-adds; the order does not depend on M, N or the tile an element falls in,
// so a token's result is the same whichever other tokens share the step.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(THREADS)
gemm_nt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias, TC* __restrict__ C,
               int M, int N, int K, long long lda, long long ldw, long long ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < (BM * BK) / THREADS; ++i) {
      const int idx = tid + i * THREADS;
      const int r = idx / BK, c = idx % BK;
      const int m = m0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? to_f(A[(long long)m * lda + k]) : 0.f;
      const int n = n0 + r;
      Ws[c][r] = (n < N && k < K) ? to_f(W[(long long)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      C[(long long)m * ldc + n] = from_f<TC>(v);
    }
  }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, long long lda,
           long long ldw, long long ldc, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_nt_kernel<TA, TW, TC><<<grid, THREADS, 0, stream>>>((const TA*)A, (const TW*)W, bias, (TC*)C, M, N, K, lda,
                                                          ldw, ldc);
  return 0;
}
}  // namespace

FMX_EXPORT int fmx_gemm_simple(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                               long long lda, long long ldw, long long ldc, int dtype_a, int dtype_w, int dtype_c,
                               cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || N < 0 || K <= 0) return fmx_fail("fmx_gemm_simple: bad sizes M=%d N=%d K=%d", M, N, K);
  if ((long long)((M + BM - 1) / BM) > 65535) return fmx_fail("fmx_gemm_simple: M=%d is too large", M);
  const int key = dtype_a * 4 + dtype_w * 2 + dtype_c;
  switch (key) {
    case 0: launch<float, float, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream); break;
    case 4: launch<bf16, float, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream); break;
    case 5: launch<bf16, float, bf16>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream); break;
    case 6: launch<bf16, bf16, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream); break;
    case 7: launch<bf16, bf16, bf16>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream); break;
    default:
      return fmx_fail("fmx_gemm_simple: no kernel for element types a=%d w=%d c=%d", dtype_a, dtype_w, dtype_c);
  }
  FMX_LAUNCH_CHECK();
  return 0;
}
