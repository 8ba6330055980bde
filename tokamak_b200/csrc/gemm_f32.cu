// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] * W[N,K]^T.
//
// Plain FFMA accumulation, no tensor cores, no TF32.  Every output element is
// summed over k in ascending order by one thread, so the value of a row of C
// does not depend on how many other rows are in the batch: a difference between
// two ways of cutting the same tokens into steps then points at the cache or
// the batch, not at the matrix product.
#include "common.cuh"

namespace tk {

constexpr int kGemmBM = 64;
constexpr int kGemmBN = 64;
constexpr int kGemmBK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sA[kGemmBK][kGemmBM + 4];
  __shared__ float sW[kGemmBK][kGemmBN + 4];

  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * kGemmBM;
  const int n0 = blockIdx.x * kGemmBN;
  const int tx = tid & 15;   // 4 output columns each
  const int ty = tid >> 4;   // 4 output rows each

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // each thread loads 4 elements of A and 4 of W per k-tile: row = tid / 4, k = (tid % 4) * 4 ..
  const int lrow = tid >> 2;
  const int lk = (tid & 3) * 4;

  for (int k0 = 0; k0 < K; k0 += kGemmBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int am = m0 + lrow;
      const int wn = n0 + lrow;
      sA[lk + i][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.0f;
      sW[lk + i][lrow] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGemmBK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sW[kk][tx * 4 + j];
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
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

}  // namespace tk

TK_API int tk_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda,
                       int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K < 0) return (int)cudaErrorInvalidValue;
  dim3 grid((N + tk::kGemmBN - 1) / tk::kGemmBN, (M + tk::kGemmBM - 1) / tk::kGemmBM);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  return (int)tk::launch(tk::gemm_f32_kernel, grid, dim3(256), 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
}
