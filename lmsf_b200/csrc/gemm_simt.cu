// C[M, N] = A[M, K] * W[N, K]^T with float32 FMA accumulation on the CUDA cores.
// This is the matrix product of the true 32-bit path (no tensor cores, no TF32) and the plain
// twin of the tensor-core products.  Counterpart in the reference: cublasLtMatmul through
// tops/csrc/tops/tensorrt_llm/common/cublasMMWrapper.cpp:122-209.
//
// Every output element is accumulated by one thread over k = 0 .. K-1 in ascending order, so a
// row's result does not depend on M or on which other rows share the launch.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_gemm_simt)

namespace lmsf {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TC>
__global__ void __launch_bounds__(256) gemm_tn_kernel(TC* __restrict__ C, const TA* __restrict__ A,
                                                      const TA* __restrict__ W, int M, int N, int K, long long lda,
                                                      long long ldw, long long ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // thread's 4x4 patch: rows ty*4.., cols tx*4..
  const int lr = tid / 4, lk = (tid % 4) * 4;  // loader: row lr of the tile, k offsets lk..lk+3

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int m = m0 + lr, n = n0 + lr;
      As[lk + e][lr] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.f;
      Ws[lk + e][lr] = (n < N && k < K) ? to_f32(W[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
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
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

}  // namespace lmsf

// in_dtype: type of A and W; out_dtype: type of C.  Leading dimensions in elements.
LMSF_API int lmsf_gemm_tn_simt(void* C, const void* A, const void* W, int M, int N, int K, long long lda,
                               long long ldw, long long ldc, int in_dtype, int out_dtype, void* stream) {
  using namespace lmsf;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) LMSF_REFUSE("gemm: K=%d must be positive", K);
  if (lda < K || ldw < K || ldc < N) LMSF_REFUSE("gemm: a leading dimension is smaller than its row");
  dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
  if (grid.y > 65535) LMSF_REFUSE("gemm: M=%d is too large for one launch", M);
  cudaStream_t s = (cudaStream_t)stream;
  if (in_dtype == LMSF_F32 && out_dtype == LMSF_F32)
    gemm_tn_kernel<float, float><<<grid, 256, 0, s>>>((float*)C, (const float*)A, (const float*)W, M, N, K, lda, ldw, ldc);
  else if (in_dtype == LMSF_BF16 && out_dtype == LMSF_BF16)
    gemm_tn_kernel<bf16, bf16><<<grid, 256, 0, s>>>((bf16*)C, (const bf16*)A, (const bf16*)W, M, N, K, lda, ldw, ldc);
  else if (in_dtype == LMSF_BF16 && out_dtype == LMSF_F32)
    gemm_tn_kernel<bf16, float><<<grid, 256, 0, s>>>((float*)C, (const bf16*)A, (const bf16*)W, M, N, K, lda, ldw, ldc);
  else
    LMSF_REFUSE("gemm: unsupported dtype pair (in %d, out %d)", in_dtype, out_dtype);
  return LMSF_LAUNCH_STATUS();
}
