// C[M, N] = A[M, K] * W[N, K]^T with float32 multiply-adds on the CUDA cores.
//
// This is the matrix product of the true 32-bit path: no tensor cores, no
// reduced-precision mode, and every output element is one thread's sum over k
// in ascending order, so a row's result does not depend on how many other rows
// the call has. Weights are [out, in] as in the reference (y = x W^T, no bias:
// engine/model.py:295,299,301 of willzeng274/kernel-rush-kawk).
//
// It also serves, with bfloat16 inputs and float32 output, for output-head
// logits at many positions, where the serving path would otherwise round its
// logits to bfloat16.
//
// 64x64 output tile, k in slices of 16, 256 threads with a 4x4 micro-tile each.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(TOut* __restrict__ C, const TIn* __restrict__ A, const TIn* __restrict__ W, int M, int N, int K,
               int lda, int ldw, int ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  const int lr = tid / 4, lk = (tid % 4) * 4;  // this thread loads row lr, k = lk..lk+3 of both tiles
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + j][lr] = (am < M && k < K) ? to_float<TIn>(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + j][lr] = (wn < N && k < K) ? to_float<TIn>(W[(size_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[k][tm + i]; w[i] = Ws[k][tn + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + tm + i, n = n0 + tn + j;
      if (m < M && n < N) C[(size_t)m * ldc + n] = from_float<TOut>(acc[i][j]);
    }
}

template <typename TIn, typename TOut>
int launch(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return -3;
  gemm_nt_kernel<TIn, TOut><<<grid, 256, 0, stream>>>((TOut*)C, (const TIn*)A, (const TIn*)W, M, N, K, lda, ldw, ldc);
  KRK_CHECK_LAUNCH();
  return 0;
}

}  // namespace

// in_dtype / out_dtype: KRK_DTYPE_F32 or KRK_DTYPE_BF16. Supported: f32->f32, bf16->f32, bf16->bf16.
KRK_API int krk_gemm_nt(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                        int in_dtype, int out_dtype, cudaStream_t stream) {
  if (in_dtype == KRK_DTYPE_F32 && out_dtype == KRK_DTYPE_F32)
    return launch<float, float>(C, A, W, M, N, K, lda, ldw, ldc, stream);
  if (in_dtype == KRK_DTYPE_BF16 && out_dtype == KRK_DTYPE_F32)
    return launch<bf16, float>(C, A, W, M, N, K, lda, ldw, ldc, stream);
  if (in_dtype == KRK_DTYPE_BF16 && out_dtype == KRK_DTYPE_BF16)
    return launch<bf16, bf16>(C, A, W, M, N, K, lda, ldw, ldc, stream);
  return -4;
}
