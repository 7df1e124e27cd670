// True 32-bit matrix product for the float32 path of the engine:
//     C[M, N] = A[M, K] (float32) . W[N, K]^T      W float32 or bfloat16 (widened exactly)
// Plain FFMA, no tensor cores, no TF32, no split along K: every output element is
// the sum over k = 0..K-1 in ascending order, so its bits do not depend on M, on
// the tile it falls into, or on what else is in the batch.  Any M, N, K.
//
// The same kernel with bfloat16 A (and a bfloat16 or float32 C, rounded once from the
// float32 sum) is the plain twin of the tensor-core products: the engine's "plain"
// kernel set runs it for every projection, so that a bfloat16 discrepancy can be put
// down to the fast kernels or to the arithmetic.
#include "common.cuh"
using namespace arle;

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                       TC* __restrict__ C, int M, int N, int K, int lda,
                                                       int ldw, int ldc) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx >> 4, c = idx & 15;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
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
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch_plain(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                        cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return ARLE_E_UNSUPPORTED;
  launch_kernel(gemm_f32_kernel<TA, TW, TC>, dim3(grid), dim3(256), 0, s, 1, (const TA*)A, (const TW*)W, (TC*)C, M, N, K,
                lda, ldw, ldc);
  return launch_status();
}

ARLE_API int arle_gemm_f32(const float* A, const void* W, int w_dtype, float* C, int M, int N, int K, int lda,
                           int ldw, int ldc, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return ARLE_E_BADARG;
  if (w_dtype == 0) return launch_plain<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, s);
  if (w_dtype == 1) return launch_plain<float, __nv_bfloat16, float>(A, W, C, M, N, K, lda, ldw, ldc, s);
  return ARLE_E_BADARG;
}

// bfloat16 A and W, float32 sums, C bfloat16 (c_dtype 1) or float32 (0).
ARLE_API int arle_gemm_plain_bf16(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int lda,
                                  int ldw, int ldc, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return ARLE_E_BADARG;
  if (c_dtype == 1) return launch_plain<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(A, W, C, M, N, K, lda, ldw, ldc, s);
  if (c_dtype == 0) return launch_plain<__nv_bfloat16, __nv_bfloat16, float>(A, W, C, M, N, K, lda, ldw, ldc, s);
  return ARLE_E_BADARG;
}
