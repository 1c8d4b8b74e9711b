// C[M,N] = A[M,K] * W[N,K]^T on CUDA cores in float32 (FFMA, no tensor cores,
// no reduced-precision mode), for the true 32-bit path and for weights that a
// checkpoint stores in 32-bit.  Weights keep the (out, in) layout of the
// checkpoint, y = x W^T (engine/layers.py:48-50).
//
// Every output element is one accumulator that walks k = 0..K-1 in ascending
// order, so a row's result does not depend on how many rows share the launch.
// A, W and C may each be float32 or bfloat16; products and sums are float32.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16
#define GS_THREADS 256

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(GS_THREADS) gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                                TC* __restrict__ C, int M, int N, int K, int lda,
                                                                int ldw, int ldc) {
  pdl_trigger();
  pdl_wait();
  __shared__ float As[GS_BK][GS_BM + 4];
  __shared__ float Ws[GS_BK][GS_BN + 4];
  const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;      // 16 x 16 threads, 4 x 4 outputs each
  const int lr = tid >> 2, lc = (tid & 3) * 4;  // loader: row 0..63, k offset 0,4,8,12
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lc + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lc + u][lr] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
      Ws[lc + u][lr] = (wn < N && k < K) ? to_f32(W[(size_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GS_BK; ++kk) {
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
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch_gemm(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                       cudaStream_t stream) {
  dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
  return launch_k(gemm_simt_kernel<TA, TW, TC>, grid, GS_THREADS, 0, stream, (const TA*)A, (const TW*)W, (TC*)C, M, N,
                  K, lda, ldw, ldc);
}

extern "C" int ie_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M,
                            int N, int K, int lda, int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IE_OK;
  if (K <= 0) return IE_BAD_SIZE;
  const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
  switch (code) {
    case 0: return launch_gemm<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 2: return launch_gemm<float, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 4: return launch_gemm<bf16, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 5: return launch_gemm<bf16, float, bf16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 6: return launch_gemm<bf16, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 7: return launch_gemm<bf16, bf16, bf16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    default: return IE_BAD_DTYPE;
  }
}
