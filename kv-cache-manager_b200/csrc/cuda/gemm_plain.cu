// Plain matrix products  Y[M,N] = X[M,K] * W[N,K]^T  (both operands K-major, as every weight of
// the model is stored: [out_features, in_features]; the reference's GEMM wrapper has the same
// contract, src/model/llama.cpp:45-52).
//
// * float x float -> float with float FMAs only: the true 32-bit path.  No tensor cores, no
//   reduced-precision mode.  Every output element is accumulated over k in ascending order by
//   one thread, so a row's result does not depend on how many other rows are in the batch.
// * the same kernel instantiated for bfloat16 operands (float accumulation) is the plain twin
//   that the fast bfloat16 kernels are checked against; Y may be float or bfloat16.
#include "common.cuh"

namespace kvcm {

constexpr int TM = 64, TN = 64, TK = 16;   // block tile; 256 threads, each a 4x4 micro-tile

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TIn* __restrict__ X, const TIn* __restrict__ W, TOut* __restrict__ Y,
                  int M, int N, int K, int ldx, int ldw, int ldy) {
  __shared__ float xs[TK][TM + 1];
  __shared__ float ws[TK][TN + 1];
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int r = i / TK, c = i % TK;
      const int gm = m0 + r, gk = k0 + c;
      xs[c][r] = (gm < M && gk < K) ? ldf(X + size_t(gm) * ldx + gk) : 0.f;
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      const int r = i / TK, c = i % TK;
      const int gn = n0 + r, gk = k0 + c;
      ws[c][r] = (gn < N && gk < K) ? ldf(W + size_t(gn) * ldw + gk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
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
      if (gn < N) stf(Y + size_t(gm) * ldy + gn, acc[i][j]);
    }
  }
}

template <typename TIn, typename TOut>
int launch_gemm_plain(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                      int ldy, cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
  gemm_plain_kernel<TIn, TOut><<<grid, 256, 0, s>>>((const TIn*)X, (const TIn*)W, (TOut*)Y, M, N, K,
                                                    ldx, ldw, ldy);
  return KVCM_LAUNCH_RESULT();
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_gemm_plain_f32(const void* X, const void* W, void* Y, int M, int N, int K, int ldx,
                                 int ldw, int ldy, void* stream) {
  return launch_gemm_plain<float, float>(X, W, Y, M, N, K, ldx, ldw, ldy, (cudaStream_t)stream);
}
KVCM_API int kvcm_gemm_plain_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int ldx,
                                  int ldw, int ldy, void* stream) {
  return launch_gemm_plain<bf16, bf16>(X, W, Y, M, N, K, ldx, ldw, ldy, (cudaStream_t)stream);
}
KVCM_API int kvcm_gemm_plain_bf16_f32out(const void* X, const void* W, void* Y, int M, int N, int K,
                                         int ldx, int ldw, int ldy, void* stream) {
  return launch_gemm_plain<bf16, float>(X, W, Y, M, N, K, ldx, ldw, ldy, (cudaStream_t)stream);
}
