// True 32-bit matrix product on CUDA cores: C[M, N] = A[M, K] . W[N, K]^T (+ bias[N]).
//
// This is the 32-bit path's stand-in for every projection the reference runs through F.linear
// (src/infer/model/layers.py:144,150,163,164; src/infer/model/qwen2.py:51-52): fp32 operands,
// fp32 fused multiply-add, no tensor-core mode of reduced precision anywhere. Each output element
// is one accumulator that walks k = 0..K-1 in order, so a row's result does not depend on how many
// other rows are in the batch. Any M, N, K >= 1; rows of A may be `lda` floats apart.
#include "common.cuh"

namespace tmk {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

__global__ void __launch_bounds__(256) gemm_f32_nt_kernel(const float* __restrict__ A, int lda,
                                                          const float* __restrict__ W,
                                                          const float* __restrict__ bias, float* __restrict__ C,
                                                          int ldc, int M, int N, int K) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Ws[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int lc = tid & 15, lr = tid >> 4;  // loader: column k0 + lc, rows lr, lr + 16, ...
  for (int k0 = 0; k0 < K; k0 += BK) {
    const int k = k0 + lc;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = lr + 16 * i;
      const int m = m0 + r, n = n0 + r;
      As[lc][r] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
      Ws[lc][r] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 w = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
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
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

}  // namespace tmk

extern "C" int tm_gemm_f32_nt(const float* A, int lda, const float* W, const float* bias, float* C, int ldc,
                              int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid((N + tmk::BN - 1) / tmk::BN, (M + tmk::BM - 1) / tmk::BM);
  if (grid.y > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  tmk::gemm_f32_nt_kernel<<<grid, 256, 0, stream>>>(A, lda, W, bias, C, ldc, M, N, K);
  return tmk::launch_status();
}
