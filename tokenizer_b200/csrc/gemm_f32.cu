// True 32-bit matrix product for the check path: C[M,N] = A[M,K] W[N,K]^T (+ bias),
// plain FMA in float, no tensor cores and no reduced-precision mode.  Each output
// element sums its K products in index order, so a row's result does not depend
// on how many other rows are in the batch.
#include "common.cuh"

#define TILE_M 64
#define TILE_N 64
#define TILE_K 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w,
                const float* __restrict__ bias, float* __restrict__ c, int M, int N, int K,
                int lda, int ldc) {
  __shared__ float a_s[TILE_K][TILE_M + 1];
  __shared__ float w_s[TILE_K][TILE_N + 1];
  const int m0 = blockIdx.y * TILE_M, n0 = blockIdx.x * TILE_N;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += TILE_K) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      const int row = idx / TILE_K, kk = idx % TILE_K;
      const int gk = k0 + kk;
      a_s[kk][row] = (m0 + row < M && gk < K) ? a[(size_t)(m0 + row) * lda + gk] : 0.f;
      w_s[kk][row] = (n0 + row < N && gk < K) ? w[(size_t)(n0 + row) * K + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TILE_K; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_s[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_s[kk][tx * 4 + j];
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
      if (n < N) c[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

TOKB200_API int tokb200_gemm_f32(const float* a, const float* w, const float* bias, float* c,
                                 int M, int N, int K, int lda, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return TOKB200_OK;
  if (K <= 0 || lda < K || ldc < N) return TOKB200_BAD_SIZE;
  const long long grid_y = (M + TILE_M - 1) / TILE_M;
  if (grid_y > 65535) return TOKB200_BAD_SIZE;
  dim3 grid((N + TILE_N - 1) / TILE_N, (unsigned)grid_y);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, w, bias, c, M, N, K, lda, ldc);
  return tokb200_launch_status();
}
