// C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]) in true 32-bit: FFMA on the CUDA cores, no
// tensor cores and therefore no reduced-precision matrix mode.  Every output element is
// accumulated over k = 0 .. K-1 in index order by one thread, so a row's result does not
// depend on M or on the row's place in the batch.
//
// Weight layout and meaning as the reference's `linear`: row-major [out, in],
// y[o] = sum_i x[i] * W[o, i] (crates/sglang-kernel/src/cpu.rs:73-108).
#include "common.cuh"

SRB_DEFINE_LAST_ERROR()

#define TILE_M 64
#define TILE_N 64
#define TILE_K 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ c, int m, int n, int k, int lda, int ldw, int ldc) {
  __shared__ float a_tile[TILE_K][TILE_M + 4];
  __shared__ float w_tile[TILE_K][TILE_N + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // 16 x 16 threads, 4 x 4 outputs each
  const int row0 = blockIdx.y * TILE_M, col0 = blockIdx.x * TILE_N;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += TILE_K) {
    for (int i = threadIdx.x; i < TILE_M * TILE_K; i += 256) {
      const int r = i / TILE_K, kk = i % TILE_K;
      const int gr = row0 + r, gk = k0 + kk;
      a_tile[kk][r] = (gr < m && gk < k) ? a[(size_t)gr * lda + gk] : 0.f;
      const int gc = col0 + r;
      w_tile[kk][r] = (gc < n && gk < k) ? w[(size_t)gc * ldw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TILE_K; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_tile[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_tile[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + ty * 4 + i;
    if (gr >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tx * 4 + j;
      if (gc < n) c[(size_t)gr * ldc + gc] = acc[i][j] + (bias ? bias[gc] : 0.f);
    }
  }
}

extern "C" int srb_gemm_f32(const float* a, const float* w, const float* bias, float* c, int m, int n, int k,
                            int lda, int ldw, int ldc, void* stream) {
  if (m <= 0 || n <= 0) return SRB_OK;
  if (k <= 0) SRB_FAIL("gemm_f32: inner size %d must be positive", k);
  if (lda < k || ldw < k || ldc < n) SRB_FAIL("gemm_f32: a leading dimension is smaller than its row");
  dim3 grid((n + TILE_N - 1) / TILE_N, (m + TILE_M - 1) / TILE_M);
  if (grid.y > 65535) SRB_FAIL("gemm_f32: %d rows exceed one launch", m);
  gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a, w, bias, c, m, n, k, lda, ldw, ldc);
  SRB_LAUNCH_CHECK("gemm_f32");
  return SRB_OK;
}
