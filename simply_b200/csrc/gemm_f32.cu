// True 32-bit matrix product on CUDA cores: out[M, N] = x[M, K] . w[N, K]^T.
//
// No tensor-core mode, no reduced-precision staging: every product and sum is a
// float32 FMA.  The sum over K runs in the same order for every row whatever M
// is, so a token's result does not depend on what else is in the batch.
// Optional epilogue: soft cap (simply/model_lib.py:107-109) for the output layer.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

__global__ void __launch_bounds__(256) gemm_f32_nt_kernel(const float* __restrict__ x,
                                                          const float* __restrict__ w,
                                                          float* __restrict__ out, int M, int N, int K,
                                                          float cap) {
  pdl_wait_block();
  pdl_launch_dependents();
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 columns per operand: 1024 values, 4 per thread.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx / BK, c = idx % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      xs[c][r] = (gm < M && gk < K) ? x[(size_t)gm * K + gk] : 0.f;
      ws[c][r] = (gn < N && gk < K) ? w[(size_t)gn * K + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
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
      if (gn >= N) continue;
      float v = acc[i][j];
      if (cap > 0.f) v = cap * tanhf(v / cap);
      out[(size_t)gm * N + gn] = v;
    }
  }
}

extern "C" int sb_gemm_f32_nt(const float* x, const float* w, float* out, int M, int N, int K, float cap,
                              cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return -6;
  sb_launch(gemm_f32_nt_kernel, grid, 256, 0, stream, x, w, out, M, N, K, cap);
  SB_LAUNCH_CHECK();
  return 0;
}
