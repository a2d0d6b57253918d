// True float32 matrix product on the CUDA cores: out[M, N] = x[M, K] * w[N, K]^T.
//
// This is the matrix product of the engine's 32-bit path.  Every product and sum is an fp32 FMA
// (no TF32, no tensor cores), and every output element adds its K products in ascending k, so the
// value of an element does not depend on M, on the tile it falls in, or on what else is in the
// batch: the 32-bit path gives bit-equal logits however the tokens are cut into steps.
// The reference has no 32-bit path (it calls cuBLAS in fp16, miniinfer/layers/linear.py:30-32).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                int M, int N, int K, int ldo) {
  mi::grid_dependency_sync();
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // tx -> n, ty -> m
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k for each operand: 1024 values, 4 per thread, k fastest for coalescing.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx / BK, kk = idx % BK;
      const int k = k0 + kk;
      xs[kk][r] = (m0 + r < M && k < K) ? x[(size_t)(m0 + r) * K + k] : 0.f;
      ws[kk][r] = (n0 + r < N && k < K) ? w[(size_t)(n0 + r) * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx + j * 16];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx + j * 16;
      if (n < N) out[(size_t)m * ldo + n] = acc[i][j];
    }
  }
}

}  // namespace

MI_API int mi_gemm_f32(float* out, const float* x, const float* w, int M, int N, int K, int ldo,
                       cudaStream_t stream) {
  MI_REQUIRE(M >= 0 && N > 0 && K > 0 && ldo >= N, "gemm_f32: bad sizes M=%d N=%d K=%d ldo=%d", M, N, K, ldo);
  if (M == 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  MI_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d is too large for one launch", M);
  mi::launch(gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, out, x, w, M, N, K, ldo);
  MI_LAUNCH_OK("gemm_f32");
  return 0;
}
