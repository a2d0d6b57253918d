// bf16 matrix product with many rows through cuBLAS: out[M, N] = x[M, K] * w[N, K]^T, float32
// accumulation, bf16 or float32 result.  This is the prefill's QKV / o / gate-up / down product,
// where the reference also calls the library (nn.Linear: miniinfer/layers/linear.py:30-32).
// The call goes straight to cublasGemmEx on the caller's stream: a prefill step issues four of
// these per layer, and the host time of each call counts (through torch.mm a call costs about
// three times as much host time).  One handle per device, made on first use.  Not for use inside
// a stream capture: the handle's workspace is the library's own.
#include <cublas_v2.h>

#include "common.cuh"

namespace {

constexpr int MAX_DEVICES = 64;
cublasHandle_t handles[MAX_DEVICES] = {};

}  // namespace

MI_API int mi_gemm_cublas_bf16(void* out, int out_dtype, const void* x, const void* w, int M, int N, int K,
                               cudaStream_t stream) {
  MI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_cublas: bad sizes M=%d N=%d K=%d", M, N, K);
  MI_REQUIRE(out_dtype == MI_BF16 || out_dtype == MI_F32, "gemm_cublas: unknown output dtype %d", out_dtype);
  if (M == 0) return 0;
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  MI_REQUIRE(ce == cudaSuccess && dev >= 0 && dev < MAX_DEVICES, "gemm_cublas: no current device");
  if (!handles[dev]) {
    cublasStatus_t st = cublasCreate(&handles[dev]);
    if (st != CUBLAS_STATUS_SUCCESS) {
      handles[dev] = nullptr;
      return mi_fail("gemm_cublas: cublasCreate failed with status %d", (int)st);
    }
  }
  cublasHandle_t h = handles[dev];
  cublasStatus_t st = cublasSetStream(h, stream);
  if (st != CUBLAS_STATUS_SUCCESS) return mi_fail("gemm_cublas: cublasSetStream failed with status %d", (int)st);
  // Row-major out[M, N] is column-major out^T[N, M] = w (as K x N column-major, transposed) * x (K x M).
  const float alpha = 1.f, beta = 0.f;
  st = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, K, x, CUDA_R_16BF, K, &beta, out,
                    out_dtype == MI_BF16 ? CUDA_R_16BF : CUDA_R_32F, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  if (st != CUBLAS_STATUS_SUCCESS) return mi_fail("gemm_cublas: cublasGemmEx failed with status %d (M=%d N=%d K=%d)", (int)st, M, N, K);
  return 0;
}
