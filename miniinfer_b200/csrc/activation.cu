// SwiGLU activation: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu in float32, one rounding.
// Stands where the reference runs a Triton kernel (kernels/triton/silu_mul.py:6-42).
#include "common.cuh"

namespace {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = mi::to_float(gu[t * 2 * I + i]);
    const float u = mi::to_float(gu[t * 2 * I + I + i]);
    out[idx] = mi::from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

}  // namespace

MI_API int mi_silu_mul(void* out, const void* gu, int dtype, int T, int I, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && I > 0, "silu_mul: bad sizes T=%d I=%d", T, I);
  if (T == 0) return 0;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == MI_BF16)
    silu_mul_kernel<<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gu, I, total);
  else if (dtype == MI_F32)
    silu_mul_kernel<<<blocks, threads, 0, stream>>>((float*)out, (const float*)gu, I, total);
  else
    return mi_fail("silu_mul: unknown dtype %d", dtype);
  MI_LAUNCH_OK("silu_mul");
  return 0;
}
