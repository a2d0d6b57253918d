// SwiGLU activation: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu in float32, one rounding
// (bfloat16: with the hardware's exponential and reciprocal; float32: exact division and expf).
// Stands where the reference runs a Triton kernel (kernels/triton/silu_mul.py:6-42).
#include "common.cuh"

namespace {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total) {
  mi::grid_dependency_sync();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = mi::to_float(gu[t * 2 * I + i]);
    const float u = mi::to_float(gu[t * 2 * I + I + i]);
    out[idx] = mi::from_float<T>(sizeof(T) == 4 ? mi::silu_mul_exact(g, u) : mi::silu_mul_fast(g, u));
  }
}

// bf16 with I a multiple of 8: 16-byte loads and stores.
__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu, int I8, size_t total8) {
  mi::grid_dependency_sync();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I8;
    const int i = (int)(idx - t * I8);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + i) * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + i) * 8);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 r;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = __bfloat1622float2(gp[k]), b = __bfloat1622float2(up[k]);
      rp[k] = __floats2bfloat162_rn(mi::silu_mul_fast(a.x, b.x), mi::silu_mul_fast(a.y, b.y));
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = r;
  }
}

}  // namespace

MI_API int mi_silu_mul(void* out, const void* gu, int dtype, int T, int I, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && I > 0, "silu_mul: bad sizes T=%d I=%d", T, I);
  if (T == 0) return 0;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  const int most = mi::sm_count() * 16;
  const int blocks = (int)((total + threads - 1) / threads < most ? (total + threads - 1) / threads : most);
  if (dtype == MI_BF16 && I % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)gu % 16) == 0) {
    const size_t total8 = total / 8;
    const int b8 = (int)((total8 + threads - 1) / threads < most ? (total8 + threads - 1) / threads : most);
    mi::launch(silu_mul_bf16x8_kernel, dim3(b8), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, I / 8, total8);
  } else if (dtype == MI_BF16)
    mi::launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, I, total);
  else if (dtype == MI_F32)
    mi::launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)out, (const float*)gu, I, total);
  else
    return mi_fail("silu_mul: unknown dtype %d", dtype);
  MI_LAUNCH_OK("silu_mul");
  return 0;
}
