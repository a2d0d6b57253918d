// RMSNorm with the residual add fused in front of it.
//
//   sum[r, :] = resid[row(r), :] (+ delta[row(r), :])         float32
//   out[r, :] = w * sum * rsqrt(mean(sum^2) + eps)            rounded once to the output type
//   resid[row(r), :] = sum                                    if write_back
//
// The reference adds in the model's type and rounds the normalised value before the weight
// multiply (kernels/triton/rms_norm.py:88-108, miniinfer/layers/layernorm.py:27-32); here the
// residual stream stays in float32 and the only rounding is the final one.
// `rows` selects rows (the final norm runs only on the rows whose logits are wanted).
#include "common.cuh"

namespace {

template <typename TOut, typename TDelta>
__global__ void add_rmsnorm_kernel(TOut* __restrict__ out, float* __restrict__ resid,
                                   const TDelta* __restrict__ delta, const float* __restrict__ w,
                                   const int* __restrict__ rows, int H, float eps, int write_back) {
  mi::grid_dependency_sync();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* x = resid + (size_t)row * H;
  const TDelta* d = delta ? delta + (size_t)row * H : nullptr;
  float ss = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = x[h];
    if (d) v += mi::to_float(d[h]);
    if (write_back && d) x[h] = v;
    ss += v * v;
  }
  const float total = mi::block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
  TOut* o = out + (size_t)r * H;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = x[h];
    if (d && !write_back) v += mi::to_float(d[h]);
    o[h] = mi::from_float<TOut>(w[h] * (v * rstd));
  }
}

// The serving case in 16-byte steps: bf16 output and delta, H a multiple of 4, a row kept in
// registers between the two passes (up to 4 * 256 * VPT values).
template <int VPT>
__global__ void __launch_bounds__(256)
add_rmsnorm_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ resid,
                            const __nv_bfloat16* __restrict__ delta, const float* __restrict__ w,
                            const int* __restrict__ rows, int H, float eps, int write_back) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int H4 = H / 4;
  // the norm weights and the row list are written by no kernel: fetched before the wait for the preceding kernel
  const int row = rows ? rows[r] : r;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 ww[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) ww[i] = w4[h];
  }
  mi::grid_dependency_sync();
  float4* x = reinterpret_cast<float4*>(resid + (size_t)row * H);
  const uint2* d = delta ? reinterpret_cast<const uint2*>(delta + (size_t)row * H) : nullptr;
  float4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) {
      v[i] = x[h];
      if (d) {
        const uint2 raw = d[h];
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[i].x += a.x; v[i].y += a.y; v[i].z += b.x; v[i].w += b.y;
        if (write_back) x[h] = v[i];
      }
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  const float total = mi::block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
  uint2* o = reinterpret_cast<uint2*>(out + (size_t)r * H);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(ww[i].x * (v[i].x * rstd), ww[i].y * (v[i].y * rstd));
      const __nv_bfloat162 hi = __floats2bfloat162_rn(ww[i].z * (v[i].z * rstd), ww[i].w * (v[i].w * rstd));
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&lo);
      packed.y = *reinterpret_cast<const uint32_t*>(&hi);
      o[h] = packed;
    }
  }
}

}  // namespace

MI_API int mi_add_rmsnorm(void* out, int out_dtype, float* resid, const void* delta, int delta_dtype,
                          const float* w, const int* rows, int R, int H, float eps, int write_back,
                          cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && H > 0, "rmsnorm: bad sizes R=%d H=%d", R, H);
  MI_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
  if (R == 0) return 0;
  const int threads = 256;  // fixed: the order of the reduction must not depend on the batch
  const bool aligned = ((uintptr_t)out % 8) == 0 && ((uintptr_t)resid % 16) == 0 && ((uintptr_t)delta % 8) == 0 && ((uintptr_t)w % 16) == 0;
  if (out_dtype == MI_BF16 && (delta == nullptr || delta_dtype == MI_BF16) && H % 4 == 0 && H <= 8192 && aligned) {
    const int vpt = (H / 4 + 255) / 256;
    if (vpt <= 1)
      mi::launch(add_rmsnorm_bf16_vec_kernel<1>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    else if (vpt <= 2)
      mi::launch(add_rmsnorm_bf16_vec_kernel<2>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    else if (vpt <= 4)
      mi::launch(add_rmsnorm_bf16_vec_kernel<4>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    else
      mi::launch(add_rmsnorm_bf16_vec_kernel<8>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    MI_LAUNCH_OK("add_rmsnorm");
    return 0;
  }
#define MI_NORM_LAUNCH(TO, TD) \
  mi::launch(add_rmsnorm_kernel<TO, TD>, dim3(R), dim3(threads), 0, stream, (TO*)out, resid, (const TD*)delta, w, rows, H, eps, write_back)
  if (out_dtype == MI_BF16 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == MI_F32 && delta_dtype == MI_F32) MI_NORM_LAUNCH(float, float);
  else if (out_dtype == MI_BF16 && delta_dtype == MI_F32) MI_NORM_LAUNCH(__nv_bfloat16, float);
  else if (out_dtype == MI_F32 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(float, __nv_bfloat16);
  else return mi_fail("rmsnorm: unknown dtypes out=%d delta=%d", out_dtype, delta_dtype);
#undef MI_NORM_LAUNCH
  MI_LAUNCH_OK("add_rmsnorm");
  return 0;
}
