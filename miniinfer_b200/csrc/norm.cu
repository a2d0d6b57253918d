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

}  // namespace

MI_API int mi_add_rmsnorm(void* out, int out_dtype, float* resid, const void* delta, int delta_dtype,
                          const float* w, const int* rows, int R, int H, float eps, int write_back,
                          cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && H > 0, "rmsnorm: bad sizes R=%d H=%d", R, H);
  MI_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
  if (R == 0) return 0;
  const int threads = 256;  // fixed: the order of the reduction must not depend on the batch
#define MI_NORM_LAUNCH(TO, TD) \
  add_rmsnorm_kernel<TO, TD><<<R, threads, 0, stream>>>((TO*)out, resid, (const TD*)delta, w, rows, H, eps, write_back)
  if (out_dtype == MI_BF16 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == MI_F32 && delta_dtype == MI_F32) MI_NORM_LAUNCH(float, float);
  else if (out_dtype == MI_BF16 && delta_dtype == MI_F32) MI_NORM_LAUNCH(__nv_bfloat16, float);
  else if (out_dtype == MI_F32 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(float, __nv_bfloat16);
  else return mi_fail("rmsnorm: unknown dtypes out=%d delta=%d", out_dtype, delta_dtype);
#undef MI_NORM_LAUNCH
  MI_LAUNCH_OK("add_rmsnorm");
  return 0;
}
