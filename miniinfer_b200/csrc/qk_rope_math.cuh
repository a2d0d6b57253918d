// The arithmetic of the per-head RMSNorm and the rotary encoding on a lane's share of a head, spelled out in
// single operations (no contraction into fused multiply-adds is left to the compiler): two kernels do this step -
// qk_norm_rope_store_fast_kernel for any step, and the cluster-scheduled decode attention kernel for its own
// query heads and new key - and the numbers must not depend on which of them ran.
// Layout: a warp takes a head; lane l holds the neighbouring elements (j, j + 1) of the head's first half and the
// pair (HALF + j, HALF + j + 1) of its second half, which are partners in the rotation.
#pragma once
#include "common.cuh"

namespace mi {

__device__ __forceinline__ float rope_sum_squares(float2 a, float2 b, float ss) {
  ss = __fmaf_rn(a.x, a.x, ss);
  ss = __fmaf_rn(a.y, a.y, ss);
  ss = __fmaf_rn(b.x, b.x, ss);
  ss = __fmaf_rn(b.y, b.y, ss);
  return ss;
}

// rstd from the head's sum of squares (already summed over the warp)
__device__ __forceinline__ float rope_rstd(float ss, int head_dim, float eps) {
  return rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)head_dim), eps));
}

__device__ __forceinline__ float2 rope_scale(float2 v, float rstd, float2 w) {
  return make_float2(__fmul_rn(v.x, __fmul_rn(rstd, w.x)), __fmul_rn(v.y, __fmul_rn(rstd, w.y)));
}

// (a, b) -> (a cos - b sin, b cos + a sin), element by element
__device__ __forceinline__ void rope_rotate(float2& a, float2& b, float2 c, float2 s) {
  const float2 ra = make_float2(__fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(b.x, s.x)), __fsub_rn(__fmul_rn(a.y, c.y), __fmul_rn(b.y, s.y)));
  const float2 rb = make_float2(__fadd_rn(__fmul_rn(b.x, c.x), __fmul_rn(a.x, s.x)), __fadd_rn(__fmul_rn(b.y, c.y), __fmul_rn(a.y, s.y)));
  a = ra;
  b = rb;
}

}  // namespace mi
