// The decode step's few-row products (up to 16 rows) with their neighbours fused to them, so that a
// layer of a decode step is five launches instead of eight:
//
//   mi_gemm_skinny_norm_bf16         out = rmsnorm(resid) * w^T            the norm in the product's prologue
//   mi_gemm_skinny_norm_swiglu_bf16  out = swiglu(rmsnorm(resid) * w^T)    the same, gate-and-up with the activation
//   mi_gemm_skinny_add_f32           resid += bf16(x * w^T)                the residual add in the product's epilogue
//
// The residual stream is float32.  The values are those of the unfused kernels up to the order of
// the norm's sum of squares: the normalised activation is rounded to bf16 once, as the norm kernel
// rounds it, and the product is rounded to bf16 before it is added, as it is when the product's
// bf16 output is handed to the norm kernel.  A row's value does not depend on the other rows.
//
// The reference runs these as separate kernels: a Triton add + RMSNorm (kernels/triton/rms_norm.py:66-149)
// and cuBLAS products (miniinfer/models/fused_qwen3.py:95,107,135,137).
#include "gemm_skinny.cuh"

#define MI_SKINNY_FUSED_CHECKS(name)                                                                      \
  MI_REQUIRE(M >= 0 && M <= 16, name ": M=%d is not in 0..16", M);                                        \
  MI_REQUIRE(N > 0 && K > 0 && ldo >= N, name ": bad sizes N=%d K=%d ldo=%d", N, K, ldo);                 \
  MI_REQUIRE(K % 8 == 0, name ": K=%d must be a multiple of 8 (16-byte loads of bf16 rows)", K);          \
  MI_REQUIRE(((uintptr_t)w % 16) == 0, name ": the weights must be 16-byte aligned");

MI_API int mi_gemm_skinny_norm_bf16(void* out, const float* resid, const float* norm_w, float eps, const void* w,
                                    int M, int N, int K, int ldo, cudaStream_t stream) {
  MI_SKINNY_FUSED_CHECKS("gemm_skinny_norm")
  MI_REQUIRE(eps > 0.f && ((uintptr_t)resid % 16) == 0 && ((uintptr_t)norm_w % 16) == 0, "gemm_skinny_norm: bad eps or alignment");
  if (M == 0) return 0;
  return dispatch16<__nv_bfloat16, FUSE_NORM>((__nv_bfloat16*)out, nullptr, (const __nv_bfloat16*)w, M, N, K, ldo, stream,
                                              FuseArgs{resid, norm_w, eps});
}

MI_API int mi_gemm_skinny_norm_swiglu_bf16(void* out, const float* resid, const float* norm_w, float eps, const void* w,
                                           int M, int N, int K, int ldo, cudaStream_t stream) {
  MI_SKINNY_FUSED_CHECKS("gemm_skinny_norm_swiglu")
  MI_REQUIRE(eps > 0.f && ((uintptr_t)resid % 16) == 0 && ((uintptr_t)norm_w % 16) == 0, "gemm_skinny_norm_swiglu: bad eps or alignment");
  if (M == 0) return 0;
  return dispatch_swiglu16<FUSE_NORM>((__nv_bfloat16*)out, nullptr, (const __nv_bfloat16*)w, M, N, K, ldo, stream,
                                      FuseArgs{resid, norm_w, eps});
}

MI_API int mi_gemm_skinny_add_f32(float* resid, const void* x, const void* w, int M, int N, int K, int ldo, cudaStream_t stream) {
  MI_SKINNY_FUSED_CHECKS("gemm_skinny_add")
  MI_REQUIRE(((uintptr_t)x % 16) == 0, "gemm_skinny_add: the activations must be 16-byte aligned");
  if (M == 0) return 0;
  return dispatch16<float, FUSE_ADD>(resid, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, M, N, K, ldo, stream,
                                     FuseArgs{nullptr, nullptr, 0.f});
}
