// The exported few-row products without anything fused to them; the kernel is in gemm_skinny.cuh.
#include "gemm_skinny.cuh"

// The gate-and-up product of a SwiGLU feed-forward with the activation in its epilogue:
// out[M, I] = silu(x w_gate^T) * (x w_up^T), w = [w_gate; w_up] of 2I rows.  Both products are
// rounded to bf16 before the activation, as mi_gemm_skinny_bf16 followed by mi_silu_mul rounds them.
MI_API int mi_gemm_skinny_swiglu_bf16(void* out, const void* x, const void* w, int M, int I, int K, int ldo,
                                      cudaStream_t stream) {
  MI_REQUIRE(M >= 0 && M <= 64, "gemm_skinny_swiglu: M=%d is not in 0..64", M);
  MI_REQUIRE(I > 0 && K > 0 && ldo >= I, "gemm_skinny_swiglu: bad sizes I=%d K=%d ldo=%d", I, K, ldo);
  MI_REQUIRE(K % 8 == 0, "gemm_skinny_swiglu: K=%d must be a multiple of 8 (16-byte loads of bf16 rows)", K);
  MI_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_skinny_swiglu: operands must be 16-byte aligned");
  if (M == 0) return 0;
  return dispatch_swiglu((__nv_bfloat16*)out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, M, I, K, ldo, stream);
}

MI_API int mi_gemm_skinny_bf16(void* out, int out_dtype, const void* x, const void* w, int M, int N, int K,
                               int ldo, cudaStream_t stream) {
  MI_REQUIRE(M >= 0 && M <= 64, "gemm_skinny: M=%d is not in 0..64 (use the large-M product)", M);
  MI_REQUIRE(N > 0 && K > 0 && ldo >= N, "gemm_skinny: bad sizes N=%d K=%d ldo=%d", N, K, ldo);
  MI_REQUIRE(K % 8 == 0, "gemm_skinny: K=%d must be a multiple of 8 (16-byte loads of bf16 rows)", K);
  MI_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_skinny: operands must be 16-byte aligned");
  if (M == 0) return 0;
  if (out_dtype == MI_BF16)
    return dispatch<__nv_bfloat16>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, M, N, K, ldo, stream);
  if (out_dtype == MI_F32)
    return dispatch<float>((float*)out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, M, N, K, ldo, stream);
  return mi_fail("gemm_skinny: unknown output dtype %d", out_dtype);
}
