// Token embedding: out[t, :] = table[ids[t], :], written as float32 because the result is the
// start of the residual stream, which is kept in 32-bit.
// Stands where the reference indexes the table in torch (miniinfer/layers/embedding.py:23-27).
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_kernel(float* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int H) {
  mi::grid_dependency_sync();
  const int t = blockIdx.x;
  const T* row = table + (size_t)ids[t] * H;
  float* o = out + (size_t)t * H;
  for (int h = threadIdx.x; h < H; h += blockDim.x) o[h] = mi::to_float(row[h]);
}

}  // namespace

// ids must already be known to lie in [0, V): the caller builds them on the host and checks there.
MI_API int mi_embedding(float* out, const void* table, int table_dtype, const int* ids, int T, int H,
                        cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && H > 0, "embedding: bad sizes T=%d H=%d", T, H);
  if (T == 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == MI_BF16)
    mi::launch(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, (const __nv_bfloat16*)table, ids, H);
  else if (table_dtype == MI_F32)
    mi::launch(embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table, ids, H);
  else
    return mi_fail("embedding: unknown table dtype %d", table_dtype);
  MI_LAUNCH_OK("embedding");
  return 0;
}
