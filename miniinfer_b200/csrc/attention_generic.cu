// Attention over the paged cache for any mix of prompt portions and decode tokens, any head size
// that is a multiple of 4 up to 256, any page size, float32 or bf16 storage, float32 arithmetic.
//
// One warp per (token, query head).  The warp walks the keys the token may see - positions
// max(0, p - window + 1) .. p of its own request, p being the token's position - in chunks of 32
// aligned to multiples of 32, with an online softmax.  The order of the arithmetic depends on
// (p, window) only, so the result for a token is bit-equal however the request was cut into steps
// and whatever else is in the batch.  This is the attention of the 32-bit path, and the reference
// against which the tensor-core kernels are checked on the device.
//
// Stands where the reference calls the FlashInfer / FlashAttention libraries
// (miniinfer/layers/attention_backend/flashinfer_backend.py:323-374); the mathematics is that of
// miniinfer/layers/attention.py:131-191 (scores * scale, causal mask, softmax, weighted values).
//
// Cache layout of one layer: [page, 2 (k, v), kv head, token in page, head_dim]; the keys of this
// step's own tokens are already in it (the QKV pass stores them first).
#include "common.cuh"

namespace {

constexpr int MAX_HD = 256;
constexpr int WARPS = 4;

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ k, const float* __restrict__ q, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ k, const float* __restrict__ q, int hd) {
  float s = 0.f;
  for (int d = 0; d < hd; d += 4) {
    const float4 v = *reinterpret_cast<const float4*>(k + d);
    s = fmaf(v.x, q[d], s);
    s = fmaf(v.y, q[d + 1], s);
    s = fmaf(v.z, q[d + 2], s);
    s = fmaf(v.w, q[d + 3], s);
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ k,
                                                        const float* __restrict__ q, int hd) {
  float s = 0.f;
  for (int d = 0; d < hd; d += 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(k + d);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    s = fmaf(__low2float(a), q[d], s);
    s = fmaf(__high2float(a), q[d + 1], s);
    s = fmaf(__low2float(b), q[d + 2], s);
    s = fmaf(__high2float(b), q[d + 3], s);
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(T* __restrict__ out, const T* __restrict__ q_base, int q_stride,
                         const T* __restrict__ kv_layer, const int* __restrict__ block_table, int bt_stride,
                         const int* __restrict__ token_item, const int* __restrict__ positions,
                         const int* __restrict__ seq_slot, int nh, int nkv, int hd, int page_size,
                         float scale, int window) {
  mi::grid_dependency_sync();
  __shared__ float qs[WARPS][MAX_HD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tkn = blockIdx.y;
  const int head = blockIdx.x * WARPS + warp;
  if (head >= nh) return;
  const int kvh = head / (nh / nkv);
  const int p = positions[tkn];
  const int slot = seq_slot[token_item[tkn]];
  const int* bt = block_table + (size_t)slot * bt_stride;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;

  const T* q = q_base + (size_t)tkn * q_stride + (size_t)head * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = mi::to_float(q[d]);
  __syncwarp();

  const size_t page_elems = (size_t)2 * nkv * page_size * hd;
  const size_t head_off = (size_t)kvh * page_size * hd;
  const size_t v_off = (size_t)nkv * page_size * hd;

  float o[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int c = (lo / 32) * 32; c <= p; c += 32) {
    const int j = c + lane;
    const bool valid = j >= lo && j <= p;
    long long koff = -1;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[j / page_size];
      koff = (long long)((size_t)page * page_elems + head_off + (size_t)(j % page_size) * hd);
      s = scale * dot_row<T>(kv_layer + koff, qs[warp], hd);
    }
    const float m_new = fmaxf(m, mi::warp_max(s));
    const float alpha = expf(m - m_new);
    const float pe = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + mi::warp_sum(pe);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) o[i] *= alpha;
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pe, jj);
      const long long off = __shfl_sync(0xffffffffu, koff, jj);
      if (off < 0) continue;  // uniform over the warp
      const T* v = kv_layer + off + v_off;
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) o[i] = fmaf(pj, mi::to_float(v[d]), o[i]);
      }
    }
  }
  const float inv = 1.f / l;
  T* dst = out + (size_t)tkn * nh * hd + (size_t)head * hd;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) dst[d] = mi::from_float<T>(o[i] * inv);
  }
}

}  // namespace

// q_base: the q part of the fused QKV rows; q_stride: elements between two tokens' rows.
MI_API int mi_attention_generic(void* out, const void* q_base, int q_stride, int dtype, const void* kv_layer,
                                const int* block_table, int bt_stride, const int* token_item,
                                const int* positions, const int* seq_slot, int T, int nh, int nkv, int hd,
                                int page_size, float scale, int window, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(hd > 0 && hd % 4 == 0 && hd <= MAX_HD, "attention: head_dim=%d must be a multiple of 4 up to %d", hd, MAX_HD);
  MI_REQUIRE(page_size > 0 && q_stride % 4 == 0, "attention: bad page_size=%d or q_stride=%d", page_size, q_stride);
  MI_REQUIRE(T <= 65535, "attention: more than 65535 tokens in one launch (T=%d)", T);
  if (T == 0) return 0;
  dim3 grid((nh + WARPS - 1) / WARPS, T);
  if (dtype == MI_BF16)
    mi::launch(attention_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(WARPS * 32), 0, stream, 
        (__nv_bfloat16*)out, (const __nv_bfloat16*)q_base, q_stride, (const __nv_bfloat16*)kv_layer, block_table,
        bt_stride, token_item, positions, seq_slot, nh, nkv, hd, page_size, scale, window);
  else if (dtype == MI_F32)
    mi::launch(attention_generic_kernel<float>, dim3(grid), dim3(WARPS * 32), 0, stream, 
        (float*)out, (const float*)q_base, q_stride, (const float*)kv_layer, block_table, bt_stride, token_item,
        positions, seq_slot, nh, nkv, hd, page_size, scale, window);
  else
    return mi_fail("attention: unknown dtype %d", dtype);
  MI_LAUNCH_OK("attention_generic");
  return 0;
}
