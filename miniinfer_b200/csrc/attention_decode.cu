// Decode attention over the paged cache in bf16: one new token per request, the keys split into
// chunks across blocks (split-KV), partial results merged by a second small kernel.
//
// This kernel is bound by reading K and V once from HBM.  A block owns (request, kv head, chunk of
// keys) and serves all query heads of that kv head from one pass over the chunk's K and V:
//   1. scores: lanes share a key 8 elements (16 bytes) each, dot with the query heads held in
//      registers, reduce across the lanes of the key; scores go to shared memory;
//   2. softmax statistics of the chunk in float32 (max, exp, sum);
//   3. values: the same lane layout accumulates p * V in float32 registers; the partial sums are
//      reduced across key slots by shuffles and across warps in shared memory.
// Each (request, head, chunk) writes an unnormalised partial output with its max and sum; the merge
// kernel combines the chunks with the usual log-sum-exp algebra (the recurrence that the reference
// sketches in flash_decode_splitk.py:76-87,129-146).  The chunk grid is aligned to multiples of
// the chunk length counted from key 0, so which chunks exist depends on the context length (and
// window) alone.
//
// Stands where the reference calls FlashInfer's / FlashAttention's decode kernels
// (miniinfer/layers/attention_backend/flashinfer_backend.py:323-327).
//
// Compiled once per head size: -DMI_HEAD_DIM=<multiple of 16, 16..256>.
#include "common.cuh"

#ifndef MI_HEAD_DIM
#error "compile with -DMI_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int HD = MI_HEAD_DIM;
constexpr int WARPS = 4;
constexpr int MAX_CHUNK = 256;
constexpr int VEC = 8;                       // bf16 elements of one 16-byte load
constexpr int ACTIVE = HD / VEC;             // lanes that hold data of one key
constexpr int LPK = ACTIVE <= 2 ? 2 : ACTIVE <= 4 ? 4 : ACTIVE <= 8 ? 8 : ACTIVE <= 16 ? 16 : 32;  // lanes per key
constexpr int KPW = 32 / LPK;                // keys a warp handles at once

__device__ __forceinline__ uint4 ld16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

struct DecodeArgs {
  const __nv_bfloat16* q_base;   // fused QKV rows; q first
  int q_stride;
  const __nv_bfloat16* kv_layer; // [page, 2, nkv, P, HD]
  const int* block_table;
  int bt_stride;
  const int* decode_items;       // item index of each decode entry
  const int* q_start;            // per item: its row
  const int* ctx_len;            // per item: keys including the new token
  const int* seq_slot;
  float* part_o;                 // [n_dec, nh, max_splits, HD]
  float* part_ml;                // [n_dec, nh, max_splits, 2]
  int nh, nkv, page_size, window, chunk, max_splits;
  float scale;
};

// GT query heads of one kv head per pass.
template <int GT>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(DecodeArgs a) {
  __shared__ float s_scores[GT][MAX_CHUNK];
  __shared__ float s_red[WARPS][GT][HD];
  __shared__ float s_stat[WARPS][GT];
  __shared__ float s_m[GT], s_l[GT];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ks = lane / LPK, dl = lane % LPK;
  const bool active = dl < ACTIVE;
  const int split = blockIdx.x, kvh = blockIdx.y, e = blockIdx.z;
  const int item = a.decode_items[e];
  const int p = a.ctx_len[item] - 1;                       // position of the query token
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int c0 = lo / a.chunk;
  const int chunk_idx = c0 + split;
  const int k_begin = max(lo, chunk_idx * a.chunk);
  const int k_end = min(p + 1, (chunk_idx + 1) * a.chunk);   // exclusive
  if (k_begin >= k_end) return;
  const int n = k_end - k_begin;
  const int G = a.nh / a.nkv;
  const int row = a.q_start[item];
  const int* bt = a.block_table + (size_t)a.seq_slot[item] * a.bt_stride;
  const size_t page_elems = (size_t)2 * a.nkv * a.page_size * HD;
  const size_t head_off = (size_t)kvh * a.page_size * HD;
  const size_t v_off = (size_t)a.nkv * a.page_size * HD;

  for (int g0 = 0; g0 < G; g0 += GT) {
    // queries of this pass, this lane's 8 elements of each
    float q[GT][VEC];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const int head = kvh * G + min(g0 + g, G - 1);
      if (active) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a.q_base + (size_t)row * a.q_stride + (size_t)head * HD + dl * VEC);
        unpack8(raw, q[g]);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) q[g][i] = 0.f;
      }
    }
    // 1. scores.  The loop bound is the same for every lane of the block (the shuffles below need
    // whole warps); lanes whose key is past the end carry zeros.
#pragma unroll 4
    for (int base = 0; base < n; base += WARPS * KPW) {
      const int jj = base + warp * KPW + ks;
      const bool has_key = jj < n;
      float kf[VEC];
      if (active && has_key) {
        const int j = k_begin + jj;
        const int page = bt[j / a.page_size];
        const __nv_bfloat16* kp = a.kv_layer + (size_t)page * page_elems + head_off + (size_t)(j % a.page_size) * HD + dl * VEC;
        unpack8(ld16(kp), kf);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) kf[i] = 0.f;
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) s = fmaf(q[g][i], kf[i], s);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (dl == 0 && has_key) s_scores[g][jj] = s * a.scale;
      }
    }
    __syncthreads();
    // 2. max and sum of exp per head
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float mx = -INFINITY;
      for (int jj = threadIdx.x; jj < n; jj += WARPS * 32) mx = fmaxf(mx, s_scores[g][jj]);
      mx = mi::warp_max(mx);
      if (lane == 0) s_stat[warp][g] = mx;
    }
    __syncthreads();
    if (threadIdx.x < GT) {
      float mx = s_stat[0][threadIdx.x];
#pragma unroll
      for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, s_stat[w][threadIdx.x]);
      s_m[threadIdx.x] = mx;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float mx = s_m[g];
      float sum = 0.f;
      for (int jj = threadIdx.x; jj < n; jj += WARPS * 32) {
        const float pe = expf(s_scores[g][jj] - mx);
        s_scores[g][jj] = pe;
        sum += pe;
      }
      sum = mi::warp_sum(sum);
      if (lane == 0) s_stat[warp][g] = sum;
    }
    __syncthreads();
    if (threadIdx.x < GT) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) sum += s_stat[w][threadIdx.x];
      s_l[threadIdx.x] = sum;
    }
    // 3. values
    float acc[GT][VEC];
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[g][i] = 0.f;
#pragma unroll 4
    for (int jj = warp * KPW + ks; jj < n; jj += WARPS * KPW) {
      if (!active) continue;
      const int j = k_begin + jj;
      const int page = bt[j / a.page_size];
      const __nv_bfloat16* vp = a.kv_layer + (size_t)page * page_elems + v_off + head_off + (size_t)(j % a.page_size) * HD + dl * VEC;
      float vf[VEC];
      unpack8(ld16(vp), vf);
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        const float pe = s_scores[g][jj];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[g][i] = fmaf(pe, vf[i], acc[g][i]);
      }
    }
    // across the key slots of the warp, then across warps
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float v = acc[g][i];
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[g][i] = v;
      }
    if (ks == 0 && active) {
#pragma unroll
      for (int g = 0; g < GT; ++g)
#pragma unroll
        for (int i = 0; i < VEC; ++i) s_red[warp][g][dl * VEC + i] = acc[g][i];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GT * HD; idx += WARPS * 32) {
      const int g = idx / HD, d = idx % HD;
      if (g0 + g >= G) continue;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += s_red[w][g][d];
      const int head = kvh * G + g0 + g;
      a.part_o[(((size_t)e * a.nh + head) * a.max_splits + split) * HD + d] = v;
    }
    if (threadIdx.x < GT && g0 + threadIdx.x < G) {
      const int head = kvh * G + g0 + threadIdx.x;
      float* ml = a.part_ml + (((size_t)e * a.nh + head) * a.max_splits + split) * 2;
      ml[0] = s_m[threadIdx.x];
      ml[1] = s_l[threadIdx.x];
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(128)
decode_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    const int* __restrict__ decode_items, const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                    int nh, int window, int chunk, int max_splits) {
  const int e = blockIdx.x, head = blockIdx.y;
  const int item = decode_items[e];
  const int p = ctx_len[item] - 1;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int splits = p / chunk - lo / chunk + 1;
  const float* ml = part_ml + ((size_t)e * nh + head) * max_splits * 2;
  const float* po = part_o + ((size_t)e * nh + head) * max_splits * HD;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
  const float inv = 1.f / l;
  __nv_bfloat16* dst = out + (size_t)q_start[item] * nh * HD + (size_t)head * HD;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += po[(size_t)s * HD + d] * expf(ml[2 * s] - m);
    dst[d] = __float2bfloat16_rn(v * inv);
  }
}

}  // namespace

// Floats of scratch the two kernels need for n_dec decode entries.
MI_API long long mi_attention_decode_scratch_floats(int n_dec, int nh, int max_splits) {
  return (long long)n_dec * nh * max_splits * (HD + 2);
}

MI_API int mi_attention_decode_bf16(void* out, const void* q_base, int q_stride, const void* kv_layer,
                                    const int* block_table, int bt_stride, const int* decode_items,
                                    const int* q_start, const int* ctx_len, const int* seq_slot, float* scratch,
                                    int n_dec, int nh, int nkv, int page_size, float scale, int window, int chunk,
                                    int max_splits, cudaStream_t stream) {
  MI_REQUIRE(n_dec >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(chunk >= 32 && chunk <= MAX_CHUNK && chunk % 32 == 0, "attention_decode: chunk=%d must be a multiple of 32 up to %d", chunk, MAX_CHUNK);
  MI_REQUIRE(max_splits >= 1 && max_splits <= 65535, "attention_decode: max_splits=%d", max_splits);
  MI_REQUIRE(page_size > 0 && q_stride % 8 == 0, "attention_decode: bad page_size=%d or q_stride=%d", page_size, q_stride);
  MI_REQUIRE(n_dec <= 65535 && nkv <= 65535, "attention_decode: too many entries for one launch");
  if (n_dec == 0) return 0;
  DecodeArgs a;
  a.q_base = (const __nv_bfloat16*)q_base;
  a.q_stride = q_stride;
  a.kv_layer = (const __nv_bfloat16*)kv_layer;
  a.block_table = block_table;
  a.bt_stride = bt_stride;
  a.decode_items = decode_items;
  a.q_start = q_start;
  a.ctx_len = ctx_len;
  a.seq_slot = seq_slot;
  a.part_o = scratch;
  a.part_ml = scratch + (size_t)n_dec * nh * max_splits * HD;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window; a.chunk = chunk; a.max_splits = max_splits;
  a.scale = scale;
  const int G = nh / nkv;
  dim3 grid(max_splits, nkv, n_dec);
  if (G == 1) decode_split_kernel<1><<<grid, WARPS * 32, 0, stream>>>(a);
  else if (G == 2) decode_split_kernel<2><<<grid, WARPS * 32, 0, stream>>>(a);
  else if (G <= 4) decode_split_kernel<4><<<grid, WARPS * 32, 0, stream>>>(a);
  else decode_split_kernel<8><<<grid, WARPS * 32, 0, stream>>>(a);
  MI_LAUNCH_OK("attention_decode split");
  decode_merge_kernel<<<dim3(n_dec, nh), 128, 0, stream>>>((__nv_bfloat16*)out, a.part_o, a.part_ml, decode_items, q_start,
                                                          ctx_len, nh, window, chunk, max_splits);
  MI_LAUNCH_OK("attention_decode merge");
  return 0;
}
