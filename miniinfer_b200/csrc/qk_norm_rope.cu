// One pass over the fused QKV activations of a step:
//   q, k heads: RMSNorm over the head (optional), then the rotary encoding (optional), in float32,
//               rounded once and written back in place;
//   k, v heads: stored into the paged cache at the token's slot (optional).
//
// Stands where the reference runs two compiled norms, a dozen torch ops for the rotation
// (miniinfer/models/fused_qwen3.py:101-105, miniinfer/layers/position_encoding.py:47-116) and an
// index assignment into the cache (miniinfer/kvcache/memory_pool.py:48-56).
//
// Rotation: half-split over the first rotary_dim elements of the head, angles taken from a float32
// table cos_sin[pos, 0:rotary_dim/2] = cos, [rotary_dim/2:rotary_dim] = sin.
// Cache layout of one layer: [page, 2 (k, v), kv head, token in page, head_dim].
#include "common.cuh"
#include "qk_rope_math.cuh"

namespace {

constexpr int MAX_HEAD_DIM = 512;
constexpr int WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_kernel(T* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                          const float* __restrict__ cos_sin, int rotary_dim,
                          const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                          T* __restrict__ kv_layer, int nh, int nkv, int hd, int page_size, float eps) {
  mi::grid_dependency_sync();
  __shared__ float buf[WARPS][MAX_HEAD_DIM];
  const int tkn = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nh + 2 * nkv;
  const int h = blockIdx.y * WARPS + warp;     // one warp per (token, head)
  if (h >= heads) return;
  T* row = qkv + (size_t)tkn * heads * hd;
  const int pos = positions[tkn];
  const int slot = (slot_mapping && kv_layer) ? slot_mapping[tkn] : -1;
  const int half = rotary_dim / 2;
  const float* cs = cos_sin ? cos_sin + (size_t)pos * rotary_dim : nullptr;

  {
    T* x = row + (size_t)h * hd;
    const bool is_q = h < nh;
    const bool is_k = !is_q && h < nh + nkv;
    const int kvh = is_q ? 0 : (is_k ? h - nh : h - nh - nkv);
    T* dst = nullptr;
    if (!is_q && slot >= 0) {
      const int page = slot / page_size, off = slot % page_size;
      dst = kv_layer + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * hd;
    }
    if (!is_q && !is_k) {  // v: copy to the cache
      if (dst)
        for (int d = lane; d < hd; d += 32) dst[d] = x[d];
      return;
    }
    const float* w = is_q ? q_w : k_w;
    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) {
      const float v = mi::to_float(x[d]);
      buf[warp][d] = v;
      ss += v * v;
    }
    float rstd = 1.f;
    if (w) {
      ss = mi::warp_sum(ss);
      rstd = rsqrtf(ss / (float)hd + eps);
    }
    __syncwarp();
    for (int d = lane; d < hd; d += 32) {
      float v = buf[warp][d] * rstd * (w ? w[d] : 1.f);
      if (cs && d < rotary_dim) {
        const int pd = d < half ? d + half : d - half;
        const float pv = buf[warp][pd] * rstd * (w ? w[pd] : 1.f);
        const int j = d < half ? d : d - half;
        const float c = cs[j], s = cs[half + j];
        v = d < half ? v * c - pv * s : v * c + pv * s;
      }
      const T r = mi::from_float<T>(v);
      x[d] = r;
      if (dst) dst[d] = r;
    }
  }
}

// The common case in one pass over registers: bf16, the whole head rotated, head_dim a multiple of
// 128 (so that a lane's partner elements d and d + head_dim/2 are its own).  A block takes one token,
// a warp every eighth head of it, four heads at a time: all their loads are issued before anything
// is computed, and the token's cosines and sines and the norm weights are loaded once per lane and
// used for every head.  A lane holds pairs of neighbouring elements (32-bit loads and stores).
template <int HD>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_fast_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                               const float* __restrict__ cos_sin, const int* __restrict__ positions,
                               const int* __restrict__ slot_mapping, __nv_bfloat16* __restrict__ kv_layer, int nh, int nkv,
                               int page_size, float eps) {
  constexpr int HALF = HD / 2;
  constexpr int NP = HALF / 64;                 // bf16 pairs per lane in each half
  constexpr int HEADS_AT_ONCE = 4;
  const int tkn = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nh + 2 * nkv;
  // what no kernel writes is fetched before the wait for the preceding kernel: weights, the table
  float2 wq[2][NP], wk[2][NP], cs_c[NP], cs_s[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int j = 64 * i + 2 * lane;
    wq[0][i] = q_w ? *reinterpret_cast<const float2*>(q_w + j) : make_float2(1.f, 1.f);
    wq[1][i] = q_w ? *reinterpret_cast<const float2*>(q_w + HALF + j) : make_float2(1.f, 1.f);
    wk[0][i] = k_w ? *reinterpret_cast<const float2*>(k_w + j) : make_float2(1.f, 1.f);
    wk[1][i] = k_w ? *reinterpret_cast<const float2*>(k_w + HALF + j) : make_float2(1.f, 1.f);
  }
  const float* cs = cos_sin ? cos_sin + (size_t)positions[tkn] * HD : nullptr;
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int j = 64 * i + 2 * lane;
    cs_c[i] = cs ? *reinterpret_cast<const float2*>(cs + j) : make_float2(1.f, 1.f);
    cs_s[i] = cs ? *reinterpret_cast<const float2*>(cs + HALF + j) : make_float2(0.f, 0.f);
  }
  const int slot = (slot_mapping && kv_layer) ? slot_mapping[tkn] : -1;
  mi::grid_dependency_sync();
  __nv_bfloat16* row = qkv + (size_t)tkn * heads * HD;
  const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;

  // gridDim.y blocks share a token (few tokens: more blocks, a head per warp; many: one block, four heads per warp)
  const int stride = 8 * (int)gridDim.y;
  for (int h0 = (int)blockIdx.y * 8 + warp; h0 < heads; h0 += stride * HEADS_AT_ONCE) {
    uint32_t raw[HEADS_AT_ONCE][2][NP];
#pragma unroll
    for (int u = 0; u < HEADS_AT_ONCE; ++u) {
      const int h = h0 + stride * u;
      if (h < heads) {
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          raw[u][0][i] = *reinterpret_cast<const uint32_t*>(row + (size_t)h * HD + 64 * i + 2 * lane);
          raw[u][1][i] = *reinterpret_cast<const uint32_t*>(row + (size_t)h * HD + HALF + 64 * i + 2 * lane);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < HEADS_AT_ONCE; ++u) {
      const int h = h0 + stride * u;
      if (h >= heads) break;                          // uniform over the warp
      __nv_bfloat16* x = row + (size_t)h * HD;
      const bool is_q = h < nh;
      const bool is_k = !is_q && h < nh + nkv;
      const int kvh = is_q ? 0 : (is_k ? h - nh : h - nh - nkv);
      __nv_bfloat16* dst = (!is_q && slot >= 0)
          ? kv_layer + (((page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * HD : nullptr;
      if (!is_q && !is_k) {                           // values: stored as they are
        if (dst) {
#pragma unroll
          for (int i = 0; i < NP; ++i) {
            *reinterpret_cast<uint32_t*>(dst + 64 * i + 2 * lane) = raw[u][0][i];
            *reinterpret_cast<uint32_t*>(dst + HALF + 64 * i + 2 * lane) = raw[u][1][i];
          }
        }
        continue;
      }
      const bool normed = is_q ? q_w != nullptr : k_w != nullptr;
      float2 v[2][NP];
      float ss = 0.f;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          v[hf][i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u][hf][i]));
        }
#pragma unroll
      for (int i = 0; i < NP; ++i) ss = mi::rope_sum_squares(v[0][i], v[1][i], ss);
      float rstd = 1.f;
      if (normed) {
        ss = mi::warp_sum(ss);
        rstd = mi::rope_rstd(ss, HD, eps);
      }
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int j = 64 * i + 2 * lane;              // index in the first half
        float2 a = v[0][i], b = v[1][i];
        if (normed) {
          a = mi::rope_scale(a, rstd, is_q ? wq[0][i] : wk[0][i]);
          b = mi::rope_scale(b, rstd, is_q ? wq[1][i] : wk[1][i]);
        }
        if (cs) mi::rope_rotate(a, b, cs_c[i], cs_s[i]);
        const __nv_bfloat162 oa = __floats2bfloat162_rn(a.x, a.y), ob = __floats2bfloat162_rn(b.x, b.y);
        const uint32_t ua = *reinterpret_cast<const uint32_t*>(&oa), ub = *reinterpret_cast<const uint32_t*>(&ob);
        *reinterpret_cast<uint32_t*>(x + j) = ua;
        *reinterpret_cast<uint32_t*>(x + HALF + j) = ub;
        if (dst) {
          *reinterpret_cast<uint32_t*>(dst + j) = ua;
          *reinterpret_cast<uint32_t*>(dst + HALF + j) = ub;
        }
      }
    }
  }
}

// Head size 128 with many tokens, in 16-byte steps: a block takes a token at a time, a warp four
// heads at a time, eight lanes per head; a lane holds elements 8l .. 8l + 7 of the head and their
// partners 64 further on, so the rotation needs no exchange and the sum of squares three shuffles.
// The norm weights and the token's row of the rotation table lie in shared memory (every head of a
// token uses the same); while a token is worked on, the first heads of the block's next token and
// its table row are already on their way.
__global__ void __launch_bounds__(256, 4)
qk_norm_rope_store_wide128_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                  const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                  const int* __restrict__ slot_mapping, __nv_bfloat16* __restrict__ kv_layer, int nh, int nkv,
                                  int page_size, float eps, int T) {
  constexpr int HD = 128, HALF = 64;
  __shared__ __align__(16) float w_s[2][HD];        // q and k norm weights (ones where there is none)
  __shared__ __align__(16) float cs_s[2][HD];       // cos | sin of the current and of the next token
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hq = lane >> 3, l8 = lane & 7;
  const int heads = nh + 2 * nkv;
  // what no kernel writes is fetched before the wait for the preceding kernel: weights, the first token's table row
  if (threadIdx.x < 64) {
    const float* w = threadIdx.x < 32 ? q_w : k_w;
    const int i = threadIdx.x & 31;
    reinterpret_cast<float4*>(w_s[threadIdx.x >> 5])[i] = w ? reinterpret_cast<const float4*>(w)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
  } else if (threadIdx.x < 96 && blockIdx.x < T) {
    const int i = threadIdx.x - 64;
    reinterpret_cast<float4*>(cs_s[0])[i] = cos_sin ? reinterpret_cast<const float4*>(cos_sin + (size_t)positions[blockIdx.x] * HD)[i]
                                                    : (i < 16 ? make_float4(1.f, 1.f, 1.f, 1.f) : make_float4(0.f, 0.f, 0.f, 0.f));
  }
  mi::grid_dependency_sync();
  __syncthreads();

  // the first four heads of this warp for the first token
  const int h0 = warp * 4 + hq;
  uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = ra;
  if (blockIdx.x < T && h0 < heads) {
    const __nv_bfloat16* x = qkv + ((size_t)blockIdx.x * heads + h0) * HD;
    ra = *reinterpret_cast<const uint4*>(x + 8 * l8);
    rb = *reinterpret_cast<const uint4*>(x + HALF + 8 * l8);
  }
  int buf = 0;
  for (int tkn = blockIdx.x; tkn < T; tkn += gridDim.x, buf ^= 1) {
    const int next = tkn + gridDim.x;
    // the next token's table row: asked for now, put into shared memory at the end of this round
    float4 cs_next = make_float4(0.f, 0.f, 0.f, 0.f);
    if (warp == 7 && next < T)
      cs_next = cos_sin ? reinterpret_cast<const float4*>(cos_sin + (size_t)positions[next] * HD)[lane]
                        : (lane < 16 ? make_float4(1.f, 1.f, 1.f, 1.f) : make_float4(0.f, 0.f, 0.f, 0.f));
    const int slot = (slot_mapping && kv_layer) ? slot_mapping[tkn] : -1;
    __nv_bfloat16* row = qkv + (size_t)tkn * heads * HD;
    const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;

    for (int hb = 0; hb < heads; hb += 32) {
      const int h = hb + h0;
      const bool live = h < heads;
      const bool is_q = h < nh;
      const bool is_k = !is_q && h < nh + nkv;
      __nv_bfloat16* x = row + (size_t)(live ? h : 0) * HD;
      uint4 xa = ra, xb = rb;
      if (hb > 0) {
        xa = xb = make_uint4(0u, 0u, 0u, 0u);
        if (live) {
          xa = *reinterpret_cast<const uint4*>(x + 8 * l8);
          xb = *reinterpret_cast<const uint4*>(x + HALF + 8 * l8);
        }
      }
      float a[8], b[8];
      {
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&xa);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&xb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
          a[2 * i] = fa.x; a[2 * i + 1] = fa.y; b[2 * i] = fb.x; b[2 * i + 1] = fb.y;
        }
      }
      if (hb == 0 && next < T && h0 < heads) {       // the same heads of the next token, in flight during what follows
        const __nv_bfloat16* xn = qkv + ((size_t)next * heads + h0) * HD;
        ra = *reinterpret_cast<const uint4*>(xn + 8 * l8);
        rb = *reinterpret_cast<const uint4*>(xn + HALF + 8 * l8);
      }
      const int kvh = is_q ? 0 : (is_k ? h - nh : h - nh - nkv);
      __nv_bfloat16* dst = (live && !is_q && slot >= 0)
          ? kv_layer + (((page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * HD : nullptr;
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
      // every lane takes part in the shuffles; the groups of eight lanes are heads
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      if (live && (is_q || is_k)) {
        if (is_q ? q_w != nullptr : k_w != nullptr) {
          const float rstd = rsqrtf(ss / (float)HD + eps);
          const float* w = w_s[is_q ? 0 : 1];
          const float4 wa0 = *reinterpret_cast<const float4*>(w + 8 * l8), wa1 = *reinterpret_cast<const float4*>(w + 8 * l8 + 4);
          const float4 wb0 = *reinterpret_cast<const float4*>(w + HALF + 8 * l8), wb1 = *reinterpret_cast<const float4*>(w + HALF + 8 * l8 + 4);
          const float wa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
          const float wb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a[i] *= rstd * wa[i];
            b[i] *= rstd * wb[i];
          }
        }
        if (cos_sin) {
          const float* cs = cs_s[buf];
          const float4 c0 = *reinterpret_cast<const float4*>(cs + 8 * l8), c1 = *reinterpret_cast<const float4*>(cs + 8 * l8 + 4);
          const float4 s0 = *reinterpret_cast<const float4*>(cs + HALF + 8 * l8), s1 = *reinterpret_cast<const float4*>(cs + HALF + 8 * l8 + 4);
          const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float na = a[i] * c[i] - b[i] * sn[i], nb = b[i] * c[i] + a[i] * sn[i];
            a[i] = na; b[i] = nb;
          }
        }
        __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&xa);
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&xb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pa[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
          pb[i] = __floats2bfloat162_rn(b[2 * i], b[2 * i + 1]);
        }
        *reinterpret_cast<uint4*>(x + 8 * l8) = xa;
        *reinterpret_cast<uint4*>(x + HALF + 8 * l8) = xb;
      }
      if (dst) {                                         // keys as normed and rotated, values as they are
        *reinterpret_cast<uint4*>(dst + 8 * l8) = xa;
        *reinterpret_cast<uint4*>(dst + HALF + 8 * l8) = xb;
      }
    }
    if (warp == 7 && next < T) reinterpret_cast<float4*>(cs_s[buf ^ 1])[lane] = cs_next;
    __syncthreads();       // the next row is in place, and nobody reads this round's row any more
  }
}

}  // namespace

MI_API int mi_qk_norm_rope_store(void* qkv, int dtype, const float* q_w, const float* k_w, const float* cos_sin,
                                 int rotary_dim, const int* positions, const int* slot_mapping, void* kv_layer,
                                 int T, int nh, int nkv, int hd, int page_size, float eps, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && hd > 0, "qk_norm_rope: bad sizes T=%d nh=%d nkv=%d hd=%d", T, nh, nkv, hd);
  MI_REQUIRE(hd <= MAX_HEAD_DIM, "qk_norm_rope: head_dim=%d is larger than %d", hd, MAX_HEAD_DIM);
  MI_REQUIRE(!cos_sin || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= hd),
             "qk_norm_rope: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, hd);
  MI_REQUIRE(!kv_layer || page_size > 0, "qk_norm_rope: page_size must be positive");
  if (T == 0) return 0;
  const dim3 grid(T, (nh + 2 * nkv + WARPS - 1) / WARPS);
  MI_REQUIRE(grid.y <= 65535, "qk_norm_rope: too many heads for one launch");
  const bool whole = !cos_sin || rotary_dim == hd;
  if (dtype == MI_BF16 && whole && (hd == 128 || hd == 256)) {
    const dim3 fast_grid(T, T <= 64 ? (nh + 2 * nkv + 7) / 8 : 1);
    const bool aligned16 = ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)kv_layer % 16) == 0 && ((uintptr_t)cos_sin % 16) == 0 &&
                           ((uintptr_t)q_w % 16) == 0 && ((uintptr_t)k_w % 16) == 0;
    if (hd == 128 && T > 64 && aligned16)
      mi::launch(qk_norm_rope_store_wide128_kernel, dim3(T < mi::sm_count() * 4 ? T : mi::sm_count() * 4), dim3(256), 0, stream, (__nv_bfloat16*)qkv, q_w, k_w,
                 cos_sin, positions, slot_mapping, (__nv_bfloat16*)kv_layer, nh, nkv, page_size, eps, T);
    else if (hd == 128)
      mi::launch(qk_norm_rope_store_fast_kernel<128>, dim3(fast_grid), dim3(256), 0, stream, (__nv_bfloat16*)qkv, q_w, k_w, cos_sin, positions,
                                                                           slot_mapping, (__nv_bfloat16*)kv_layer, nh, nkv, page_size, eps);
    else
      mi::launch(qk_norm_rope_store_fast_kernel<256>, dim3(fast_grid), dim3(256), 0, stream, (__nv_bfloat16*)qkv, q_w, k_w, cos_sin, positions,
                                                                           slot_mapping, (__nv_bfloat16*)kv_layer, nh, nkv, page_size, eps);
    MI_LAUNCH_OK("qk_norm_rope_store");
    return 0;
  }
  if (dtype == MI_BF16)
    mi::launch(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3(grid), dim3(WARPS * 32), 0, stream, (__nv_bfloat16*)qkv, q_w, k_w, cos_sin, rotary_dim, positions,
                                                           slot_mapping, (__nv_bfloat16*)kv_layer, nh, nkv, hd, page_size, eps);
  else if (dtype == MI_F32)
    mi::launch(qk_norm_rope_store_kernel<float>, dim3(grid), dim3(WARPS * 32), 0, stream, (float*)qkv, q_w, k_w, cos_sin, rotary_dim, positions,
                                                           slot_mapping, (float*)kv_layer, nh, nkv, hd, page_size, eps);
  else
    return mi_fail("qk_norm_rope: unknown dtype %d", dtype);
  MI_LAUNCH_OK("qk_norm_rope_store");
  return 0;
}
