// Decode attention over the paged cache in bf16: one new token per request, the keys split into
// chunks across blocks (split-KV), the last block of a (request, kv head) to finish merges the chunks.
//
// The kernel is bound by reading K and V once from HBM, so it is built around keeping bytes in
// flight.  A block owns (request, kv head, chunk of keys).  First thing, it asks the bulk-copy
// engine (TMA, cp.async.bulk) for the chunk's K rows and V rows: in the pool's layout the rows of
// one page and one head are contiguous, so one copy per page piece brings them into shared memory,
// and an mbarrier counts the bytes.  All of a block's traffic is in flight from its first
// instructions; several blocks per SM keep the memory system full.  Then, from shared memory:
//   1. scores: lanes share a key 8 elements (16 bytes) each, dot with all query heads of this kv
//      head (held in registers), reduce across the lanes of the key;
//   2. softmax statistics in float32, first per warp over the warp's own keys (no block barrier),
//      merged across the four warps at the end;
//   3. values (behind their own mbarrier, so they stream in while 1 and 2 run): the same lane
//      layout accumulates p * V in float32; partial sums are reduced by shuffles, then across warps.
// Each (request, head, chunk) writes an unnormalised partial output with its max and sum to scratch
// memory; a counter per (request, kv head) tells the last block to arrive that it is the last, and
// that block merges the chunks with the log-sum-exp algebra (the recurrence the reference sketches
// in flash_decode_splitk.py:76-87,129-146) and writes the output rows.  The chunk grid is aligned
// to multiples of the chunk length counted from key 0, so which chunks exist - and the order of
// every sum - depends on the context length (and window) alone.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets an error word and the block
// leaves.
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
constexpr int MAX_CHUNK = 128;
constexpr int VEC = 8;                       // bf16 elements of one 16-byte load
constexpr int ACTIVE = HD / VEC;             // lanes that hold data of one key
constexpr int LPK = ACTIVE <= 2 ? 2 : ACTIVE <= 4 ? 4 : ACTIVE <= 8 ? 8 : ACTIVE <= 16 ? 16 : 32;  // lanes per key
constexpr int KPW = 32 / LPK;                // keys a warp handles at once
constexpr int WAIT_LIMIT = 1 << 22;          // polls of an mbarrier before giving up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t phase) {
  const uint32_t addr = smem_u32(bar);
  for (int i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(phase) : "memory");
    if (done) return true;
  }
  return false;
}
// One contiguous run of bytes from global to shared memory; both addresses and the size are
// multiples of 16.  Completion is counted on the mbarrier.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
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
  __nv_bfloat16* out;            // [T, nh * HD]
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
  int* counters;                 // [n_dec, nkv], zero between launches
  int* status;                   // set to 1 when a bounded wait ran out
  int nh, nkv, page_size, window, chunk, max_splits;
  float scale;
};

// GT query heads of one kv head per pass.
template <int GT>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(DecodeArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);             // [chunk][HD]
  __nv_bfloat16* v_s = k_s + (size_t)a.chunk * HD;                            // [chunk][HD]
  float* s_scores = reinterpret_cast<float*>(v_s + (size_t)a.chunk * HD);     // [WARPS][GT][chunk / WARPS]: a warp's own keys
  const int chunk64 = (a.chunk + 63) / 64 * 64;                               // room for every warp's keys at any head size
  float* s_red = s_scores + GT * chunk64;                                     // [WARPS][GT][HD]
  float* s_stat = s_red + WARPS * GT * HD;                                    // [WARPS][GT][2]: max, sum
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_stat + WARPS * GT * 2);      // [2]; the float count before it is even
  __shared__ int s_last;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ks = lane / LPK, dl = lane % LPK;
  const bool active = dl < ACTIVE;
  const int split = blockIdx.x, kvh = blockIdx.y, e = blockIdx.z;
  const int item = a.decode_items[e];
  const int p = a.ctx_len[item] - 1;                       // position of the query token
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int c0 = lo / a.chunk;
  const int n_splits = p / a.chunk - c0 + 1;
  if (split >= n_splits) return;
  const int chunk_idx = c0 + split;
  const int k_begin = max(lo, chunk_idx * a.chunk);
  const int k_end = min(p + 1, (chunk_idx + 1) * a.chunk);   // exclusive; the range is never empty
  const int n = k_end - k_begin;
  const int G = a.nh / a.nkv;
  const int row = a.q_start[item];
  const int* bt = a.block_table + (size_t)a.seq_slot[item] * a.bt_stride;
  const size_t page_elems = (size_t)2 * a.nkv * a.page_size * HD;
  const size_t head_off = (size_t)kvh * a.page_size * HD;
  const size_t v_off = (size_t)a.nkv * a.page_size * HD;
  const float scale2 = a.scale * 1.4426950408889634f;      // scores are kept in the base-2 domain

  // ---- ask for the chunk's K and V: one bulk copy per page piece, each counted on its barrier
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars[0], (uint32_t)(n * HD * 2));
      mbar_expect_tx(&bars[1], (uint32_t)(n * HD * 2));
    }
    __syncwarp();
    const int first_page = k_begin / a.page_size, last_page = (k_end - 1) / a.page_size;
    for (int which = 0; which < 2; ++which) {
      for (int pg = first_page + lane; pg <= last_page; pg += 32) {
        const int j0 = max(k_begin, pg * a.page_size), j1 = min(k_end, (pg + 1) * a.page_size);
        const __nv_bfloat16* src = a.kv_layer + (size_t)bt[pg] * page_elems + (which ? v_off : 0) + head_off +
                                   (size_t)(j0 - pg * a.page_size) * HD;
        bulk_load((which ? v_s : k_s) + (size_t)(j0 - k_begin) * HD, src, (uint32_t)((j1 - j0) * HD * 2), &bars[which]);
      }
    }
  }

  // A warp's keys are jj = it * (WARPS * KPW) + warp * KPW + ks; its own index for them is it * KPW + ks.
  const int per_warp = chunk64 / WARPS;                    // at least the most keys a warp can have
  float* my_scores = s_scores + (size_t)warp * GT * per_warp;
  int my_n = 0;                                            // keys of this warp: same for all its lanes
  for (int base = 0; base < n; base += WARPS * KPW) my_n += min(KPW, max(0, n - base - warp * KPW));

  bool ok = mbar_wait(&bars[0], 0);
  if (__syncthreads_or(!ok)) {
    if (threadIdx.x == 0) atomicExch(a.status, 1);
    return;
  }

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
    // 1. scores of the warp's keys.  The loop bound is the same for every lane (the shuffles need whole
    // warps); lanes whose key is past the end carry zeros.
#pragma unroll 2
    for (int it = 0; it * (WARPS * KPW) < n; ++it) {
      const int jj = it * (WARPS * KPW) + warp * KPW + ks;
      const bool has_key = jj < n;
      float kf[VEC];
      if (active && has_key) {
        unpack8(*reinterpret_cast<const uint4*>(k_s + (size_t)jj * HD + dl * VEC), kf);
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
        if (dl == 0 && has_key) my_scores[g * per_warp + it * KPW + ks] = s * scale2;
      }
    }
    __syncwarp();
    // 2. the warp's own max and sum of exp2 per head
    float m_w[GT], l_w[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float mx = -INFINITY;
      for (int i = lane; i < my_n; i += 32) mx = fmaxf(mx, my_scores[g * per_warp + i]);
      mx = mi::warp_max(mx);
      const float m_use = mx == -INFINITY ? 0.f : mx;      // a warp without keys
      float sum = 0.f;
      for (int i = lane; i < my_n; i += 32) {
        const float pe = exp2f(my_scores[g * per_warp + i] - m_use);
        my_scores[g * per_warp + i] = pe;
        sum += pe;
      }
      m_w[g] = mx;
      l_w[g] = mi::warp_sum(sum);
    }
    __syncwarp();
    // 3. values, once they are there
    if (g0 == 0) {
      ok = mbar_wait(&bars[1], 0);
      if (__syncthreads_or(!ok)) {
        if (threadIdx.x == 0) atomicExch(a.status, 1);
        return;
      }
    }
    float acc[GT][VEC];
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[g][i] = 0.f;
    if (active) {
#pragma unroll 2
      for (int it = 0; it * (WARPS * KPW) + warp * KPW + ks < n; ++it) {
        const int jj = it * (WARPS * KPW) + warp * KPW + ks;
        float vf[VEC];
        unpack8(*reinterpret_cast<const uint4*>(v_s + (size_t)jj * HD + dl * VEC), vf);
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          const float pe = my_scores[g * per_warp + it * KPW + ks];
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[g][i] = fmaf(pe, vf[i], acc[g][i]);
        }
      }
    }
    // across the key slots of the warp
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
        for (int i = 0; i < VEC; ++i) s_red[(warp * GT + g) * HD + dl * VEC + i] = acc[g][i];
    }
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        s_stat[(warp * GT + g) * 2] = m_w[g];
        s_stat[(warp * GT + g) * 2 + 1] = l_w[g];
      }
    }
    __syncthreads();
    // across the warps: the chunk's max, sum and unnormalised output, in a fixed order
    for (int idx = threadIdx.x; idx < GT * HD; idx += WARPS * 32) {
      const int g = idx / HD, d = idx % HD;
      if (g0 + g >= G) continue;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m = fmaxf(m, s_stat[(w * GT + g) * 2]);
      float v = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float mw = s_stat[(w * GT + g) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
        v = fmaf(s_red[(w * GT + g) * HD + d], f, v);
        l = fmaf(s_stat[(w * GT + g) * 2 + 1], f, l);
      }
      const int head = kvh * G + g0 + g;
      a.part_o[(((size_t)e * a.nh + head) * a.max_splits + split) * HD + d] = v;
      if (d == 0) {
        float* ml = a.part_ml + (((size_t)e * a.nh + head) * a.max_splits + split) * 2;
        ml[0] = m;
        ml[1] = l;
      }
    }
    __syncthreads();
  }

  // ---- the last block of this (request, kv head) merges the chunks
  __threadfence();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&a.counters[e * a.nkv + kvh], 1);
    s_last = prev == n_splits - 1;
    if (s_last) a.counters[e * a.nkv + kvh] = 0;     // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // work items: (head of this kv head, 32 dims); a warp takes items in turn, a lane one dim
  constexpr int DS = (HD + 31) / 32;
  for (int item_idx = warp; item_idx < G * DS; item_idx += WARPS) {
    const int g = item_idx / DS, d = (item_idx % DS) * 32 + lane;
    const int head = kvh * G + g;
    const float* ml = a.part_ml + ((size_t)e * a.nh + head) * a.max_splits * 2;
    const float* po = a.part_o + ((size_t)e * a.nh + head) * a.max_splits * HD;
    // lanes over chunks: max and sum
    float m = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, __ldcg(ml + 2 * s));
    m = mi::warp_max(m);
    float l = 0.f, w_lane = 0.f;
    for (int s = lane; s < n_splits; s += 32) {
      const float f = exp2f(__ldcg(ml + 2 * s) - m);
      if (s < 32) w_lane = f;
      l = fmaf(__ldcg(ml + 2 * s + 1), f, l);
    }
    l = mi::warp_sum(l);
    const float inv = 1.f / l;
    float o = 0.f;
    const int first = min(n_splits, 32);
#pragma unroll 4
    for (int s = 0; s < first; ++s) {
      const float f = __shfl_sync(0xffffffffu, w_lane, s);
      if (d < HD) o = fmaf(__ldcg(po + (size_t)s * HD + d), f, o);
    }
    for (int s = 32; s < n_splits; ++s) {
      const float f = exp2f(__ldcg(ml + 2 * s) - m);
      if (d < HD) o = fmaf(__ldcg(po + (size_t)s * HD + d), f, o);
    }
    if (d < HD) a.out[(size_t)row * a.nh * HD + (size_t)head * HD + d] = __float2bfloat16_rn(o * inv);
  }
}

size_t smem_bytes(int chunk, int gt) {
  return (size_t)2 * chunk * HD * 2 + (size_t)gt * ((chunk + 63) / 64 * 64) * 4 + (size_t)WARPS * gt * HD * 4 + (size_t)WARPS * gt * 2 * 4 +
         2 * 8 + 16;
}

template <int GT>
int launch(const DecodeArgs& a, int n_dec, cudaStream_t stream) {
  const size_t smem = smem_bytes(a.chunk, GT);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_split_kernel<GT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(MAX_CHUNK, GT));
    if (e != cudaSuccess) return mi_fail("attention_decode: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem_bytes(MAX_CHUNK, GT);
  }
  decode_split_kernel<GT><<<dim3(a.max_splits, a.nkv, n_dec), WARPS * 32, smem, stream>>>(a);
  MI_LAUNCH_OK("attention_decode");
  return 0;
}

}  // namespace

// Scratch of the kernel for n_dec decode entries: floats for the partial results, then ints for the
// arrival counters (which must be zero before the first launch; the kernel leaves them zero) and
// one status word.
MI_API long long mi_attention_decode_scratch_floats(int n_dec, int nh, int max_splits) {
  return (long long)n_dec * nh * max_splits * (HD + 2);
}

MI_API int mi_attention_decode_bf16(void* out, const void* q_base, int q_stride, const void* kv_layer,
                                    const int* block_table, int bt_stride, const int* decode_items,
                                    const int* q_start, const int* ctx_len, const int* seq_slot, float* scratch,
                                    int* counters, int* status, int n_dec, int nh, int nkv, int page_size, float scale,
                                    int window, int chunk, int max_splits, cudaStream_t stream) {
  MI_REQUIRE(n_dec >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(chunk >= 32 && chunk <= MAX_CHUNK && chunk % 32 == 0, "attention_decode: chunk=%d must be a multiple of 32 up to %d", chunk, MAX_CHUNK);
  MI_REQUIRE(max_splits >= 1 && max_splits <= 65535, "attention_decode: max_splits=%d", max_splits);
  MI_REQUIRE(page_size > 0 && q_stride % 8 == 0, "attention_decode: bad page_size=%d or q_stride=%d", page_size, q_stride);
  MI_REQUIRE(n_dec <= 65535 && nkv <= 65535, "attention_decode: too many entries for one launch");
  MI_REQUIRE(((uintptr_t)kv_layer % 16) == 0 && ((uintptr_t)q_base % 16) == 0, "attention_decode: operands must be 16-byte aligned");
  if (n_dec == 0) return 0;
  DecodeArgs a;
  a.out = (__nv_bfloat16*)out;
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
  a.counters = counters;
  a.status = status;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window; a.chunk = chunk; a.max_splits = max_splits;
  a.scale = scale;
  const int G = nh / nkv;
  if (G == 1) return launch<1>(a, n_dec, stream);
  if (G == 2) return launch<2>(a, n_dec, stream);
  if (G <= 4) return launch<4>(a, n_dec, stream);
  return launch<8>(a, n_dec, stream);
}
