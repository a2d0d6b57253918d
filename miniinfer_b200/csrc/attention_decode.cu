// Decode attention over the paged cache in bf16: one new token per request, the keys split into
// chunks across blocks (split-KV), the last block of a (request, kv head) to finish merges the chunks.
//
// The kernel has to read K and V once from HBM and do as little else as possible: a first version
// that multiplied on the CUDA cores spent one instruction per 6 bytes and was bound by issue
// slots, not by memory.  So the products run on the tensor cores.  A block owns (request, kv head,
// chunk of keys); the query heads that share the kv head are the rows of one 16-row MMA tile
// (zero-padded; more than 16 heads take another pass).  Keys come in blocks of 64: their K and V
// rows are gathered page by page into padded shared-memory rows with cp.async, three blocks in
// flight; each of the four warps takes 16 keys of a block: S = Q K^T (mma.m16n8k16, bf16 in, fp32
// accumulate), online softmax in float32 (base 2, scale folded in), O += P V.  At the end the four
// warps' (max, sum, O) are merged in shared memory in a fixed order and written as the chunk's
// partial result; a counter per (request, kv head) tells the last block to arrive that it is the
// last, and that block merges the chunks with the log-sum-exp algebra (the recurrence the
// reference sketches in flash_decode_splitk.py:76-87,129-146) and writes the output rows.  The
// chunk grid is aligned to multiples of the chunk length counted from key 0, so which chunks
// exist - and the order of every sum - depends on the context length (and window) alone.
//
// No block waits for another: the merge is done by whichever block finds the counter full.
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
constexpr int BK = 64;             // keys of a block; 16 per warp
constexpr int STAGES = 2;
constexpr int MAX_CHUNK = 1024;    // keys of a (request, kv head) that one block may take
constexpr int LDS = HD + 8;        // shared-memory row stride in elements (odd number of 16-byte units)
constexpr int CHUNKS = HD / 8;     // 16-byte chunks of a row
constexpr int KSTEPS = HD / 16;
constexpr int NT_O = HD / 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
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
  int nh, nkv, page_size, window, chunk, max_splits;
  float scale;
};

// Gathers keys first .. first + BK of one kv head (K and V rows) into a stage; rows from `end` on are
// zeros.  Consecutive lanes take consecutive 16-byte chunks of a row, so a warp's copy instruction
// covers whole 128-byte lines; the page of a row is looked up only when it changes.
__device__ __forceinline__ void load_block(__nv_bfloat16* ks, __nv_bfloat16* vs, const DecodeArgs& a, const int* bt,
                                           size_t page_elems, size_t head_off, size_t v_off, int first, int end) {
  int last_pg = -1;
  size_t page_base = 0;
#pragma unroll
  for (int i = 0; i < (BK * CHUNKS + WARPS * 32 - 1) / (WARPS * 32); ++i) {
    const int idx = threadIdx.x + i * WARPS * 32;
    if ((BK * CHUNKS) % (WARPS * 32) != 0 && idx >= BK * CHUNKS) break;
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const int j = first + r;
    const bool valid = j < end;
    const __nv_bfloat16* src = a.kv_layer;
    if (valid) {
      const int pg = j / a.page_size;
      if (pg != last_pg) {
        last_pg = pg;
        page_base = (size_t)bt[pg] * page_elems + head_off;
      }
      src = a.kv_layer + page_base + (size_t)(j - pg * a.page_size) * HD + c * 8;
    }
    cp_async16(ks + r * LDS + c * 8, src, valid);
    cp_async16(vs + r * LDS + c * 8, valid ? src + v_off : src, valid);
  }
}

__global__ void __launch_bounds__(WARPS * 32, 3)
decode_split_kernel(DecodeArgs a) {
  mi::grid_dependency_sync();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16][LDS]
  __nv_bfloat16* stage0 = q_s + 16 * LDS;                            // [STAGES][2 (k, v)][BK][LDS]
  float* red = reinterpret_cast<float*>(stage0);                     // after the loop: [WARPS][16][HD] + [WARPS][16][2]
  __shared__ int s_last;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int lm = lane >> 3, lr = lane & 7;     // ldmatrix: lane gives the address of row lr of 8x8 matrix lm
  // kv heads vary fastest: blocks that run side by side read neighbouring segments of the same pages
  const int kvh = blockIdx.x, split = blockIdx.y, e = blockIdx.z;
  const int item = a.decode_items[e];
  const int p = a.ctx_len[item] - 1;                       // position of the query token
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int c0 = lo / a.chunk;
  const int n_splits = p / a.chunk - c0 + 1;
  if (split >= n_splits) return;
  const int chunk_idx = c0 + split;
  const int k_begin = max(lo, chunk_idx * a.chunk);
  const int k_end = min(p + 1, (chunk_idx + 1) * a.chunk);   // exclusive; the range is never empty
  const int nb = (k_end - k_begin + BK - 1) / BK;
  const int G = a.nh / a.nkv;
  const int row = a.q_start[item];
  const int* bt = a.block_table + (size_t)a.seq_slot[item] * a.bt_stride;
  const size_t page_elems = (size_t)2 * a.nkv * a.page_size * HD;
  const size_t head_off = (size_t)kvh * a.page_size * HD;
  const size_t v_off = (size_t)a.nkv * a.page_size * HD;
  const float scale2 = a.scale * 1.4426950408889634f;      // scores are kept in the base-2 domain

  for (int g0 = 0; g0 < G; g0 += 16) {
    const int heads = min(16, G - g0);
    // ---- queries of this pass (rows past `heads` are zeros) and the first blocks of keys
    for (int idx = threadIdx.x; idx < 16 * CHUNKS; idx += WARPS * 32) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      const bool valid = r < heads;
      const __nv_bfloat16* src = valid ? a.q_base + (size_t)row * a.q_stride + (size_t)(kvh * G + g0 + r) * HD + c * 8 : a.q_base;
      cp_async16(q_s + r * LDS + c * 8, src, valid);
    }
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      if (s < nb) load_block(stage0 + (size_t)s * 2 * BK * LDS, stage0 + (size_t)(s * 2 + 1) * BK * LDS, a, bt, page_elems, head_off,
                             v_off, k_begin + s * BK, k_end);
      cp_async_commit();
    }

    uint32_t qf[KSTEPS][4];
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int b = 0; b < nb; ++b) {
      cp_async_wait<STAGES - 2>();      // block b (and the queries) have landed
      __syncthreads();                  // ... for every thread; and everyone is done with block b - 1
      {
        const int nxt = b + STAGES - 1;
        if (nxt < nb) {
          const int s = nxt % STAGES;
          load_block(stage0 + (size_t)s * 2 * BK * LDS, stage0 + (size_t)(s * 2 + 1) * BK * LDS, a, bt, page_elems, head_off, v_off,
                     k_begin + nxt * BK, k_end);
        }
        cp_async_commit();
      }
      if (b == 0) {
#pragma unroll
        for (int k = 0; k < KSTEPS; ++k) ldmatrix_x4(qf[k], q_s + ((lm & 1) * 8 + lr) * LDS + k * 16 + (lm >> 1) * 8);
      }
      const int st = b % STAGES;
      const __nv_bfloat16* ks = stage0 + (size_t)st * 2 * BK * LDS + (size_t)warp * 16 * LDS;   // this warp's 16 keys
      const __nv_bfloat16* vs = ks + (size_t)BK * LDS;

      // S = Q K^T: 16 heads x 16 keys
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        // matrices: (keys 0..7, d k*16 + 0..7), (same keys, d + 8), (keys 8..15, d), (keys 8..15, d + 8)
        uint32_t kf[4];
        ldmatrix_x4(kf, ks + ((lm >> 1) * 8 + lr) * LDS + k * 16 + (lm & 1) * 8);
        mma_bf16(s[0], qf[k], kf[0], kf[1]);
        mma_bf16(s[1], qf[k], kf[2], kf[3]);
      }
      // keys past the end of the chunk do not count; softmax update per row (rows g and g + 8)
      const int key0 = k_begin + b * BK + warp * 16;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = key0 + i * 8 + 2 * t + (c & 1);
          const float v = j < k_end ? s[i][c] * scale2 : -INFINITY;
          s[i][c] = v;
          mx[c >> 1] = fmaxf(mx[c >> 1], v);
        }
      float alpha[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[h], mx[h]);
        m_use[h] = m_new == -INFINITY ? 0.f : m_new;
        alpha[h] = exp2f(m_run[h] - m_use[h]);
        m_run[h] = m_new;
        l_run[h] *= alpha[h];
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float pe = exp2f(s[i][c] - m_use[c >> 1]);
          s[i][c] = pe;
          l_run[c >> 1] += pe;
        }
#pragma unroll
      for (int i = 0; i < NT_O; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
        o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
      // O += P V: one k16 step over the warp's 16 keys
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int nbk = 0; nbk < HD / 16; ++nbk) {
        // transposed loads: (keys 0..7, d nbk*16 + 0..7), (keys 8..15, d), (keys 0..7, d + 8), (keys 8..15, d + 8)
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vs + ((lm & 1) * 8 + lr) * LDS + nbk * 16 + (lm >> 1) * 8);
        mma_bf16(o[2 * nbk], pa, vf[0], vf[1]);
        mma_bf16(o[2 * nbk + 1], pa, vf[2], vf[3]);
      }
    }
    cp_async_wait<0>();
    __syncthreads();     // the stages are free: they now carry the warps' results

    // ---- the four warps' results -> shared memory, merged in warp order
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* red_o = red + (size_t)warp * 16 * HD;
    float* red_ml = red + (size_t)WARPS * 16 * HD + (size_t)warp * 16 * 2;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      red_o[g * HD + i * 8 + 2 * t] = o[i][0];
      red_o[g * HD + i * 8 + 2 * t + 1] = o[i][1];
      red_o[(g + 8) * HD + i * 8 + 2 * t] = o[i][2];
      red_o[(g + 8) * HD + i * 8 + 2 * t + 1] = o[i][3];
    }
    if (t == 0) {
      red_ml[g * 2] = m_run[0]; red_ml[g * 2 + 1] = l_run[0];
      red_ml[(g + 8) * 2] = m_run[1]; red_ml[(g + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < heads * HD; idx += WARPS * 32) {
      const int r = idx / HD, d = idx % HD;
      const float* ml = red + (size_t)WARPS * 16 * HD;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m = fmaxf(m, ml[(w * 16 + r) * 2]);
      float v = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float mw = ml[(w * 16 + r) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
        v = fmaf(red[((size_t)w * 16 + r) * HD + d], f, v);
        l = fmaf(ml[(w * 16 + r) * 2 + 1], f, l);
      }
      const int head = kvh * G + g0 + r;
      a.part_o[(((size_t)e * a.nh + head) * a.max_splits + split) * HD + d] = v;
      if (d == 0) {
        float* pml = a.part_ml + (((size_t)e * a.nh + head) * a.max_splits + split) * 2;
        pml[0] = m;
        pml[1] = l;
      }
    }
    __syncthreads();     // before the next pass overwrites the stages
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
    const int gh = item_idx / DS, d = (item_idx % DS) * 32 + lane;
    const int head = kvh * G + gh;
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
    float acc = 0.f;
    const int first = min(n_splits, 32);
#pragma unroll 4
    for (int s = 0; s < first; ++s) {
      const float f = __shfl_sync(0xffffffffu, w_lane, s);
      if (d < HD) acc = fmaf(__ldcg(po + (size_t)s * HD + d), f, acc);
    }
    for (int s = 32; s < n_splits; ++s) {
      const float f = exp2f(__ldcg(ml + 2 * s) - m);
      if (d < HD) acc = fmaf(__ldcg(po + (size_t)s * HD + d), f, acc);
    }
    if (d < HD) a.out[(size_t)row * a.nh * HD + (size_t)head * HD + d] = __float2bfloat16_rn(acc * inv);
  }
}

constexpr size_t SMEM_BYTES = (size_t)(16 + STAGES * 2 * BK) * LDS * sizeof(__nv_bfloat16);
static_assert((size_t)WARPS * 16 * HD * 4 + WARPS * 16 * 2 * 4 <= (size_t)STAGES * 2 * BK * LDS * 2,
              "the warps' results must fit into the stages");

}  // namespace

// Scratch of the kernel for n_dec decode entries: floats for the partial results; and n_dec * nkv
// ints for the arrival counters (zero before the first launch; the kernel leaves them zero).
MI_API long long mi_attention_decode_scratch_floats(int n_dec, int nh, int max_splits) {
  return (long long)n_dec * nh * max_splits * (HD + 2);
}

MI_API int mi_attention_decode_bf16(void* out, const void* q_base, int q_stride, const void* kv_layer,
                                    const int* block_table, int bt_stride, const int* decode_items,
                                    const int* q_start, const int* ctx_len, const int* seq_slot, float* scratch,
                                    int* counters, int n_dec, int nh, int nkv, int page_size, float scale,
                                    int window, int chunk, int max_splits, cudaStream_t stream) {
  MI_REQUIRE(n_dec >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(chunk >= BK && chunk <= MAX_CHUNK && chunk % BK == 0, "attention_decode: chunk=%d must be a multiple of %d up to %d", chunk, BK, MAX_CHUNK);
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
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window; a.chunk = chunk; a.max_splits = max_splits;
  a.scale = scale;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(decode_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (err != cudaSuccess) return mi_fail("attention_decode: cannot get %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  mi::launch(decode_split_kernel, dim3(dim3(nkv, max_splits, n_dec)), dim3(WARPS * 32), SMEM_BYTES, stream, a);
  MI_LAUNCH_OK("attention_decode");
  return 0;
}
