// Prefill attention over the paged cache in bf16 on the tensor cores: portions of prompts (any
// number of new tokens at any offset) against all keys of their request that the mask allows.
//
// A block of four warps owns 64 query rows of one request and one query head (a "tile" of the
// step's work list); each warp owns 16 rows.  It walks the keys in blocks of 64: K and V rows are
// gathered page by page into shared memory with cp.async (two stages: the next block loads while
// this one is multiplied), S = Q K^T and O += P V run as mma.m16n8k16 (bf16 in, fp32 accumulate),
// softmax is the online form in float32 with exp2 and the scale folded in, P is rounded to bf16
// for the second product.  Causal and window masks are applied by absolute position, so a portion
// that starts in the middle of a prompt sees the cached keys before it.
//
// Shared-memory rows are padded by 16 bytes; with head sizes that are multiples of 16 the row
// stride is an odd number of 16-byte units, which keeps the 8-row ldmatrix reads free of bank
// conflicts at every head size.
//
// Stands where the reference calls flash_attn_varlen_func / FlashInfer's prefill wrapper
// (miniinfer/layers/attention_backend/flashattention_backend.py:441-452,
// flashinfer_backend.py:352-374).
//
// Compiled once per head size: -DMI_HEAD_DIM=<multiple of 16, 16..256>.
#include "common.cuh"

#ifndef MI_HEAD_DIM
#error "compile with -DMI_HEAD_DIM=<head size>"
#endif

MI_DEFINE_LAST_ERROR()

namespace {

constexpr int HD = MI_HEAD_DIM;
constexpr int BQ = 64;            // query rows of a tile
constexpr int BK = 64;            // keys of a block
constexpr int WARPS = 4;
constexpr int LDS = HD + 8;       // shared-memory row stride in elements
constexpr int CHUNKS = HD / 8;    // 16-byte chunks of a row
constexpr int KSTEPS = HD / 16;   // k16 steps of Q K^T
constexpr int NT_S = BK / 8;      // n8 tiles of S
constexpr int NT_O = HD / 8;      // n8 tiles of O
constexpr bool Q_IN_REGS = HD <= 128;

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

struct PrefillArgs {
  __nv_bfloat16* out;            // [T, nh * HD]
  const __nv_bfloat16* q_base;   // fused QKV rows; q first
  int q_stride;
  const __nv_bfloat16* kv_layer; // [page, 2, nkv, P, HD]
  const int* block_table;
  int bt_stride;
  const int* tiles;              // [n_tiles, 2]: item, first row of the tile within the item's new tokens
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  const int* seq_slot;
  int nh, nkv, page_size, window;
  float scale_log2;              // scale * log2(e)
};

// Gathers keys kb*BK .. kb*BK+BK of one kv head (K and V) into a stage; rows past `last_key` are zeros.
__device__ __forceinline__ void load_kv_block(__nv_bfloat16* ks, __nv_bfloat16* vs, const PrefillArgs& a, const int* bt,
                                              size_t page_elems, size_t head_off, size_t v_off, int kb, int last_key) {
  for (int idx = threadIdx.x; idx < BK * CHUNKS; idx += WARPS * 32) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const int j = kb * BK + r;
    const bool valid = j <= last_key;
    const __nv_bfloat16* src = a.kv_layer;
    if (valid) {
      const int page = bt[j / a.page_size];
      src = a.kv_layer + (size_t)page * page_elems + head_off + (size_t)(j % a.page_size) * HD + c * 8;
    }
    cp_async16(ks + r * LDS + c * 8, src, valid);
    cp_async16(vs + r * LDS + c * 8, valid ? src + v_off : src, valid);
  }
}

__global__ void __launch_bounds__(WARPS * 32)
attention_prefill_kernel(PrefillArgs a) {
  mi::grid_dependency_sync();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [BQ][LDS]
  __nv_bfloat16* kbuf = qs + BQ * LDS;                              // [2][BK][LDS]
  __nv_bfloat16* vbuf = kbuf + 2 * BK * LDS;                        // [2][BK][LDS]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int item = a.tiles[2 * blockIdx.x], off = a.tiles[2 * blockIdx.x + 1];
  const int head = blockIdx.y;
  const int kvh = head / (a.nh / a.nkv);
  const int n_new = a.q_len[item];
  const int rows = min(BQ, n_new - off);
  const int row0 = a.q_start[item] + off;
  const int p0 = a.ctx_len[item] - n_new + off;           // position of the tile's first row
  const int p_last = p0 + rows - 1;
  const int lo_tile = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
  const int kb_begin = lo_tile / BK, kb_end = p_last / BK;   // inclusive
  const int* bt = a.block_table + (size_t)a.seq_slot[item] * a.bt_stride;
  const size_t page_elems = (size_t)2 * a.nkv * a.page_size * HD;
  const size_t head_off = (size_t)kvh * a.page_size * HD;
  const size_t v_off = (size_t)a.nkv * a.page_size * HD;

  // Q tile -> shared memory (rows past the portion are zeros), with the first K/V block behind it
  for (int idx = threadIdx.x; idx < BQ * CHUNKS; idx += WARPS * 32) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool valid = r < rows;
    const __nv_bfloat16* src = valid ? a.q_base + (size_t)(row0 + r) * a.q_stride + (size_t)head * HD + c * 8 : a.q_base;
    cp_async16(qs + r * LDS + c * 8, src, valid);
  }
  load_kv_block(kbuf, vbuf, a, bt, page_elems, head_off, v_off, kb_begin, p_last);
  cp_async_commit();

  uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int pr[2] = {p0 + warp * 16 + g, p0 + warp * 16 + g + 8};    // positions of this thread's two rows
  const bool row_ok[2] = {warp * 16 + g < rows, warp * 16 + g + 8 < rows};

  // ldmatrix lane addressing: lane l gives the row address of 8x8 matrix l/8, row l%8
  const int lm = lane >> 3, lr = lane & 7;
  const __nv_bfloat16* q_lane = qs + (warp * 16 + (lm & 1) * 8 + lr) * LDS + (lm >> 1) * 8;

  for (int kb = kb_begin; kb <= kb_end; ++kb) {
    const int stage = (kb - kb_begin) & 1;
    __nv_bfloat16* ks = kbuf + stage * BK * LDS;
    __nv_bfloat16* vs = vbuf + stage * BK * LDS;
    if (kb < kb_end) {
      load_kv_block(kbuf + (stage ^ 1) * BK * LDS, vbuf + (stage ^ 1) * BK * LDS, a, bt, page_elems, head_off, v_off, kb + 1, p_last);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (Q_IN_REGS && kb == kb_begin) {
#pragma unroll
      for (int k = 0; k < (Q_IN_REGS ? KSTEPS : 1); ++k) ldmatrix_x4(qf[k], q_lane + k * 16);
    }

    // S = Q K^T for this warp's 16 rows and the block's 64 keys
    float s[NT_S][4];
#pragma unroll
    for (int i = 0; i < NT_S; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
      uint32_t qa[4];
      if (Q_IN_REGS) {
#pragma unroll
        for (int c = 0; c < 4; ++c) qa[c] = qf[Q_IN_REGS ? k : 0][c];
      } else {
        ldmatrix_x4(qa, q_lane + k * 16);
      }
#pragma unroll
      for (int nb = 0; nb < BK / 16; ++nb) {
        // matrices: (keys nb*16 + 0..7, d k*16 + 0..7), (same keys, d + 8), (keys + 8, d), (keys + 8, d + 8)
        uint32_t kf[4];
        ldmatrix_x4(kf, ks + (nb * 16 + (lm >> 1) * 8 + lr) * LDS + k * 16 + (lm & 1) * 8);
        mma_bf16(s[2 * nb], qa, kf[0], kf[1]);
        mma_bf16(s[2 * nb + 1], qa, kf[2], kf[3]);
      }
    }

    // mask by absolute position, online softmax in float32 (base 2, scale folded in)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < NT_S; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = kb * BK + i * 8 + 2 * t + (c & 1);
        const int h = c >> 1;
        const bool see = row_ok[h] && j <= pr[h] && (a.window <= 0 || j > pr[h] - a.window);
        const float v = see ? s[i][c] * a.scale_log2 : -INFINITY;
        s[i][c] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;       // a row that has seen no key yet
      alpha[h] = exp2f(m_run[h] - m_use[h]);              // exp2(-inf) = 0 on the first block
      m_run[h] = m_new;
      l_run[h] *= alpha[h];
    }
#pragma unroll
    for (int i = 0; i < NT_S; ++i)
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

    // O += P V
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nb = 0; nb < HD / 16; ++nb) {
        // transposed loads: (keys kk*16 + 0..7, d nb*16 + 0..7), (keys + 8, d), (keys, d + 8), (keys + 8, d + 8)
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vs + (kk * 16 + (lm & 1) * 8 + lr) * LDS + nb * 16 + (lm >> 1) * 8);
        mma_bf16(o[2 * nb], pa, vf[0], vf[1]);
        mma_bf16(o[2 * nb + 1], pa, vf[2], vf[3]);
      }
    }
    __syncthreads();   // everyone is done with this stage before the next load overwrites it
  }

  // finish: row sums across the quad, normalise, store
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!row_ok[h]) continue;
    const float inv = 1.f / l_run[h];
    __nv_bfloat16* dst = a.out + (size_t)(row0 + warp * 16 + g + 8 * h) * a.nh * HD + (size_t)head * HD;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      const uint32_t v = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = v;
    }
  }
}

}  // namespace

MI_API int mi_attention_head_dim() { return HD; }

MI_API int mi_attention_prefill_bf16(void* out, const void* q_base, int q_stride, const void* kv_layer,
                                     const int* block_table, int bt_stride, const int* tiles, int n_tiles,
                                     const int* q_start, const int* q_len, const int* ctx_len, const int* seq_slot,
                                     int nh, int nkv, int page_size, float scale, int window, cudaStream_t stream) {
  MI_REQUIRE(n_tiles >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_prefill: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(page_size > 0 && q_stride % 8 == 0, "attention_prefill: bad page_size=%d or q_stride=%d", page_size, q_stride);
  MI_REQUIRE(nh <= 65535, "attention_prefill: too many heads for one launch");
  if (n_tiles == 0) return 0;
  PrefillArgs a;
  a.out = (__nv_bfloat16*)out;
  a.q_base = (const __nv_bfloat16*)q_base;
  a.q_stride = q_stride;
  a.kv_layer = (const __nv_bfloat16*)kv_layer;
  a.block_table = block_table;
  a.bt_stride = bt_stride;
  a.tiles = tiles;
  a.q_start = q_start; a.q_len = q_len; a.ctx_len = ctx_len; a.seq_slot = seq_slot;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  const size_t smem = (size_t)(BQ + 4 * BK) * LDS * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return mi_fail("attention_prefill: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  mi::launch(attention_prefill_kernel, dim3(dim3(n_tiles, nh)), dim3(WARPS * 32), smem, stream, a);
  MI_LAUNCH_OK("attention_prefill");
  return 0;
}
