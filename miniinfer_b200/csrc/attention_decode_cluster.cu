// Decode attention over the paged cache in bf16 for steps with little to read - a few requests, or
// short contexts - where the time of the persistent kernel (attention_decode_tma.cu) is not the
// bytes but what surrounds them: a work list to walk, partial results that travel through L2 to
// whichever block arrives last (a request of 2048 tokens alone: 15 us for 8 MB; of 60 tokens: 9 us).
// The same tiles, the same tile computation (attention_decode_tile.cuh), another schedule:
//
//   * one block per (request, kv head, piece of the key tiles); the blocks that share a (request,
//     kv head) are a thread-block cluster (1 to 16 blocks) and take equal runs of 64-key tiles;
//   * what a block needs to know it reads before it waits for its predecessor: the request's length
//     and row, and its tiles' pages from the block table, into shared memory.  After the wait one
//     thread asks the TMA engine for the block's tiles - all of them at once if the ring of stages
//     holds them, so that the step's whole cache is in flight after one round trip;
//   * four warps take tiles in turn (tile t to warp t mod 4) and compute them on the tensor cores;
//     their (max, sum, weighted values) are merged in shared memory in the order of the tiles, and
//     the blocks of a cluster are merged through distributed shared memory: every block leaves its
//     result in its own shared memory, the cluster meets at its hardware barrier, and each block
//     combines a slice of the output rows from all of them.  Nothing goes through global memory but
//     the output; there are no counters, and no block waits in a loop for another;
//   * for a step of decode tokens only (head size 128) the kernel also does what otherwise a kernel of
//     its own does before it - the QK norm, the rotation, the new token's key and value into the cache
//     (mi_attention_decode_cluster_rope): 2.4 us a layer less at the Qwen3-0.6B shape;
//   * every wait on a copy's mbarrier is bounded: one that runs out raises a flag that ends the
//     block's other waits, sets the status word, and the block runs to its end.
//
// (Tried and dropped: letting this kernel ask for the weights that the step's next kernels stream - the output
// product, the feed-forward's matrices, the next layer's QKV matrix, 31 MB at the Qwen3-0.6B shape - into L2 with
// cp.async.bulk.prefetch.L2 while it runs.  The prefetches compete with the kernel's own copies and the products
// gain less than that costs: a batch-1 decode step took 0.80 ms with them against 0.73 ms without, a batch-8 step
// 1.00 ms against 0.99 ms, whether they were issued before or behind the block's own copies.)
//
// Page sizes and head sizes that are multiples of 64 (the tiles' geometry); up to 8 query heads per kv
// head.  The sums of a request are added in an order that depends on the cluster size, which the
// launcher chooses from the number of requests: outputs vary with the batch by rounding, as the
// bf16 path allows.
//
// Stands where the reference calls FlashInfer's / FlashAttention's decode kernels
// (miniinfer/layers/attention_backend/flashinfer_backend.py:323-327).
//
// Compiled once per head size: -DMI_HEAD_DIM=<multiple of 16, 16..256>.
#include <cooperative_groups.h>
#include <string.h>

#include "common.cuh"
#include "qk_rope_math.cuh"

#ifndef MI_HEAD_DIM
#error "compile with -DMI_HEAD_DIM=<head size>"
#endif

#if MI_HEAD_DIM % 64 == 0

#include "attention_decode_tile.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int CW = 4;                        // warps that compute
constexpr int CTHREADS = (CW + 1) * 32;      // + the warp that asks for the copies
constexpr int CMAX_STAGES = 8;
constexpr int ROW = HD + 2;                  // a head's partial result: HD weighted values, max, sum
constexpr int GP = 8;                        // heads per kv head the tile computation is laid out for
constexpr int MAX_CLUSTER = 16;
// What the blocks of a cluster send each other at the end: a block's share of every block's output sums (G x HD
// values over the cluster, rounded up per block) and every block's maximum and sum per head.
constexpr int RECV_FLOATS = GP * HD + MAX_CLUSTER * (2 * GP + 1);

struct ClusterArgs {
  __nv_bfloat16* out;              // [T, nh * HD]
  const __nv_bfloat16* q_base;     // fused QKV rows; q first
  int q_stride;
  const int* block_table;
  int bt_stride;
  const int* decode_items;         // the items that bring one token (null: all of the step's items do)
  const int* q_start;
  const int* ctx_len;
  const int* seq_slot;
  int* status;
  int nh, nkv, page_size, window, stages, max_tiles;
  float scale;
  // The step before attention - QK norm, rotation, the new token's K and V into the cache - done here (head size 128):
  int rope;                        // 0: the rows of q_base are normed and rotated and the cache holds the new token
  const float* q_w;                // norm weights [HD] (null: no norm)
  const float* k_w;
  const float* cos_sin;            // [position][cos 0..HD/2 | sin 0..HD/2] (null: no rotation)
  const int* slot_mapping;         // per row of the step: page * page_size + offset of the token's cache entry (null: no store)
  __nv_bfloat16* kv_layer;         // the layer's cache, [page][2][kv head][token][HD]
  float eps;
};

__global__ void __launch_bounds__(CTHREADS, 1)
decode_cluster_kernel(const __grid_constant__ CUtensorMap kv_map, ClusterArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the swizzle pattern is a function of the address: the tiles start on a 1024-byte boundary
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // [stages][K tile, V tile] | recv [RECV_FLOATS] | red [CW][GP][ROW] | barriers | pages [max_tiles] | flag
  unsigned char* stage0 = smem;
  float* recv = reinterpret_cast<float*>(smem + (size_t)a.stages * STAGE_BYTES);   // [block of the cluster][its sums of my slice | max, sum per head]
  float* red = recv + RECV_FLOATS;
  uint64_t* full = reinterpret_cast<uint64_t*>(red + CW * GP * ROW);
  uint64_t* empty = full + CMAX_STAGES;
  uint64_t* patched = empty + CMAX_STAGES;                       // rope: the new token's key and value are in the last tile
  int* pages = reinterpret_cast<int*>(patched + 1);
  volatile int* abort = pages + a.max_tiles;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(pages + ((a.max_tiles + 4 + 3) & ~3));   // [GP][HD]: the query heads, normed and rotated here (rope)

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int C = (int)gridDim.x, r = (int)blockIdx.x, kvh = (int)blockIdx.y, e = (int)blockIdx.z;
  const int G = a.nh / a.nkv;
  // The blocks of a cluster write into one another's shared memory at the end, which needs them all to have
  // started: every thread says so here and waits for the others only then.
  if (C > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(patched, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Read before the wait for the preceding kernel: only what the host uploaded.
  const int item = a.decode_items ? a.decode_items[e] : e;     // null: every item of the step brings one token, in order
  const int p = a.ctx_len[item] - 1;
  const int row = a.q_start[item];
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int j_first = lo / BK * BK;                              // first key of the request's first tile
  const int tiles = (p + 1 - j_first + BK - 1) / BK;
  const int per = (tiles + C - 1) / C;                           // tiles per block
  const int b0 = min(tiles, r * per), b1 = min(tiles, (r + 1) * per);
  const int nb = b1 - b0;
  {
    const int* bt = a.block_table + (size_t)a.seq_slot[item] * a.bt_stride;
    for (int i = threadIdx.x; i < nb && i < a.max_tiles; i += CTHREADS) pages[i] = bt[(j_first + (b0 + i) * BK) / a.page_size];
  }
  // The kernel that norms and rotates q and k and stores the new token's k and v may be this kernel's work (rope):
  // each computing warp then prepares a query head of this kv head in shared memory, and in the block that holds the
  // request's last tile the copying warp puts the new token's key and value into that tile in shared memory once its
  // copy has landed (whatever the cache held at that place), tells the warp that computes the tile, and writes the
  // entry into the cache for the steps to come.
  // The arithmetic is qk_norm_rope_store_fast_kernel's, operation for operation (qk_rope_math.cuh; a lane holds the
  // pairs 2 l and 64 + 2 l of a head), so the step's numbers do not depend on which of the two did it.  The norm
  // weights and the position's row of the table are read here, before the wait: no kernel writes them.
  constexpr int HALF = HD / 2;
  const bool rope = HD == 128 && a.rope != 0;
  const int j = 2 * lane;
  const float2 one = make_float2(1.f, 1.f), zero = make_float2(0.f, 0.f);
  float2 w0 = one, w1 = one, c = one, sn = zero;             // this warp's norm weights (q, or k in the copying warp)
  bool has_table = false;
  if (rope) {
    const float* w = warp == CW ? a.k_w : a.q_w;
    if (w) {
      w0 = *reinterpret_cast<const float2*>(w + j);
      w1 = *reinterpret_cast<const float2*>(w + HALF + j);
    }
    if (a.cos_sin) {
      const float* cs = a.cos_sin + (size_t)max(p, 0) * HD;    // (an item without a token, p = -1, has no tile either)
      c = *reinterpret_cast<const float2*>(cs + j);
      sn = *reinterpret_cast<const float2*>(cs + HALF + j);
      has_table = true;
    }
  }
  auto norm_rotate = [&](const __nv_bfloat16* x, bool normed, uint32_t& ua, uint32_t& ub) {
    const uint32_t r0 = *reinterpret_cast<const uint32_t*>(x + j), r1 = *reinterpret_cast<const uint32_t*>(x + HALF + j);
    float2 va = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r0));
    float2 vb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r1));
    if (normed) {
      const float rstd = mi::rope_rstd(mi::warp_sum(mi::rope_sum_squares(va, vb, 0.f)), HD, a.eps);
      va = mi::rope_scale(va, rstd, w0);
      vb = mi::rope_scale(vb, rstd, w1);
    }
    if (has_table) mi::rope_rotate(va, vb, c, sn);
    const __nv_bfloat162 oa = __floats2bfloat162_rn(va.x, va.y), ob = __floats2bfloat162_rn(vb.x, vb.y);
    ua = *reinterpret_cast<const uint32_t*>(&oa);
    ub = *reinterpret_cast<const uint32_t*>(&ob);
  };
  // this block holds the tile with position p, and the new token's entry is this kernel's to write
  const bool patch = rope && nb > 0 && b1 == tiles && a.slot_mapping != nullptr && a.kv_layer != nullptr;
  auto ask = [&](int b) {                                    // lane 0 of the copying warp
    const int s = b % a.stages;
    mbar_wait(&empty[s], ((b / a.stages) & 1) ^ 1, abort, a.status);
    const int jb = j_first + (b0 + b) * BK;
    const int y_k = ((pages[b] * 2) * a.nkv + kvh) * a.page_size + jb % a.page_size;
    const int y_v = y_k + a.nkv * a.page_size;
    unsigned char* dst = stage0 + (size_t)s * STAGE_BYTES;
    mbar_expect_tx(&full[s], (uint32_t)STAGE_BYTES);
#pragma unroll
    for (int x = 0; x < NBOX; ++x) {
      tma_load_2d(dst + x * BOX_BYTES, &kv_map, x * 64, y_k, &full[s]);
      tma_load_2d(dst + TILE_BYTES + x * BOX_BYTES, &kv_map, x * 64, y_v, &full[s]);
    }
  };
  // When this kernel stores the new token itself, no kernel of the step has written this layer's cache before it:
  // what the cache holds is older than the kernel before the preceding one, which has completed (a kernel lets its
  // successor onto the SMs only after its own wait).  The first tiles - as many as the ring holds - can therefore be
  // asked for before the wait, while the QKV product still runs; the new token's row is put into its tile afterwards.
  // (Worth 0.4 % of a decode step at batch 8 and 0.3 % at batch 1: a block of this kernel gets onto an SM only when the
  // product's block there has left, so little of the product is left to hide the copies behind.)
  __syncthreads();                                           // the barriers and the page numbers are in shared memory
  int asked = 0;
  if (rope && warp == CW && lane == 0)
    for (; asked < nb && asked < a.stages; ++asked) ask(asked);       // the ring is empty: no wait in here
  mi::grid_dependency_sync();

  if (warp == CW) {
    // ------------------------------------------------------------------ the warp that asks for the copies
    if (lane == 0)
      for (; asked < nb && asked < a.stages; ++asked) ask(asked);     // the ring is empty: no wait in here
    const int slot = patch ? a.slot_mapping[row] : -1;
    uint32_t ka = 0u, kb = 0u, va = 0u, vb = 0u;               // this lane's pairs of the new key (normed, rotated) and value
    if (patch && slot >= 0) {
      const __nv_bfloat16* qkv_row = a.q_base + (size_t)row * a.q_stride;
      const __nv_bfloat16* xv = qkv_row + (size_t)(a.nh + a.nkv + kvh) * HD;
      va = *reinterpret_cast<const uint32_t*>(xv + j);
      vb = *reinterpret_cast<const uint32_t*>(xv + HALF + j);
      norm_rotate(qkv_row + (size_t)(a.nh + kvh) * HD, a.k_w != nullptr, ka, kb);
    }
    if (lane == 0)
      for (; asked < nb; ++asked) ask(asked);
    if (patch) {
      // The lanes meet here: a lane that looked at the last tile's barrier before lane 0 had asked for that tile could
      // take an earlier use of the stage - two phases back, the same parity - for it.
      __syncwarp();
      if (slot >= 0) {
        const int last = nb - 1, s = last % a.stages;
        mbar_wait(&full[s], (last / a.stages) & 1, abort, a.status);   // the last tile has landed
        const uint32_t kt = smem_u32(stage0 + (size_t)s * STAGE_BYTES);
        const int rp = p - (j_first + (b0 + last) * BK);       // the new token's row of the tile
        const uint32_t in_chunk = (uint32_t)((lane & 3) * 4);
        auto put = [](uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); };
        put(tile_addr(kt, rp, lane >> 2) + in_chunk, ka);
        put(tile_addr(kt, rp, 8 + (lane >> 2)) + in_chunk, kb);
        put(tile_addr(kt + TILE_BYTES, rp, lane >> 2) + in_chunk, va);
        put(tile_addr(kt + TILE_BYTES, rp, 8 + (lane >> 2)) + in_chunk, vb);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(patched);
      if (slot >= 0) {
        const size_t page = slot / a.page_size, off = slot % a.page_size;
        __nv_bfloat16* dk = a.kv_layer + (((page * 2 + 0) * a.nkv + kvh) * a.page_size + off) * HD;
        __nv_bfloat16* dv = a.kv_layer + (((page * 2 + 1) * a.nkv + kvh) * a.page_size + off) * HD;
        *reinterpret_cast<uint32_t*>(dk + j) = ka;
        *reinterpret_cast<uint32_t*>(dk + HALF + j) = kb;
        *reinterpret_cast<uint32_t*>(dv + j) = va;
        *reinterpret_cast<uint32_t*>(dv + HALF + j) = vb;
      }
    }
  } else {
    // ------------------------------------------------------------------ the warps that compute
    const int g = lane >> 2, t4 = lane & 3;
    const float scale2 = a.scale * 1.4426950408889634f;
    // query fragments straight from the row: head g, dims 16k + 2t.. and + 8
    uint32_t qf[KSTEPS][2];
    {
      const __nv_bfloat16* qrow = a.q_base + (size_t)row * a.q_stride + (size_t)(kvh * G + g) * HD;
      if (rope) {
        const __nv_bfloat16* qkv_row = a.q_base + (size_t)row * a.q_stride;
        for (int h = warp; h < G; h += CW) {                  // a head per warp
          uint32_t ua, ub;
          norm_rotate(qkv_row + (size_t)(kvh * G + h) * HD, a.q_w != nullptr, ua, ub);
          *reinterpret_cast<uint32_t*>(q_s + h * HD + j) = ua;
          *reinterpret_cast<uint32_t*>(q_s + h * HD + HALF + j) = ub;
        }
        asm volatile("bar.sync 2, %0;" ::"n"(CW * 32) : "memory");      // the computing warps have left the query heads in shared memory
        qrow = q_s + (g < G ? g : 0) * HD;
      }
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        const int c0 = k * 16 + 2 * t4;
        qf[k][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + c0) : 0u;
        qf[k][1] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + c0 + 8) : 0u;
      }
    }
    float o[HD / 16][4];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // heads 2t and 2t + 1
    for (int b = warp; b < nb; b += CW) {
      const int s = b % a.stages;
      mbar_wait(&full[s], (b / a.stages) & 1, abort, a.status);
      if (patch && b == nb - 1) mbar_wait(patched, 0, abort, a.status);
      const uint32_t kt = smem_u32(stage0 + (size_t)s * STAGE_BYTES);
      consume_tile(kt, kt + TILE_BYTES, qf, o, m_run, l_run, j_first + (b0 + b) * BK, lo, p + 1, scale2, lane);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    // the warp's sums over the lanes that held different keys, then its result into shared memory
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
    }
    float* mine = red + (size_t)warp * GP * ROW;
#pragma unroll
    for (int i = 0; i < HD / 16; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) mine[(2 * t4 + (c & 1)) * ROW + i * 16 + g + 8 * (c >> 1)] = o[i][c];
    if (g == 0) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        mine[(2 * t4 + c) * ROW + HD] = m_run[c];
        mine[(2 * t4 + c) * ROW + HD + 1] = l_run[c];
      }
    }
  }
  __syncthreads();
  // The warps of the block, in warp order (which is the order of their first tiles).  In a cluster every block then
  // owns a slice of the output values: each block puts its sums of a slice into the owner's shared memory, and its
  // maximum and sum per head into everybody's; one barrier over the cluster later each block finds all it needs
  // at home, combines in rank order and leaves - nobody reads a neighbour's memory after the barrier.
  cg::cluster_group cluster = cg::this_cluster();
  const int total = G * HD;
  const int slice = (total + C - 1) / C;
  const int rs = slice + 2 * GP;                           // floats a block receives from one block
  if (C > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");     // every block of the cluster has started
  for (int idx = threadIdx.x; idx < total; idx += CTHREADS) {
    const int h = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < CW; ++w) M = fmaxf(M, red[((size_t)w * GP + h) * ROW + HD]);
    float L = 0.f, A = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < CW; ++w) {
        const float* src = red + ((size_t)w * GP + h) * ROW;
        const float f = src[HD] == -INFINITY ? 0.f : exp2f(src[HD] - M);
        L = fmaf(src[HD + 1], f, L);
        A = fmaf(src[d], f, A);
      }
    }
    if (C == 1) {
      a.out[(size_t)row * a.nh * HD + (size_t)(kvh * G + h) * HD + d] = __float2bfloat16_rn(A / L);
    } else {
      const int owner = idx / slice;
      cluster.map_shared_rank(recv, owner)[(size_t)r * rs + (idx - owner * slice)] = A;
      if (d == 0) {
        for (int rr = 0; rr < C; ++rr) {
          float* to = cluster.map_shared_rank(recv, rr) + (size_t)r * rs + slice;
          to[2 * h] = M;
          to[2 * h + 1] = L;
        }
      }
    }
  }
  if (C == 1) return;
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

  // the blocks of the cluster, in rank order
  for (int t = threadIdx.x; t < slice && r * slice + t < total; t += CTHREADS) {
    const int idx = r * slice + t;
    const int h = idx / HD, d = idx % HD;
    float M = -INFINITY;
    for (int rr = 0; rr < C; ++rr) M = fmaxf(M, recv[(size_t)rr * rs + slice + 2 * h]);
    float L = 0.f, A = 0.f;
    for (int rr = 0; rr < C; ++rr) {
      const float* src = recv + (size_t)rr * rs;
      const float mr = src[slice + 2 * h];
      if (mr == -INFINITY) continue;
      const float f = exp2f(mr - M);
      L = fmaf(src[slice + 2 * h + 1], f, L);
      A = fmaf(src[t], f, A);
    }
    a.out[(size_t)row * a.nh * HD + (size_t)(kvh * G + h) * HD + d] = __float2bfloat16_rn(A / L);
  }
}

size_t cluster_smem(int stages, int max_tiles) {
  return (size_t)stages * STAGE_BYTES + (size_t)RECV_FLOATS * sizeof(float) + (size_t)CW * GP * ROW * sizeof(float) + (2 * CMAX_STAGES + 1) * 8 +
         (size_t)(max_tiles + 8) * sizeof(int) + (size_t)GP * HD * sizeof(__nv_bfloat16) + 1024;
}

// Stages for blocks of up to `max_tiles` tiles: one per tile if they fit (every copy is then asked for at once and
// no stage is used twice); otherwise a multiple of the number of computing warps, so that a stage always goes to
// the same warp and that warp sees every phase of the stage's barriers (a parity wait cannot tell phases two
// apart: a warp that came to a stage it has never used could take the phase before last for its own).  0: none fits.
int cluster_stages(int max_tiles) {
  int cap = CMAX_STAGES;
  while (cap > 0 && cluster_smem(cap, max_tiles) > 200 * 1024) --cap;
  if (max_tiles <= cap) return max_tiles < 1 ? 1 : max_tiles;
  return cap / CW * CW;
}

}  // namespace

MI_API int mi_attention_decode_cluster_supported() { return 1; }

// How many clusters of `cluster` blocks with `tiles_per_block` stages can be on the GPU at once (0: the size is
// not available).  The launcher's caller picks the largest cluster whose clusters all run together.
MI_API int mi_attention_decode_cluster_fit(int cluster, int tiles_per_block) {
  const int stages = cluster_stages(tiles_per_block);
  if (stages < 1) return 0;
  const size_t smem = cluster_smem(stages, tiles_per_block);
  if (smem > 227 * 1024) return 0;
  if (cudaFuncSetAttribute(decode_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return 0;
  if (cluster > 8 && cudaFuncSetAttribute(decode_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, 1, 1);
  cfg.blockDim = dim3(CTHREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, decode_cluster_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

namespace {
int launch_cluster(void* out, const void* q_base, int q_stride, const void* kv_map,
                   const int* block_table, int bt_stride, const int* decode_items, const int* q_start,
                   const int* ctx_len, const int* seq_slot, int* status, int n_dec, int nh, int nkv,
                   int page_size, float scale, int window, int cluster, int max_ctx_len, cudaStream_t stream,
                   int rope, const float* q_w, const float* k_w, const float* cos_sin, const int* slot_mapping, void* kv_layer, float eps) {
  MI_REQUIRE(n_dec >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode_cluster: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(nh / nkv <= GP, "attention_decode_cluster: at most %d query heads per kv head (got %d)", GP, nh / nkv);
  MI_REQUIRE(cluster >= 1 && cluster <= 16, "attention_decode_cluster: cluster=%d is not in 1..16", cluster);
  MI_REQUIRE(page_size % BK == 0, "attention_decode_cluster: page_size=%d must be a multiple of %d", page_size, BK);
  MI_REQUIRE(q_stride % 8 == 0 && max_ctx_len > 0, "attention_decode_cluster: bad q_stride=%d or max_ctx_len=%d", q_stride, max_ctx_len);
  MI_REQUIRE(n_dec <= 65535 && nkv <= 65535, "attention_decode_cluster: too many entries for one launch");
  MI_REQUIRE(((uintptr_t)q_base % 16) == 0, "attention_decode_cluster: q must be 16-byte aligned");
  if (n_dec == 0) return 0;
  ClusterArgs a;
  a.out = (__nv_bfloat16*)out;
  a.q_base = (const __nv_bfloat16*)q_base;
  a.q_stride = q_stride;
  a.block_table = block_table;
  a.bt_stride = bt_stride;
  a.decode_items = decode_items;
  a.q_start = q_start;
  a.ctx_len = ctx_len;
  a.seq_slot = seq_slot;
  a.status = status;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale = scale;
  a.rope = rope; a.q_w = q_w; a.k_w = k_w; a.cos_sin = cos_sin; a.slot_mapping = slot_mapping;
  a.kv_layer = (__nv_bfloat16*)kv_layer; a.eps = eps;
  MI_REQUIRE(!rope || HD == 128, "attention_decode_cluster: norm and rotation inside the kernel are for head size 128 (got %d)", HD);
  // the most tiles a request can have (a window may start anywhere in its first tile), and a block's share
  const int span = window > 0 && window < max_ctx_len ? window : max_ctx_len;
  const int tiles = (span + BK - 1) / BK + 1;
  a.max_tiles = (tiles + cluster - 1) / cluster;
  const int stages = cluster_stages(a.max_tiles);
  MI_REQUIRE(stages >= 1, "attention_decode_cluster: head size %d with %d tiles per block has no ring of stages that fits", HD, a.max_tiles);
  a.stages = stages;
  const size_t smem = cluster_smem(stages, a.max_tiles);
  MI_REQUIRE(smem <= 227 * 1024, "attention_decode_cluster: shared memory does not suffice (%zu bytes)", smem);
  static bool configured = false, wide = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(decode_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (err != cudaSuccess) return mi_fail("attention_decode_cluster: cannot get shared memory: %s", cudaGetErrorString(err));
    configured = true;
  }
  if (cluster > 8 && !wide) {
    cudaError_t err = cudaFuncSetAttribute(decode_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (err != cudaSuccess) return mi_fail("attention_decode_cluster: clusters of %d blocks are not available: %s", cluster, cudaGetErrorString(err));
    wide = true;
  }
  CUtensorMap map;
  memcpy(&map, kv_map, sizeof(map));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, nkv, n_dec);
  cfg.blockDim = dim3(CTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (mi::pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (cluster > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t err = cudaLaunchKernelEx(&cfg, decode_cluster_kernel, map, a);
  if (err != cudaSuccess) return mi_fail("attention_decode_cluster: launch failed: %s", cudaGetErrorString(err));
  return 0;
}
}  // namespace

// cluster: blocks that share a (request, kv head), 1 .. 16.  max_ctx_len: no request of the step is longer.
MI_API int mi_attention_decode_cluster(void* out, const void* q_base, int q_stride, const void* kv_map,
                                       const int* block_table, int bt_stride, const int* decode_items, const int* q_start,
                                       const int* ctx_len, const int* seq_slot, int* status, int n_dec, int nh, int nkv,
                                       int page_size, float scale, int window, int cluster, int max_ctx_len, cudaStream_t stream) {
  return launch_cluster(out, q_base, q_stride, kv_map, block_table, bt_stride, decode_items, q_start, ctx_len, seq_slot, status, n_dec,
                        nh, nkv, page_size, scale, window, cluster, max_ctx_len, stream, 0, nullptr, nullptr, nullptr, nullptr, nullptr, 0.f);
}

// The same for a step of decode tokens only, with the step before attention inside (head size 128, the whole head
// rotated): q_base holds the raw QKV rows; q and k are normed (weights, or null) and rotated (table [position][128], or
// null) as qk_norm_rope_store does, and the new token's k and v go into the cache at slot_mapping[row] (null: no store).
MI_API int mi_attention_decode_cluster_rope(void* out, const void* qkv, int q_stride, const void* kv_map,
                                            const int* block_table, int bt_stride, const int* decode_items, const int* q_start,
                                            const int* ctx_len, const int* seq_slot, int* status, int n_dec, int nh, int nkv,
                                            int page_size, float scale, int window, int cluster, int max_ctx_len,
                                            const float* q_w, const float* k_w, const float* cos_sin, const int* slot_mapping,
                                            void* kv_layer, float eps, cudaStream_t stream) {
  return launch_cluster(out, qkv, q_stride, kv_map, block_table, bt_stride, decode_items, q_start, ctx_len, seq_slot, status, n_dec,
                        nh, nkv, page_size, scale, window, cluster, max_ctx_len, stream, 1, q_w, k_w, cos_sin, slot_mapping, kv_layer, eps);
}

#else  // head sizes that are not multiples of 64 have no TMA tiles

MI_API int mi_attention_decode_cluster_supported() { return 0; }
MI_API int mi_attention_decode_cluster_fit(int, int) { return 0; }
MI_API int mi_attention_decode_cluster(void*, const void*, int, const void*, const int*, int, const int*, const int*, const int*,
                                       const int*, int*, int, int, int, int, float, int, int, int, cudaStream_t) {
  return mi_fail("attention_decode_cluster: head size %d has no such kernel", MI_HEAD_DIM);
}
MI_API int mi_attention_decode_cluster_rope(void*, const void*, int, const void*, const int*, int, const int*, const int*, const int*,
                                            const int*, int*, int, int, int, int, float, int, int, int, const float*, const float*,
                                            const float*, const int*, void*, float, cudaStream_t) {
  return mi_fail("attention_decode_cluster: head size %d has no such kernel", MI_HEAD_DIM);
}

#endif
