// Decode attention over the paged cache in bf16, fed by TMA: the kernel for page sizes that are
// multiples of 64 and head sizes that are multiples of 64 (the other sizes take the cp.async kernel
// of attention_decode.cu, which computes the same thing).
//
// Reading K and V once from HBM is all the time this kernel should take, and at B200's bandwidth
// per SM that leaves no room for per-thread copy instructions or for blocks that start and stop:
//   * one persistent block per SM; the step's 64-key tiles - all (request, kv head, tile) triples -
//     are dealt out evenly over the blocks, so every block reads the same number of bytes;
//   * a producer warp asks the TMA engine for 64-key tiles of K and V - one tensor copy per
//     64 x 64-element box, written to shared memory in the 128-byte swizzle that makes the later
//     ldmatrix reads conflict-free - several tiles ahead, across item boundaries, counted on
//     mbarriers (full / empty per stage);
//   * three consumer warps take tiles in turn; the number of stages is a multiple of three, so a
//     stage always goes to the same warp and that warp sees every phase of the stage's barriers
//     (a parity wait cannot tell phases two apart).  Each warp computes its whole tile on the
//     tensor cores (mma.m16n8k16, bf16 in, fp32 accumulate) with the products transposed:
//     S^T = K Q^T and O^T += V^T P^T, the 16-row operand being keys (or dims of V) and the 8-column
//     operand the query heads that share the kv head.  A decode step has few heads per kv head and
//     many keys; this way the padding is to 8 heads, not 16, and the scores, the exponentials and
//     the accumulators per thread are half of what heads-as-rows needs.  P^T comes from the
//     scores' fragments by an 8x8 transpose inside the warp (movmatrix).  The softmax is online,
//     in float32, base 2 with the scale folded in.  More than 8 heads per kv head: further passes;
//   * at the end of an item the three warps' (max, sum, O) are merged in shared memory in the
//     order of the tiles they took.  If the item is the request's only chunk, that is the output.
//     Otherwise it is written
//     as the chunk's partial result and handed to an epilogue warp, which does what needs round
//     trips through L2 off the consumers' path: it counts the item on a counter per (request, kv
//     head); the block whose count is the last one merges the chunks (the recurrence the reference
//     sketches in flash_decode_splitk.py:76-87,129-146) and writes the output rows.
// Where a request is cut between blocks depends on what else is in the step, so the sums of a
// request are added in an order that varies with the batch: its output varies by rounding, as the
// bf16 path allows (the 32-bit path has its own kernel, whose order is fixed).
//
// (Dealing only three quarters of the tiles out evenly and handing the rest out in runs of two
// tiles from a counter, so that blocks whose copies come in slowly end up with fewer tiles, was
// tried: every further item costs a merge of the three warps and a partial result, which outweighed
// the balance gained - a batch-8 decode step took 1.46 ms against 1.15 ms.  Letting the warp that
// reaches the end of an item last do the merge alone, with two buffers taking turns and no barrier
// among the consumer warps, was tried as well: one warp merges slower than three, 1.143 ms against
// 1.123 ms.)
//
// No block waits for another block.  Inside a block every wait on an mbarrier is bounded: a wait
// that runs out raises a flag in shared memory that ends all later waits at once, sets the status
// word in global memory, and the block runs to its end (its results are then garbage and the host
// raises an error when it reads the status).
//
// Stands where the reference calls FlashInfer's / FlashAttention's decode kernels
// (miniinfer/layers/attention_backend/flashinfer_backend.py:323-327).
//
// Compiled once per head size: -DMI_HEAD_DIM=<multiple of 16, 16..256>.
#include <cuda.h>

#include "common.cuh"

#ifndef MI_HEAD_DIM
#error "compile with -DMI_HEAD_DIM=<head size>"
#endif

#if MI_HEAD_DIM % 64 == 0

#include "attention_decode_tile.cuh"

namespace {

constexpr int CONSUMERS = 3;                 // consumer warps; the number of stages is a multiple of it
constexpr int THREADS = (CONSUMERS + 2) * 32;   // + producer warp + epilogue warp
constexpr int NI = 4;                        // items in flight between producer, consumers and epilogue
constexpr int MAX_STAGES = 12;

struct Item {                                // what the producer tells the consumers about an item
  int nb;                                    // tiles; -1: no more items
  int e, kvh, split, n_splits;
  int j0;                                    // first key of tile 0 (a multiple of 64)
  int k_lo, k_end;                           // keys that count: k_lo <= j < k_end
  int row;                                   // the request's row in the step
  int pad;                                   // keeps the size a multiple of 8 bytes
};

struct Args {
  __nv_bfloat16* out;            // [T, nh * HD]
  const __nv_bfloat16* q_base;   // fused QKV rows; q first
  int q_stride;
  const int* block_table;
  int bt_stride;
  const int* decode_items;
  const int* q_start;
  const int* ctx_len;
  const int* seq_slot;
  float* part_o;                 // [n_dec, nh, max_splits, HD]
  float* part_ml;                // [n_dec, nh, max_splits, 2]
  int* counters;                 // [n_dec, nkv], zero between launches
  int* status;
  int n_dec, nh, nkv, page_size, window, chunk, max_splits, stages, gp;   // gp = min(G, 16)
  float scale;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory"); }
// Barrier of the consumer warps that also tells every one of them whether any passed a true flag.
__device__ __forceinline__ bool consumer_any(bool flag) {
  uint32_t out;
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, 1, %2, q;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(out) : "r"((uint32_t)flag), "n"(CONSUMERS * 32) : "memory");
  return out != 0;
}
__global__ void __launch_bounds__(THREADS, 1)
decode_tma_kernel(const __grid_constant__ CUtensorMap kv_map, Args a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the swizzle pattern is a function of the address: the tiles start on a 1024-byte boundary
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // [stages][K tile, V tile] | q[NI][gp][HD] bf16 | red [4][gp][HD] + [4][gp][2] floats | items[NI] | barriers | flag
  unsigned char* stage0 = smem;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem + (size_t)a.stages * STAGE_BYTES);
  float* red = reinterpret_cast<float*>(q_s + NI * a.gp * HD);
  Item* items = reinterpret_cast<Item*>(red + CONSUMERS * a.gp * (HD + 2));
  uint64_t* full = reinterpret_cast<uint64_t*>(items + NI);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* qfull = empty + MAX_STAGES;     // item described and its queries landed
  uint64_t* qempty = qfull + NI;            // consumers and epilogue are done with the item's slot
  uint64_t* efull = qempty + NI;            // the item's partial results are written
  volatile int* abort = reinterpret_cast<volatile int*>(efull + NI);
  float* merge_s = reinterpret_cast<float*>(efull + NI) + 4;   // [gp][max_splits][2]: the epilogue warp's scratch
  int* prefix_s = reinterpret_cast<int*>(merge_s + a.gp * a.max_splits * 2);   // [n_dec + 1]: tiles before each request

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = a.nh / a.nkv;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < NI; ++i) {
      mbar_init(&qfull[i], 1);
      mbar_init(&qempty[i], CONSUMERS + 1);
      mbar_init(&efull[i], 1);
    }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Before this kernel waits for its predecessor it reads only what the host uploaded (lengths, the
  // list of decode entries): the producer warp counts the tiles of every request into a prefix array.
  if (warp == CONSUMERS) {
    int carry = 0;
    for (int base = 0; base < a.n_dec; base += 32) {
      const int e = base + lane;
      int v = 0;
      if (e < a.n_dec) {
        const int p = a.ctx_len[a.decode_items[e]] - 1;
        const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
        v = (p + 1 - lo / BK * BK + BK - 1) / BK;
      }
      int x = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (e < a.n_dec) prefix_s[e] = carry + x - v;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
    if (lane == 0) prefix_s[a.n_dec] = carry;
    __syncwarp();
  }
  __syncthreads();

  if (warp == CONSUMERS) {
    // ------------------------------------------------------------------ producer
    // The step's tiles - all (request, kv head, 64-key tile) triples in that order - are dealt out
    // evenly: block c takes the tiles bound(c) .. bound(c + 1), bound(c) = floor(c * total / blocks).
    // A (request, kv head) that falls into one block is finished there; one that straddles blocks
    // becomes one item in each, with partial results.  The whole warp walks this block's range in
    // step (so that its lanes can fetch a run of page numbers at once); lane 0 alone talks to the
    // barriers and the copy engines.  What describes an item comes from arrays the host uploaded,
    // so the warp works out its first item before it waits for the preceding kernel, whose output
    // (the queries, this step's keys and values) only the copies read.
    bool waited = false;
    const long long total = (long long)prefix_s[a.n_dec] * a.nkv;
    // with fewer tiles than blocks only the first `total` blocks work, one tile each
    const long long nblk = min((long long)gridDim.x, total);
    const long long t_begin = blockIdx.x < nblk ? (long long)blockIdx.x * total / nblk : total;
    const long long t_end = blockIdx.x < nblk ? (long long)(blockIdx.x + 1) * total / nblk : total;
    int it = 0, blk = 0;
    // the request that holds tile t_begin: the last e with prefix[e] * nkv <= t_begin
    int e = 0;
    {
      int lo_e = 0, hi_e = a.n_dec;          // prefix[lo_e] * nkv <= t_begin < prefix[hi_e] * nkv (when the range is not empty)
      while (hi_e - lo_e > 1) {
        const int mid = (lo_e + hi_e) / 2;
        if ((long long)prefix_s[mid] * a.nkv <= t_begin) lo_e = mid; else hi_e = mid;
      }
      e = lo_e;
    }
    for (long long t = t_begin; t < t_end;) {
      while ((long long)prefix_s[e + 1] * a.nkv <= t) ++e;         // skips requests without tiles
      const int nt = prefix_s[e + 1] - prefix_s[e];
      const long long first = (long long)prefix_s[e] * a.nkv;      // the request's first tile
      const int kvh = (int)((t - first) / nt);
      const int b0 = (int)((t - first) % nt);
      const int b1 = (int)min((long long)nt, b0 + (t_end - t));
      const int item = a.decode_items[e];
      const int p = a.ctx_len[item] - 1;
      const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
      const int j_first = lo / BK * BK;
      const int j0 = j_first + b0 * BK;
      const int nb = b1 - b0;
      const int k_lo = max(lo, j0);
      const int k_end = min(p + 1, j_first + b1 * BK);
      const int row = a.q_start[item];
      const int* bt = a.block_table + (size_t)a.seq_slot[item] * a.bt_stride;
      // which blocks share this (request, kv head): those that hold its first and its last tile
      const long long s_first = first + (long long)kvh * nt, s_last = s_first + nt - 1;
      const int c_first = (int)(((s_first + 1) * nblk - 1) / total);
      const int c_last = (int)(((s_last + 1) * nblk - 1) / total);
      const int n_splits = c_last - c_first + 1;
      const int split = (int)blockIdx.x - c_first;

      const int qp = it % NI;
      // asks for the tiles from .. to of this item, 32 page numbers at a time
      auto issue_tiles = [&](int from, int to) {
        for (int c0 = from; c0 < to; c0 += 32) {
          const int page = bt[(j0 + min(c0 + lane, nb - 1) * BK) / a.page_size];
          const int run = min(32, to - c0);
          for (int u = 0; u < run; ++u, ++blk) {
            const int pg = __shfl_sync(0xffffffffu, page, u);
            if (lane == 0) {
              const int s = blk % a.stages;
              mbar_wait(&empty[s], ((blk / a.stages) & 1) ^ 1, abort, a.status);
              const int jb = j0 + (c0 + u) * BK;
              const int y_k = ((pg * 2) * a.nkv + kvh) * a.page_size + jb % a.page_size;
              const int y_v = y_k + a.nkv * a.page_size;
              unsigned char* dst = stage0 + (size_t)s * STAGE_BYTES;
              mbar_expect_tx(&full[s], (uint32_t)STAGE_BYTES);
#pragma unroll
              for (int x = 0; x < NBOX; ++x) {
                tma_load_2d(dst + x * BOX_BYTES, &kv_map, x * 64, y_k, &full[s]);
                tma_load_2d(dst + TILE_BYTES + x * BOX_BYTES, &kv_map, x * 64, y_v, &full[s]);
              }
            }
          }
        }
      };
      if (!waited) {
        // (Asking for the block's first tiles before the wait - they hold only what earlier steps
        // wrote - was tried and made the step slower: the early copies compete with the kernel that
        // is still running.)
        mi::grid_dependency_sync();
        waited = true;
      }
      if (lane == 0) {
        mbar_wait(&qempty[qp], ((it / NI) & 1) ^ 1, abort, a.status);
        Item d;
        d.nb = nb; d.e = e; d.kvh = kvh; d.split = split; d.n_splits = n_splits;
        d.j0 = j0; d.k_lo = k_lo; d.k_end = k_end; d.row = row;
        items[qp] = d;
        // the query heads of this kv head are neighbours in the row: one copy
        mbar_expect_tx(&qfull[qp], (uint32_t)(G * HD * 2));
        bulk_load_1d(q_s + (size_t)qp * a.gp * HD, a.q_base + (size_t)row * a.q_stride + (size_t)kvh * G * HD, (uint32_t)(G * HD * 2), &qfull[qp]);
      }
      issue_tiles(0, nb);
      ++it;
      t += nb;
    }
    if (!waited) mi::grid_dependency_sync();
    // no more items
    if (lane == 0) {
      const int qp = it % NI;
      mbar_wait(&qempty[qp], ((it / NI) & 1) ^ 1, abort, a.status);
      items[qp].nb = -1;
      mbar_arrive(&qfull[qp]);
    }
    return;
  }
  mi::grid_dependency_sync();   // consumers and the epilogue warp: before anything a kernel wrote is read, or anything is written

  if (warp == CONSUMERS + 1) {
    // ------------------------------------------------------------------ epilogue warp
    // Items whose request has several chunks: count the item; the block that counts last merges.
    for (int it = 0;; ++it) {
      const int qp = it % NI;
      mbar_wait(&efull[qp], (it / NI) & 1, abort, a.status);
      const Item d = items[qp];
      if (d.nb < 0 || *abort) break;
      if (d.n_splits > 1) {
        int prev = 0;
        if (lane == 0) {
          __threadfence();                 // the consumers' partial results (ordered before by the barrier) go first
          prev = atomicAdd(&a.counters[d.e * a.nkv + d.kvh], 1);
        }
        prev = __shfl_sync(0xffffffffu, prev, 0);
        const bool last = prev == d.n_splits - 1;
        if (last && lane == 0) a.counters[d.e * a.nkv + d.kvh] = 0;     // ready for the next launch
        if (last) {
          __threadfence();
          // All heads of this kv head at once: every chunk's max and sum go to shared memory, from
          // which the weights follow; the chunks' partial outputs are asked for at the same time.
          constexpr int DS = (HD + 31) / 32;
          const int ns = d.n_splits;
          const float* ml0 = a.part_ml + ((size_t)d.e * a.nh + (size_t)d.kvh * G) * a.max_splits * 2;
          const float* po0 = a.part_o + ((size_t)d.e * a.nh + (size_t)d.kvh * G) * a.max_splits * HD;
          // four chunks of one head's partial output at a time, many loads in flight per lane
          auto load_batch = [&](float (&v)[4][DS], int gh, int sp0) {
            const float* po = po0 + (size_t)gh * a.max_splits * HD;
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
              for (int i = 0; i < DS; ++i) {
                const int dd = i * 32 + lane;
                v[u][i] = (sp0 + u < ns && dd < HD) ? __ldcg(po + (size_t)(sp0 + u) * HD + dd) : 0.f;
              }
          };
          float cur[4][DS], nxt[4][DS];
          // one round trip through L2 for every chunk's max and sum and for the first batch of outputs
          for (int idx = lane; idx < G * ns; idx += 32) {
            const int gh = idx / ns, sp = idx % ns;
            const float2 v = __ldcg(reinterpret_cast<const float2*>(ml0 + ((size_t)gh * a.max_splits + sp) * 2));
            merge_s[2 * idx] = v.x;
            merge_s[2 * idx + 1] = v.y;
          }
          load_batch(cur, 0, 0);
          __syncwarp();
          for (int gh = 0; gh < G; ++gh) {
            float m = -INFINITY;
            for (int sp = lane; sp < ns; sp += 32) m = fmaxf(m, merge_s[2 * (gh * ns + sp)]);
            m = mi::warp_max(m);
            float l = 0.f;
            for (int sp = lane; sp < ns; sp += 32) l = fmaf(merge_s[2 * (gh * ns + sp) + 1], exp2f(merge_s[2 * (gh * ns + sp)] - m), l);
            l = mi::warp_sum(l);
            const float inv = 1.f / l;
            __syncwarp();
            for (int sp = lane; sp < ns; sp += 32) merge_s[2 * (gh * ns + sp)] = exp2f(merge_s[2 * (gh * ns + sp)] - m) * inv;   // the chunk's weight
          }
          __syncwarp();
          // the batches in order (head by head); the next one is on its way while this one is added up
          const int per_head = (ns + 3) / 4;
          float acc[DS];
          for (int bi = 0; bi < G * per_head; ++bi) {
            const int gh = bi / per_head, sp0 = (bi % per_head) * 4;
            if (bi + 1 < G * per_head) load_batch(nxt, (bi + 1) / per_head, ((bi + 1) % per_head) * 4);
            if (sp0 == 0) {
#pragma unroll
              for (int i = 0; i < DS; ++i) acc[i] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float f = sp0 + u < ns ? merge_s[2 * (gh * ns + sp0 + u)] : 0.f;
#pragma unroll
              for (int i = 0; i < DS; ++i) acc[i] = fmaf(cur[u][i], f, acc[i]);
            }
            if (sp0 + 4 >= ns) {
              const int head = d.kvh * G + gh;
#pragma unroll
              for (int i = 0; i < DS; ++i) {
                const int dd = i * 32 + lane;
                if (dd < HD) a.out[(size_t)d.row * a.nh * HD + (size_t)head * HD + dd] = __float2bfloat16_rn(acc[i]);
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
              for (int i = 0; i < DS; ++i) cur[u][i] = nxt[u][i];
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&qempty[qp]);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int g = lane >> 2, t4 = lane & 3;
  const float scale2 = a.scale * 1.4426950408889634f;
  const int gp = a.gp;
  int blk_base = 0;
  for (int it = 0;; ++it) {
    const int qp = it % NI;
    mbar_wait(&qfull[qp], (it / NI) & 1, abort, a.status);
    const Item d = items[qp];
    // all consumer warps take the same decision, or the barriers below would not be met by all
    if (consumer_any(d.nb < 0 || *abort != 0)) {
      if (threadIdx.x == 0) mbar_arrive(&efull[qp]);     // the epilogue warp sees the end as well
      break;
    }

    for (int g0 = 0; g0 < G; g0 += 8) {        // more than 8 heads per kv head: the tiles are walked again
      const int heads = min(8, G - g0);
      // The products are taken transposed, keys as the 16-row operand and the (few) heads as the
      // 8-column one: S^T = K Q^T, O^T = V^T P^T.  Query fragments: head g, dims 16k + 2t.. and + 8.
      uint32_t qf[KSTEPS][2];
      {
        const __nv_bfloat16* qrow = q_s + (size_t)qp * gp * HD + (size_t)(g0 + g) * HD;
#pragma unroll
        for (int k = 0; k < KSTEPS; ++k) {
          const int c0 = k * 16 + 2 * t4;
          qf[k][0] = g < heads ? *reinterpret_cast<const uint32_t*>(qrow + c0) : 0u;
          qf[k][1] = g < heads ? *reinterpret_cast<const uint32_t*>(qrow + c0 + 8) : 0u;
        }
      }
      // o[db][c]: dim db*16 + g + 8*(c/2), head 2t + (c&1)
      float o[HD / 16][4];
#pragma unroll
      for (int i = 0; i < HD / 16; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
      float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // heads 2t and 2t + 1

      // tile gb of this block's stream goes to warp gb mod 3 (it owns the stages gb mod `stages` can be);
      // `rank` is the warp's place among the item's tiles, which fixes the order of the merge
      const int rank = (warp + CONSUMERS - blk_base % CONSUMERS) % CONSUMERS;
      for (int b = rank; b < d.nb; b += CONSUMERS) {
        const int gb = blk_base + b;
        const int s = gb % a.stages;
        if (g0 == 0) mbar_wait(&full[s], (gb / a.stages) & 1, abort, a.status);
        const uint32_t kt = smem_u32(stage0 + (size_t)s * STAGE_BYTES);
        const uint32_t vt = kt + TILE_BYTES;

        consume_tile(kt, vt, qf, o, m_run, l_run, d.j0 + b * BK, d.k_lo, d.k_end, scale2, lane);
        if (g0 + 8 >= G) {           // last pass over this tile: hand the stage back
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);
        }
      }

      // ---- the four warps' results -> shared memory, merged in warp order
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
      }
      float* red_o = red + (size_t)rank * gp * HD;
      float* red_ml = red + (size_t)CONSUMERS * gp * HD;
#pragma unroll
      for (int i = 0; i < HD / 16; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int h = 2 * t4 + (c & 1);
          if (h < heads) red_o[h * HD + i * 16 + g + 8 * (c >> 1)] = o[i][c];
        }
      if (g == 0) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int h = 2 * t4 + c;
          if (h < heads) { red_ml[(rank * gp + h) * 2] = m_run[c]; red_ml[(rank * gp + h) * 2 + 1] = l_run[c]; }
        }
      }
      consumer_sync();
      for (int idx = threadIdx.x; idx < heads * HD; idx += CONSUMERS * 32) {
        const int r = idx / HD, dd = idx % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, red_ml[(w * gp + r) * 2]);
        float v = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) {
          const float mw = red_ml[(w * gp + r) * 2];
          const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
          v = fmaf(red[((size_t)w * gp + r) * HD + dd], f, v);
          l = fmaf(red_ml[(w * gp + r) * 2 + 1], f, l);
        }
        const int head = d.kvh * G + g0 + r;
        if (d.n_splits == 1) {            // the only chunk: this is the output
          a.out[(size_t)d.row * a.nh * HD + (size_t)head * HD + dd] = __float2bfloat16_rn(v / l);
        } else {
          a.part_o[(((size_t)d.e * a.nh + head) * a.max_splits + d.split) * HD + dd] = v;
          if (dd == 0) {
            float* pml = a.part_ml + (((size_t)d.e * a.nh + head) * a.max_splits + d.split) * 2;
            pml[0] = m;
            pml[1] = l;
          }
        }
      }
      consumer_sync();      // red is free again; the results of this pass are written
    }
    blk_base += d.nb;
    // hand the item to the epilogue warp and go on
    if (threadIdx.x == 0) mbar_arrive(&efull[qp]);
    if (lane == 0) mbar_arrive(&qempty[qp]);
  }
}


size_t smem_bytes(int stages, int gp, int max_splits, int n_dec) {
  return (size_t)stages * STAGE_BYTES + (size_t)NI * gp * HD * 2 + (size_t)CONSUMERS * gp * (HD + 2) * 4 + NI * sizeof(Item) +
         (size_t)(2 * MAX_STAGES + 3 * NI) * 8 + 16 + (size_t)gp * max_splits * 2 * 4 + (size_t)(n_dec + 1) * 4 + 1024;
}

}  // namespace

// Describes one layer of the cache - [page, 2, kv head, token, HD] seen as rows of HD elements - to
// the TMA engine: boxes of 64 rows x 64 elements, 128-byte swizzle.  `out_map` receives 128 bytes.
MI_API int mi_kv_tensor_map(void* out_map, const void* kv_layer, long long rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return mi_fail("kv_tensor_map: the driver does not offer cuTensorMapEncodeTiled");
    encode = (EncodeFn)fn;
  }
  MI_REQUIRE(((uintptr_t)kv_layer % 128) == 0, "kv_tensor_map: the cache layer must be 128-byte aligned");
  MI_REQUIRE(rows > 0, "kv_tensor_map: no rows");
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)BK};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv_layer), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mi_fail("kv_tensor_map: cuTensorMapEncodeTiled failed with code %d", (int)r);
  memcpy(out_map, &map, sizeof(map));
  return 0;
}

MI_API int mi_attention_decode_tma_supported() { return 1; }

// counters: n_dec * nkv ints, zero before the first launch; status: one int, 0 until a wait runs out.
MI_API int mi_attention_decode_tma(void* out, const void* q_base, int q_stride, const void* kv_map,
                                   const int* block_table, int bt_stride, const int* decode_items, const int* q_start,
                                   const int* ctx_len, const int* seq_slot, float* scratch, int* counters, int* status,
                                   int n_dec, int nh, int nkv, int page_size, float scale, int window, int chunk,
                                   int max_splits, int num_sms, cudaStream_t stream) {
  MI_REQUIRE(n_dec >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode_tma: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(page_size % BK == 0, "attention_decode_tma: page_size=%d must be a multiple of %d", page_size, BK);
  MI_REQUIRE(chunk >= BK && chunk % BK == 0, "attention_decode_tma: chunk=%d must be a multiple of %d", chunk, BK);
  MI_REQUIRE(max_splits >= 1 && max_splits <= 512 && q_stride % 8 == 0, "attention_decode_tma: bad max_splits=%d (1..512) or q_stride=%d", max_splits, q_stride);
  MI_REQUIRE(((uintptr_t)q_base % 16) == 0, "attention_decode_tma: q must be 16-byte aligned");
  MI_REQUIRE(num_sms > 0, "attention_decode_tma: num_sms");
  if (n_dec == 0) return 0;
  const int G = nh / nkv;
  MI_REQUIRE(G <= 16, "attention_decode_tma: at most 16 query heads per kv head (got %d)", G);
  Args a;
  a.out = (__nv_bfloat16*)out;
  a.q_base = (const __nv_bfloat16*)q_base;
  a.q_stride = q_stride;
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
  a.n_dec = n_dec; a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window; a.chunk = chunk;
  a.max_splits = max_splits;
  a.gp = G < 16 ? G : 16;
  a.scale = scale;
  int stages = MAX_STAGES;
  while (stages > CONSUMERS && smem_bytes(stages, a.gp, max_splits, n_dec) > 220 * 1024) stages -= CONSUMERS;
  MI_REQUIRE(smem_bytes(stages, a.gp, max_splits, n_dec) <= 227 * 1024, "attention_decode_tma: shared memory does not suffice");
  a.stages = stages;
  const size_t smem = smem_bytes(stages, a.gp, max_splits, n_dec);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (err != cudaSuccess) return mi_fail("attention_decode_tma: cannot get shared memory: %s", cudaGetErrorString(err));
    configured = 227 * 1024;
  }
  CUtensorMap map;
  memcpy(&map, kv_map, sizeof(map));
  MI_REQUIRE(n_dec <= 4096, "attention_decode_tma: at most 4096 decode entries per launch (got %d)", n_dec);
  const int grid = num_sms;
  mi::launch(decode_tma_kernel, dim3(grid), dim3(THREADS), smem, stream, map, a);
  MI_LAUNCH_OK("attention_decode_tma");
  return 0;
}

#else  // head sizes that are not multiples of 64 have no TMA kernel

#include <string.h>

MI_API int mi_attention_decode_tma_supported() { return 0; }
MI_API int mi_kv_tensor_map(void*, const void*, long long) { return mi_fail("kv_tensor_map: head size %d has no TMA kernel", MI_HEAD_DIM); }
MI_API int mi_attention_decode_tma(void*, const void*, int, const void*, const int*, int, const int*, const int*, const int*,
                                   const int*, float*, int*, int*, int, int, int, int, float, int, int, int, int, cudaStream_t) {
  return mi_fail("attention_decode_tma: head size %d has no TMA kernel", MI_HEAD_DIM);
}

#endif
