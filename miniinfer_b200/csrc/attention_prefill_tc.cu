// Prefill attention over the paged cache in bf16 on the fifth-generation tensor cores (tcgen05):
// the kernel for head sizes 64 and 128 and page sizes that are multiples of 64.  The other sizes
// take the mma.sync kernel of attention_prefill.cu, which computes the same thing.
//
// A piece of work is 128 query rows that share one kv head - 128 tokens of one query head, or, when
// the number of query heads per kv head is even, 64 tokens of two neighbouring heads (so K and V are
// read once for both) - and the keys the mask allows, walked in tiles of 128.  Two blocks may also share
// a work of 128 tokens of two neighbouring heads, a head each (a cluster of two, tcgen05 cta_group::2:
// one instruction stream for 256 rows; a block then holds its own Q rows, 64 of a tile's 128 keys and 64
// of the 128 dims of its values, so each SM asks L2 for half the bytes and the ring has four stages
// instead of two; the copies of both blocks count on the first block's barriers, its commits arrive on
// both blocks' barriers, both blocks' softmax warps tell the first block when S is read and P written).
// Blocks are persistent,
// one per SM (a block takes all of an SM's tensor memory): the works are dealt out longest first, in
// rounds that go back and forth over the blocks, and a block's barriers run on from one work to the
// next, so that the next work's Q and first keys are copied and its first S is computed while the
// softmax warps finish the work before.  Within a work:
//   * a producer warp asks the TMA engine for the Q rows once and for K and V tile by tile (boxes
//     of 64 rows x 64 elements, one page and one half of the head size each, written in the
//     128-byte swizzle), two stages each (four in a pair), counted on mbarriers; K and V are counted apart, since
//     K is free again as soon as S is computed;
//   * the key tiles are dealt to two streams, the even and the odd ones.  A stream has four softmax
//     warps, an output accumulator (head size columns of tensor memory), 64 columns for P, and a running
//     maximum and sum per row of its own, as if it were a request with half the keys; the two are merged
//     at the end;
//   * S = Q K^T of every tile goes into ONE buffer of 128 columns.  A softmax thread owns a query row (its
//     lane of tensor memory): it reads the row's 128 scores into registers with one tcgen05.ld and hands
//     the buffer back at once, so the S of the next tile - the other stream's - follows as soon as its K
//     is there, whatever the P V products do.  One thread issues the S products (tcgen05.mma, M = 128,
//     N = 128, K = 16, operands described in shared memory, K-major);
//   * the softmax thread then works in registers: the mask (only in tiles that it touches: the scores a
//     row may not see are set to -inf once), the maximum, the exponentials in float32, base 2 with the
//     scale folded in, the sum, and P in bf16 into the stream's own columns.  The output row stays in
//     tensor memory; it is rescaled there only when a row's maximum moves up by more than 2^8 (until then
//     sums and P are taken against the older maximum, which costs no accuracy in float32 and bf16), and
//     read once at the end;
//   * a second thread issues O += P V (P from tensor memory, V from shared memory, MN-major: dims
//     contiguous, as the cache stores it) when a stream's P is written; tcgen05.commit tells the
//     mbarriers when products are done.  Nothing orders an S behind a P V any more, and the softmax warps
//     of a stream go from one tile to the next without waiting for either;
//   * at the end of a work each thread reads its half of the two streams' output rows with one wait, and
//     the rows go to global memory through shared memory, so that a store of the warp covers whole
//     128-byte lines.
// Causal and window masks go by absolute position.  Rows past the end of the item's tokens are computed on
// whatever the Q copy brought and never stored.
//
// How it got here (2048 tokens of 16 heads of 128, microseconds per launch).  The first forms kept an S buffer per
// stream, with P written over the S it came from: S of a stream's next tile then had to wait for the P V that read
// that P, and a tile's chain S - softmax - P V ran 5000 to 5800 cycles, two such chains interleaved (40.9; with
// persistent blocks 38.5; with the block set up before it waits for its predecessor 37.9).  A timeline of one
// block (clock64 stamps of the issuing thread and the softmax warps) showed what bound it: not a pipe - with the
// exponential replaced by a multiply-add the launch took as long, the tensor cores were busy ~1100 of ~2900 cycles
// a tile - but the chain, and in it the one issuing thread, whose every look at a barrier in shared memory costs
// 350 to 600 cycles while S products read Q and K at the full width of shared memory.  Tried on that form and not
// faster: the scores held in registers by two threads a row (spills at the 96 registers 18 warps leave), one
// arrival per warp on the barriers, the block table read 32 entries at a time by the whole producer warp, the
// next tile's barriers looked at early, an issuing thread per stream (46.2: the streams fall into step), every
// other exponential as a polynomial (45.7), the keys of a block split over two blocks (61).  One thread per row
// with the row in registers (10 warps, 168 registers, no exchange between threads) took 40.6 as it was; what it
// made possible is what counts: the S buffer shared and handed back at once, P in columns of its own (36.8), an
// issuing thread for S and one for P V (36.1), the mask applied once to the scores instead of in both passes - a
// masked tile took 6800 cycles against 2000, one warp per scheduler has nobody to hide its instructions behind -
// (31.5), the epilogue's loads under one wait and its stores through shared memory (30.2).  A tile now takes ~2250
// cycles, of which the tensor cores are busy ~1500: eight products of S and eight of P V at ~95 cycles each, which is
// the rate the library's products reach too (1.5 PFLOP/s while they run).  The rest is the chain again - a stream's
// softmax takes ~2500 cycles from S computed to P written, with two streams the tensor cores wait 500 to 1000 cycles
// before every P V - and it is not the softmax's arithmetic: without the exponential, the maximum, the sum or the
// conversion to bf16 (each left out in turn) a launch takes as long.  Per work there are ~6500 cycles (3.4 us) beside
// the tiles: 3500 until the first scores are there (the work's description three dependent loads deep, the first
// Q and K copies ~1300 cycles each, the first S cold) and 2500 for the merge and the output rows; 8192 tokens of 16
// heads run at 907 TFLOP/s, 2048 at 564.  Measured against this form and not faster: the works' descriptions worked
// out once into shared memory and the page numbers of sixteen tiles kept in the producer warp's registers (31.8
// against 31.1 in a graph of launches), named barriers instead of mbarriers for "S is read" and "P is written"
// (30.5), half of every K and V copy left out (28.8: the copies' latency, ~3000 cycles under load, is part of the
// chain - with two stages the K of tile j + 2 can only be asked for when S of tile j is done, so two tiles cannot
// take less than that latency and an S product, and shared memory has no room for a third stage of K and of V
// beside Q - their bandwidth is not the bound), and pairs of blocks (31.4 at 2048 tokens, 291 against 303
// at 8192, 56.3 against 57.7 at 32 heads): pairs run where a step brings many tokens.  P handed to the P V products
// in two halves of 64 keys, so that the first four products run while the other half is still exponentiated, was
// slower (31.9 against 31.1 at 2048 tokens, 317 against 303 at 8192): a second wait for the stores, a second arrival
// and a second wait of the issuing thread cost more than the earlier start gains.  With an odd number of
// query heads per kv head a block takes 128 tokens of one head from a list of 128-token tiles (41 against 66 us
// on three prompts of 24 heads when half the works of a 64-token list were skipped one by one).
//
// Every wait on an mbarrier is bounded: a wait that runs out raises a flag in shared memory that
// ends all later waits at once and sets the status word, and the block runs to its end, where the
// tensor memory is given back.
//
// Stands where the reference calls flash_attn_varlen_func / FlashInfer's prefill wrapper
// (miniinfer/layers/attention_backend/flashattention_backend.py:441-452,
// flashinfer_backend.py:352-374).
//
// Compiled once per head size: -DMI_HEAD_DIM=<head size>.
#include <cuda.h>
#include <string.h>

#include <type_traits>

#include "common.cuh"

#ifndef MI_HEAD_DIM
#error "compile with -DMI_HEAD_DIM=<head size>"
#endif

#if MI_HEAD_DIM == 64 || MI_HEAD_DIM == 128

namespace {

constexpr int HD = MI_HEAD_DIM;
constexpr int BM = 128;                       // query rows of a block
constexpr int BN = 128;                       // keys of a tile
constexpr int MAX_STAGES = 4;
constexpr int NHALF = HD / 64;                // 64-element (128-byte) halves of a row
constexpr int HALF_BYTES = 128 * 128;         // 128 rows x 128 bytes
constexpr int Q_BYTES = NHALF * HALF_BYTES;
constexpr int K_BYTES = NHALF * HALF_BYTES;   // and V
constexpr int STAGE_BYTES = 2 * K_BYTES;
constexpr int KV_RING_BYTES = 2 * STAGE_BYTES;  // shared memory of the K / V ring: two stages of a block that works alone, four of a block of a pair
constexpr uint32_t PAIR_LEADER_MASK = 0xFEFFFFFFu;   // clears the bit of a shared::cluster address that tells the two blocks of a pair apart
// CTAS: blocks that share a tile's instruction stream (1, or 2 as a cluster - tcgen05 cta_group::2).  A block of a
// pair holds its own 128 query rows, the first or second 64 keys of a K tile and the first or second 64 dims of
// a V tile: half the bytes per tile, so the same shared memory holds twice the stages.
template <int CTAS> struct Ring {
  static constexpr int KEYS = BN / CTAS;                   // keys of a K tile that a block holds
  static constexpr int K_HALF = KEYS * 128;                // one 64-element half of those keys' rows
  static constexpr int K_HELD = NHALF * K_HALF;
  static constexpr int V_HELD = K_BYTES / CTAS;
  static constexpr int STAGE = K_HELD + V_HELD;
  static constexpr int STAGES = KV_RING_BYTES / STAGE;
};
constexpr int STREAMS = 2;                      // the key tiles are dealt to two streams (even, odd) with sums of their own
constexpr int TPR = 1;                          // softmax threads per query row and stream: one, with the whole row of scores in registers
constexpr int SOFTMAX_WARPS = 4 * TPR * STREAMS;
constexpr int PRODUCER_WARP = SOFTMAX_WARPS, MMA_WARP = SOFTMAX_WARPS + 1;
constexpr int PV_WARP = MMA_WARP + 1;             // the thread that issues the P V products (MMA_WARP's issues the S products)
constexpr int THREADS = (SOFTMAX_WARPS + 3) * 32;
constexpr int TMEM_COLS = 512;
// Tensor memory: one S accumulator (128 float32 columns) that the streams take turns at, and per stream 64 columns
// of P (bf16, two keys to a column) and an output accumulator (head size columns).
constexpr int S_COL = 0, P_COL = 128, O_COL = 256;      // S: one buffer both streams take their scores from; stream s: P at P_COL + 64 s, O at O_COL + 128 s
constexpr int WAIT_LIMIT = 1 << 22;
constexpr int OUT_ROW_BYTES = HD;                       // a softmax thread's half of an output row in bf16
constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + KV_RING_BYTES + 256 + (2 * STREAMS * TPR + 2 * STREAMS * (TPR + 1)) * BM * sizeof(float) +
                              (size_t)SOFTMAX_WARPS * 32 * OUT_ROW_BYTES;

struct Args {
  __nv_bfloat16* out;            // [T, nh * HD]
  const int* block_table;
  int bt_stride;
  const int* tiles;              // [n_tiles, 2]: item, first row of the tile within the item's new tokens (multiples of 64, or of 128 when hpt = 1 and nothing is skipped)
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  const int* seq_slot;
  int* status;
  int n_tiles, nh, nkv, page_size, window;
  int hpt;                       // query heads of a block: 1 (128 tokens) or 2 (64 tokens each)
  int hw;                        // query heads of a work: hpt, or 2 x hpt when a pair of blocks shares the work
  int skip_odd;                  // hpt = 1 on a list of 64-token tiles: the tiles that start at an odd multiple of 64 are covered by the tile before
  float scale_log2;              // scale * log2(e)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait.  `abort` is a flag in shared memory: once any wait has run out, all waits return.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort, int* status) {
  const uint32_t addr = smem_u32(bar);
  for (int i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return;
    if ((i & 63) == 63 && *abort) return;
  }
  *abort = 1;
  atomicExch(status, 2);
}
// One look at a barrier, without blocking: has the phase of this parity completed?
__device__ __forceinline__ uint32_t mbar_peek(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// The same from a block of a pair: the bytes are counted on the barrier of the pair's first block.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar) & PAIR_LEADER_MASK) : "memory");
}
template <int CTAS>
__device__ __forceinline__ void tma_load(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  if (CTAS == 1) tma_load_2d(dst, map, x, y, bar);
  else tma_load_2d_pair(dst, map, x, y, bar);
}
// One more arrival on a barrier of the block that issues the products (in a pair: the first block, from either).
template <int CTAS>
__device__ __forceinline__ void mbar_arrive_issuer(uint64_t* bar) {
  if (CTAS == 1) mbar_arrive(bar);
  else asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PAIR_LEADER_MASK) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- tensor memory and tcgen05 (in a pair: the same warp of both blocks allocates, each for its own SM)
template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_in_smem, uint32_t cols) {
  if (CTAS == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_in_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_in_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}
template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  if (CTAS == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
  else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The barrier gets an arrival when all products issued so far by this thread are done; in a pair the barrier at
// the same place in both blocks does.
template <int CTAS>
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  if (CTAS == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
  } else {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
  }
}
// D[tmem] (+)= A[smem] * B[smem], bf16 in, float32 out; one thread issues it for the block, or for the pair
// (A: 128 rows in each block, B: half of its rows in each block, D: 128 rows in each block's tensor memory).
template <int CTAS>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (CTAS == 1) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    const uint32_t z = 0;      // no output lane is masked
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z) : "memory");
  }
}
// The same with A in tensor memory: lane = row, two bf16 of consecutive k to a column.
template <int CTAS>
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (CTAS == 1) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    const uint32_t z = 0;
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z) : "memory");
  }
}
// 16 consecutive columns of this thread's lane, written.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
// 32 consecutive columns of this thread's lane, written.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31]) : "memory");
}
// 32 consecutive columns of this thread's lane (lane = 32 * (warp % 4) + lane of the warp).
__device__ __forceinline__ void tmem_ld32(float (&v)[32], uint32_t taddr) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 128 consecutive columns of this thread's lane - a whole row of S - with one wait.
__device__ __forceinline__ void tmem_ld128(float (&v)[128], uint32_t taddr) {
  uint32_t r[128];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x128.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63,%64,%65,%66,%67,%68,%69,%70,%71,%72,%73,%74,%75,%76,%77,%78,%79,%80,%81,%82,%83,%84,%85,%86,%87,%88,%89,%90,%91,%92,%93,%94,%95,%96,%97,%98,%99,%100,%101,%102,%103,%104,%105,%106,%107,%108,%109,%110,%111,%112,%113,%114,%115,%116,%117,%118,%119,%120,%121,%122,%123,%124,%125,%126,%127}, [%128];\n"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]), "=r"(r[64]), "=r"(r[65]), "=r"(r[66]), "=r"(r[67]), "=r"(r[68]), "=r"(r[69]), "=r"(r[70]), "=r"(r[71]), "=r"(r[72]), "=r"(r[73]), "=r"(r[74]), "=r"(r[75]), "=r"(r[76]), "=r"(r[77]), "=r"(r[78]), "=r"(r[79]), "=r"(r[80]), "=r"(r[81]), "=r"(r[82]), "=r"(r[83]), "=r"(r[84]), "=r"(r[85]), "=r"(r[86]), "=r"(r[87]), "=r"(r[88]), "=r"(r[89]), "=r"(r[90]), "=r"(r[91]), "=r"(r[92]), "=r"(r[93]), "=r"(r[94]), "=r"(r[95]), "=r"(r[96]), "=r"(r[97]), "=r"(r[98]), "=r"(r[99]), "=r"(r[100]), "=r"(r[101]), "=r"(r[102]), "=r"(r[103]), "=r"(r[104]), "=r"(r[105]), "=r"(r[106]), "=r"(r[107]), "=r"(r[108]), "=r"(r[109]), "=r"(r[110]), "=r"(r[111]), "=r"(r[112]), "=r"(r[113]), "=r"(r[114]), "=r"(r[115]), "=r"(r[116]), "=r"(r[117]), "=r"(r[118]), "=r"(r[119]), "=r"(r[120]), "=r"(r[121]), "=r"(r[122]), "=r"(r[123]), "=r"(r[124]), "=r"(r[125]), "=r"(r[126]), "=r"(r[127])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 128; ++i) v[i] = __uint_as_float(r[i]);
}

// Two stretches of this thread's lane, N columns each, with one wait: the two streams' halves of an output row.
template <int N>
__device__ __forceinline__ void tmem_ld_pair(float (&v0)[N], float (&v1)[N], uint32_t a0, uint32_t a1) {
  static_assert(N == 64 || N == 32, "half a head of 128 or of 64");
  uint32_t r[2 * N];
  if constexpr (N == 64) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%128];\n"
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%64,%65,%66,%67,%68,%69,%70,%71,%72,%73,%74,%75,%76,%77,%78,%79,%80,%81,%82,%83,%84,%85,%86,%87,%88,%89,%90,%91,%92,%93,%94,%95,%96,%97,%98,%99,%100,%101,%102,%103,%104,%105,%106,%107,%108,%109,%110,%111,%112,%113,%114,%115,%116,%117,%118,%119,%120,%121,%122,%123,%124,%125,%126,%127}, [%129];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]), "=r"(r[64]), "=r"(r[65]), "=r"(r[66]), "=r"(r[67]), "=r"(r[68]), "=r"(r[69]), "=r"(r[70]), "=r"(r[71]), "=r"(r[72]), "=r"(r[73]), "=r"(r[74]), "=r"(r[75]), "=r"(r[76]), "=r"(r[77]), "=r"(r[78]), "=r"(r[79]), "=r"(r[80]), "=r"(r[81]), "=r"(r[82]), "=r"(r[83]), "=r"(r[84]), "=r"(r[85]), "=r"(r[86]), "=r"(r[87]), "=r"(r[88]), "=r"(r[89]), "=r"(r[90]), "=r"(r[91]), "=r"(r[92]), "=r"(r[93]), "=r"(r[94]), "=r"(r[95]), "=r"(r[96]), "=r"(r[97]), "=r"(r[98]), "=r"(r[99]), "=r"(r[100]), "=r"(r[101]), "=r"(r[102]), "=r"(r[103]), "=r"(r[104]), "=r"(r[105]), "=r"(r[106]), "=r"(r[107]), "=r"(r[108]), "=r"(r[109]), "=r"(r[110]), "=r"(r[111]), "=r"(r[112]), "=r"(r[113]), "=r"(r[114]), "=r"(r[115]), "=r"(r[116]), "=r"(r[117]), "=r"(r[118]), "=r"(r[119]), "=r"(r[120]), "=r"(r[121]), "=r"(r[122]), "=r"(r[123]), "=r"(r[124]), "=r"(r[125]), "=r"(r[126]), "=r"(r[127])
        : "r"(a0), "r"(a1)
        : "memory");
  } else {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(a0), "r"(a1)
        : "memory");
  }
#pragma unroll
  for (int i = 0; i < N; ++i) {
    v0[i] = __uint_as_float(r[i]);
    v1[i] = __uint_as_float(r[N + i]);
  }
}


// Shared-memory operand descriptor, 128-byte swizzle: start address, leading and stride byte offsets
// in 16-byte units, descriptor version 1 (bits 46..47), layout type 2 = 128-byte swizzle (bits 61..63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: float32 accumulator (bits 4..5 = 1), bf16 A and B (bits 7..9
// and 10..12 = 1), B K-major or MN-major (bit 16), N / 8 at bits 17..22, M / 16 at bits 24..28.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// What a block works on at a time: 128 query rows that share one kv head, and the key tiles they see.
struct Work {
  int item, o, head0, kvh, rows_tok, start, p_first, p_last, lo_last, t_begin, n, row0;
  const int* bt;
  bool skip;
};

// Work number w of the step, longest first: all head groups of the last 64-token tile, then of the tile
// before, ...  (Later tiles of a request see more keys.)
__device__ __forceinline__ Work work_of(const Args& a, int w, int rank) {
  Work k;
  const int X = a.nh / a.hw;
  const int tile = a.n_tiles - 1 - w / X;
  k.item = a.tiles[2 * tile];
  k.o = a.tiles[2 * tile + 1];
  k.skip = a.skip_odd && (k.o & 64);                      // the work of the tile before covers these 64 tokens too
  const int G = a.nh / a.nkv;
  k.head0 = (w % X) * a.hw + rank * a.hpt;                // in a pair the second block takes the work's second head
  k.kvh = k.head0 / G;
  const int qlen = a.q_len[k.item], ctx = a.ctx_len[k.item];
  k.start = ctx - qlen;                                   // position of the item's first new token
  const int tok_per_block = BM / a.hpt;
  k.rows_tok = min(tok_per_block, qlen - k.o);            // tokens of this work that exist
  k.p_first = k.start + k.o;
  k.p_last = k.start + k.o + k.rows_tok - 1;
  const int lo_first = a.window > 0 ? max(0, k.p_first - a.window + 1) : 0;
  k.lo_last = a.window > 0 ? max(0, k.p_last - a.window + 1) : 0;
  k.t_begin = lo_first / BN;
  k.n = k.p_last / BN - k.t_begin + 1;                    // key tiles to walk
  k.row0 = a.q_start[k.item] + k.o;                       // the first row in the step
  k.bt = a.block_table + (size_t)a.seq_slot[k.item] * a.bt_stride;
  return k;
}

// The i-th work of block b of `blocks`: the works are dealt out in rounds, back and forth (0 .. blocks-1,
// then blocks-1 .. 0, ...), so that the block that got the longest work of one round gets the shortest of
// the next.  Returns -1 past the end.
__device__ __forceinline__ int nth_work(int i, int b, int blocks, int total) {
  const int w = i * blocks + ((i & 1) ? blocks - 1 - b : b);
  return w < total ? w : -1;
}

template <int CTAS>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, Args a) {
  using R = Ring<CTAS>;
  constexpr int STAGES = R::STAGES;
  const int total_work = (a.nh / a.hw) * a.n_tiles;
  const int blocks = (int)gridDim.x / CTAS, me = (int)blockIdx.x / CTAS;      // pairs (or blocks) and this one's number
  const int rank = CTAS == 1 ? 0 : (int)cluster_rank();                      // place in the pair; its first block issues the products
  const bool leader = rank == 0;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* kv_s = q_s + Q_BYTES;                    // [stage][K, V]
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + KV_RING_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                            // K and V of a tile are counted apart: K is free again
  uint64_t* k_empty = k_full + MAX_STAGES;                // once S is computed, long before P V is
  uint64_t* v_full = k_empty + MAX_STAGES;
  uint64_t* v_empty = v_full + MAX_STAGES;
  uint64_t* s_full = v_empty + MAX_STAGES;                // [stream]: S of the stream's tile is computed
  uint64_t* p_full = s_full + STREAMS;                    // [stream]: its P is written
  uint64_t* o_full = p_full + STREAMS;                    // [stream]: its P V is added to the output row
  uint64_t* q_empty = o_full + STREAMS;                   // the work's last S is computed: the Q rows may be replaced
  uint64_t* o_free = q_empty + 1;                         // the work's output rows are read: the next work's P V may overwrite them
  uint64_t* s_free = o_free + 1;                          // the scores in the S buffer are in their stream's registers: the next S may overwrite them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* fin_l = reinterpret_cast<float*>(bars + 32);     // [2][stream][BM]: at the end of a work, each thread's sum
  float* fin_m = fin_l + 2 * STREAMS * BM;                // [2][stream][BM]: and each stream's maximum (two works take turns)
  unsigned char* out_s = reinterpret_cast<unsigned char*>(fin_l + (2 * STREAMS * TPR + 2 * STREAMS * (TPR + 1)) * BM);   // [softmax warp][32 rows][half a row]: output rows on their way to global memory

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // In a pair the barriers that the issuing threads wait on (Q, K, V copied; S read; P written; output rows read) are
  // the first block's and count both blocks' copies and arrivals; the barriers that copies and softmax warps wait on
  // are each block's own, and a commit of the first block arrives on both.
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_free, SOFTMAX_WARPS * CTAS);
    mbar_init(s_free, 4 * CTAS);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < STREAMS; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 4 * CTAS);
      mbar_init(&o_full[b], 1);
    }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc<CTAS>(tmem_slot, TMEM_COLS);
  if (warp == PRODUCER_WARP && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&q_map)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&kv_map)) : "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync();     // the other block's barriers are set up before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Up to here the block has touched nothing that a kernel writes: set up beside its predecessor in the stream, it
  // also reads the description of its first work (the step's lists, which the host uploaded) so that the roles find
  // it in the cache, and only then waits for the predecessor - the kernel that wrote the Q rows and the cache.
  {
    const int w0 = nth_work(0, me, blocks, total_work);
    if (w0 >= 0) {
      const Work k0 = work_of(a, w0, rank);
      asm volatile("" ::"r"(k0.n), "r"(k0.row0), "l"(k0.bt));
    }
  }
  mi::grid_dependency_sync();

  // A block is persistent: it takes one work after the other.  The barriers' phases run on across works -
  // every role counts the works (Q), the key tiles (the K / V ring) and each stream's tiles (S, P, O) it has
  // seen - so the copies of the next work's Q and first keys, and its first S, are under way while the
  // softmax warps still finish the work before.
  if (warp == PRODUCER_WARP) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int gi = 0, it = 0;                                  // key tiles and works so far
      for (int i = 0;; ++i) {
        const int w = nth_work(i, me, blocks, total_work);
        if (w < 0 || *abort) break;
        const Work k = work_of(a, w, rank);
        if (k.skip) continue;
        mbar_wait(q_empty, (it & 1) ^ 1, abort, a.status);   // the S products of the work before have read the Q rows
        if (leader) mbar_expect_tx(q_full, (uint32_t)(CTAS * Q_BYTES));
#pragma unroll
        for (int rb = 0; rb < 2; ++rb) {
          const int head = k.head0 + (a.hpt == 2 ? rb : 0);
          const int y = k.row0 + (a.hpt == 2 ? 0 : 64 * rb);
#pragma unroll
          for (int h = 0; h < NHALF; ++h)
            tma_load<CTAS>(q_s + h * HALF_BYTES + rb * 64 * 128, &q_map, head * HD + h * 64, y, q_full);
        }
        // K of tile i goes first, then V of tile i - 1: S of the next tile never waits for a V copy
        auto load = [&](int li, bool values) {
          const int g = gi + li;                           // the tile's number among all tiles of this block
          const int s = g % STAGES;
          uint64_t* full = values ? &v_full[s] : &k_full[s];
          mbar_wait(values ? &v_empty[s] : &k_empty[s], ((g / STAGES) & 1) ^ 1, abort, a.status);
          unsigned char* dst = kv_s + (size_t)s * R::STAGE + (values ? R::K_HELD : 0);
          if (leader) mbar_expect_tx(full, (uint32_t)K_BYTES);     // of both blocks of a pair together
          const int key0 = (k.t_begin + li) * BN;
#pragma unroll
          for (int pg = 0; pg < 2; ++pg) {
            if (CTAS == 2 && !values && pg != rank) continue;      // K: a block of a pair holds its 64 keys, all dims
            const int key = key0 + 64 * pg;
            const int page = k.bt[min(key / a.page_size, a.bt_stride - 1)];   // past the context: the dummy page, masked below
            const int y = ((page * 2 + (values ? 1 : 0)) * a.nkv + k.kvh) * a.page_size + key % a.page_size;
#pragma unroll
            for (int h = 0; h < NHALF; ++h) {
              if (CTAS == 2 && values && h != rank) continue;      // V: all 128 keys, its 64 dims
              unsigned char* to = CTAS == 1 ? dst + h * HALF_BYTES + pg * 64 * 128
                                            : (values ? dst + pg * 64 * 128 : dst + h * R::K_HALF);
              tma_load<CTAS>(to, &kv_map, h * 64, y, full);
            }
          }
        };
        for (int step = 0; step <= k.n && !*abort; ++step) {
          if (step < k.n) load(step, false);
          if (step >= 1) load(step - 1, true);
        }
        gi += k.n;
        ++it;
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ the thread that issues S = Q K^T
    // S goes into one buffer of tensor memory that both streams take their scores from: a stream's softmax warps
    // read their row of a tile into registers at once and hand the buffer back, so S of the next tile - of the
    // other stream - can follow as soon as that has happened and its K is copied, whatever the P V products do.
    if (lane == 0 && leader) {
      constexpr uint32_t IDESC_S = instr_desc(BM * CTAS, BN, false);
      const uint64_t q_desc = smem_desc(smem_u32(q_s), 16, 1024);
      auto q_step = [](int ks) { return (uint64_t)((ks >> 2) * (HALF_BYTES >> 4) + (ks & 3) * 2); };
      auto k_step = [](int ks) { return (uint64_t)((ks >> 2) * (R::K_HALF >> 4) + (ks & 3) * 2); };
      int gi = 0, it = 0, s_count = 0;                     // key tiles, works and S products so far
      for (int i = 0;; ++i) {
        const int w = nth_work(i, me, blocks, total_work);
        if (w < 0 || *abort) break;
        const Work k = work_of(a, w, rank);
        if (k.skip) continue;
        const int n = k.n;
        mbar_wait(q_full, it & 1, abort, a.status);
        for (int j = 0; j < n && !*abort; ++j, ++s_count) {
          const int g = gi + j, st_ = g % STAGES;
          const uint32_t k_ready = mbar_peek(&k_full[st_], (g / STAGES) & 1);
          if (s_count > 0) mbar_wait(s_free, (s_count - 1) & 1, abort, a.status);   // the scores before are in registers
          if (!k_ready) mbar_wait(&k_full[st_], (g / STAGES) & 1, abort, a.status);
          if (*abort) break;
          tc_fence_after();
          const uint64_t k_desc = smem_desc(smem_u32(kv_s + (size_t)st_ * R::STAGE), 16, 1024);
          const uint32_t d = tmem_base + S_COL;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            tc_mma<CTAS>(d, q_desc + q_step(ks), k_desc + k_step(ks), IDESC_S, ks > 0 ? 1u : 0u);
          tc_commit<CTAS>(&s_full[j & 1]);
          tc_commit<CTAS>(&k_empty[st_]);
          if (j == n - 1) tc_commit<CTAS>(q_empty);        // the work's last S: the Q rows are free once it is done
        }
        gi += n;
        ++it;
      }
    }
  } else if (warp == PV_WARP) {
    // ------------------------------------------------------------------ the thread that issues O += P V
    if (lane == 0 && leader) {
      constexpr uint32_t IDESC_PV = instr_desc(BM * CTAS, HD, true);
      int gi = 0, it = 0;
      int sb[STREAMS] = {0, 0};                            // tiles of each stream so far
      for (int i = 0;; ++i) {
        const int w = nth_work(i, me, blocks, total_work);
        if (w < 0 || *abort) break;
        const Work k = work_of(a, w, rank);
        if (k.skip) continue;
        const int n = k.n;
        // the output rows in tensor memory are the work before's until its softmax warps have read them
        if (it > 0) mbar_wait(o_free, (it - 1) & 1, abort, a.status);
        for (int j = 0; j < n && !*abort; ++j) {
          const int g = gi + j, st_ = g % STAGES, b = j & 1;
          const uint32_t v_ready = mbar_peek(&v_full[st_], (g / STAGES) & 1);
          mbar_wait(&p_full[b], (sb[b] + j / 2) & 1, abort, a.status);
          if (!v_ready) mbar_wait(&v_full[st_], (g / STAGES) & 1, abort, a.status);
          if (*abort) break;
          tc_fence_after();
          const uint64_t v_desc = smem_desc(smem_u32(kv_s + (size_t)st_ * R::STAGE + R::K_HELD), HALF_BYTES, 1024);
          const uint32_t p_tmem = tmem_base + P_COL + 64 * b;   // lane = row, two keys to a column
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)                   // 16 keys further: 2048 bytes of V
            tc_mma_ts<CTAS>(tmem_base + O_COL + 128 * b, p_tmem + (uint32_t)(8 * ks),
                      v_desc + (uint64_t)(ks * (2048 >> 4)), IDESC_PV,
                      (j >= 2 || ks > 0) ? 1u : 0u);         // the stream's output row is summed over the work's tiles in tensor memory
          tc_commit<CTAS>(&o_full[b]);
          tc_commit<CTAS>(&v_empty[st_]);
        }
        gi += n;
        sb[0] += (n + 1) / 2;
        sb[1] += n / 2;
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax
    // Warp w: tensor-memory lanes 32 (w & 3) .. + 31 (a warp reaches the lanes of its number mod
    // 4), stream st = w >> 2; a thread owns a row.  A stream keeps a maximum, a sum and an output row
    // of its own over its tiles (the even or the odd ones); the two are merged at the end.
    const int q = warp & 3, st = warp >> 2;
    const int r = q * 32 + lane;                           // row of the block = lane of the tensor memory
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
    const float sc = a.scale_log2;
    int o_seen = 0;
    auto wait_o = [&](int upto) {
      while (o_seen <= upto) {
        mbar_wait(&o_full[st], o_seen & 1, abort, a.status);
        ++o_seen;
      }
      tc_fence_after();
    };
    const uint32_t s_addr = t_lane + S_COL;
    const uint32_t p_addr = t_lane + P_COL + 64 * st;
    const uint32_t o_addr = t_lane + O_COL + 128 * st;
    int base = 0, it = 0;                                  // tiles of this stream and works so far

    for (int i = 0;; ++i) {
      const int w = nth_work(i, me, blocks, total_work);
      if (w < 0) break;
      const Work wk = work_of(a, w, rank);
      if (wk.skip) continue;
      const int n = wk.n, start = wk.start, o = wk.o, rows_tok = wk.rows_tok;
      const int p_first = wk.p_first, p_last = wk.p_last, lo_last = wk.lo_last, t_begin = wk.t_begin;
      const int tok = a.hpt == 2 ? (r & 63) : r;
      const int head = wk.head0 + (a.hpt == 2 ? (r >> 6) : 0);
      const bool row_valid = tok < rows_tok;
      const int pos = row_valid ? start + o + tok : p_last;
      const int lo_r = a.window > 0 ? max(0, pos - a.window + 1) : 0;
      float m_run = -INFINITY, l_run = 0.f;
      const int n_mine = (n - st + 1) / 2;                 // tiles of this stream

      for (int k = 0; k < n_mine; ++k) {
        const int j = 2 * k + st;
        const int kk = base + k;
        const int key0 = (t_begin + j) * BN;
        const bool masked = !((t_begin + j) * BN + BN - 1 <= p_first && (t_begin + j) * BN >= lo_last);
        mbar_wait(&s_full[st], kk & 1, abort, a.status);
        tc_fence_after();
        float v[BN];
        tmem_ld128(v, s_addr);
        // the scores are in registers: the S buffer may take the next tile's (of either stream)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_issuer<CTAS>(s_free);
        if (masked) {
          // A tile that the mask touches: the scores a row may not see are set to -inf once, here, and everything
          // after treats the tile like any other (a maximum ignores them, their exponentials are 0).  The visible
          // columns of a row are one stretch, first .. last.
          int first = lo_r - key0, last = pos - key0;
          if (last < first) first = BN + 1;                // none: no column passes the test below
          const unsigned span = (unsigned)(last - first);
#pragma unroll
          for (int e = 0; e < BN; ++e) v[e] = (unsigned)(e - first) <= span ? v[e] : -INFINITY;
        }
        {
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int e = 0; e < BN; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], v[e]);
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          const float m_new = fmaxf(m_run, mx * sc);       // the scale is positive
          const bool move = m_new > m_run + 8.f || m_run == -INFINITY;
          if (__any_sync(0xffffffffu, move)) {
            const float m_next = move ? m_new : m_run;
            const float m_to = m_next == -INFINITY ? 0.f : m_next;
            const float alpha = move ? exp2f(m_run - m_to) : 1.f;
            if (k > 0) {
              wait_o(kk - 1);
#pragma unroll 1
              for (int c = 0; c < HD / 32; ++c) {
                float op[32];
                tmem_ld32(op, o_addr + c * 32);
                uint32_t wv[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) wv[e] = __float_as_uint(op[e] * alpha);
                tmem_st32(o_addr + c * 32, wv);
              }
              asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            l_run *= alpha;
            m_run = m_next;
          }
          const float m_use = m_run == -INFINITY ? 0.f : m_run;
          float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t packed[16];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float x = fmaf(v[32 * c + e], sc, -m_use);     // -inf where the row may not see the key
              float pe;
              asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pe) : "f"(x));
              v[32 * c + e] = pe;
              part[e & 3] += pe;
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) packed[e] = pack_bf16(v[32 * c + 2 * e], v[32 * c + 2 * e + 1]);
            if (c == 0 && kk > 0) wait_o(kk - 1);          // the product that read the stream's P before has run
            tmem_st16(p_addr + 16 * c, packed);            // P: two keys to a column
          }
          l_run += (part[0] + part[1]) + (part[2] + part[3]);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_issuer<CTAS>(&p_full[st]);
      }
      if (n_mine > 0) wait_o(base + n_mine - 1);
      // ---- the two streams' sums are merged: every thread leaves its sum and maximum in shared memory, all
      // softmax warps meet, and each thread finishes half of its row's output
      float* fl = fin_l + (it & 1) * STREAMS * BM;
      float* fm = fin_m + (it & 1) * STREAMS * BM;
      fl[st * BM + r] = l_run;
      fm[st * BM + r] = m_run;
      tc_fence_before();
      asm volatile("bar.sync 9, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
      tc_fence_after();
      const float m0 = fm[r], m1 = fm[BM + r];
      const float m_all = fmaxf(m0, m1);
      const float w0 = m0 == -INFINITY ? 0.f : exp2f(m0 - m_all);
      const float w1 = m1 == -INFINITY ? 0.f : exp2f(m1 - m_all);
      const float l_all = fl[r] * w0 + fl[BM + r] * w1;
      constexpr int OD = HD / 2;                           // output columns of this thread
      const bool has1 = n > 1;
      const float f0 = w0 / l_all, f1 = has1 ? w1 / l_all : 0.f;
      (void)head; (void)row_valid;
      float o0[OD], o1[OD];
      if (has1) {
        tmem_ld_pair<OD>(o0, o1, t_lane + O_COL + st * OD, t_lane + O_COL + 128 + st * OD);
      } else {
        tmem_ld_pair<OD>(o0, o1, t_lane + O_COL + st * OD, t_lane + O_COL + st * OD);
      }
      // the output rows are in registers: the next work's products may overwrite them in tensor memory
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_issuer<CTAS>(o_free);
      // A thread's half row goes through shared memory (16-byte chunks, swizzled by the row), so that a store of
      // the warp covers whole 128-byte lines of four rows instead of 16 bytes of each of 32 rows.
      constexpr int CH = OUT_ROW_BYTES / 16;               // chunks of a half row: 8 (head size 128) or 4
      unsigned char* mine = out_s + (size_t)warp * 32 * OUT_ROW_BYTES;
#pragma unroll
      for (int d = 0; d < OD; d += 8) {
        uint4 wv;
        wv.x = pack_bf16(o0[d] * f0 + o1[d] * f1, o0[d + 1] * f0 + o1[d + 1] * f1);
        wv.y = pack_bf16(o0[d + 2] * f0 + o1[d + 2] * f1, o0[d + 3] * f0 + o1[d + 3] * f1);
        wv.z = pack_bf16(o0[d + 4] * f0 + o1[d + 4] * f1, o0[d + 5] * f0 + o1[d + 5] * f1);
        wv.w = pack_bf16(o0[d + 6] * f0 + o1[d + 6] * f1, o0[d + 7] * f0 + o1[d + 7] * f1);
        *reinterpret_cast<uint4*>(mine + lane * OUT_ROW_BYTES + (((d / 8) ^ (lane & (CH - 1))) << 4)) = wv;
      }
      __syncwarp();
      if (!*abort) {
#pragma unroll
        for (int i2 = 0; i2 < CH; ++i2) {
          const int rw = i2 * (32 / CH) + lane / CH, chunk = lane % CH;     // row of the warp, chunk of its half row
          const int rg = q * 32 + rw;                                       // row of the block
          const int tok2 = a.hpt == 2 ? (rg & 63) : rg;
          const int head2 = wk.head0 + (a.hpt == 2 ? (rg >> 6) : 0);
          if (tok2 < rows_tok) {
            const uint4 wv = *reinterpret_cast<const uint4*>(mine + rw * OUT_ROW_BYTES + ((chunk ^ (rw & (CH - 1))) << 4));
            *reinterpret_cast<uint4*>(a.out + (size_t)(wk.row0 + tok2) * a.nh * HD + (size_t)head2 * HD + st * OD + chunk * 8) = wv;
          }
        }
      }
      __syncwarp();                                        // the warp's rows are out before the next work's are put there
      base += n_mine;
      ++it;
    }
  }
  // ---- teardown: every tensor-memory access is done, then the columns go back
  tc_fence_before();
  __syncthreads();
  // neither block of a pair leaves, or frees its tensor memory, while the other may still signal it or work on
  // a tile they share
  if (CTAS == 2) cluster_sync();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, TMEM_COLS);
  }
}

}  // namespace

MI_API int mi_attention_prefill_tc_supported() { return 1; }

// Describes the step's fused QKV rows - [rows, width] bf16, row-major - to the TMA engine: boxes of
// 64 rows x 64 elements, 128-byte swizzle, zeros past the last row.  `out_map` receives 128 bytes.
MI_API int mi_qkv_tensor_map(void* out_map, const void* qkv, long long rows, long long width) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return mi_fail("qkv_tensor_map: the driver does not offer cuTensorMapEncodeTiled");
    encode = (EncodeFn)fn;
  }
  MI_REQUIRE(((uintptr_t)qkv % 16) == 0 && rows > 0 && width >= 64 && width % 8 == 0,
             "qkv_tensor_map: rows=%lld, width=%lld (a multiple of 8, at least 64) or the address do not fit", rows, width);
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)width * 2};
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mi_fail("qkv_tensor_map: cuTensorMapEncodeTiled failed with code %d", (int)r);
  memcpy(out_map, &map, sizeof(map));
  return 0;
}

namespace {

// Launches the kernel for blocks that work alone (CTAS = 1) or in pairs (2).  `placed` tells whether pairs can be
// resident on this device at all; if not, nothing was launched and the caller takes the other form.
template <int CTAS>
int launch_prefill_tc(const CUtensorMap& qm, const CUtensorMap& km, const Args& a, int num_sms, cudaStream_t stream, bool* placed) {
  auto kernel = attention_prefill_tc_kernel<CTAS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (err != cudaSuccess) return mi_fail("attention_prefill_tc: cannot get %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  int groups = num_sms / CTAS;       // persistent blocks, one per SM (a block takes all of an SM's tensor memory)
  if (CTAS == 2) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
    static int max_pairs = -1;       // how many pairs can be resident; asked once
    if (max_pairs < 0) {
      cfg.gridDim = dim3(num_sms / 2 * 2);
      cfg.attrs = attr;
      cfg.numAttrs = n_attr;
      int n = 0;
      cudaError_t err = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
      max_pairs = (err == cudaSuccess) ? n : 0;
      cudaGetLastError();
    }
    if (max_pairs < 1) {
      *placed = false;
      return 0;
    }
    groups = min(groups, max_pairs);
  }
  if (mi::pdl_enabled()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  const int total_work = (a.nh / a.hw) * a.n_tiles;
  cfg.gridDim = dim3(CTAS * max(1, min(groups, total_work)));      // no more blocks (pairs) than there is work
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, qm, km, a);
  if (err != cudaSuccess) return mi_fail("attention_prefill_tc: launch failed: %s", cudaGetErrorString(err));
  *placed = true;
  return 0;
}

}  // namespace

// q_map: mi_qkv_tensor_map of the step's QKV rows; kv_map: mi_kv_tensor_map of the layer's cache.
// status: one word, set to 2 if a bounded wait ran out.  tiles128: the tiles of 128 tokens of the same items (item,
// first row), or null.  pairs: whether two blocks may share a work - 128 tokens of two neighbouring heads, a head
// each - which takes heads of 128, an even number of query heads per kv head and the list of 128-token tiles;
// otherwise, and where pairs cannot be placed, blocks work alone.
MI_API int mi_attention_prefill_tc(void* out, const void* q_map, const void* kv_map, const int* block_table, int bt_stride,
                                   const int* tiles, int n_tiles, const int* q_start, const int* q_len, const int* ctx_len,
                                   const int* seq_slot, int* status, int nh, int nkv, int page_size, float scale, int window,
                                   int num_sms, cudaStream_t stream, const int* tiles128, int n_tiles128, int pairs) {
  MI_REQUIRE(num_sms > 0, "attention_prefill_tc: num_sms");
  MI_REQUIRE(n_tiles >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_prefill_tc: bad head counts nh=%d nkv=%d", nh, nkv);
  MI_REQUIRE(page_size % 64 == 0, "attention_prefill_tc: page_size=%d must be a multiple of 64", page_size);
  MI_REQUIRE(scale > 0.f, "attention_prefill_tc: the scale must be positive");
  MI_REQUIRE(n_tiles <= 65535, "attention_prefill_tc: more than 65535 tiles in one launch (%d)", n_tiles);
  if (n_tiles == 0) return 0;
  Args a;
  a.out = (__nv_bfloat16*)out;
  a.block_table = block_table;
  a.bt_stride = bt_stride;
  a.tiles = tiles;
  a.q_start = q_start;
  a.q_len = q_len;
  a.ctx_len = ctx_len;
  a.seq_slot = seq_slot;
  a.status = status;
  a.n_tiles = n_tiles; a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap qm, km;
  memcpy(&qm, q_map, sizeof(qm));
  memcpy(&km, kv_map, sizeof(km));
  const bool even_group = (nh / nkv) % 2 == 0;
  bool placed = false;
  if (pairs && HD == 128 && even_group && num_sms >= 2 && tiles128 != nullptr && n_tiles128 > 0) {
    // a pair of blocks: 128 tokens of two neighbouring heads, a head each
    Args p = a;
    p.tiles = tiles128;
    p.n_tiles = n_tiles128;
    p.hpt = 1;
    p.hw = 2;
    p.skip_odd = 0;
    const int r = launch_prefill_tc<2>(qm, km, p, num_sms, stream, &placed);
    if (r != 0) return r;
  }
  if (!placed) {
    a.hpt = even_group ? 2 : 1;
    a.hw = a.hpt;
    a.skip_odd = a.hpt == 1 ? 1 : 0;
    if (a.hpt == 1 && tiles128 != nullptr && n_tiles128 > 0) {
      a.tiles = tiles128;
      a.n_tiles = n_tiles128;
      a.skip_odd = 0;
    }
    const int r = launch_prefill_tc<1>(qm, km, a, num_sms, stream, &placed);
    if (r != 0) return r;
  }
  MI_LAUNCH_OK("attention_prefill_tc");
  return 0;
}

#else  // other head sizes have no tcgen05 kernel

MI_API int mi_attention_prefill_tc_supported() { return 0; }
MI_API int mi_qkv_tensor_map(void*, const void*, long long, long long) { return mi_fail("qkv_tensor_map: head size %d has no tcgen05 kernel", MI_HEAD_DIM); }
MI_API int mi_attention_prefill_tc(void*, const void*, const void*, const int*, int, const int*, int, const int*, const int*, const int*,
                                   const int*, int*, int, int, int, float, int, int, cudaStream_t, const int*, int, int) {
  return mi_fail("attention_prefill_tc: head size %d has no tcgen05 kernel", MI_HEAD_DIM);
}

#endif
