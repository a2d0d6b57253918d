// Prefill attention over the paged cache in bf16 on the fifth-generation tensor cores (tcgen05):
// the kernel for head sizes 64 and 128 and page sizes that are multiples of 64.  The other sizes
// take the mma.sync kernel of attention_prefill.cu, which computes the same thing.
//
// A piece of work is 128 query rows that share one kv head - 128 tokens of one query head, or, when
// the number of query heads per kv head is even, 64 tokens of two neighbouring heads (so K and V are
// read once for both) - and the keys the mask allows, walked in tiles of 128.  Blocks are persistent,
// one per SM (a block takes all of an SM's tensor memory): the works are dealt out longest first, in
// rounds that go back and forth over the blocks, and a block's barriers run on from one work to the
// next, so that the next work's Q and first keys are copied and its first S is computed while the
// softmax warps finish the work before (2048 tokens of 16 heads: 40.1 -> 38.5 us).  Within a work:
//   * a producer warp asks the TMA engine for the Q rows once and for K and V tile by tile (boxes
//     of 64 rows x 64 elements, one page and one half of the head size each, written in the
//     128-byte swizzle), two stages each, counted on mbarriers; K and V are counted apart, since
//     K is free again as soon as S is computed;
//   * the key tiles are dealt to two streams, the even and the odd ones.  A stream has an S
//     accumulator (128 columns of tensor memory), an output accumulator (head size columns), and
//     a running maximum and sum per row of its own, as if it were a request with half the keys;
//     the two are merged at the end.  Inside a stream everything follows in order - S, softmax,
//     P V, S of its next tile - and the two streams take turns on the tensor cores, which so have
//     the products of one stream to do while the softmax warps of the other work;
//   * one thread of the MMA warp issues S = Q K^T (tcgen05.mma, M = 128, N = 128, K = 16 per
//     instruction, operands described in shared memory, K-major) and, once the stream's softmax
//     warps have written P, O += P V (P from tensor memory, where it overwrites the columns of S
//     it came from; V from shared memory, MN-major: dims contiguous, as the cache stores it);
//     tcgen05.commit tells the mbarriers when the products are done;
//   * eight softmax warps per stream - two threads per query row (tensor-memory lane = row), 64
//     columns each - read S with tcgen05.ld (once for the maximum, again for the exponentials),
//     keep the maximum and the sum in float32, base 2 with the scale folded in, and write P in
//     bf16 back into tensor memory.  The output row stays in tensor memory; it is rescaled there
//     only when a row's maximum moves up by more than 2^8 (until then sums and P are taken
//     against the older maximum, which costs no accuracy in float32 and bf16), and read once at
//     the end.
// Causal and window masks go by absolute position; tiles that the mask does not touch skip the
// comparisons.  Rows past the end of the item's tokens are computed on whatever the Q copy brought
// and never stored.
//
// (Tried and not kept, at 2048 tokens of 16 heads, 40.9 us per launch as it stands: the scores read
// once and held in registers between the maximum and the exponentials, 44.5 us; the keys of a block
// split over two blocks, 61 us; every other exponential as a polynomial on the FMA pipe instead
// of the special-function unit, 45.7 us - the softmax warps wait on the latencies of tensor
// memory and of each other, not on a pipe, and more instructions only lengthen their path.
// With persistent blocks, 38.5 us as it stands: one softmax thread per row that reads the row's 128
// scores once and holds them in registers (four warps per stream, 200 registers a thread by
// setmaxnreg, no exchange between threads), 96 us - half as many warps hide the latencies of
// tensor memory and of the exponentials half as well.  Two threads per row that hold their 64
// scores in registers between the maximum and the exponentials need about 112 registers each; the
// block is launched with 96 for each of its 640 threads, and setmaxnreg only moves registers that the
// block already has between its warpgroups - four softmax warpgroups at 112 and the fifth at 56
// are more than that, and a setmaxnreg.inc that cannot be met waits for ever.  Not built.
// A timeline of one block (clock64 stamps of the issuing thread and of the softmax warps, 16 tiles of
// one work) shows what binds: a stream's tile takes S (~600 cycles on the tensor cores), the softmax
// warps' round (~2600: 1400 for the pass over the scores, where the stream's two warps per scheduler
// share one special-function unit, 200 for the exchange of maxima, 500 to 800 for the store of P and
// its wait, 350 for the barriers), P V (~500), and two looks at barriers in between, each of which
// costs 350 to 600 cycles even when the barrier completed long before: while S products run, the
// tensor cores read Q and K at the full width of shared memory, and everything else that goes to
// shared memory queues behind them.  Two such chains, interleaved, give the ~2900 cycles a tile
// takes; the tensor cores are busy for ~1100 of them.  The issuing thread spends a tile's time as 16
// products (60 to 80 cycles each), five commits (55 each), a fence (100), the wait for P (600) and the
// looks at V and the next K.  Tried against that, none faster (38.5 us as it stands): later tiles of a
// stream in one pass over the scores (exponentials against the old maximum, redone only if the maximum
// moves by more than 2^8: 38.6 us, and the kernel spills at its 96 registers); one arrival per warp
// instead of per thread on the barriers the softmax warps complete (no change); the block table read
// by the whole producer warp, 32 entries at a time (no change: the copies do not wait for those reads);
// the barriers of the next tile looked at while this tile's products are issued (40.8 -> 41.7 us in the
// build that could switch it: the look comes too early to find P written); an issuing thread per
// stream (46.2 us: the two streams fall into step, both in the softmax and then both on the tensor
// cores, instead of taking turns).  Nor does the special-function unit bind: with the exponential replaced by a
// multiply-add (wrong numbers, for the time only) the launch takes as long.)
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

#include "common.cuh"

#ifndef MI_HEAD_DIM
#error "compile with -DMI_HEAD_DIM=<head size>"
#endif

#if MI_HEAD_DIM == 64 || MI_HEAD_DIM == 128

namespace {

constexpr int HD = MI_HEAD_DIM;
constexpr int BM = 128;                       // query rows of a block
constexpr int BN = 128;                       // keys of a tile
constexpr int STAGES = 2;
constexpr int NHALF = HD / 64;                // 64-element (128-byte) halves of a row
constexpr int HALF_BYTES = 128 * 128;         // 128 rows x 128 bytes
constexpr int Q_BYTES = NHALF * HALF_BYTES;
constexpr int K_BYTES = NHALF * HALF_BYTES;   // and V
constexpr int STAGE_BYTES = 2 * K_BYTES;
constexpr int STREAMS = 2;                      // the key tiles are dealt to two streams (even, odd) with sums of their own
constexpr int TPR = 2;                          // softmax threads per query row and stream, half of the columns each
constexpr int COLS = BN / TPR;                  // columns of S per softmax thread
constexpr int SOFTMAX_WARPS = 4 * TPR * STREAMS;
constexpr int PRODUCER_WARP = SOFTMAX_WARPS, MMA_WARP = SOFTMAX_WARPS + 1;
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
constexpr int TMEM_COLS = 512;
// Tensor memory: per stream an S accumulator (128 float32 columns; P overwrites part of it) and an
// output accumulator (head size columns).
constexpr int S_COL = 0, O_COL = 256;                  // stream s: S at S_COL + 128 s, O at O_COL + 128 s
constexpr int WAIT_LIMIT = 1 << 22;
constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + STAGES * STAGE_BYTES + 256 + (2 * STREAMS * TPR + 2 * STREAMS * (TPR + 1)) * BM * sizeof(float);

struct Args {
  __nv_bfloat16* out;            // [T, nh * HD]
  const int* block_table;
  int bt_stride;
  const int* tiles;              // [n_tiles, 2]: item, first row of the tile within the item's new tokens (multiples of 64)
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  const int* seq_slot;
  int* status;
  int n_tiles, nh, nkv, page_size, window;
  int hpt;                       // query heads of a block: 1 (128 tokens) or 2 (64 tokens each)
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

// ---- tensor memory and tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_in_smem)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 in, float32 out; one thread issues it for the block.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with A in tensor memory: lane = row, two bf16 of consecutive k to a column.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive columns of this thread's lane, written.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
// 16 consecutive columns of this thread's lane, read.
__device__ __forceinline__ void tmem_ld16(float (&v)[16], uint32_t taddr) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
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

// by the length of the array
__device__ __forceinline__ void tmem_ld(float (&v)[32], uint32_t taddr) { tmem_ld32(v, taddr); }
__device__ __forceinline__ void tmem_ld(float (&v)[16], uint32_t taddr) { tmem_ld16(v, taddr); }
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[32]) { tmem_st32(taddr, r); }
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }

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
__device__ __forceinline__ Work work_of(const Args& a, int w) {
  Work k;
  const int X = a.nh / a.hpt;
  const int tile = a.n_tiles - 1 - w / X;
  k.item = a.tiles[2 * tile];
  k.o = a.tiles[2 * tile + 1];
  k.skip = a.hpt == 1 && (k.o & 64);                      // the work of the tile before covers these 64 tokens too
  const int G = a.nh / a.nkv;
  k.head0 = (w % X) * a.hpt;
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

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, Args a) {
  const int total_work = (a.nh / a.hpt) * a.n_tiles;
  const int blocks = (int)gridDim.x, me = (int)blockIdx.x;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* kv_s = q_s + Q_BYTES;                    // [stage][K, V]
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + STAGES * STAGE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                            // K and V of a tile are counted apart: K is free again
  uint64_t* k_empty = k_full + STAGES;                    // once S is computed, long before P V is
  uint64_t* v_full = k_empty + STAGES;
  uint64_t* v_empty = v_full + STAGES;
  uint64_t* s_full = v_empty + STAGES;                    // [stream]: S of the stream's tile is computed
  uint64_t* p_full = s_full + STREAMS;                    // [stream]: its P is written
  uint64_t* o_full = p_full + STREAMS;                    // [stream]: its P V is added to the output row
  uint64_t* q_empty = o_full + STREAMS;                   // the work's last S is computed: the Q rows may be replaced
  uint64_t* o_free = q_empty + 1;                         // the work's output rows are read: the next work's P V may overwrite them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(bars + 32);       // [stream][2][TPR][BM]: the maxima the threads of a row tell each other
  float* fin_l = xch + 2 * STREAMS * TPR * BM;            // [2][stream][TPR][BM]: at the end of a work, each thread's sum
  float* fin_m = fin_l + 2 * STREAMS * TPR * BM;          // [2][stream][BM]: and each stream's maximum (two works take turns)

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_free, SOFTMAX_WARPS * 32);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < STREAMS; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 4 * TPR * 32);
      mbar_init(&o_full[b], 1);
    }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Up to here the block has touched nothing that a kernel writes: set up beside its predecessor in the stream, it
  // also reads the description of its first work (the step's lists, which the host uploaded) so that the roles find
  // it in the cache, and only then waits for the predecessor - the kernel that wrote the Q rows and the cache.
  {
    const int w0 = nth_work(0, me, blocks, total_work);
    if (w0 >= 0) {
      const Work k0 = work_of(a, w0);
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
        const Work k = work_of(a, w);
        if (k.skip) continue;
        mbar_wait(q_empty, (it & 1) ^ 1, abort, a.status);   // the S products of the work before have read the Q rows
        mbar_expect_tx(q_full, (uint32_t)Q_BYTES);
#pragma unroll
        for (int rb = 0; rb < 2; ++rb) {
          const int head = k.head0 + (a.hpt == 2 ? rb : 0);
          const int y = k.row0 + (a.hpt == 2 ? 0 : 64 * rb);
#pragma unroll
          for (int h = 0; h < NHALF; ++h)
            tma_load_2d(q_s + h * HALF_BYTES + rb * 64 * 128, &q_map, head * HD + h * 64, y, q_full);
        }
        // K of tile i goes first, then V of tile i - 1: S of the next tile never waits for a V copy
        auto load = [&](int li, bool values) {
          const int g = gi + li;                           // the tile's number among all tiles of this block
          const int s = g % STAGES;
          uint64_t* full = values ? &v_full[s] : &k_full[s];
          mbar_wait(values ? &v_empty[s] : &k_empty[s], ((g / STAGES) & 1) ^ 1, abort, a.status);
          unsigned char* dst = kv_s + (size_t)s * STAGE_BYTES + (values ? K_BYTES : 0);
          mbar_expect_tx(full, (uint32_t)K_BYTES);
          const int key0 = (k.t_begin + li) * BN;
#pragma unroll
          for (int pg = 0; pg < 2; ++pg) {
            const int key = key0 + 64 * pg;
            const int page = k.bt[min(key / a.page_size, a.bt_stride - 1)];   // past the context: the dummy page, masked below
            const int y = ((page * 2 + (values ? 1 : 0)) * a.nkv + k.kvh) * a.page_size + key % a.page_size;
#pragma unroll
            for (int h = 0; h < NHALF; ++h) tma_load_2d(dst + h * HALF_BYTES + pg * 64 * 128, &kv_map, h * 64, y, full);
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
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_S = instr_desc(BM, BN, false);
      constexpr uint32_t IDESC_PV = instr_desc(BM, HD, true);
      const uint32_t q_addr = smem_u32(q_s);
      // Tile j of a work belongs to stream j & 1.  The products of a stream follow each other - S, (softmax,)
      // P V, S of its next tile, ... - and the two streams take turns, so the tensor cores have the
      // products of one stream to do while the softmax warps of the other work.  The tensor cores
      // run the products in the order they are issued: P V of a tile (which reads P from the
      // columns of S) is issued before S of the stream's next tile overwrites them.
      // What this one thread issues is on the path of both streams, so it is kept short: the
      // descriptors are made once and stepped by addition (the address field counts 16 bytes), a
      // barrier that copies complete is looked at before the thread blocks on the softmax warps'
      // barrier (the look's latency passes meanwhile), and only that barrier - behind which other
      // threads wrote P with tcgen05.st - is followed by a fence.
      const uint64_t q_desc = smem_desc(q_addr, 16, 1024);
      auto k_step = [](int ks) { return (uint64_t)((ks >> 2) * (HALF_BYTES >> 4) + (ks & 3) * 2); };
      int gi = 0, it = 0;                                  // key tiles and works so far
      int sb[STREAMS] = {0, 0};                            // tiles of each stream so far
      for (int i = 0;; ++i) {
        const int w = nth_work(i, me, blocks, total_work);
        if (w < 0 || *abort) break;
        const Work k = work_of(a, w);
        if (k.skip) continue;
        const int n = k.n;
        auto issue_s = [&](int li, uint32_t ready) {
          const int g = gi + li;
          const int s = g % STAGES, b = li & 1;
          if (!ready) mbar_wait(&k_full[s], (g / STAGES) & 1, abort, a.status);
          const uint64_t k_desc = smem_desc(smem_u32(kv_s + (size_t)s * STAGE_BYTES), 16, 1024);
          const uint32_t d = tmem_base + S_COL + 128 * b;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            tc_mma(d, q_desc + k_step(ks), k_desc + k_step(ks), IDESC_S, ks > 0 ? 1u : 0u);
          tc_commit(&s_full[b]);
          tc_commit(&k_empty[s]);
          if (li == n - 1) tc_commit(q_empty);             // the work's last S: the Q rows are free once it is done
        };
        mbar_wait(q_full, it & 1, abort, a.status);
        if (!*abort) issue_s(0, 0u);
        if (!*abort && n > 1) issue_s(1, 0u);
        // the output rows in tensor memory are the work before's until its softmax warps have read them
        if (it > 0) mbar_wait(o_free, (it - 1) & 1, abort, a.status);
        for (int j = 0; j < n && !*abort; ++j) {
          const int g = gi + j;
          const int s = g % STAGES, b = j & 1;
          const uint32_t v_ready = mbar_peek(&v_full[s], (g / STAGES) & 1);
          const uint32_t k_ready = j + 2 < n ? mbar_peek(&k_full[(g + 2) % STAGES], ((g + 2) / STAGES) & 1) : 1u;
          mbar_wait(&p_full[b], (sb[b] + j / 2) & 1, abort, a.status);
          if (!v_ready) mbar_wait(&v_full[s], (g / STAGES) & 1, abort, a.status);
          if (*abort) break;
          tc_fence_after();
          const uint64_t v_desc = smem_desc(smem_u32(kv_s + (size_t)s * STAGE_BYTES + K_BYTES), HALF_BYTES, 1024);
          const uint32_t p_tmem = tmem_base + S_COL + 128 * b;   // thread `ch` of a row leaves its 64 keys in its first 32 columns
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)                   // 16 keys further: 2048 bytes of V
            tc_mma_ts(tmem_base + O_COL + 128 * b, p_tmem + (uint32_t)(64 * (ks >> 2) + 8 * (ks & 3)),
                      v_desc + (uint64_t)(ks * (2048 >> 4)), IDESC_PV,
                      (j >= 2 || ks > 0) ? 1u : 0u);         // the stream's output row is summed over the work's tiles in tensor memory
          tc_commit(&o_full[b]);
          tc_commit(&v_empty[s]);
          if (j + 2 < n) issue_s(j + 2, k_ready);
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
    // 4), half ch = (w >> 2) & 1 of the columns, stream st = w >> 3.  A stream keeps a maximum, a sum
    // and an output row of its own over its tiles (the even or the odd ones); the two are merged at
    // the end.  The two threads of a row and stream tell each other their half's maximum through
    // shared memory, with a barrier of the 64 threads that share the rows.
    const int q = warp & 3, ch = (warp >> 2) & 1, st = warp >> 3;
    const int r = q * 32 + lane;                           // row of the block = lane of the tensor memory
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
    const float sc = a.scale_log2;
    auto row_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + st * 4 + q) : "memory"); };
    // o_full of the stream completes once per tile of the stream; every thread takes the phases in
    // order, each at most one tile late, and remembers how many it has seen
    int o_seen = 0;
    auto wait_o = [&](int upto) {
      while (o_seen <= upto) {
        mbar_wait(&o_full[st], o_seen & 1, abort, a.status);
        ++o_seen;
      }
      tc_fence_after();
    };
    const uint32_t s_addr = t_lane + S_COL + 128 * st + ch * COLS;
    const uint32_t o_addr = t_lane + O_COL + 128 * st + ch * (HD / 2);   // for rescaling: this thread's half of the stream's output row
    int base = 0, it = 0;                                  // tiles of this stream and works so far

    for (int i = 0;; ++i) {
      const int w = nth_work(i, me, blocks, total_work);
      if (w < 0) break;
      const Work wk = work_of(a, w);
      if (wk.skip) continue;
      const int n = wk.n, start = wk.start, o = wk.o, rows_tok = wk.rows_tok;
      const int p_first = wk.p_first, p_last = wk.p_last, lo_last = wk.lo_last, t_begin = wk.t_begin;
      const int tok = a.hpt == 2 ? (r & 63) : r;
      const int head = wk.head0 + (a.hpt == 2 ? (r >> 6) : 0);
      const bool row_valid = tok < rows_tok;
      const int pos = row_valid ? start + o + tok : p_last;
      const int lo_r = a.window > 0 ? max(0, pos - a.window + 1) : 0;
      float m_run = -INFINITY, l_run = 0.f;                // m_run: the maximum the stream's sums are taken against
      const int n_mine = (n - st + 1) / 2;                 // tiles of this stream

      for (int k = 0; k < n_mine; ++k) {
        const int j = 2 * k + st;
        const int kk = base + k;                           // the tile's number among all tiles of this stream and block
        const int key0 = (t_begin + j) * BN + ch * COLS;   // first key of this thread's columns
        const bool masked = !((t_begin + j) * BN + BN - 1 <= p_first && (t_begin + j) * BN >= lo_last);   // some (row, key) of the tile is hidden
        // (after a wait has run out the loop goes on without waiting, so that the warps of a row
        // still meet at every row barrier; what it computes then is never stored)
        mbar_wait(&s_full[st], kk & 1, abort, a.status);
        tc_fence_after();
        // first pass over this thread's 64 scores: their maximum
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one of 64 links
#pragma unroll
        for (int c = 0; c < COLS / 32; ++c) {
          float v[32];
          tmem_ld32(v, s_addr + 32 * c);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int key = key0 + 32 * c + e;
            if (!masked || (key >= lo_r && key <= pos)) mx4[e & 3] = fmaxf(mx4[e & 3], v[e]);
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        float* my_xch = xch + ((st * 2 + (kk & 1)) * TPR) * BM;
        my_xch[ch * BM + r] = mx;
        row_sync();
        mx = fmaxf(mx, my_xch[(ch ^ 1) * BM + r]);
        // The sums stay relative to the old maximum while the new one is at most 2^8 above it (the
        // exponentials then stay below 2^8, which float32 sums and bf16 P hold easily); only a larger
        // move - the first tile, mostly - rescales the sum and the output row in tensor memory.  The
        // decision is taken for the warp, so that the tensor-memory accesses stay warp-wide; both
        // threads of a row see the same maxima and decide alike.
        const float m_new = fmaxf(m_run, mx * sc);         // the scale is positive
        const bool move = m_new > m_run + 8.f || m_run == -INFINITY;
        if (__any_sync(0xffffffffu, move)) {
          const float m_next = move ? m_new : m_run;
          const float m_to = m_next == -INFINITY ? 0.f : m_next;
          const float alpha = move ? exp2f(m_run - m_to) : 1.f;   // 0 for a row that had no key yet
          if (k > 0) {
            wait_o(kk - 1);                                // the stream's products so far are in its output row
#pragma unroll
            for (int c = 0; c < HD / 2 / 32; ++c) {
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
        // exponentials, their sum, and P in bf16 into tensor memory, where the second product reads
        // its A operand (lane = row, two keys to a column): this thread's 64 keys go to the first 32
        // of its own 64 columns of S, which it has read
        // (32 scores at a time: the first 32 are read before P overwrites the first 16 columns, and
        // the P of the second 32 goes to the columns 16..31, read by then)
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < COLS / 32; ++c) {
          float v[32];
          tmem_ld32(v, s_addr + 32 * c);
          uint32_t packed[16];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int key = key0 + 32 * c + e;
            float x = fmaf(v[e], sc, -m_use);
            if (masked) x = (key >= lo_r && key <= pos) ? x : -INFINITY;
            float pe;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pe) : "f"(x));
            v[e] = pe;
            part[e & 3] += pe;
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) packed[e] = pack_bf16(v[2 * e], v[2 * e + 1]);
          tmem_st16(s_addr + 16 * c, packed);
        }
        l_run += (part[0] + part[1]) + (part[2] + part[3]);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        // Every phase of o_full is taken no later than one tile after it completes (a waiter two
        // phases behind would read the parity of the wrong phase).  The product waited for here was
        // issued a whole tile of the stream ago.
        if (kk > 0) wait_o(kk - 1);
        tc_fence_before();
        mbar_arrive(&p_full[st]);
      }
      if (n_mine > 0) wait_o(base + n_mine - 1);
      // ---- the two streams' sums are merged: every thread leaves its sum (and the stream's maximum)
      // in shared memory, all softmax warps meet, and each thread finishes a quarter of the output row
      float* fl = fin_l + (it & 1) * STREAMS * TPR * BM;
      float* fm = fin_m + (it & 1) * STREAMS * BM;
      fl[(st * TPR + ch) * BM + r] = l_run;
      if (ch == 0) fm[st * BM + r] = m_run;
      tc_fence_before();
      asm volatile("bar.sync 9, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
      tc_fence_after();
      const float m0 = fm[r], m1 = fm[BM + r];
      const float m_all = fmaxf(m0, m1);
      const float w0 = m0 == -INFINITY ? 0.f : exp2f(m0 - m_all);     // a stream without tiles, or without a visible key, counts nothing
      const float w1 = m1 == -INFINITY ? 0.f : exp2f(m1 - m_all);
      const float l_all = (fl[r] + fl[BM + r]) * w0 + (fl[2 * BM + r] + fl[3 * BM + r]) * w1;
      constexpr int OD = HD / 4;                           // output columns of this thread: 32 or 16
      const int part_no = st * 2 + ch;
      float o0[OD], o1[OD];
      const bool has1 = n > 1;                             // the second stream has an output row only if it had a tile
      tmem_ld(o0, t_lane + O_COL + part_no * OD);
      if (has1) {
        tmem_ld(o1, t_lane + O_COL + 128 + part_no * OD);
      } else {
#pragma unroll
        for (int e = 0; e < OD; ++e) o1[e] = 0.f;
      }
      // the output rows are in registers: the next work's products may overwrite them in tensor memory
      tc_fence_before();
      mbar_arrive(o_free);
      if (row_valid && !*abort) {
        const float f0 = w0 / l_all, f1 = has1 ? w1 / l_all : 0.f;
        __nv_bfloat16* dst = a.out + (size_t)(wk.row0 + tok) * a.nh * HD + (size_t)head * HD + part_no * OD;
#pragma unroll
        for (int d = 0; d < OD; d += 8) {
          uint4 wv;
          wv.x = pack_bf16(o0[d] * f0 + o1[d] * f1, o0[d + 1] * f0 + o1[d + 1] * f1);
          wv.y = pack_bf16(o0[d + 2] * f0 + o1[d + 2] * f1, o0[d + 3] * f0 + o1[d + 3] * f1);
          wv.z = pack_bf16(o0[d + 4] * f0 + o1[d + 4] * f1, o0[d + 5] * f0 + o1[d + 5] * f1);
          wv.w = pack_bf16(o0[d + 6] * f0 + o1[d + 6] * f1, o0[d + 7] * f0 + o1[d + 7] * f1);
          *reinterpret_cast<uint4*>(dst + d) = wv;
        }
      }
      base += n_mine;
      ++it;
    }
  }
  // ---- teardown: every tensor-memory access is done, then the columns go back
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
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

// q_map: mi_qkv_tensor_map of the step's QKV rows; kv_map: mi_kv_tensor_map of the layer's cache.
// status: one word, set to 2 if a bounded wait ran out.
MI_API int mi_attention_prefill_tc(void* out, const void* q_map, const void* kv_map, const int* block_table, int bt_stride,
                                   const int* tiles, int n_tiles, const int* q_start, const int* q_len, const int* ctx_len,
                                   const int* seq_slot, int* status, int nh, int nkv, int page_size, float scale, int window,
                                   int num_sms, cudaStream_t stream) {
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
  a.hpt = ((nh / nkv) % 2 == 0) ? 2 : 1;
  a.scale_log2 = scale * 1.4426950408889634f;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (err != cudaSuccess) return mi_fail("attention_prefill_tc: cannot get %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  CUtensorMap qm, km;
  memcpy(&qm, q_map, sizeof(qm));
  memcpy(&km, kv_map, sizeof(km));
  // persistent blocks, one per SM (a block takes all of an SM's tensor memory), no more than there is work
  const int total_work = (nh / a.hpt) * n_tiles;
  mi::launch(attention_prefill_tc_kernel, dim3(total_work < num_sms ? total_work : num_sms), dim3(THREADS), SMEM_BYTES, stream, qm, km, a);
  MI_LAUNCH_OK("attention_prefill_tc");
  return 0;
}

#else  // other head sizes have no tcgen05 kernel

MI_API int mi_attention_prefill_tc_supported() { return 0; }
MI_API int mi_qkv_tensor_map(void*, const void*, long long, long long) { return mi_fail("qkv_tensor_map: head size %d has no tcgen05 kernel", MI_HEAD_DIM); }
MI_API int mi_attention_prefill_tc(void*, const void*, const void*, const int*, int, const int*, int, const int*, const int*, const int*,
                                   const int*, int*, int, int, int, float, int, int, cudaStream_t) {
  return mi_fail("attention_prefill_tc: head size %d has no tcgen05 kernel", MI_HEAD_DIM);
}

#endif
