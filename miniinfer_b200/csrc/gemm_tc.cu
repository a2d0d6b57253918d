// Matrix product with many activation rows on the tcgen05 tensor cores, with the SwiGLU activation
// in its epilogue:  out[M, I] = silu(x w_gate^T) * (x w_up^T),  x [M, K] and w = [w_gate; w_up]
// [2I, K] in bf16, K contiguous in both.  The library product that runs elsewhere for many rows has
// no such epilogue: it writes [M, 2I], which a second kernel reads again; here the gate and the up
// half of an output tile are accumulated side by side in tensor memory and only their product
// leaves the SM.  (The plain product out = x w^T runs through the same kernel, for tests and as a
// stand-in where the library is not wanted.)
//
// Persistent blocks walk output tiles of 128 rows x 128 (SwiGLU) or 256 (plain) columns:
//   * warp 4, one thread: asks the TMA engine for 64-element slices of K - boxes of 128 rows of x
//     and of w - into a ring of stages, 128-byte swizzled as the tensor cores read them;
//   * warp 5, one thread: issues tcgen05.mma (bf16 in, float32 accumulators in tensor memory), four
//     per stage, and hands the stage back with tcgen05.commit; the accumulators of consecutive
//     tiles alternate between the two halves of the 512 columns, so the products of the next tile
//     run while the last one is written out;
//   * warps 0-3: the epilogue.  A thread owns one row of the tile (its lane of tensor memory); it
//     reads 32 columns of the gate and of the up half at a time, rounds both to bf16 (as the
//     two-kernel path does), applies silu(g) * u in float32 and stores 64 bytes of the row.
// Rows past M and columns past the edge are zero-filled by TMA on the way in and not stored.
//
// What limits a block that works alone is the traffic from L2: a 128 x 256 accumulator needs
// 48 KB per 64 elements of K, and all SMs together then ask L2 for more than it delivers.  So the
// blocks work in pairs (a cluster of two, tcgen05 cta_group::2): the pair computes 256 rows x 256
// accumulator columns with one instruction stream, each block holding its own 128 rows of x and
// one half of the rows of w (the first block the gate rows, the second the up rows), 32 KB per
// block and slice.  The first block of the pair issues the products for both; the copies of both
// blocks count on its barrier; its commits free the stages and hand over the accumulators in both
// blocks at once (tcgen05.commit with a multicast to the pair); both blocks' epilogue warps tell
// the first block when an accumulator has been read.  The single-block variant remains for a
// device where pairs cannot be placed.
//
// (The fused QKV product with the per-head norm, the rotation and the store into the cache in this
// kernel's epilogue was tried and is not here: a thread owns a row, so it reads its own 512-byte
// row of the rotation table, and the rows of a tile's 128 threads do not fit into what the stages
// leave of L1 - 32 us against 23.4 us for the library product followed by the norm-and-rotate
// kernel, at 2048 rows.)
//
// Every wait on an mbarrier is bounded: a wait that runs out raises a flag that ends all other
// waits of the block, sets the status word to 4, and the block runs to its end, tensor memory freed.
//
// Stands where the reference calls torch.nn.functional.linear followed by its Triton silu_mul
// kernel (miniinfer/models/fused_qwen3.py:111-138, kernels/triton/silu_mul.py:6-42).
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;                      // rows of a block's tile
constexpr int BN = 256;                      // accumulator columns of a tile: two boxes of 128 rows of w
constexpr int BK = 64;                       // elements of K per stage: 128 bytes, one swizzle row
constexpr int BOX_BYTES = 128 * BK * 2;      // 128 rows of x or of w
constexpr int EPILOGUE_WARPS = 4, PRODUCER_WARP = 4, MMA_WARP = 5;
constexpr int THREADS = 6 * 32;
constexpr int TMEM_COLS = 512;               // two accumulators of 256 columns
constexpr int WAIT_LIMIT = 1 << 22;
constexpr uint32_t PAIR_LEADER_MASK = 0xFEFFFFFFu;   // clears the bit of a shared::cluster address that tells the two blocks of a pair apart

// CTAS: blocks that share a tile's instruction stream (1, or 2 as a cluster).
template <int CTAS> struct Shape {
  static constexpr int B_BOXES = CTAS == 1 ? 2 : 1;                // boxes of w a block loads per stage
  static constexpr int STAGE_BYTES = (1 + B_BOXES) * BOX_BYTES;
  static constexpr int STAGES = CTAS == 1 ? 4 : 6;
  static constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + 256;
};

struct Args {
  __nv_bfloat16* out;
  int* status;
  int M, N;              // output rows and columns (SwiGLU: N = I)
  int K, ldo;
  int second;            // row of w where the second box of a tile starts, relative to the first (SwiGLU: I; plain: 128)
  int tiles_m, tiles_n;
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
  atomicExch(status, 4);
}
// One look at the barrier: has the phase of this parity completed?  The answer is not needed at once,
// so the instruction's latency passes behind what the thread issues next.
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
// One more arrival on a barrier of the pair's first block, from either block.
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PAIR_LEADER_MASK) : "memory");
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
// Tensor memory: one warp allocates (in a pair: the same warp of both blocks, each for its own SM).
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
// The barrier gets an arrival when all products issued so far by this thread are done; in a pair the
// barrier at the same place in both blocks does.
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
// D[tmem] (+)= A[smem] * B[smem]^T, bf16 in, float32 out; one thread issues it for the block, or
// for the pair (A: 128 rows in each block, B: half of its rows in each block).
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
// Shared-memory operand descriptor, K-major with the 128-byte swizzle: start address, leading and
// stride byte offsets in 16-byte units (groups of 8 rows are 1024 bytes apart), descriptor version 1
// (bits 46..47), layout type 2 = 128-byte swizzle (bits 61..63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: float32 accumulator (bits 4..5 = 1), bf16 A and B (bits 7..9
// and 10..12 = 1), both K-major, N / 8 at bits 17..22, M / 16 at bits 24..28 (M: rows of the pair).
constexpr uint32_t instr_desc(int m) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <bool SWIGLU, int CTAS>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, Args a) {
  using S = Shape<CTAS>;
  constexpr int STAGES = S::STAGES, STAGE_BYTES = S::STAGE_BYTES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the swizzle pattern is a function of the address: the stages start on a 1024-byte boundary
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;       // [2]: the tile's products are all in tensor memory
  uint64_t* acc_empty = acc_full + 2;        // [2]: the epilogue warps have read the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rank = CTAS == 1 ? 0 : (int)cluster_rank();     // place in the pair; block 0 issues the products
  const bool leader = rank == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], EPILOGUE_WARPS * CTAS);
    }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc<CTAS>(tmem_slot, TMEM_COLS);
  if (warp == PRODUCER_WARP && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&x_map)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync();     // the other block's barriers are set up before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  mi::grid_dependency_sync();        // x is the output of the kernel before

  // tiles of the pair (or of the block): CTAS * 128 rows each
  const int tiles_m = (a.tiles_m + CTAS - 1) / CTAS;
  const int n_tiles = tiles_m * a.tiles_n;
  const int first_tile = (int)blockIdx.x / CTAS, tile_step = (int)gridDim.x / CTAS;
  const int kblocks = (a.K + BK - 1) / BK;
  constexpr int TILE_COLS = SWIGLU ? BN / 2 : BN;      // output columns of a tile
  constexpr uint32_t IDESC = instr_desc(BM * CTAS);

  if (warp == PRODUCER_WARP) {
    if (lane == 0) {
      // The thread looks at the barrier of the next stage before it issues this stage's copies, so
      // that the look's latency is not added to every step.
      int it = 0;
      uint32_t ready = mbar_peek(&empty[0], 1);
      for (int tile = first_tile; tile < n_tiles && !*abort; tile += tile_step) {
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        const int row0 = (tm * CTAS + rank) * BM, n0 = tn * TILE_COLS;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ready) {
            mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort, a.status);
            if (*abort) break;
          }
          const int nx = it + 1;
          ready = mbar_peek(&empty[nx % STAGES], ((nx / STAGES) & 1) ^ 1);
          unsigned char* st = smem + (size_t)s * STAGE_BYTES;
          if (CTAS == 1) {
            mbar_expect_tx(&full[s], (uint32_t)STAGE_BYTES);
            tma_load_2d(st, &x_map, kb * BK, row0, &full[s]);
            tma_load_2d(st + BOX_BYTES, &w_map, kb * BK, n0, &full[s]);
            tma_load_2d(st + 2 * BOX_BYTES, &w_map, kb * BK, n0 + a.second, &full[s]);
          } else {
            // both blocks' bytes are counted on the first block's barrier, which expects them all
            if (leader) mbar_expect_tx(&full[s], (uint32_t)(2 * STAGE_BYTES));
            tma_load_2d_pair(st, &x_map, kb * BK, row0, &full[s]);
            tma_load_2d_pair(st + BOX_BYTES, &w_map, kb * BK, n0 + rank * a.second, &full[s]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    if (lane == 0 && leader) {
      // What this thread issues per 64 elements of K - a look at the next stage's barrier, four
      // products, a commit - has to take less time than the products themselves: the descriptors
      // are made once per stage and stepped by addition, and no wait stands between the products
      // unless the copies have fallen behind.  (Copies by TMA and products by tcgen05 both work
      // through the asynchronous proxy: the barrier the copy completes on orders them, no fence
      // is needed in the loop.)
      int it = 0, t = 0;
      uint32_t ready = 0;
      for (int tile = first_tile; tile < n_tiles && !*abort; tile += tile_step, ++t) {
        const int buf = t & 1;
        mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, abort, a.status);
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)buf * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ready) {
            mbar_wait(&full[s], (it / STAGES) & 1, abort, a.status);
            if (*abort) break;
          }
          const int nx = it + 1;
          ready = mbar_peek(&full[nx % STAGES], (nx / STAGES) & 1);
          const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + BOX_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)      // 32 bytes further along K: 2 in the descriptor's units of 16 bytes
            tc_mma<CTAS>(d, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit<CTAS>(&empty[s]);
        }
        tc_commit<CTAS>(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue warps 0..3
    int t = 0;
    for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++t) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int buf = t & 1;
      mbar_wait(&acc_full[buf], (t >> 1) & 1, abort, a.status);
      if (*abort) break;
      tc_fence_after();
      const int row = (tm * CTAS + rank) * BM + warp * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)buf * BN;
      __nv_bfloat16* orow = a.out + (size_t)row * a.ldo;
#pragma unroll 1
      for (int c = 0; c < TILE_COLS / 32; ++c) {
        float g[32];
        uint32_t packed[16];
        tmem_ld32(g, taddr + c * 32);
        if (SWIGLU) {
          float u[32];
          tmem_ld32(u, taddr + BN / 2 + c * 32);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float gg = round_bf16(g[i]), uu = round_bf16(u[i]);
            g[i] = mi::silu_mul_fast(gg, uu);
          }
        }
        if (c == TILE_COLS / 32 - 1) {
          // the accumulator has been read: the products of the tile after next may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CTAS == 1) mbar_arrive(&acc_empty[buf]);
            else mbar_arrive_leader(&acc_empty[buf]);
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) packed[i] = pack_bf16(g[2 * i], g[2 * i + 1]);
        const int col = tn * TILE_COLS + c * 32;
        if (row < a.M) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (col + q * 8 + 8 <= a.N)
              *reinterpret_cast<uint4*>(orow + col + q * 8) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  // neither block of a pair leaves, or frees its tensor memory, while the other may still signal it
  // or work on a tile they share
  if (CTAS == 2) cluster_sync();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, TMEM_COLS);
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, cols] bf16, row-major: boxes of 128 rows x 64 elements, 128-byte swizzle, zeros outside.
int encode_map(CUtensorMap* map, const void* base, long long rows, long long cols) {
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return mi_fail("gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
    encode = (EncodeFn)fn;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, 128};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mi_fail("gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

template <bool SWIGLU, int CTAS>
int launch_tc(const CUtensorMap& xm, const CUtensorMap& wm, const Args& a, int sms, cudaStream_t stream, bool* placed) {
  using S = Shape<CTAS>;
  auto kernel = gemm_tc_kernel<SWIGLU, CTAS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM_BYTES);
    if (err != cudaSuccess) return mi_fail("gemm_tc: cannot get %zu bytes of shared memory: %s", S::SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  const int tiles = ((a.tiles_m + CTAS - 1) / CTAS) * a.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = S::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (CTAS == 2) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  int groups = sms / CTAS;           // persistent: as many blocks (pairs) as the device places at once
  if (CTAS == 2) {
    static int max_pairs = -1;       // how many pairs can be resident; asked once
    if (max_pairs < 0) {
      cfg.gridDim = dim3(sms / 2 * 2);
      cfg.attrs = attr;
      cfg.numAttrs = n_attr;
      int n = 0;
      cudaError_t err = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
      max_pairs = (err == cudaSuccess) ? n : 0;
      cudaGetLastError();
    }
    if (max_pairs < 1) {
      *placed = false;               // pairs cannot be placed here: the caller takes the single-block kernel
      return 0;
    }
    groups = min(groups, max_pairs);
  }
  if (mi::pdl_enabled()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.gridDim = dim3(CTAS * max(1, min(groups, tiles)));
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, xm, wm, a);
  if (err != cudaSuccess) return mi_fail("gemm_tc: launch failed: %s", cudaGetErrorString(err));
  *placed = true;
  return 0;
}

template <bool SWIGLU>
int run(void* out, const void* x, const void* w, int M, int N, int K, int ldo, int* status, int pairs, cudaStream_t stream) {
  // N: output columns; w has N rows (plain) or 2 N rows (SwiGLU)
  MI_REQUIRE(M > 0 && N > 0 && K >= BK && K % 8 == 0 && N % 8 == 0 && ldo % 8 == 0 && ldo >= N,
             "gemm_tc: M=%d N=%d K=%d ldo=%d: K (at least 64), N and the row stride must be multiples of 8", M, N, K, ldo);
  MI_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0, "gemm_tc: operands must be 16-byte aligned");
  CUtensorMap xm, wm;
  if (int e = encode_map(&xm, x, M, K)) return e;
  if (int e = encode_map(&wm, w, SWIGLU ? 2LL * N : (long long)N, K)) return e;
  Args a;
  a.out = (__nv_bfloat16*)out;
  a.status = status;
  a.M = M; a.N = N; a.K = K; a.ldo = ldo;
  a.second = SWIGLU ? N : 128;
  constexpr int TILE_COLS = SWIGLU ? BN / 2 : BN;
  a.tiles_m = (M + BM - 1) / BM;
  a.tiles_n = (N + TILE_COLS - 1) / TILE_COLS;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms < 2) pairs = 0;
  bool placed = false;
  if (pairs) {
    if (int e = launch_tc<SWIGLU, 2>(xm, wm, a, sms, stream, &placed)) return e;
  }
  if (!placed) {
    if (int e = launch_tc<SWIGLU, 1>(xm, wm, a, sms > 0 ? sms : 1, stream, &placed)) return e;
  }
  return 0;
}

}  // namespace

// out[M, I] = silu(x w[0:I]^T) * (x w[I:2I]^T), all bf16; status: one word, set to 4 if a bounded wait ran out.
// pairs: non-zero to let two blocks share a tile (the default of the engine), zero for blocks that work alone.
MI_API int mi_gemm_tc_swiglu_bf16(void* out, const void* x, const void* w, int M, int I, int K, int ldo, int* status,
                                  int pairs, cudaStream_t stream) {
  return run<true>(out, x, w, M, I, K, ldo, status, pairs, stream);
}

// out[M, N] = x w^T, all bf16.
MI_API int mi_gemm_tc_bf16(void* out, const void* x, const void* w, int M, int N, int K, int ldo, int* status,
                           int pairs, cudaStream_t stream) {
  return run<false>(out, x, w, M, N, K, ldo, status, pairs, stream);
}
