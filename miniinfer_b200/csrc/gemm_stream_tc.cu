// Matrix product for few activation rows and a large weight matrix on the tcgen05 tensor cores:
//   out[M, N] = x[M, K] w[N, K]^T          (M <= 16; bf16 in, float32 sums, bf16 or float32 out), or
//   out[M, I] = silu(x w_gate^T) * (x w_up^T)   with w = [w_gate; w_up]  [2I, K].
// This is a decode step's product at the sizes of larger models, where the time is the one pass over
// the weights from HBM and the question is only how evenly and how deeply the SMs keep asking for
// them.  The product is turned around: 128 weight rows are the rows of the tensor-core tile (its A
// operand, lanes of tensor memory), the activation rows its 16 columns.
//   * The work is the list of (tile of 128 weight rows, slice of 256 elements of K), tile after tile.
//     Each of the persistent blocks - one per SM - takes an equal, contiguous stretch of that list,
//     whatever tiles it cuts: every SM streams the same number of bytes and all end together.  A block
//     starts with the tiles its stretch cuts and goes on to the whole tiles between them.
//   * warp 0 asks the TMA engine for the slices, a lane per copy - eight boxes of 64 weight rows x 64
//     elements (512 bytes of each row at a time: slices of 128 elements streamed 5 % slower) and
//     four 16 x 64 boxes of the activations beside them - into a ring of three stages of 72 KB,
//     128-byte swizzled as the tensor cores read them.  The weight boxes of the first three slices are
//     asked for at once, before the block has met and before the kernel waits for its predecessor in
//     the stream: no kernel writes weights.
//   * warp 1, one thread: sixteen tcgen05.mma (M = 128, N = 16, K = 16) per slice into one of two
//     accumulators of 16 columns of tensor memory; tcgen05.commit hands the stage back and, at the end
//     of a stretch of one tile, the accumulator over.
//   * warps 2-5, a thread per weight row: read the accumulator (tcgen05.ld), and either store the 16
//     results of a whole tile, or - where a block's stretch began or ended inside a tile - leave the
//     partial sums in a workspace and count the tile's parts; the block that arrives last adds the
//     parts in the order of K and stores.  No block waits for another, and the order of the sums
//     behind an output is a function of (N, K) and the number of SMs alone: a request's value does
//     not depend on what else is in the batch.
// With SwiGLU a tile is 64 gate rows and the 64 up rows of the same columns; the up threads pass
// their sums to the gate threads through shared memory, and both are rounded to bf16 before the
// activation, as the product followed by the activation kernel rounds them.
//
// Measured on B200 with 8 rows, cold weights, launches chained in a graph (this kernel / the mma.sync kernel
// of gemm_skinny.cuh / the library's product at 17 rows): 5120 x 25600 (262 MB) 49.2 / 64.1 / 47.2 us, 10240 x 5120
// (105 MB) 23.6 / 26.1 / 22.3, SwiGLU 2 x 25600 x 5120 (524 MB) 84.3 / 93.4 / 90.8 (+ the activation), SwiGLU
// 2 x 12288 x 4096 (201 MB) 38.8 / 41.7 / 37.2 (+ the activation), 151936 x 1024 (311 MB) 55.1 / 56.2; but 4096 x 12288
// (101 MB) 23.1 / 19.7 / 22.4, 6144 x 4096 (50 MB) 14.2 / 11.7 / 11.6, 4096 x 1024 (8 MB) 6.2 / 2.8.  Once it runs
// it streams at 6.0 to 6.6 TB/s (the 1.2 GB head of the 8B shape: 188 us, the mma.sync kernel 216 us, the library
// 207 us).  What this kernel adds is the even split - the other kernel's blocks make 2.2 rounds over the SMs for
// 10240 weight rows, or fill 72 % of them for 5120 - and what it costs is its start and its end: 1.2 us until
// tensor memory is allocated and the block has met, 3 us from the first request to the first slice, and for a
// matrix with fewer tiles than SMs every sum goes through the workspace, a round trip of 3 to 5 us.  So the engine
// takes it from 160 MiB of weights on, and from 80 MiB for more than 4096 rows (ops.STREAM_TC_MIN_BYTES): a decode
// step of the Qwen3-32B shape goes from 15.4 to 13.7 ms at batch 8.
//
// Every wait on an mbarrier is bounded: a wait that runs out raises a flag that ends all other waits
// of the block, sets the status word to 8, and the block runs to its end, tensor memory freed.
//
// The reference calls cuBLAS through nn.Linear for these products
// (miniinfer/models/fused_qwen3.py:95,107,135,137; miniinfer/layers/embedding.py:29-32).
#include <cuda.h>
#include <string.h>

#include "common.cuh"

namespace {

constexpr int TILE_ROWS = 128;                 // weight rows of a tile: the lanes of tensor memory
constexpr int HALF_ROWS = 64;                  // rows of a weight box
constexpr int BK = 64;                         // elements of K in a box: 128 bytes, one swizzle row
constexpr int KBOX = 4;                        // boxes of K in a slice
constexpr int SLICE_K = KBOX * BK;             // 128
constexpr int NB = 16;                         // activation rows = accumulator columns
constexpr int W_BOX_BYTES = HALF_ROWS * BK * 2;            // 8 KB
constexpr int W_KBOX_BYTES = 2 * W_BOX_BYTES;              // 128 rows x 128 bytes
constexpr int W_STAGE_BYTES = KBOX * W_KBOX_BYTES;         // 32 KB
constexpr int X_BOX_BYTES = NB * BK * 2;                   // 2 KB
constexpr int STAGE_BYTES = W_STAGE_BYTES + KBOX * X_BOX_BYTES;   // 36 KB
constexpr int STAGES = 3;                      // 108 KB: two blocks - of this launch and of the next - have room on an SM
constexpr int PRODUCER_WARP = 0, MMA_WARP = 1, EPILOGUE_WARP0 = 2, EPILOGUE_WARPS = 4;
constexpr int THREADS = (2 + EPILOGUE_WARPS) * 32;
constexpr int TMEM_COLS = 32;                  // two accumulators of 16 columns
constexpr int WAIT_LIMIT = 1 << 22;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 256 + HALF_ROWS * NB * sizeof(float);
constexpr int PART_FLOATS = NB * TILE_ROWS;    // a block's partial sums of a tile: [16][128]

struct Args {
  void* out;
  float* parts;          // [blocks][2][16][128]: a block's partial sums of the tile it begins in, and of the tile it ends in
  int* counters;         // [tiles]: parts of a tile that have arrived; all zero between launches
  int* status;
  int M, N, K, ldo;      // N: output columns (SwiGLU: I)
  int up_row0;           // SwiGLU: row of w where the up rows start (I); plain: unused
  int tiles, slices;     // tiles of weight rows; slices of K in a tile
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
  atomicExch(status, 8);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
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
// D[tmem] (+)= A[smem] * B[smem]^T, bf16 in, float32 out; one thread issues it for the block.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive columns of this thread's lane (lane = 32 * (warp % 4) + lane of the warp).
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
// Shared-memory operand descriptor, K-major with the 128-byte swizzle: start address, leading and
// stride byte offsets in 16-byte units (groups of 8 rows are 1024 bytes apart), descriptor version 1
// (bits 46..47), layout type 2 = 128-byte swizzle (bits 61..63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: float32 accumulator (bits 4..5 = 1), bf16 A and B (bits 7..9
// and 10..12 = 1), both K-major, N / 8 at bits 17..22, M / 16 at bits 24..28.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);

template <typename TOut>
__device__ __forceinline__ void store_out(TOut* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// The stretch of block b of `blocks` in a list of `units` (fewer than 2^31): [first, first of b + 1).
__device__ __forceinline__ int stretch_begin(int b, int blocks, int units) { return (int)((long long)b * units / blocks); }
// The block whose stretch holds unit u.
__device__ __forceinline__ int block_of(int u, int blocks, int units) {
  int b = (int)((long long)u * blocks / units);
  while (b + 1 < blocks && stretch_begin(b + 1, blocks, units) <= u) ++b;
  while (b > 0 && stretch_begin(b, blocks, units) > u) --b;
  return b;
}

// A block's stretch [begin, end) of the list as segments of one tile each: first the tile it begins inside and
// the tile it ends inside (whose sums other blocks wait to add up, or this block adds up when it comes last -
// the sooner they are in the workspace, the less of that is left for the end), then the whole tiles between.
struct Walk {
  int begin, end, head_end, tail_begin;
  int slices;
  __device__ Walk(int b, int e, int s) : begin(b), end(e), slices(s) {
    head_end = (b % s != 0) ? min((b / s + 1) * s, e) : b;
    const int last_tile = (e / s) * s;
    tail_begin = (e % s != 0 && last_tile >= head_end) ? last_tile : e;
  }
  // segment i: units [u0, u1) of one tile; false past the last
  __device__ bool segment(int i, int& u0, int& u1) const {
    if (head_end > begin) {
      if (i == 0) { u0 = begin; u1 = head_end; return true; }
      --i;
    }
    if (tail_begin < end) {
      if (i == 0) { u0 = tail_begin; u1 = end; return true; }
      --i;
    }
    u0 = head_end + i * slices;
    u1 = u0 + slices;
    return u0 < tail_begin;
  }
  // the n-th unit in that order (n below the stretch's length)
  __device__ int unit(int n) const {
    int u0, u1;
    for (int i = 0; segment(i, u0, u1); ++i) {
      if (n < u1 - u0) return u0 + n;
      n -= u1 - u0;
    }
    return begin;
  }
};

// Waits for the predecessor in the stream.  Unlike the other kernels of this library, this one does not let its
// successor be placed before it has ended: a block holds nearly all of an SM's shared memory, and a successor
// placed beside it early made the step slower, not faster (a decode step of 6 layers of the Qwen3-8B shape, this
// kernel for the gate-and-up product, the mma.sync kernel behind it: 0.983 ms with the early placement - at the
// kernel's start or when its last copy was asked for, alike - and 0.843 ms without; all products on the
// mma.sync kernel: 0.868 ms).
__device__ __forceinline__ void dep_sync() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_tc_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, Args a) {
  // The stages are read in the 128-byte swizzle, whose pattern repeats every 1024 bytes of address: the kernel has no
  // other shared memory, so its dynamic part starts at the block's window and is so aligned; were it not, the block
  // says so and leaves (no spare kilobyte is asked for: two blocks of 113 KB fit an SM, two of 114 do not).
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(a.status, 16);
    return;
  }
  unsigned char* stages = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stages + (size_t)STAGES * STAGE_BYTES);
  uint64_t* full = bars;                       // [STAGES]: a slice has landed
  uint64_t* empty = full + STAGES;             // [STAGES]: its products are done
  uint64_t* acc_full = empty + STAGES;         // [2]: a stretch's sums are in the accumulator
  uint64_t* acc_empty = acc_full + 2;          // [2]: the epilogue has read them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort) + 1;
  float* up_s = reinterpret_cast<float*>(bars + 32);       // [64][16]: the up rows' sums, for the gate threads

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blocks = (int)gridDim.x, me = (int)blockIdx.x;
  const int units = a.tiles * a.slices;
  const int u_begin = stretch_begin(me, blocks, units), u_end = stretch_begin(me + 1, blocks, units);
  const Walk walk(u_begin, u_end, a.slices);

  // Warp 0 is the producer.  Its first thread sets the barriers up, and the warp asks for the first weights at once,
  // before the block meets (the other warps have tensor memory to allocate and nothing to do until a slice has
  // landed) and before the predecessor in the stream is waited for (no kernel writes weights).  A slice is twelve
  // copies - eight boxes of weights, four of activations -, each asked for by a lane of its own: one thread
  // issuing them one after the other took 2 us for the first three slices.
  constexpr int W_BOXES = 2 * KBOX;                        // weight boxes of a slice
  static_assert(STAGES * W_BOXES <= 32 && STAGES * KBOX <= 32 && W_BOXES + KBOX <= 32, "a lane per copy");
  auto weight_box = [&](int u, int s, int box) {           // box: 2 * (box of K) + (half of the rows)
    const int t = u / a.slices, k = u % a.slices;
    const int kb = box >> 1, hi = box & 1;
    const int row = SWIGLU ? (hi ? a.up_row0 + t * HALF_ROWS : t * HALF_ROWS) : t * TILE_ROWS + hi * HALF_ROWS;
    tma_load_2d(stages + (size_t)s * STAGE_BYTES + kb * W_KBOX_BYTES + hi * W_BOX_BYTES, &w_map, k * SLICE_K + kb * BK, row, &full[s]);
  };
  auto activation_box = [&](int u, int s, int kb) {
    const int k = u % a.slices;
    tma_load_2d(stages + (size_t)s * STAGE_BYTES + W_STAGE_BYTES + kb * X_BOX_BYTES, &x_map, k * SLICE_K + kb * BK, 0, &full[s]);
  };
  const int early = min(STAGES, u_end - u_begin);
  if (warp == PRODUCER_WARP) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&x_map)) : "memory");
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&acc_full[i], 1);
        mbar_init(&acc_empty[i], EPILOGUE_WARPS);
      }
      *abort = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      for (int i = 0; i < early; ++i) mbar_expect_tx(&full[i], (uint32_t)STAGE_BYTES);
    }
    __syncwarp();
    if (lane < early * W_BOXES) weight_box(walk.unit(lane / W_BOXES), lane / W_BOXES, lane % W_BOXES);
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == PRODUCER_WARP) {
    // ------------------------------------------------------------------ producer
    dep_sync();
    if (lane < early * KBOX) activation_box(walk.unit(lane / KBOX), lane / KBOX, lane % KBOX);
    int n = 0;
    int u0, u1;
    bool stop = false;
    for (int i = 0; walk.segment(i, u0, u1) && !stop; ++i) {
      for (int u = u0; u < u1; ++u, ++n) {
        if (n < early) continue;
        const int s = n % STAGES;
        if (lane == 0) {
          mbar_wait(&empty[s], ((n / STAGES) & 1) ^ 1, abort, a.status);
          if (!*abort) mbar_expect_tx(&full[s], (uint32_t)STAGE_BYTES);
        }
        stop = __shfl_sync(0xffffffffu, (int)*abort, 0) != 0;   // after a wait has run out nothing more is asked for
        if (stop) break;
        if (lane < W_BOXES) weight_box(u, s, lane);
        else if (lane < W_BOXES + KBOX) activation_box(u, s, lane - W_BOXES);
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    dep_sync();
    if (lane == 0) {
      int n = 0;
      int u0, u1;
      for (int seg = 0; walk.segment(seg, u0, u1) && !*abort; ++seg) {
        const int k0 = u0 % a.slices;
        const int k1 = k0 + (u1 - u0);
        const int acc = seg & 1;
        mbar_wait(&acc_empty[acc], ((seg >> 1) & 1) ^ 1, abort, a.status);   // the epilogue has read what was there
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(acc * NB);
        for (int k = k0; k < k1 && !*abort; ++k, ++n) {
          const int s = n % STAGES;
          mbar_wait(&full[s], (n / STAGES) & 1, abort, a.status);
          tc_fence_after();
          const uint32_t base = smem_u32(stages + (size_t)s * STAGE_BYTES);
#pragma unroll
          for (int kb = 0; kb < KBOX; ++kb) {
            const uint64_t a_desc = smem_desc(base + kb * W_KBOX_BYTES);
            const uint64_t b_desc = smem_desc(base + W_STAGE_BYTES + kb * X_BOX_BYTES);
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks)     // 16 elements further: 32 bytes, 2 in the address field
              tc_mma(d, a_desc + (uint64_t)(2 * ks), b_desc + (uint64_t)(2 * ks), IDESC, (k > k0 || kb > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(&empty[s]);
        }
        tc_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: a thread per weight row
    dep_sync();
    const int q = warp & 3;                                // the quarter of the lanes this warp reaches
    const int r = q * 32 + lane;                           // row of the tile
    const int et = threadIdx.x - EPILOGUE_WARP0 * 32;      // 0..127 among the epilogue threads
    TOut* out = reinterpret_cast<TOut*>(a.out);
    int u0, u1;
    for (int seg = 0; walk.segment(seg, u0, u1); ++seg) {
      const int t = u0 / a.slices;
      const int k0 = u0 % a.slices;
      const int k1 = k0 + (u1 - u0);
      const int acc = seg & 1;
      mbar_wait(&acc_full[acc], (seg >> 1) & 1, abort, a.status);
      tc_fence_after();
      float v[NB];
      tmem_ld16(v, tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * NB));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      bool finish = true;
      if (k0 > 0 || k1 < a.slices) {
        // part of a tile: leave the sums in the workspace; whoever brings a tile's last part adds them all
        const int slot = k0 > 0 ? 0 : 1;
        float* mine = a.parts + ((size_t)me * 2 + slot) * PART_FLOATS;
#pragma unroll
        for (int m = 0; m < NB; ++m) mine[m * TILE_ROWS + r] = v[m];
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(EPILOGUE_WARPS * 32) : "memory");
        const int tile_first = t * a.slices, tile_last = tile_first + a.slices - 1;
        const int b_first = block_of(tile_first, blocks, units), b_last = block_of(tile_last, blocks, units);
        if (et == 0) {
          const int before = atomicAdd(&a.counters[t], 1);
          const int last = before == b_last - b_first;
          if (last) a.counters[t] = 0;                     // as the next launch expects it
          *last_flag = last;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPILOGUE_WARPS * 32) : "memory");
        finish = *last_flag != 0;
        if (finish) {
          __threadfence();
#pragma unroll
          for (int m = 0; m < NB; ++m) v[m] = 0.f;
          for (int b = b_first; b <= b_last; ++b) {        // in the order of K, whoever came when
            const float* part = a.parts + ((size_t)b * 2 + (b == b_first ? 1 : 0)) * PART_FLOATS;
#pragma unroll
            for (int m = 0; m < NB; ++m) v[m] += __ldcg(part + m * TILE_ROWS + r);
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPILOGUE_WARPS * 32) : "memory");   // last_flag may be written again
      }
      if (finish) {
        const bool ok = !*abort;                           // (the barriers below are passed whatever it says)
        if (SWIGLU) {
          // lanes 64..127 hold the up rows of the columns whose gate rows lanes 0..63 hold
          if (r >= HALF_ROWS) {
#pragma unroll
            for (int m = 0; m < NB; ++m) up_s[(r - HALF_ROWS) * NB + m] = v[m];
          }
          asm volatile("bar.sync 1, %0;" ::"n"(EPILOGUE_WARPS * 32) : "memory");
          if (r < HALF_ROWS) {
            const int n = t * HALF_ROWS + r;
            if (n < a.N && ok) {
#pragma unroll
              for (int m = 0; m < NB; ++m)
                if (m < a.M) store_out<TOut>(out + (size_t)m * a.ldo + n, mi::silu_mul_fast(round_bf16(v[m]), round_bf16(up_s[r * NB + m])));
            }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(EPILOGUE_WARPS * 32) : "memory");   // up_s may be written again
        } else {
          const int n = t * TILE_ROWS + r;
          if (n < a.N && ok) {
#pragma unroll
            for (int m = 0; m < NB; ++m)
              if (m < a.M) store_out<TOut>(out + (size_t)m * a.ldo + n, v[m]);
          }
        }
      }
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

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, cols] bf16, row-major: boxes of `box_rows` rows x 64 elements, 128-byte swizzle, zeros outside.
int encode_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return mi_fail("gemm_stream_tc: the driver does not offer cuTensorMapEncodeTiled");
    encode = (EncodeFn)fn;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mi_fail("gemm_stream_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

template <bool SWIGLU, typename TOut>
int run(void* out, const void* x, const void* w, int M, int N, int K, int ldo, float* parts, int* counters, int counters_len,
        int parts_blocks, int* status, cudaStream_t stream) {
  MI_REQUIRE(M > 0 && M <= NB && N > 0 && K >= BK && K % 8 == 0 && ldo >= N,
             "gemm_stream_tc: M=%d (at most 16) N=%d K=%d (a multiple of 8, at least 64) ldo=%d", M, N, K, ldo);
  MI_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_stream_tc: operands must be 16-byte aligned");
  Args a;
  a.out = out;
  a.parts = parts;
  a.counters = counters;
  a.status = status;
  a.M = M; a.N = N; a.K = K; a.ldo = ldo;
  a.up_row0 = N;
  a.tiles = SWIGLU ? (N + HALF_ROWS - 1) / HALF_ROWS : (N + TILE_ROWS - 1) / TILE_ROWS;
  a.slices = (K + SLICE_K - 1) / SLICE_K;
  const long long units = (long long)a.tiles * a.slices;
  MI_REQUIRE(units < (1LL << 30), "gemm_stream_tc: %lld slices of tiles are more than the kernel counts", units);
  const int sms = mi::sm_count();
  const int blocks = (int)(units < sms ? units : sms);
  MI_REQUIRE(a.tiles <= counters_len && blocks <= parts_blocks,
             "gemm_stream_tc: the workspace holds %d tiles and %d blocks, the product has %d and %d", counters_len, parts_blocks, a.tiles, blocks);
  CUtensorMap xm, wm;
  if (int e = encode_map(&xm, x, M, K, NB)) return e;
  if (int e = encode_map(&wm, w, SWIGLU ? 2LL * N : (long long)N, K, HALF_ROWS)) return e;
  auto kernel = gemm_stream_tc_kernel<SWIGLU, TOut>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (err != cudaSuccess) return mi_fail("gemm_stream_tc: cannot get %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  mi::launch(kernel, dim3(blocks), dim3(THREADS), SMEM_BYTES, stream, xm, wm, a);
  MI_LAUNCH_OK("gemm_stream_tc");
  return 0;
}

}  // namespace

// Floats of partial sums and ints of counters that the kernels below want: `parts` for as many blocks as the device has
// SMs, `counters` (all zero) for the tiles of the largest product.
MI_API int mi_gemm_stream_tc_workspace(long long* part_floats, int* blocks) {
  *blocks = mi::sm_count();
  *part_floats = (long long)mi::sm_count() * 2 * PART_FLOATS;
  return 0;
}

// out[M, N] = x w^T; out_dtype: 1 bf16, 0 float32 (the codes of the other products).  status: one word, set to 8 if a
// bounded wait ran out.
MI_API int mi_gemm_stream_tc_bf16(void* out, int out_dtype, const void* x, const void* w, int M, int N, int K, int ldo,
                                  float* parts, int* counters, int counters_len, int parts_blocks, int* status, cudaStream_t stream) {
  if (out_dtype == MI_BF16) return run<false, __nv_bfloat16>(out, x, w, M, N, K, ldo, parts, counters, counters_len, parts_blocks, status, stream);
  if (out_dtype == MI_F32) return run<false, float>(out, x, w, M, N, K, ldo, parts, counters, counters_len, parts_blocks, status, stream);
  return mi_fail("gemm_stream_tc: out must be bf16 or float32");
}

// out[M, I] = silu(x w[0:I]^T) * (x w[I:2I]^T), all bf16.
MI_API int mi_gemm_stream_tc_swiglu_bf16(void* out, const void* x, const void* w, int M, int I, int K, int ldo,
                                         float* parts, int* counters, int counters_len, int parts_blocks, int* status, cudaStream_t stream) {
  return run<true, __nv_bfloat16>(out, x, w, M, I, K, ldo, parts, counters, counters_len, parts_blocks, status, stream);
}
