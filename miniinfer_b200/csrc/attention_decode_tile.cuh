// What the two TMA-fed decode attention kernels share (attention_decode_tma.cu: persistent blocks for
// steps with much to read; attention_decode_cluster.cu: thread-block clusters for steps with little):
// the geometry of a 64-key tile in shared memory, the barrier and copy instructions with bounded
// waits, and the tile computation on the tensor cores.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int HD = MI_HEAD_DIM;
constexpr int BK = 64;                       // keys of a tile
constexpr int NBOX = HD / 64;                // 64-element (128-byte) boxes across a row
constexpr int BOX_BYTES = BK * 128;          // 64 rows x 128 bytes
constexpr int TILE_BYTES = NBOX * BOX_BYTES; // K (or V) of one tile
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int KSTEPS = HD / 16;
constexpr int WAIT_LIMIT = 1 << 18;          // polls of an mbarrier before giving up

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
  atomicExch(status, 1);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Transposes an 8x8 matrix of 16-bit values held in fragment layout (lane 4r + c holds row r, columns 2c, 2c + 1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// Address of the 16-byte chunk `c` (0 .. HD/8) of row `r` (0 .. 63) of a swizzled tile.
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, int r, int c) {
  return tile + (uint32_t)((c >> 3) * BOX_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}


// One 64-key tile for up to 8 query heads of a kv head, on the tensor cores with the products transposed
// (keys as the 16-row operand, heads as the 8-column one): S^T = K Q^T, the online softmax (base 2,
// `scale2` = scale * log2 e folded in) over the keys k_lo <= j < k_end, and O^T += V^T P^T.  `kt`, `vt`:
// the tile's keys and values in shared memory as the tensor copies write them (128-byte swizzle);
// `jb`: the token of the tile's first row; qf: the query fragments (head lane / 4, dims 16k + 2(lane % 4) ..
// and + 8); o[db][c]: dim db*16 + lane/4 + 8*(c/2), head 2(lane % 4) + (c & 1); m_run, l_run: heads
// 2(lane % 4) and + 1, the sums still spread over the lanes that hold different keys.
__device__ __forceinline__ void consume_tile(uint32_t kt, uint32_t vt, const uint32_t (&qf)[KSTEPS][2], float (&o)[HD / 16][4],
                                             float (&m_run)[2], float (&l_run)[2], int jb, int k_lo, int k_end, float scale2,
                                             int lane) {
  const int g = lane >> 2;
  const int lm = lane >> 3, lr = lane & 7;
  // S^T = K Q^T: 64 keys x 8 heads; sc[mb][c]: key mb*16 + g + 8*(c/2), head 2t + (c&1)
  float sc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) sc[i][c] = 0.f;
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
#pragma unroll
    for (int mb = 0; mb < 4; ++mb) {
      // matrices: (keys mb*16 + 0..7, d k*16 + 0..7), (keys + 8, d), (keys, d + 8), (keys + 8, d + 8)
      uint32_t kf[4];
      ldmatrix_x4(kf, tile_addr(kt, mb * 16 + (lm & 1) * 8 + lr, k * 2 + (lm >> 1)));
      mma_bf16(sc[mb], kf, qf[k][0], qf[k][1]);
    }
  }
  // keys outside k_lo .. k_end do not count; softmax update per head (a column)
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = jb + i * 16 + g + 8 * (c >> 1);
      const float v = (j >= k_lo && j < k_end) ? sc[i][c] * scale2 : -INFINITY;
      sc[i][c] = v;
      mx[c & 1] = fmaxf(mx[c & 1], v);
    }
  float alpha[2], m_use[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
    const float m_new = fmaxf(m_run[h], mx[h]);
    m_use[h] = m_new == -INFINITY ? 0.f : m_new;
    alpha[h] = exp2f(m_run[h] - m_use[h]);
    m_run[h] = m_new;
    l_run[h] *= alpha[h];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float pe = exp2f(sc[i][c] - m_use[c & 1]);
      sc[i][c] = pe;
      l_run[c & 1] += pe;
    }
#pragma unroll
  for (int i = 0; i < HD / 16; ++i) {
    o[i][0] *= alpha[0]; o[i][1] *= alpha[1];
    o[i][2] *= alpha[0]; o[i][3] *= alpha[1];
  }
  // O^T += V^T P^T
#pragma unroll
  for (int kb = 0; kb < 4; ++kb) {
    // P^T as the 8-column operand: the 8x8 blocks (keys x heads) of the scores, transposed
    const uint32_t pb0 = movmatrix_trans(pack_bf16(sc[kb][0], sc[kb][1]));
    const uint32_t pb1 = movmatrix_trans(pack_bf16(sc[kb][2], sc[kb][3]));
#pragma unroll
    for (int db = 0; db < HD / 16; ++db) {
      // transposed: (keys kb*16 + 0..7, d db*16 + 0..7), (keys, d + 8), (keys + 8, d), (keys + 8, d + 8)
      uint32_t vf[4];
      ldmatrix_x4_trans(vf, tile_addr(vt, kb * 16 + (lm >> 1) * 8 + lr, db * 2 + (lm & 1)));
      mma_bf16(o[db], vf, pb0, pb1);
    }
  }
}

}  // namespace
