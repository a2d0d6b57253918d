// (shared by gemm_skinny.cu and gemm_skinny_fused.cu)
// bf16 matrix product for few rows (M <= 64): out[M, N] = x[M, K] * w[N, K]^T, fp32 accumulate,
// bf16 or fp32 result.  This is the decode step's and the LM head's product, where the time goes
// into reading the weight matrix once from HBM.
//
// Shape of the work: the weight rows are the long axis.  A warp owns 8*NT weight rows and one
// eighth of K; it streams its weights with 16-byte loads that bypass L1 (each byte is used once),
// reads the matching activations (small, L1/L2 resident) and multiplies on the tensor cores with
// mma.m16n8k16 (activations as the 16-row operand, 8 weight rows as the 8-column operand).  The
// warps that share a group of weight rows (1, 2, 4 or 8 of them, chosen from N alone) cover K
// between them and add their partial tiles in shared memory in a fixed order.  No split across
// blocks, no atomics: the value of an output element is a function of (N, K) alone, so a request's
// logits do not depend on what else is in the batch.
//
// The k index inside a 32-wide block is permuted the same way for both operands so that a thread's
// 16-byte load is exactly its fragment of two consecutive MMAs (thread t of a quad loads
// k = 8t..8t+7; MMA s uses elements 4s..4s+3 of it).
//
// At the sizes of larger models the kernel is further from the memory system's speed than at the
// benchmark's (measured alone with cold weights, 8 rows: 8B-shape QKV, 50 MB, 17.5 us; o, 34 MB,
// 11.1 us; gate-up with SwiGLU, 201 MB, 43 us; down, 101 MB, 22.9 us; the LM head's 1.2 GB stream
// at 5.8 TB/s).  Two variants that keep more bytes in flight were tried for those sizes and were no
// faster: the activations in shared memory and three groups of weight registers (QKV 20.5 us,
// gate-up 49.6 us), and the weights through shared memory with cp.async, three groups deep (gate-up
// 49.0 us, down 27.1 us).  So it is not the depth of the queue of loads that limits these launches;
// their times fit 4 to 5 us per launch for starting and ending plus the bytes at 5.3 TB/s.
//
// The reference calls cuBLAS through nn.Linear for these products
// (miniinfer/models/fused_qwen3.py:95,107,135,137; miniinfer/layers/embedding.py:29-32).
#pragma once
#include "common.cuh"

namespace {

constexpr int WARPS = 8;        // warps of a block; 16 for matrices with so few rows that 8 would leave SMs without a block

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ld_cached(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TOut>
__device__ __forceinline__ void store_out(TOut* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
// out += the product rounded to bf16 (each element has one writer, so no atomics)
__device__ __forceinline__ void add_out(float* p, float v) { *p += __bfloat162float(__float2bfloat16_rn(v)); }
template <int FUSE, typename TOut>
__device__ __forceinline__ void put_out(TOut* p, float v) {
  if constexpr (FUSE == 2) add_out(p, v);
  else store_out<TOut>(p, v);
}

// Eight normalised activations as bf16, from float32 residual values: w * (x * rstd), rounded once.
__device__ __forceinline__ uint4 normed8(const float* x, const float* w, float rstd) {
  const float4 x0 = __ldg(reinterpret_cast<const float4*>(x)), x1 = __ldg(reinterpret_cast<const float4*>(x) + 1);
  const float4 w0 = __ldg(reinterpret_cast<const float4*>(w)), w1 = __ldg(reinterpret_cast<const float4*>(w) + 1);
  const __nv_bfloat162 a = __floats2bfloat162_rn(w0.x * (x0.x * rstd), w0.y * (x0.y * rstd));
  const __nv_bfloat162 b = __floats2bfloat162_rn(w0.z * (x0.z * rstd), w0.w * (x0.w * rstd));
  const __nv_bfloat162 c = __floats2bfloat162_rn(w1.x * (x1.x * rstd), w1.y * (x1.y * rstd));
  const __nv_bfloat162 d = __floats2bfloat162_rn(w1.z * (x1.z * rstd), w1.w * (x1.w * rstd));
  uint4 r;
  r.x = *reinterpret_cast<const uint32_t*>(&a); r.y = *reinterpret_cast<const uint32_t*>(&b);
  r.z = *reinterpret_cast<const uint32_t*>(&c); r.w = *reinterpret_cast<const uint32_t*>(&d);
  return r;
}

// MT: 16-row tiles of x (M <= 16*MT; HALF: M <= 8, the upper 8 rows of the tile are never loaded).
// NT: 8-row tiles of w per warp.  KSPLIT: warps that share a group of weight rows and split K between
// them; a block's 8 warps hold 8 / KSPLIT such groups.  KSPLIT is chosen from N alone.
// SWIGLU (NT == 2): w holds 2N rows, gate rows first; a warp's first tile is 8 gate rows, its second
// the 8 up rows of the same columns, and the result is silu(gate) * up of the bf16-rounded products,
// as the product followed by the activation kernel rounds them.
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float swiglu(float gate, float up) {
  const float g = round_bf16(gate), u = round_bf16(up);
  return mi::silu_mul_fast(g, u);
}

// What may be fused to the product (FUSE; MT == 1 only, the decode step's products):
//   FUSE_NORM   the RMSNorm in front of it: x is not given; `xf` are the float32 residual rows and the
//               activation is norm_w * (xf * rsqrt(mean(xf^2) + eps)) rounded to bf16, the value the norm
//               kernel writes.  Every block works out the (few) rows' sums of squares itself, a warp per
//               row in an order that depends on K alone.
//   FUSE_ADD    the residual add behind it: out is the float32 residual stream and receives
//               out += bf16(product), the value the norm kernel adds when it is given the bf16 product.
enum { FUSE_NONE = 0, FUSE_NORM = 1, FUSE_ADD = 2 };

struct FuseArgs {
  const float* xf;       // FUSE_NORM: residual rows [M, K]
  const float* norm_w;   // FUSE_NORM: norm weights [K]
  float eps;
};

template <int MT, int NT, int KSPLIT, bool HALF, typename TOut, bool SWIGLU = false, int W = WARPS, int FUSE = FUSE_NONE>
__global__ void __launch_bounds__(W * 32, (MT == 1 && W == 8) ? 2 : 1)   // few activation rows: two blocks of 8 warps per SM
gemm_skinny_kernel(TOut* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, int M, int N, int K, int ldo, FuseArgs fa) {
  extern __shared__ float red[];  // [W][MT*16][NT*8 + 1]
  __shared__ float rstd_s[FUSE == FUSE_NORM ? 16 : 1];
  static_assert(FUSE == FUSE_NONE || MT == 1, "the fused forms are for up to 16 rows");
  constexpr int RS = NT * 8 + 1;
  constexpr int GROUPS = W / KSPLIT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int group = warp / KSPLIT, kpart = warp % KSPLIT;
  static_assert(!SWIGLU || NT == 2, "the fused activation pairs one gate tile with one up tile");
  constexpr int COLS = SWIGLU ? 8 : NT * 8;   // output columns of a group of warps
  const int n0 = (blockIdx.x * GROUPS + group) * COLS;

  const int nkb = (K + 31) / 32;
  const int per = (nkb + KSPLIT - 1) / KSPLIT;
  const int kb_begin = kpart * per;
  const int kb_end = min(nkb, kb_begin + per);

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  const __nv_bfloat16* wrow[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j)
    wrow[j] = SWIGLU ? w + ((size_t)min(n0 + g, N - 1) + (size_t)j * N) * K
                     : w + (size_t)min(n0 + j * 8 + g, N - 1) * K;

  // k-blocks are taken U at a time; the loads of the next group are issued before the products of
  // this one, so a warp always has a whole group of 16-byte loads in flight.
  constexpr int LOADS = (HALF ? MT : 2 * MT) + NT;
  constexpr int U = LOADS <= 3 ? 4 : (LOADS <= 6 ? 2 : 1);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 wv[U][NT], xa[U][MT], xb[U][HALF ? 1 : MT];
  uint4 wn[U][NT], xan[U][MT], xbn[U][HALF ? 1 : MT];

  auto load_w = [&](int kb0, uint4 (&w_)[U][NT]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb0 + u) * 32 + 8 * t;
      const bool in = (kb0 + u) < kb_end && k < K;
#pragma unroll
      for (int j = 0; j < NT; ++j) w_[u][j] = in ? ld_stream(wrow[j] + k) : zero;
    }
  };
  auto load_x = [&](int kb0, uint4 (&a_)[U][MT], uint4 (&b_)[U][HALF ? 1 : MT]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb0 + u) * 32 + 8 * t;
      const bool in = (kb0 + u) < kb_end && k < K;
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const int ma = i * 16 + g, mb = ma + 8;
        if constexpr (FUSE == FUSE_NORM) {
          a_[u][i] = (in && ma < M) ? normed8(fa.xf + (size_t)ma * K + k, fa.norm_w + k, rstd_s[ma]) : zero;
          if (!HALF) b_[u][i] = (in && mb < M) ? normed8(fa.xf + (size_t)mb * K + k, fa.norm_w + k, rstd_s[mb]) : zero;
        } else {
          a_[u][i] = (in && ma < M) ? ld_cached(x + (size_t)ma * K + k) : zero;
          if (!HALF) b_[u][i] = (in && mb < M) ? ld_cached(x + (size_t)mb * K + k) : zero;
        }
      }
    }
  };

  // The first two groups of weights are on their way before this kernel waits for its predecessor:
  // the weights are written by no kernel, the activations are.
  if (kb_begin < kb_end) load_w(kb_begin, wv);
  if (kb_begin + U < kb_end) load_w(kb_begin + U, wn);
  mi::grid_dependency_sync();
  if constexpr (FUSE == FUSE_NORM) {
    // a warp per row: lane-strided sum of squares, then the warp's tree - an order that K alone fixes
    for (int m = warp; m < M; m += W) {
      const float4* row = reinterpret_cast<const float4*>(fa.xf + (size_t)m * K);
      float ss = 0.f;
      for (int i = lane; i < K / 4; i += 32) {
        const float4 v = row[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = mi::warp_sum(ss);
      if (lane == 0) rstd_s[m] = rsqrtf(ss / (float)K + fa.eps);
    }
    __syncthreads();
  }
  if (kb_begin < kb_end) load_x(kb_begin, xa, xb);
  for (int kb = kb_begin; kb < kb_end; kb += U) {
    const bool more = kb + U < kb_end;
    if (more) {
      if (kb != kb_begin) load_w(kb + U, wn);
      load_x(kb + U, xan, xbn);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const uint4 b = HALF ? zero : xb[u][HALF ? 0 : i];
          mma_bf16(acc[i][j], xa[u][i].x, b.x, xa[u][i].y, b.y, wv[u][j].x, wv[u][j].y);
          mma_bf16(acc[i][j], xa[u][i].z, b.z, xa[u][i].w, b.w, wv[u][j].z, wv[u][j].w);
        }
    if (more) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int j = 0; j < NT; ++j) wv[u][j] = wn[u][j];
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          xa[u][i] = xan[u][i];
          if (!HALF) xb[u][i] = xbn[u][i];
        }
      }
    }
  }

  const int rows = min(M, MT * 16);
  if (KSPLIT == 1) {
    // no partner: straight from the fragments; element c of (i, j): row i*16 + g + 8*(c/2), col j*8 + 2t + (c&1)
    if constexpr (SWIGLU) {
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int m = i * 16 + g + 8 * (c >> 1), n = n0 + 2 * t + (c & 1);
          if (m < rows && n < N) put_out<FUSE, TOut>(out + (size_t)m * ldo + n, swiglu(acc[i][0][c], acc[i][NT - 1][c]));
        }
      return;
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int m = i * 16 + g + 8 * (c >> 1), n = n0 + j * 8 + 2 * t + (c & 1);
          if (m < rows && n < N) put_out<FUSE, TOut>(out + (size_t)m * ldo + n, acc[i][j][c]);
        }
    return;
  }
  // partial tiles -> shared memory, then the KSPLIT partials of a group are added in a fixed order
  float* mine = red + (size_t)warp * (MT * 16) * RS;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        mine[(i * 16 + g + 8 * (c >> 1)) * RS + j * 8 + 2 * t + (c & 1)] = acc[i][j][c];
  __syncthreads();
  constexpr int PER_GROUP = KSPLIT * 32;           // threads of a group
  const int tid_in_group = kpart * 32 + lane;
  for (int idx = tid_in_group; idx < rows * COLS; idx += PER_GROUP) {
    const int m = idx / COLS, c = idx % COLS;
    const int n = n0 + c;
    if (n >= N) continue;
    float s = 0.f, s_up = 0.f;
#pragma unroll
    for (int ww = 0; ww < KSPLIT; ++ww) {
      const float* tile = red + ((size_t)(group * KSPLIT + ww) * (MT * 16) + m) * RS;
      s += tile[c];
      if (SWIGLU) s_up += tile[8 + c];
    }
    put_out<FUSE, TOut>(out + (size_t)m * ldo + n, SWIGLU ? swiglu(s, s_up) : s);
  }
}

template <int MT, int NT, int KSPLIT, bool HALF, typename TOut, bool SWIGLU, int W = WARPS, int FUSE = FUSE_NONE>
int launch(TOut* out, const __nv_bfloat16* x, const __nv_bfloat16* w, int M, int N, int K, int ldo,
           cudaStream_t stream, FuseArgs fa = FuseArgs{nullptr, nullptr, 0.f}) {
  const size_t smem = KSPLIT == 1 ? 0 : (size_t)W * (MT * 16) * (NT * 8 + 1) * sizeof(float);
  auto kernel = gemm_skinny_kernel<MT, NT, KSPLIT, HALF, TOut, SWIGLU, W, FUSE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return mi_fail("gemm_skinny: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  }
  const int cols_per_block = (W / KSPLIT) * (SWIGLU ? 8 : NT * 8);
  const int blocks = (N + cols_per_block - 1) / cols_per_block;
  mi::launch(kernel, dim3(blocks), dim3(W * 32), smem, stream, out, x, w, M, N, K, ldo, fa);
  MI_LAUNCH_OK("gemm_skinny");
  return 0;
}

template <int MT, int NT, bool HALF, typename TOut, bool SWIGLU = false, int FUSE = FUSE_NONE>
int pick_ksplit(TOut* out, const __nv_bfloat16* x, const __nv_bfloat16* w, int M, int N, int K, int ldo,
                cudaStream_t stream, FuseArgs fa = FuseArgs{nullptr, nullptr, 0.f}) {
  // As few warps per group of rows as still gives every SM about two blocks: long-lived warps that
  // stream many rows keep more bytes in flight than many short-lived blocks.  A function of N and K
  // only, so that the order of the additions behind an output does not depend on the batch.
  const int target = 2 * mi::sm_count();       // two blocks of 8 warps per SM
  const int cols = SWIGLU ? 8 : NT * 8;
  int ks = 1;
  while (ks < 8 && (N + (WARPS / ks) * cols - 1) / ((WARPS / ks) * cols) < target) ks *= 2;
  if (K < 64 * ks) ks = 1;   // nothing to split
  // A little more than one block for every place on the SMs is the worst case: a second round runs
  // with most SMs idle.  Twice the split gives twice the blocks - two to three rounds, far better
  // filled - as long as a warp still walks a stretch of K worth streaming.  (The 8B shape's gate-up
  // product, 201 MB of weights: 384 blocks 46.6 us, 768 blocks 36.6 us.)
  {
    const int blocks = (N + (WARPS / ks) * cols - 1) / ((WARPS / ks) * cols);
    if (ks < 8 && blocks > target && blocks < target * 3 / 2 && K >= 512 * (2 * ks)) ks *= 2;
  }
  // Few rows (a hidden-size output): even one group of rows per block leaves SMs without a block, and
  // each warp would walk a long stretch of K.  Sixteen warps per block halve the stretch and double
  // the bytes in flight.  Few activation rows only: the wide tiles need the registers.
  if constexpr (MT == 1) {
    if (ks == 8 && (N + cols - 1) / cols < mi::sm_count() && K >= 64 * 16)
      return launch<MT, NT, 16, HALF, TOut, SWIGLU, 16, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
  }
  switch (ks) {
    case 1: return launch<MT, NT, 1, HALF, TOut, SWIGLU, WARPS, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
    case 2: return launch<MT, NT, 2, HALF, TOut, SWIGLU, WARPS, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
    case 4: return launch<MT, NT, 4, HALF, TOut, SWIGLU, WARPS, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
    default: return launch<MT, NT, 8, HALF, TOut, SWIGLU, WARPS, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
  }
}

// Up to 16 rows (the decode step's products), with or without a fused norm or residual add.
template <typename TOut, int FUSE>
int dispatch16(TOut* out, const __nv_bfloat16* x, const __nv_bfloat16* w, int M, int N, int K, int ldo,
               cudaStream_t stream, FuseArgs fa) {
  const bool wide = N >= 2048;
  const int blocks16 = (N + 15) / 16;
  if (blocks16 > 2 * mi::sm_count() && blocks16 <= 3 * mi::sm_count() && K >= 512)
    return M <= 8 ? launch<1, 3, 8, true, TOut, false, WARPS, FUSE>(out, x, w, M, N, K, ldo, stream, fa)
                  : launch<1, 3, 8, false, TOut, false, WARPS, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
  if (M <= 8) return wide ? pick_ksplit<1, 2, true, TOut, false, FUSE>(out, x, w, M, N, K, ldo, stream, fa)
                          : pick_ksplit<1, 1, true, TOut, false, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
  return wide ? pick_ksplit<1, 2, false, TOut, false, FUSE>(out, x, w, M, N, K, ldo, stream, fa)
              : pick_ksplit<1, 1, false, TOut, false, FUSE>(out, x, w, M, N, K, ldo, stream, fa);
}

template <typename TOut>
int dispatch(TOut* out, const __nv_bfloat16* x, const __nv_bfloat16* w, int M, int N, int K, int ldo,
             cudaStream_t stream) {
  // Wider warp tiles re-use the activation fragments; narrower ones make more blocks.
  const bool wide = N >= 2048;
  // (16 weight rows per warp where there are many rows: half as many blocks, all of them on the SMs at once)
  // With 16 rows per warp and K split eight ways a block covers 16 rows.  If that makes a little more
  // blocks than the SMs hold at once (two each), 24 rows per warp bring them back under: one round of
  // blocks that all run together instead of a full round and a nearly empty one.
  if (M <= 16) return dispatch16<TOut, FUSE_NONE>(out, x, w, M, N, K, ldo, stream, FuseArgs{nullptr, nullptr, 0.f});
  if (M <= 32) return wide ? pick_ksplit<2, 2, false, TOut>(out, x, w, M, N, K, ldo, stream)
                           : pick_ksplit<2, 1, false, TOut>(out, x, w, M, N, K, ldo, stream);
  return wide ? pick_ksplit<4, 2, false, TOut>(out, x, w, M, N, K, ldo, stream)
              : pick_ksplit<4, 1, false, TOut>(out, x, w, M, N, K, ldo, stream);
}

// out[M, I] = silu(x * w[0:I]^T) * (x * w[I:2I]^T), bf16
template <int FUSE>
int dispatch_swiglu16(__nv_bfloat16* out, const __nv_bfloat16* x, const __nv_bfloat16* w, int M, int I, int K, int ldo,
                      cudaStream_t stream, FuseArgs fa) {
  if (M <= 8) return pick_ksplit<1, 2, true, __nv_bfloat16, true, FUSE>(out, x, w, M, I, K, ldo, stream, fa);
  return pick_ksplit<1, 2, false, __nv_bfloat16, true, FUSE>(out, x, w, M, I, K, ldo, stream, fa);
}

inline int dispatch_swiglu(__nv_bfloat16* out, const __nv_bfloat16* x, const __nv_bfloat16* w, int M, int I, int K, int ldo,
                    cudaStream_t stream) {
  if (M <= 16) return dispatch_swiglu16<FUSE_NONE>(out, x, w, M, I, K, ldo, stream, FuseArgs{nullptr, nullptr, 0.f});
  if (M <= 32) return pick_ksplit<2, 2, false, __nv_bfloat16, true>(out, x, w, M, I, K, ldo, stream);
  return pick_ksplit<4, 2, false, __nv_bfloat16, true>(out, x, w, M, I, K, ldo, stream);
}

}  // namespace
