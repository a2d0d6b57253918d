// Shared declarations of the sm_100a kernel libraries: the C calling convention, element types,
// error reporting and a few device helpers.
//
// Every exported function returns 0 on success.  On a refused size or a failed launch it returns a
// non-zero code and leaves a message that mi_last_error() of the same library hands out.  Nothing
// is allocated here; callers pass every buffer and the stream.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <utility>

#define MI_API extern "C" __attribute__((visibility("default")))

enum MiDtype { MI_F32 = 0, MI_BF16 = 1 };

inline thread_local char mi_error_text[1024] = "";

inline int mi_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(mi_error_text, sizeof(mi_error_text), fmt, ap);
  va_end(ap);
  return 1;
}

#define MI_REQUIRE(cond, ...)              \
  do {                                     \
    if (!(cond)) return mi_fail(__VA_ARGS__); \
  } while (0)

#define MI_LAUNCH_OK(name)                                                              \
  do {                                                                                  \
    cudaError_t mi_e = cudaGetLastError();                                              \
    if (mi_e != cudaSuccess) return mi_fail("%s: launch failed: %s", name, cudaGetErrorString(mi_e)); \
  } while (0)

// Each library defines mi_last_error once with this.
#define MI_DEFINE_LAST_ERROR() \
  MI_API const char* mi_last_error() { return mi_error_text; }

namespace mi {

// Programmatic dependent launch (on; MINIINFER_B200_PDL=0 turns it off): a kernel launched with
// the attribute may be placed on the SMs while its predecessor in the stream is still running.
// Every kernel of these libraries calls grid_dependency_sync() before it reads anything that a
// kernel writes and before it writes anything at all: it waits until the predecessor has completed
// and its memory operations are visible, and only then lets its own successor be placed.  So at
// most one successor waits on the SMs beside a running kernel, and the order of the work is what
// plain stream order gives.  Before the wait a kernel may only fetch what no kernel writes (weights,
// the step's description that the host uploaded).  Without the attribute both instructions do nothing.
// Measured on a decode step of 229 short kernels: 1.31 ms with it, 1.39 ms without.
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("MINIINFER_B200_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// SMs of the current device, asked once per device (launchers size their grids in SMs; B200 has 148).
inline int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
  }
  return cached[dev];
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ void grid_dependency_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// silu(g) * u as the bfloat16 paths compute it: in float32 with the hardware's exponential and
// reciprocal (errors of a few units in the last place of float32, far below the rounding to bf16
// that follows).  Every bf16 kernel that applies SwiGLU uses this one function, so the fused and the
// two-kernel path agree bit for bit on the same products; the float32 path divides exactly.
__device__ __forceinline__ float silu_mul_fast(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }
__device__ __forceinline__ float silu_mul_exact(float g, float u) { return g / (1.f + expf(-g)) * u; }

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of the additions
// depends only on blockDim, so equal rows give equal sums whatever else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float t = lane < nw ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace mi
