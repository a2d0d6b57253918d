// The sampler: one block per row of float32 logits.
//
//   temperature <= 0      arg-max, lowest index among equals
//   otherwise             z = logit / temperature; keep the top_k largest (0: all), then the
//                         smallest set of the most likely tokens whose probability reaches top_p
//                         (1: all); draw from softmax(kept z) by the Gumbel-max rule:
//                         token = argmax_i (z_i - log(-log u_i)),
//                         u_i = uniform(seed, counter, i) from a counter-based generator.
//
// The reference samples with temperature, top-k and top-p through a library softmax and inverse
// CDF (miniinfer/layers/sample.py:111-128) from the global generator, so its draws depend on what
// else is in the batch.  Here a draw is a function of (logits row, seed, counter) alone.
//
// Thresholds are found exactly by a 4 x 8-bit radix walk over the order-preserving integer image
// of z: counts per bin for top-k, probability mass per bin for top-p.  Mass is held as 64-bit
// fixed point (exp(z - max) * 2^40, integer adds), so the walk does not depend on the order in
// which threads add.  Entries equal to a threshold are all kept.  The histograms are kept per warp
// and added up at the end of a pass, and a row is spread over a cluster of up to eight blocks (a row of 151936
// logits: top-p 0.13 ms, top-k 0.05 ms; with one block per row and one histogram that a thousand threads add to
// with 64-bit shared-memory atomics, most of them to the same few bins, top-p took 2.2 ms).
//
// Two launches: (1) a cluster of up to eight blocks per row finds the row's threshold, each block on its part of
// the row, the blocks' histograms added up through distributed shared memory (rows without top-k/top-p leave at
// once); (2) the vocabulary of each row is cut into slices, one block per (slice, row) finds the
// slice's best perturbed score, and the last block of a row to finish picks the row's best.  The
// arg-max with its lowest-index rule is associative, so the slicing does not change the result.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

// The 23 random bits of (key, index).
__device__ __forceinline__ uint32_t uniform_bits(uint64_t key, int index) {
  return (uint32_t)(mix64(key ^ ((uint64_t)index * 0xD1342543DE82EF95ull)) >> 41);
}
__device__ __forceinline__ float uniform_of_bits(uint32_t n) {
  // 23 bits: (n + 0.5) * 2^-23 is exact in float32 and lies in [2^-24, 1 - 2^-24], strictly inside
  // (0, 1).  With 24 bits the largest n + 0.5 would round up and give u = 1, whose noise is +inf.
  return ((float)n + 0.5f) * (1.0f / 8388608.0f);
}
// Seven draws in eight have u < 7/8, whose noise -log(-log(u)) is below 2.0135: a bound that needs no logarithm.
constexpr uint32_t SMALL_NOISE_BITS = 7u << 20;         // n below this: u < 7/8
constexpr float SMALL_NOISE = 2.02f;

__device__ __forceinline__ uint32_t ordered(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Best {
  float v;
  int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ Best block_argmax(Best mine, Best* scratch /* 32 */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
    mine = better(mine, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    Best b = scratch[lane];  // THREADS / 32 == 32 warps
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other;
      other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = better(b, other);
    }
    if (lane == 0) scratch[0] = b;
  }
  __syncthreads();
  return scratch[0];
}

// Histograms without contention.  The top byte of the ordered image takes a handful of values for real
// logits, so a block-wide histogram in shared memory has a thousand threads adding to three or four
// words - and 64-bit shared-memory adds are compare-and-swap loops.  Here every warp has a histogram of
// its own for the mass; in each step the lanes of a warp that hit the same bin find each other (match.any), one of them
// takes the group's sum (redux) and adds it to the warp's bin with plain loads and stores - the groups of a
// step hit different bins, and a warp's steps follow each other - and at the end of a pass the warps'
// histograms are added up, bin by bin.  Integer sums: the result does not depend on the order.
constexpr int WARPS_T = THREADS / 32;

__device__ __forceinline__ void warp_hist_add(unsigned long long* mine /* [256] of this warp */, bool active, unsigned bin,
                                              unsigned long long value) {
  const unsigned live = __ballot_sync(0xffffffffu, active);
  if (!active) return;
  const unsigned group = __match_any_sync(live, bin);
  // the sum of a group's values, 24 bits at a time (32 lanes of 24 bits fit a 32-bit redux)
  const unsigned lo = __reduce_add_sync(group, (unsigned)(value & 0xffffffull));
  const unsigned mid = __reduce_add_sync(group, (unsigned)((value >> 24) & 0xffffffull));
  const unsigned hi = __reduce_add_sync(group, (unsigned)(value >> 48));
  if ((threadIdx.x & 31) == __ffs(group) - 1)
    mine[bin] += (unsigned long long)lo + ((unsigned long long)mid << 24) + ((unsigned long long)hi << 48);
}

// Launch 1: thresholds.  thr[row] = smallest ordered image that is kept (0: everything).
__global__ void __launch_bounds__(THREADS)
sample_threshold_kernel(uint32_t* __restrict__ thr_out, const float* __restrict__ logits,
                        const float* __restrict__ temperature, const int* __restrict__ top_k,
                        const float* __restrict__ top_p, int V) {
  mi::grid_dependency_sync();
  extern __shared__ unsigned long long warp_hist[];          // [WARPS_T][256]
  __shared__ Best best_scratch[32];
  __shared__ unsigned long long hist[256];                   // the warps' histograms added up
  __shared__ unsigned int sh_prefix;
  __shared__ unsigned long long sh_above;
  __shared__ unsigned long long sh_rank;

  // A row belongs to a cluster of C blocks (gridDim.x = C), each of which walks a C-th of the row; after a pass
  // the blocks' histograms are added up through distributed shared memory, and every block walks the sum.
  __shared__ float sh_max;
  const int C = (int)gridDim.x, rank = (int)blockIdx.x;
  const int row = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* x = logits + (size_t)row * V;
  const float temp = temperature[row];
  const int k = top_k[row];
  const float p = top_p[row];
  const bool use_k = k > 0 && k < V, use_p = p < 1.f;
  if (!(temp > 0.f) || (!use_k && !use_p)) {                  // the same for every block of the cluster
    if (threadIdx.x == 0 && rank == 0) thr_out[row] = 0u;
    return;
  }
  uint32_t thr_k = 0u, thr_p = 0u;  // keep entries whose ordered image is >= both
  unsigned long long* mine = warp_hist + (size_t)warp * 256;
  const int part = ((V + C - 1) / C + 31) / 32 * 32;          // this block's part of the row: whole warps walk it together
  const int i_begin = rank * part, i_end = min(V, i_begin + part);
  // the sum over the cluster of what every block has in hist[] (nothing to do for a cluster of one)
  auto cluster_sum = [&]() {
    if (C == 1) return;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    unsigned long long t = 0ull;
    if (threadIdx.x < 256)
      for (int r = 0; r < C; ++r) t += cluster.map_shared_rank(hist, r)[threadIdx.x];
    cluster.sync();                                           // everybody has read: hist may be overwritten
    if (threadIdx.x < 256) hist[threadIdx.x] = t;
    __syncthreads();
  };

  // One pass of a radix walk: the histogram, over bin = byte `shift` of the ordered image, of value(i) over the
  // entries whose higher bytes equal `prefix` (and that `keep` lets through).  Result in hist[].
  // Counts go to one histogram of the block with 32-bit shared-memory adds, which the hardware does itself (a
  // row of 151936 logits, top-k: 150 us that way, 430 us through the warps' histograms).
  auto count_pass = [&](int shift, uint32_t prefix, uint32_t mask) {
    unsigned int* counts = reinterpret_cast<unsigned int*>(warp_hist);
    if (threadIdx.x < 256) counts[threadIdx.x] = 0u;
    __syncthreads();
    for (int i = i_begin + threadIdx.x; i < i_end; i += THREADS) {
      const uint32_t u = ordered(x[i] / temp);
      if ((u & mask) == prefix) atomicAdd(&counts[(u >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x < 256) hist[threadIdx.x] = counts[threadIdx.x];
    __syncthreads();
    cluster_sum();
  };
  auto pass = [&](int shift, uint32_t prefix, uint32_t mask, auto value_of) {
    for (int b = lane; b < 256; b += 32) mine[b] = 0ull;
    __syncwarp();
    for (int i = i_begin + threadIdx.x; i < i_begin + part; i += THREADS) {
      bool active = i < i_end;
      unsigned bin = 0;
      unsigned long long val = 0ull;
      if (active) {
        const float z = x[i] / temp;
        const uint32_t u = ordered(z);
        active = u >= thr_k && (u & mask) == prefix;
        if (active) {
          bin = (u >> shift) & 255u;
          val = value_of(z);
          active = val != 0ull;
        }
      }
      warp_hist_add(mine, active, bin, val);
      __syncwarp();
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      unsigned long long t = 0ull;
#pragma unroll 8
      for (int w = 0; w < WARPS_T; ++w) t += warp_hist[(size_t)w * 256 + threadIdx.x];
      hist[threadIdx.x] = t;
    }
    __syncthreads();
    cluster_sum();
  };

  if (use_k) {
    // the k-th largest z: walk the bits from the top, keeping the rank still wanted
    if (threadIdx.x == 0) { sh_prefix = 0u; sh_rank = (unsigned long long)k; }
    __syncthreads();
    for (int ps = 0; ps < 4; ++ps) {
      const int shift = 24 - 8 * ps;
      const uint32_t prefix = sh_prefix;
      const uint32_t mask = ps == 0 ? 0u : (0xffffffffu << (shift + 8));
      count_pass(shift, prefix, mask);
      if (threadIdx.x == 0) {
        unsigned long long want = sh_rank, seen = 0;
        int b = 255;
        for (; b > 0; --b) {
          if (seen + hist[b] >= want) break;
          seen += hist[b];
        }
        sh_rank = want - seen;
        sh_prefix = prefix | ((uint32_t)b << shift);
      }
      __syncthreads();
    }
    thr_k = sh_prefix;
    __syncthreads();
  }

  if (use_p) {
    // max of the kept entries, then their total mass in fixed point
    float mx = -INFINITY;
    for (int i = i_begin + threadIdx.x; i < i_end; i += THREADS) {
      const float z = x[i] / temp;
      if (ordered(z) >= thr_k) mx = fmaxf(mx, z);
    }
    mx = block_argmax(Best{mx, 0}, best_scratch).v;
    if (C > 1) {                                              // the largest of the blocks' maxima
      cg::cluster_group cluster = cg::this_cluster();
      if (threadIdx.x == 0) sh_max = mx;
      cluster.sync();
      for (int r = 0; r < C; ++r) mx = fmaxf(mx, *cluster.map_shared_rank(&sh_max, r));
      cluster.sync();
    }
    if (threadIdx.x == 0) { sh_prefix = 0u; sh_above = 0ull; }
    __syncthreads();
    unsigned long long target = 0ull;  // used by thread 0 only
    for (int ps = 0; ps < 4; ++ps) {
      const int shift = 24 - 8 * ps;
      const uint32_t prefix = sh_prefix;
      const uint32_t mask = ps == 0 ? 0u : (0xffffffffu << (shift + 8));
      pass(shift, prefix, mask, [mx](float z) { return (unsigned long long)(expf(z - mx) * 1099511627776.0f); });
      if (threadIdx.x == 0) {
        if (ps == 0) {
          unsigned long long total = 0ull;
          for (int b = 0; b < 256; ++b) total += hist[b];
          target = (unsigned long long)((double)total * (double)p);
          if (target < 1ull) target = 1ull;
        }
        // first bin, from the top, at which the inclusive mass reaches the target
        unsigned long long above = sh_above;
        int b = 255;
        for (; b > 0; --b) {
          if (above + hist[b] >= target) break;
          above += hist[b];
        }
        sh_above = above;
        sh_prefix = prefix | ((uint32_t)b << shift);
      }
      __syncthreads();
    }
    thr_p = sh_prefix;
  }
  if (threadIdx.x == 0 && rank == 0) thr_out[row] = thr_k > thr_p ? thr_k : thr_p;
}

constexpr size_t THRESHOLD_SMEM = (size_t)WARPS_T * 256 * sizeof(unsigned long long);   // 64 KB

// The threshold kernel's shared memory is more than a kernel gets without asking; asked once per process.
static int configure_threshold_kernel() {
  static bool done = false;
  if (done) return 0;
  cudaError_t e = cudaFuncSetAttribute(sample_threshold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)THRESHOLD_SMEM);
  if (e != cudaSuccess) return mi_fail("sample: cannot get %zu bytes of shared memory: %s", THRESHOLD_SMEM, cudaGetErrorString(e));
  done = true;
  return 0;
}

// Blocks per row of the threshold kernel: a cluster of up to 8, each block at least 8192 logits.
static int threshold_cluster(int V) {
  int c = 1;
  while (c < 8 && V >= 2 * 8192 * c) c *= 2;
  return c;
}

static int launch_thresholds(uint32_t* thr, const float* logits, const float* temperature, const int* top_k, const float* top_p,
                             int R, int V, cudaStream_t stream) {
  if (configure_threshold_kernel()) return 1;
  const int C = threshold_cluster(V);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C, R);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = THRESHOLD_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (mi::pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (C > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = C;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, sample_threshold_kernel, thr, logits, temperature, top_k, top_p, V);
  if (e != cudaSuccess) return mi_fail("sample thresholds: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

constexpr int PICK_THREADS = 256;
constexpr int PICK_BATCH = 8;           // logits a thread loads before it looks at any of them

// Launch 2: best perturbed score of each slice; the last block of a row picks the row's best.
__global__ void __launch_bounds__(PICK_THREADS)
sample_pick_kernel(int* __restrict__ out, const float* __restrict__ logits, const float* __restrict__ temperature,
                   const long long* __restrict__ seed, const long long* __restrict__ counter,
                   const uint32_t* __restrict__ thr_in, float* __restrict__ part_v, int* __restrict__ part_i,
                   int* __restrict__ arrivals, int V, int slices, int slice_len) {
  mi::grid_dependency_sync();
  __shared__ Best scratch[PICK_THREADS / 32];
  __shared__ int s_last;
  const int row = blockIdx.y, slice = blockIdx.x;
  const float* x = logits + (size_t)row * V;
  const float temp = temperature[row];
  const int begin = slice * slice_len, end = min(V, begin + slice_len);
  Best b{-INFINITY, 0x7fffffff};
  // A thread walks its logits in the order of their indices, PICK_BATCH of them loaded at a time: with few rows a
  // slice is long, and a load per turn of the loop would make the walk a chain of memory latencies.
  if (!(temp > 0.f)) {
    for (int i0 = begin + threadIdx.x; i0 < end; i0 += PICK_THREADS * PICK_BATCH) {
      float v[PICK_BATCH];
#pragma unroll
      for (int u = 0; u < PICK_BATCH; ++u) {
        const int i = i0 + u * PICK_THREADS;
        v[u] = i < end ? x[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < PICK_BATCH; ++u) {
        const int i = i0 + u * PICK_THREADS;
        if (i < end) b = better(b, Best{v[u], i});
      }
    }
  } else {
    const uint32_t thr = thr_in[row];
    const uint64_t key = mix64((uint64_t)seed[row] ^ mix64((uint64_t)counter[row] + 0x9E3779B97F4A7C15ull));
    for (int i0 = begin + threadIdx.x; i0 < end; i0 += PICK_THREADS * PICK_BATCH) {
      float v[PICK_BATCH];
#pragma unroll
      for (int u = 0; u < PICK_BATCH; ++u) {
        const int i = i0 + u * PICK_THREADS;
        v[u] = i < end ? x[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < PICK_BATCH; ++u) {
        const int i = i0 + u * PICK_THREADS;
        if (i >= end) continue;
        const float z = v[u] / temp;
        if (ordered(z) < thr || !(z > -INFINITY)) continue;
        // u <= 1 - 2^-24, so the noise -log(-log(u)) stays below 16.7 < 17.4: a score that far under this
        // thread's best cannot win, and its draw need not be worked out
        if (z + 17.4f < b.v) continue;
        const uint32_t n = uniform_bits(key, i);
        if (n < SMALL_NOISE_BITS && z + SMALL_NOISE < b.v) continue;      // the same reasoning with the draw's own bound
        b = better(b, Best{z - logf(-logf(uniform_of_bits(n))), i});
      }
    }
  }
  // block arg-max
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    b = better(b, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = b;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < PICK_THREADS / 32; ++w) b = better(b, scratch[w]);
    part_v[(size_t)row * slices + slice] = b.v;
    part_i[(size_t)row * slices + slice] = b.i;
    __threadfence();
    const int prev = atomicAdd(&arrivals[row], 1);
    s_last = prev == slices - 1;
    if (s_last) arrivals[row] = 0;     // ready for the next launch
  }
  __syncthreads();
  if (!s_last || warp != 0) return;
  __threadfence();
  Best r{-INFINITY, 0x7fffffff};
  for (int s = lane; s < slices; s += 32)
    r = better(r, Best{__ldcg(part_v + (size_t)row * slices + s), __ldcg(part_i + (size_t)row * slices + s)});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, other);
  }
  if (lane == 0) out[row] = r.i < V ? r.i : 0;
}

}  // namespace

// Scratch: `scratch_words` 32-bit words laid out as thr[R], part_v[R * slices], part_i[R * slices];
// `arrivals[R]` must be zero before the first launch (the kernel leaves it zero).
MI_API int mi_sample_scratch_words(int R, int slices) { return R + 2 * R * slices; }

MI_API int mi_sample(int* out, const float* logits, const float* temperature, const int* top_k, const float* top_p,
                     const long long* seed, const long long* counter, void* scratch, int* arrivals, int R, int V,
                     int slices, cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && V > 0, "sample: bad sizes R=%d V=%d", R, V);
  MI_REQUIRE(slices >= 1 && slices <= 65535 && R <= 65535, "sample: bad slicing R=%d slices=%d", R, slices);
  if (R == 0) return 0;
  uint32_t* thr = (uint32_t*)scratch;
  float* part_v = (float*)scratch + R;
  int* part_i = (int*)scratch + R + (size_t)R * slices;
  if (launch_thresholds(thr, logits, temperature, top_k, top_p, R, V, stream)) return 1;
  const int slice_len = (V + slices - 1) / slices;
  mi::launch(sample_pick_kernel, dim3(dim3(slices, R)), dim3(PICK_THREADS), 0, stream, out, logits, temperature, seed, counter, thr, part_v,
                                                                  part_i, arrivals, V, slices, slice_len);
  MI_LAUNCH_OK("sample pick");
  return 0;
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (declared and described in no_alloc_api.h).  Its scratch is a
// fixed array in the library's device image instead of memory the caller passes.
#include "no_alloc_api.h"

#define MI_SAMPLE_STATIC_WORDS 1024   /* thr[R] + best value and index per (row, slice): R + 2 * R * slices, with R * slices <= 384 */
#define MI_SAMPLE_STATIC_MAX_DEVICES 64

// 4 KiB of per-slice results and thresholds, then one arrival counter per row.
static __device__ __align__(256) unsigned int g_sample_static_scratch[MI_SAMPLE_STATIC_WORDS + MI_SAMPLE_STATIC_MAX_ROWS];
static_assert(sizeof(g_sample_static_scratch) == MI_SAMPLE_STATIC_SCRATCH_BYTES, "the header states the size");

// In host code the array's name is only a handle; the kernels need its address on the device,
// which differs from GPU to GPU.  Looked up once per device.
static void* g_sample_static_addr[MI_SAMPLE_STATIC_MAX_DEVICES] = {};

MI_API int mi_sample_static(int* out, const float* logits, const float* temperature, const int* top_k, const float* top_p,
                            const long long* seed, const long long* counter, int R, int V, cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && V > 0, "sample_static: bad sizes R=%d V=%d", R, V);
  MI_REQUIRE(R <= MI_SAMPLE_STATIC_MAX_ROWS, "sample_static: R=%d rows is more than the %d this entry point has scratch for",
             R, MI_SAMPLE_STATIC_MAX_ROWS);
  if (R == 0) return 0;
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return mi_fail("sample_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
  MI_REQUIRE(device >= 0 && device < MI_SAMPLE_STATIC_MAX_DEVICES, "sample_static: device %d is out of range", device);
  if (!g_sample_static_addr[device]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_sample_static_scratch);
    if (e != cudaSuccess || !p) return mi_fail("sample_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_sample_static_addr[device] = p;
  }
  unsigned int* base = (unsigned int*)g_sample_static_addr[device];
  // slices of the vocabulary per row: about two blocks of the pick kernel per SM, bounded so that
  // the results fit the fixed scratch.  Callers of mi_sample choose their own count (the engine asks for
  // more); the token is the same for any count, since the arg-max over slices is associative.
  int slices = (2 * mi::sm_count() < 384 ? 2 * mi::sm_count() : 384) / R;
  if (slices > 64) slices = 64;
  if (slices > (V + 1023) / 1024) slices = (V + 1023) / 1024;
  if (slices < 1) slices = 1;
  MI_REQUIRE(R + 2 * R * slices <= MI_SAMPLE_STATIC_WORDS, "sample_static: scratch too small for R=%d slices=%d", R, slices);
  uint32_t* thr = base;
  float* part_v = (float*)base + R;
  int* part_i = (int*)base + R + (size_t)R * slices;
  int* arrivals = (int*)base + MI_SAMPLE_STATIC_WORDS;
  // the arrival counters must start at zero whatever an earlier call left behind
  e = cudaMemsetAsync(arrivals, 0, sizeof(int) * R, stream);
  if (e != cudaSuccess) return mi_fail("sample_static: cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  if (launch_thresholds(thr, logits, temperature, top_k, top_p, R, V, stream)) return 1;
  const int slice_len = (V + slices - 1) / slices;
  mi::launch(sample_pick_kernel, dim3(slices, R), dim3(PICK_THREADS), 0, stream, out, logits, temperature, seed, counter, thr,
             part_v, part_i, arrivals, V, slices, slice_len);
  MI_LAUNCH_OK("sample_static pick");
  return 0;
}
