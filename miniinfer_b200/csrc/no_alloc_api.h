// One entry point of the common kernel library that never allocates.
//
// It has no counterpart in tom-jerr/MiniInfer; it exists for the callers of THIS library that
// must not allocate device memory at the moment they sample: an embedding application that has
// handed the whole device to its own pool (the engine itself gives nearly all free memory to the
// key/value cache), a serving loop that forbids cudaMalloc on its hot path because the call
// synchronises the device and can fail late under memory pressure, or a host that only lends this
// library its inputs, outputs and a stream.  The regular entry point, mi_sample, asks its caller
// for scratch memory; this one keeps its scratch inside the library.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of rows one call may sample.  The scratch behind the call is a fixed array of
// MI_SAMPLE_STATIC_SCRATCH_BYTES bytes in the library's device image: every GPU that loads the
// library holds that much until the process exits, whether or not the entry point is ever called.
#define MI_SAMPLE_STATIC_MAX_ROWS 256
#define MI_SAMPLE_STATIC_SCRATCH_BYTES 5120

// Samples one token per row of float32 logits [R, V], by the same rule and with the same kernels as
// mi_sample (temperature <= 0: arg-max; otherwise temperature, top-k, top-p and a Gumbel-max draw
// from the counter-based generator keyed by seed and counter), writing int32 tokens to `out`.
// All pointers are device pointers supplied by the caller; the call runs on `stream`.
//
// It calls no cudaMalloc, cudaFree or other allocating routine.  Returns 0, or non-zero with a
// message in mi_last_error() - in particular when R exceeds MI_SAMPLE_STATIC_MAX_ROWS.
//
// The first call on a device looks up the device address of the scratch array (once per device,
// with that device current) and remembers it; make that first call outside of any stream capture.
//
// All calls on a device share the one scratch array.  The part that must start at zero is cleared
// at the start of every call (on `stream`), so an earlier call's contents do no harm; but two calls
// that overlap on the GPU - on different streams, or from different threads - race on it.  Calls on
// one stream are safe.
int mi_sample_static(int* out, const float* logits, const float* temperature, const int* top_k, const float* top_p,
                     const long long* seed, const long long* counter, int R, int V, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
