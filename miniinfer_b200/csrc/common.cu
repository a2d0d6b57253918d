// The common library's error text and a version probe.
#include "common.cuh"

MI_DEFINE_LAST_ERROR()

// Compute capability the library was compiled for; callers compare it with the device's.
MI_API int mi_compiled_arch() { return 100; }
