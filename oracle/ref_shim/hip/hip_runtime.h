// Stand-in for <hip/hip_runtime.h>: the reference's simple_device_mem.hpp names hipMalloc/hipFree
// (simple_device_mem.hpp:20,25).  The oracle build never allocates device memory; these fail loudly if called.
#pragma once
#include <cstddef>
#include <cstdlib>
#include "hip_fp16.h"
typedef int hipError_t;
static inline hipError_t hipMalloc(void**, std::size_t) { std::abort(); }
static inline hipError_t hipFree(void*) { return 0; }
