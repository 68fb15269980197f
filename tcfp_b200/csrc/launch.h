// Host-side plumbing shared by the translation units of libtcfp_b200:
// thread-local error text, CUDA error mapping, device properties.
#pragma once

#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>

#include "../../include/tcfp_b200.h"

namespace tcfp {

// records a printf-style message for tcfp_last_error() and returns `code`
int fail(int code, const char* fmt, ...);
// number of SMs of the current device (cached per device)
int sm_count();

}  // namespace tcfp

#define CUDA_TRY(expr)                                                                         \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return ::tcfp::fail(TCFP_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));      \
  } while (0)
