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
// SMs the persistent GEMM grids may occupy: sm_count() minus the calling thread's
// tcfp_set_sm_reserve() (SMs left free for a collective running beside the GEMM)
int gemm_sm_budget();

}  // namespace tcfp

#define CUDA_TRY(expr)                                                                         \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return ::tcfp::fail(TCFP_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));      \
  } while (0)
