// Library-level entry points of libtcfp_b200: version, error text, device
// status.  The compute entry points live next to their kernels.
#include <stdio.h>
#include <string.h>

#include "launch.h"

namespace tcfp {

static thread_local char t_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static thread_local int t_sm_reserve = 0;

int gemm_sm_budget() {
  const int n = sm_count() - t_sm_reserve;
  return n < 2 ? 2 : n;
}

}  // namespace tcfp

extern "C" int32_t tcfp_version(void) { return 100; }

extern "C" int32_t tcfp_set_sm_reserve(int32_t n) {
  if (n < 0 || n > 128) return tcfp::fail(TCFP_ERR_INVALID, "sm_reserve must be in [0, 128], got %d", n);
  const int prev = tcfp::t_sm_reserve;
  tcfp::t_sm_reserve = n;
  return prev;
}

extern "C" int32_t tcfp_last_error(char* buf, size_t n) {
  if (!buf || n == 0) return TCFP_ERR_INVALID;
  strncpy(buf, tcfp::t_error, n - 1);
  buf[n - 1] = '\0';
  return TCFP_OK;
}

