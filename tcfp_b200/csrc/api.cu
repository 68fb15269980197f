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

}  // namespace tcfp

extern "C" int32_t tcfp_version(void) { return 100; }

extern "C" int32_t tcfp_last_error(char* buf, size_t n) {
  if (!buf || n == 0) return TCFP_ERR_INVALID;
  strncpy(buf, tcfp::t_error, n - 1);
  buf[n - 1] = '\0';
  return TCFP_OK;
}

