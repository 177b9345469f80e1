// Error text of the C entry points.  Every entry returns 0 or a non-zero code after
// leaving a message here; the Python side raises it.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include "common.cuh"

static thread_local char g_error[512] = "";

const char* fmx_set_error(const char* msg) {
  snprintf(g_error, sizeof g_error, "%s", msg);
  return g_error;
}

int fmx_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return 1;
}

// Programmatic dependent launch is on; fmx_set_pdl(0) turns it off for this library (every
// kernel then waits for the one before it to finish before it is scheduled), which is how
// its effect is measured.
static int g_pdl = 1;
bool fmx_pdl_enabled() { return g_pdl == 1; }
FMX_EXPORT void fmx_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// Multiprocessors of the current device, asked once per device.
int fmx_num_sms() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

FMX_EXPORT const char* fmx_last_error() { return g_error; }

FMX_EXPORT int fmx_abi_version() { return 1; }
