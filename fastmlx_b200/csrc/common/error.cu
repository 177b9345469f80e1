// Error text of the C entry points.  Every entry returns 0 or a non-zero code after
// leaving a message here; the Python side raises it.
#include <stdarg.h>
#include <stdio.h>
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

FMX_EXPORT const char* fmx_last_error() { return g_error; }

FMX_EXPORT int fmx_abi_version() { return 1; }
