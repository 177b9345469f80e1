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

// FASTMLX_PDL=0 turns programmatic dependent launch off (every kernel then waits for the one
// before it to finish before it is scheduled).
static int g_pdl = -1;
bool fmx_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("FASTMLX_PDL");
    g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_pdl == 1;
}
FMX_EXPORT void fmx_set_pdl(int on) { g_pdl = on ? 1 : 0; }

FMX_EXPORT const char* fmx_last_error() { return g_error; }

FMX_EXPORT int fmx_abi_version() { return 1; }
