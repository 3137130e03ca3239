// Per-thread last-error message and library version.
#include <stdarg.h>
#include <stdio.h>

#include "ri_common.cuh"

static thread_local char g_last_error[512] = "";

int ri_fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

extern "C" const char* ri_last_error(void) { return g_last_error; }

extern "C" int ri_version(void) { return 1; }
