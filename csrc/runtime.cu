// Library-wide host utilities: thread-local error message, version.
#include <stdarg.h>
#include <string.h>

#include "api.h"
#include "common.cuh"

static thread_local char g_err[512] = "";

void pg_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

extern "C" const char* pg_last_error(void) { return g_err; }
extern "C" int pg_version(void) { return 1; }
