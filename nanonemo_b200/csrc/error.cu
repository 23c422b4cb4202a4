// Error channel of the launchers and a build-identification symbol.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_err[512] = {0};

void nnb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

extern "C" const char* nnb_last_error() { return g_err; }

extern "C" int nnb_build_arch() {
#ifdef NNB_ARCH
  return NNB_ARCH;
#else
  return 0;
#endif
}
