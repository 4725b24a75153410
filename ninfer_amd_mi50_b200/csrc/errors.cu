// Error reporting of the kernel library (see common.cuh).
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace nf {
static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return 2;
  }
  return 0;
}
}  // namespace nf

extern "C" const char* nf_last_error() { return nf::g_error; }

extern "C" int nf_abi_version() { return 1; }
