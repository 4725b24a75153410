// Error reporting of the kernel library (see common.cuh).
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace nf {
int g_chained_launch = -1;
static thread_local bool g_chain_break = false;
bool take_chain_break() {
  const bool b = g_chain_break;
  g_chain_break = false;
  return b;
}
void set_chain_break() { g_chain_break = true; }
int g_chain_outside_capture = 1;      // nf_set_chained_launch_outside_capture(0): chain only while a stream captures
bool chain_this_launch(int cls, cudaStream_t stream) {
  const bool pending_break = take_chain_break();          // consumed by this launch either way
  if (!(g_chained_launch & cls) || pending_break) return false;
  if (g_chain_outside_capture) return true;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return st == cudaStreamCaptureStatusActive;
}
static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static thread_local cudaError_t g_noted = cudaSuccess;

void note_launch_error(cudaError_t e) { g_noted = e; }

int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e == cudaSuccess) e = g_noted;
  g_noted = cudaSuccess;
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

// 1 (default): kernels are launched with programmatic stream serialization (they may begin while
// their predecessor drains) whether or not the stream is being captured; 0: only inside a capture.
extern "C" int nf_set_chained_launch_outside_capture(int on) {
  nf::g_chain_outside_capture = on ? 1 : 0;
  return 0;
}

extern "C" int nf_chain_break() {
  nf::set_chain_break();
  return 0;
}

extern "C" int nf_set_chained_launch(int on) {
  nf::g_chained_launch = on;
  return 0;
}
