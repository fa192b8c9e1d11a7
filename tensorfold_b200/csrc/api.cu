// Library-wide state behind the C ABI: the last error text, the device status word, launch options.

#include "api.h"
#include "common.cuh"

#include <mutex>

namespace tfb {

int g_use_pdl = 0;
static int g_wait_limit_ms = 1000;

uint64_t wait_limit_ns() { return (uint64_t)g_wait_limit_ms * 1000000ull; }

static thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace tfb

using namespace tfb;

extern "C" const char* tfb_last_error(void) { return g_error; }

extern "C" int tfb_version(void) { return 1; }

extern "C" int tfb_set_pdl(int on) {
  const int was = g_use_pdl;
  g_use_pdl = on ? 1 : 0;
  return was;
}

// Sets how long the barriers of an expert-parallel step (csrc/peer.cu) wait for the other ranks, in milliseconds
// (1 .. 600000; one second unless set); returns the previous limit, or -1 for a value out of range.  The limit is read
// when a step is launched or captured.  Long enough for the slowest rank's host to reach its launch (first calls,
// graph instantiation), short enough that a rank that died is reported instead of waited for.
extern "C" int tfb_set_wait_limit_ms(int ms) {
  if (ms < 1 || ms > 600000) return fail(TFB_ERR_ARG, "set_wait_limit_ms: %d ms outside 1..600000", ms);
  const int was = g_wait_limit_ms;
  g_wait_limit_ms = ms;
  return was;
}

// Reads the current device's status word (0 = no kernel recorded a failure) and clears it; synchronises `stream`.
extern "C" int tfb_kernel_status(int* status, void* stream) {
  TFB_REQUIRE(status, "kernel_status: null pointer");
  auto st = static_cast<cudaStream_t>(stream);
  int v = 0;
  TFB_CUDA(cudaMemcpyFromSymbolAsync(&v, g_kernel_status, sizeof v, 0, cudaMemcpyDeviceToHost, st),
           "kernel_status: read");
  TFB_CUDA(cudaStreamSynchronize(st), "kernel_status: synchronize");
  if (v != 0) {
    const int zero = 0;
    TFB_CUDA(cudaMemcpyToSymbolAsync(g_kernel_status, &zero, sizeof zero, 0, cudaMemcpyHostToDevice, st),
             "kernel_status: clear");
    TFB_CUDA(cudaStreamSynchronize(st), "kernel_status: synchronize");
  }
  *status = v;
  return TFB_OK;
}
