// Library-wide state behind the C ABI: the last error text, the device status word, launch options.

#include "api.h"
#include "common.cuh"

#include <mutex>

namespace tfb {

int g_use_pdl = 0;

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
