// Host-side helpers shared by the C-ABI entry points: status codes, last-error text, launch checks.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#define TFB_OK 0
#define TFB_ERR_ARG (-1)      // a bad argument; nothing was launched
#define TFB_ERR_CUDA (-2)     // the CUDA runtime refused a call
#define TFB_ERR_DEVICE (-3)   // a kernel recorded a failure in the device status word

namespace tfb {

// printf-style: stores the message for tfb_last_error() and returns `code`
int fail(int code, const char* fmt, ...);

inline int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return TFB_OK;
  return fail(TFB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

inline int check_launch(const char* what) { return check_cuda(cudaGetLastError(), what); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// When set (tfb_set_pdl), kernels are launched with programmatic stream serialization: a kernel may start while the
// one before it in the stream drains, and waits (griddepcontrol.wait) before it touches global memory.
extern int g_use_pdl;

// How long a barrier between expert-parallel ranks waits before it gives up (tfb_set_wait_limit_ms), in nanoseconds.
uint64_t wait_limit_ns();

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tfb

#define TFB_REQUIRE(cond, ...)                                  \
  do {                                                          \
    if (!(cond)) return ::tfb::fail(TFB_ERR_ARG, __VA_ARGS__);  \
  } while (0)

#define TFB_CUDA(call, what)                      \
  do {                                            \
    int rc_ = ::tfb::check_cuda((call), (what));  \
    if (rc_ != TFB_OK) return rc_;                \
  } while (0)
