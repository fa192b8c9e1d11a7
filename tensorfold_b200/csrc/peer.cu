// Expert parallelism over NVLink peer memory: the two exchanges of an expert-parallel step done by this library's own
// kernels with plain loads and stores to the peers' buffers (no NCCL call, no TMA, no multicast):
//   * tokens: every rank copies its rows into its own window; after a flag barrier each rank PULLS all ranks' rows into
//     a local buffer (a few hundred KB) and the layer's kernels read only local memory;
//   * results: the kernel that forms a rank's per-token partial sums (its experts' slots, weights applied, slot order)
//     PUSHES each token's row straight into the home rank's slot for this rank; after a second flag barrier the home
//     rank adds the ranks' rows in rank order and rounds to bf16.
// Buffers are double-buffered by the parity of a device-side step counter, so two barriers a step suffice and the
// whole step can be replayed from a CUDA graph.  Every wait is bounded (about a second): on a time-out the device
// status word is set and the kernel returns.  (No counterpart in the reference, which has no expert parallelism:
// src/tensorfold/cuda/comm.py is a 2-rank all-gather.)

#include "api.h"
#include "common.cuh"

namespace tfb {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 r;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p)
               : "memory");
  return r;
}

// One warp.  Lane i < world tells rank i "rank `rank` reached barrier number v" and waits until rank i said the same.
// flags: each rank's window starts with [2][world] counters (which = 0: tokens ready, 1: results ready).
// `count` is this rank's local count of barriers of each kind.
__global__ void __launch_bounds__(32)
peer_barrier_kernel(uint8_t* const* __restrict__ windows, int rank, int world, int which, uint32_t* __restrict__ count) {
  pdl_wait();
  const int lane = threadIdx.x;
  const uint32_t v = count[which] + 1;
  __syncwarp();
  if (lane == 0) count[which] = v;
  __threadfence_system();                              // what this GPU wrote before the barrier is visible to the peers
  if (lane < world) {
    uint32_t* theirs = reinterpret_cast<uint32_t*>(windows[lane]) + which * world + rank;
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(windows[rank]) + which * world + lane;
    st_release_sys(theirs, v);
    uint64_t start = 0;
    bool ok = false;
    for (uint32_t spin = 0; spin < (1u << 28); ++spin) {
      if ((int32_t)(ld_acquire_sys(mine) - v) >= 0) {
        ok = true;
        break;
      }
      if ((spin & 255u) == 255u) {
        const uint64_t now = global_ns();
        if (start == 0) start = now;
        else if (now - start > 1000000000ull) break;
      }
    }
    if (!ok) atomicExch(&g_kernel_status, ST_WAIT_TIMEOUT);
  }
  __syncwarp();
  __threadfence_system();
  pdl_launch_dependents();
}

// x_local [rows, D] bf16 -> this rank's token window of the current parity.
__global__ void __launch_bounds__(256)
peer_stage_kernel(const uint4* __restrict__ x_local, uint8_t* __restrict__ window, int64_t x_offset, int64_t x_bytes,
                  const uint32_t* __restrict__ count) {
  pdl_wait();
  const int parity = count[0] & 1;                     // barriers of kind 0 passed so far = steps completed
  uint4* dst = reinterpret_cast<uint4*>(window + x_offset + parity * x_bytes);
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < x_bytes / 16; i += (int64_t)gridDim.x * 256) dst[i] = x_local[i];
  pdl_launch_dependents();
}

// After the tokens barrier: x_all [world * rows, D] <- every rank's window (parity of the step just opened).
__global__ void __launch_bounds__(256)
peer_gather_kernel(uint8_t* const* __restrict__ windows, int world, int64_t x_offset, int64_t x_bytes,
                   uint4* __restrict__ x_all, const uint32_t* __restrict__ count) {
  pdl_wait();
  const int parity = (count[0] - 1) & 1;               // the tokens barrier of this step has been counted already
  const int64_t per = x_bytes / 16;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < per * world; i += (int64_t)gridDim.x * 256) {
    const int r = (int)(i / per);
    const int64_t j = i - (int64_t)r * per;
    x_all[i] = ld_relaxed_sys_v4(windows[r] + x_offset + parity * x_bytes + j * 16);
  }
  pdl_launch_dependents();
}

// This rank's partial sum of every token (slots whose expert lies in [lo, lo + n), fp32 fma chain in slot order),
// written into the token's home rank: windows[home] + p_offset + parity * p_bytes + ((rank * rows + j) * D) * 4.
__global__ void __launch_bounds__(256)
combine_push_kernel(const float* __restrict__ y, const float* __restrict__ wts, const int* __restrict__ pick, int lo,
                    int n, uint8_t* const* __restrict__ windows, int64_t p_offset, int64_t p_bytes, int rank, int rows,
                    int S, int D, const uint32_t* __restrict__ count) {
  const int r = blockIdx.x;
  const int d = (blockIdx.y * 256 + threadIdx.x) * 4;
  if (d >= D) return;
  pdl_wait();
  const int parity = (count[0] - 1) & 1;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < S; ++s) {
    const int e = pick[(size_t)r * S + s] - lo;
    if (e < 0 || e >= n) continue;
    const float w = wts[(size_t)r * S + s];
    const float4 f = *reinterpret_cast<const float4*>(y + ((size_t)r * S + s) * D + d);
    acc[0] = fmaf(w, f.x, acc[0]);
    acc[1] = fmaf(w, f.y, acc[1]);
    acc[2] = fmaf(w, f.z, acc[2]);
    acc[3] = fmaf(w, f.w, acc[3]);
  }
  const int home = r / rows, j = r - home * rows;
  float* dst = reinterpret_cast<float*>(windows[home] + p_offset + parity * p_bytes) + ((size_t)rank * rows + j) * D + d;
  *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  pdl_launch_dependents();
}

// After the results barrier: out [rows, D] bf16 = the ranks' rows added in rank order.
__global__ void __launch_bounds__(256)
peer_sum_kernel(const uint8_t* __restrict__ window, int64_t p_offset, int64_t p_bytes, int world, int rows, int D,
                __nv_bfloat16* __restrict__ out, const uint32_t* __restrict__ count) {
  pdl_wait();
  const int parity = (count[0] - 1) & 1;
  const float* part = reinterpret_cast<const float*>(window + p_offset + parity * p_bytes);
  const int64_t n4 = (int64_t)rows * D / 4;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (int64_t)gridDim.x * 256) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const uint4 u = ld_relaxed_sys_v4(part + (size_t)r * rows * D + i * 4);
      acc.x += __uint_as_float(u.x);
      acc.y += __uint_as_float(u.y);
      acc.z += __uint_as_float(u.z);
      acc.w += __uint_as_float(u.w);
    }
    __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    reinterpret_cast<uint2*>(out)[i] = o;
  }
  pdl_launch_dependents();
}

}  // namespace tfb

using namespace tfb;

// windows: DEVICE array of `world` pointers, entry i = rank i's window as mapped into this process (entry `rank` is
// this rank's own).  A window holds: [2][world] uint32 barrier counters, then at x_offset two token buffers of x_bytes,
// then at p_offset two result buffers of p_bytes = world * rows * D * 4.  count: 2 local uint32 (zero at start).

extern "C" int tfb_peer_barrier(void* const* windows, int rank, int world, int which, void* count, void* stream) {
  TFB_REQUIRE(windows && count, "peer_barrier: null pointer");
  TFB_REQUIRE(world >= 1 && world <= 32 && rank >= 0 && rank < world, "peer_barrier: rank %d of %d", rank, world);
  TFB_REQUIRE(which == 0 || which == 1, "peer_barrier: which is 0 (tokens) or 1 (results)");
  return check_cuda(launch(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                           reinterpret_cast<uint8_t* const*>(windows), rank, world, which,
                           static_cast<uint32_t*>(count)),
                    "peer_barrier");
}

extern "C" int tfb_peer_stage(const void* x_local, void* window, int64_t x_offset, int64_t x_bytes, const void* count,
                              void* stream) {
  TFB_REQUIRE(x_local && window && count, "peer_stage: null pointer");
  TFB_REQUIRE(x_bytes > 0 && x_bytes % 16 == 0 && x_offset % 16 == 0 && aligned16(x_local), "peer_stage: 16-byte units");
  const int grid = (int)((x_bytes / 16 + 255) / 256 < 592 ? (x_bytes / 16 + 255) / 256 : 592);
  return check_cuda(launch(peer_stage_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const uint4*>(x_local), static_cast<uint8_t*>(window), x_offset, x_bytes,
                           static_cast<const uint32_t*>(count)),
                    "peer_stage");
}

extern "C" int tfb_peer_gather(void* const* windows, int world, int64_t x_offset, int64_t x_bytes, void* x_all,
                               const void* count, void* stream) {
  TFB_REQUIRE(windows && x_all && count, "peer_gather: null pointer");
  TFB_REQUIRE(x_bytes > 0 && x_bytes % 16 == 0 && x_offset % 16 == 0 && aligned16(x_all), "peer_gather: 16-byte units");
  const int64_t n = x_bytes / 16 * world;
  const int grid = (int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  return check_cuda(launch(peer_gather_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           reinterpret_cast<uint8_t* const*>(windows), world, x_offset, x_bytes,
                           static_cast<uint4*>(x_all), static_cast<const uint32_t*>(count)),
                    "peer_gather");
}

extern "C" int tfb_combine_push(const float* y, const float* wts, const int32_t* pick, int lo, int n,
                                void* const* windows, int64_t p_offset, int64_t p_bytes, int rank, int rows_local,
                                int T, int slots, int D, const void* count, void* stream) {
  TFB_REQUIRE(y && wts && pick && windows && count, "combine_push: null pointer");
  TFB_REQUIRE(D > 0 && D % 4 == 0 && slots >= 1 && rows_local >= 1 && T % rows_local == 0,
              "combine_push: D %% 4 == 0 and T a multiple of the rows a rank");
  TFB_REQUIRE(p_offset % 16 == 0 && p_bytes % 16 == 0, "combine_push: 16-byte units");
  if (T <= 0) return TFB_OK;
  return check_cuda(launch(combine_push_kernel, dim3(T, (D + 1023) / 1024), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), y, wts, pick, lo, n,
                           reinterpret_cast<uint8_t* const*>(windows), p_offset, p_bytes, rank, rows_local, slots, D,
                           static_cast<const uint32_t*>(count)),
                    "combine_push");
}

extern "C" int tfb_peer_sum(const void* window, int64_t p_offset, int64_t p_bytes, int world, int rows_local, int D,
                            void* out, const void* count, void* stream) {
  TFB_REQUIRE(window && out && count, "peer_sum: null pointer");
  TFB_REQUIRE(D > 0 && D % 4 == 0 && rows_local >= 1 && world >= 1, "peer_sum: bad sizes");
  const int64_t n4 = (int64_t)rows_local * D / 4;
  const int grid = (int)((n4 + 255) / 256 < 592 ? (n4 + 255) / 256 : 592);
  return check_cuda(launch(peer_sum_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const uint8_t*>(window), p_offset, p_bytes, world, rows_local, D,
                           static_cast<__nv_bfloat16*>(out), static_cast<const uint32_t*>(count)),
                    "peer_sum");
}
