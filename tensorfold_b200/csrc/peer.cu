// Expert parallelism over NVLink peer memory: the two exchanges of an expert-parallel step done by this library's own
// kernels with plain loads and stores to the peers' buffers (no NCCL call, no TMA, no multicast):
//   * tokens: every rank has its rows, and the experts and weights it selected for them, in its own window; after a
//     flag barrier each rank PULLS all ranks' rows and selections into local buffers (a few hundred KB) and the layer's
//     kernels read only local memory;
//   * results: the kernel that forms a rank's per-token partial sums (its experts' slots, weights applied, slot order)
//     PUSHES each token's row straight into the home rank's slot for this rank; after a second flag barrier the home
//     rank adds the ranks' rows in rank order and rounds to bf16.
// The two barriers order every reuse: a rank overwrites its token buffer only after it passed the results barrier,
// which every peer signals after its pull; peers overwrite a rank's result buffer only after they passed the next
// tokens barrier, which the rank signals after its sum.  Barrier numbers come from a device-side step counter, so a
// step can be replayed from a CUDA graph.  Every wait is bounded (tfb_set_wait_limit_ms, one second unless set): on a
// time-out the status word records WHICH barrier ran out and the lowest RANK that had not arrived, the kernel returns
// without touching any peer's memory, and every later kernel of this file on that GPU does the same until the host has
// read (and so cleared) the status word.  A step's output is valid only if the status read after it is 0.
// (No counterpart in the reference, which has no expert parallelism: src/tensorfold/cuda/comm.py is a 2-rank
// all-gather.)

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

// Flag barrier folded into the kernel that needs it.  Block 0 tells every rank "rank `rank` reached barrier `target` of
// kind `which`" (what this GPU wrote in earlier kernels is complete by stream order; the fence orders it before the
// flag); then every block waits until all ranks said the same in THIS rank's window.  flags: [2][world] uint32 at the
// start of a window.  Bounded by `limit_ns`: a wait that runs out records (time-out, barrier kind, lowest missing rank)
// in the status word and the call returns false to every thread of the block.  All threads must call it.
__device__ __forceinline__ bool peer_barrier(uint8_t* const* __restrict__ windows, int rank, int world, int which,
                                             uint32_t target, uint64_t limit_ns) {
  __shared__ int arrived;
  if (threadIdx.x == 0) arrived = 1;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    if (blockIdx.x == 0 && blockIdx.y == 0) {
      __threadfence_system();
      if (lane < world) st_release_sys(reinterpret_cast<uint32_t*>(windows[lane]) + which * world + rank, target);
    }
    bool ok = true;
    if (lane < world) {
      const uint32_t* mine = reinterpret_cast<const uint32_t*>(windows[rank]) + which * world + lane;
      uint64_t start = 0;
      ok = false;
      for (uint32_t spin = 0; spin < (1u << 30); ++spin) {
        if ((int32_t)(ld_acquire_sys(mine) - target) >= 0) {
          ok = true;
          break;
        }
        if ((spin & 63u) == 63u) {
          const uint64_t now = global_ns();
          if (start == 0) start = now;
          else if (now - start > limit_ns) break;
        }
      }
    }
    const unsigned late = __ballot_sync(0xffffffffu, !ok);
    if (late != 0u && lane == 0) {
      atomicCAS(&g_kernel_status, 0, status_word(ST_WAIT_TIMEOUT, which + 1, __ffs(late) - 1));
      arrived = 0;
    }
  }
  __syncthreads();
  return arrived != 0;
}

// True when an earlier kernel recorded a failure that the host has not read yet: peers' memory is then left alone.
__device__ __forceinline__ bool step_failed() { return *reinterpret_cast<volatile int*>(&g_kernel_status) != 0; }

// x_local [rows, D] bf16 -> this rank's token buffer (for callers that do not write their tokens there themselves).
__global__ void __launch_bounds__(256)
peer_stage_kernel(const uint4* __restrict__ x_local, uint8_t* __restrict__ window, int64_t x_offset, int64_t x_bytes) {
  pdl_wait();
  uint4* dst = reinterpret_cast<uint4*>(window + x_offset);
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < x_bytes / 16; i += (int64_t)gridDim.x * 256) dst[i] = x_local[i];
  pdl_launch_dependents();
}

// Tokens barrier, then up to PEER_SEGS regions of every rank's window are pulled into local buffers:
// dst[s][r * bytes[s] ...] <- windows[r] + offset[s], for every rank r.  step[0] = steps completed so far.
constexpr int PEER_SEGS = 4;
struct PeerSegs {
  int64_t offset[PEER_SEGS], units[PEER_SEGS];   // units of 16 bytes
  uint4* dst[PEER_SEGS];
  int n;
};

__global__ void __launch_bounds__(256)
peer_gather_kernel(uint8_t* const* __restrict__ windows, int rank, int world, PeerSegs segs,
                   const uint32_t* __restrict__ step, uint64_t limit_ns) {
  pdl_wait();
  if (!peer_barrier(windows, rank, world, 0, step[0] + 1, limit_ns)) return;   // nothing is pulled
  int64_t per = 0;
  for (int s = 0; s < segs.n; ++s) per += segs.units[s];
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < per * world; i += (int64_t)gridDim.x * 256) {
    const int r = (int)(i / per);
    int64_t j = i - (int64_t)r * per;
    int sg = 0;
    while (sg + 1 < segs.n && j >= segs.units[sg]) j -= segs.units[sg++];
    segs.dst[sg][(int64_t)r * segs.units[sg] + j] = ld_relaxed_sys_v4(windows[r] + segs.offset[sg] + j * 16);
  }
  pdl_launch_dependents();
}

// This rank's partial sum of every token (slots whose expert lies in [lo, lo + n), fp32 fma chain in slot order),
// written into the token's home rank: windows[home] + p_offset + ((rank * rows + j) * D) * 4.  Counts the step.
__global__ void __launch_bounds__(256)
combine_push_kernel(const float* __restrict__ y, const float* __restrict__ wts, const int* __restrict__ pick, int lo,
                    int n, uint8_t* const* __restrict__ windows, int64_t p_offset, int rank, int rows, int S, int D,
                    uint32_t* __restrict__ step) {
  const int r = blockIdx.x;
  const int d = (blockIdx.y * 256 + threadIdx.x) * 4;
  pdl_wait();
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) step[0] += 1;     // read by the kernels before and after only
  if (step_failed()) return;                          // a barrier of this step ran out: store nothing into the peers
  if (d < D) {
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
    float* dst = reinterpret_cast<float*>(windows[home] + p_offset) + ((size_t)rank * rows + j) * D + d;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  }
  pdl_launch_dependents();
}

// A rank's partial sums that some other kernel formed (partial [T, D] fp32, row r = token r of the gathered order):
// each row goes to its home rank's result buffer, slot `rank`.  Counts the step, like combine_push_kernel.
__global__ void __launch_bounds__(256)
peer_push_kernel(const float4* __restrict__ partial, uint8_t* const* __restrict__ windows, int64_t p_offset, int rank,
                 int rows, int D, uint32_t* __restrict__ step) {
  const int r = blockIdx.x;
  pdl_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) step[0] += 1;
  if (step_failed()) return;                          // a barrier of this step ran out: store nothing into the peers
  const int home = r / rows, j = r - home * rows;
  float4* dst = reinterpret_cast<float4*>(windows[home] + p_offset) + ((size_t)rank * rows + j) * (D / 4);
  for (int i = threadIdx.x; i < D / 4; i += 256) dst[i] = partial[(size_t)r * (D / 4) + i];
  pdl_launch_dependents();
}

// Selections as one rank sees them: ids of its experts [lo, lo + n) renumbered from 0 with their weights, every other
// slot as id n (which the expert kernels skip) with weight 0.
__global__ void __launch_bounds__(256)
window_picks_kernel(const int* __restrict__ pick, const float* __restrict__ wts, int lo, int n,
                    int* __restrict__ pick_out, float* __restrict__ wts_out, int count) {
  pdl_wait();
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < count) {
    const int e = pick[i] - lo;
    const bool mine = e >= 0 && e < n;
    pick_out[i] = mine ? e : n;
    wts_out[i] = mine ? wts[i] : 0.f;
  }
  pdl_launch_dependents();
}

// Results barrier, then out [rows, D] = the ranks' rows added in rank order, then (when given) extra_w[j] * extra[j, :]
// (the replicated shared expert of the rank's own rows), then (when given) the residual row (bf16; the layer's input:
// out = h + layer(h) without a pass of its own), rounded once to bf16 or stored as fp32.
template <typename TO>
__global__ void __launch_bounds__(256)
peer_sum_kernel(uint8_t* const* __restrict__ windows, int rank, int64_t p_offset, int world, int rows, int D,
                TO* __restrict__ out, const float* __restrict__ extra, const float* __restrict__ extra_w,
                int extra_w_stride, const __nv_bfloat16* __restrict__ residual, const uint32_t* __restrict__ step,
                uint64_t limit_ns) {
  pdl_wait();
  if (step_failed()) return;                          // the tokens barrier ran out: out keeps what it held
  if (!peer_barrier(windows, rank, world, 1, step[0], limit_ns)) return;
  const float* part = reinterpret_cast<const float*>(windows[rank] + p_offset);
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
    if (extra != nullptr) {
      const float w = extra_w[(i * 4 / D) * extra_w_stride];
      const float4 f = reinterpret_cast<const float4*>(extra)[i];
      acc.x = fmaf(w, f.x, acc.x);
      acc.y = fmaf(w, f.y, acc.y);
      acc.z = fmaf(w, f.z, acc.z);
      acc.w = fmaf(w, f.w, acc.w);
    }
    if (residual != nullptr) {
      const uint2 h = reinterpret_cast<const uint2*>(residual)[i];
      acc.x += bf16_lo(h.x);
      acc.y += bf16_hi(h.x);
      acc.z += bf16_lo(h.y);
      acc.w += bf16_hi(h.y);
    }
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(out)[i] = acc;
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(out)[i] = o;
    }
  }
  pdl_launch_dependents();
}

}  // namespace tfb

using namespace tfb;

// windows: DEVICE array of `world` pointers, entry i = rank i's window as mapped into this process (entry `rank` is
// this rank's own).  A window holds: [2][world] uint32 barrier flags, the regions the peers pull (tokens, selections),
// the result buffer of world * rows * D * 4 bytes at p_offset.  step: 1 uint32 in device memory (zero at start).

extern "C" int tfb_peer_stage(const void* x_local, void* window, int64_t x_offset, int64_t x_bytes, void* stream) {
  TFB_REQUIRE(x_local && window, "peer_stage: null pointer");
  TFB_REQUIRE(x_bytes > 0 && x_bytes % 16 == 0 && x_offset % 16 == 0 && aligned16(x_local), "peer_stage: 16-byte units");
  const int grid = (int)((x_bytes / 16 + 255) / 256 < 592 ? (x_bytes / 16 + 255) / 256 : 592);
  return check_cuda(launch(peer_stage_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const uint4*>(x_local), static_cast<uint8_t*>(window), x_offset, x_bytes),
                    "peer_stage");
}

extern "C" int tfb_peer_gather(void* const* windows, int rank, int world, int nseg, const int64_t* seg_offset,
                               const int64_t* seg_bytes, void* const* seg_dst, const void* step, void* stream) {
  TFB_REQUIRE(windows && seg_offset && seg_bytes && seg_dst && step, "peer_gather: null pointer");
  TFB_REQUIRE(world >= 1 && world <= 32 && rank >= 0 && rank < world, "peer_gather: rank %d of %d", rank, world);
  TFB_REQUIRE(nseg >= 1 && nseg <= PEER_SEGS, "peer_gather: 1..%d regions, not %d", PEER_SEGS, nseg);
  PeerSegs segs = {};
  segs.n = nseg;
  int64_t n = 0;
  for (int s = 0; s < nseg; ++s) {
    TFB_REQUIRE(seg_bytes[s] > 0 && seg_bytes[s] % 16 == 0 && seg_offset[s] % 16 == 0 && seg_dst[s] &&
                    aligned16(seg_dst[s]),
                "peer_gather: region %d is not in 16-byte units", s);
    segs.offset[s] = seg_offset[s];
    segs.units[s] = seg_bytes[s] / 16;
    segs.dst[s] = static_cast<uint4*>(seg_dst[s]);
    n += segs.units[s] * world;
  }
  const int grid = (int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  return check_cuda(launch(peer_gather_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           reinterpret_cast<uint8_t* const*>(windows), rank, world, segs,
                           static_cast<const uint32_t*>(step), wait_limit_ns()),
                    "peer_gather");
}

extern "C" int tfb_combine_push(const float* y, const float* wts, const int32_t* pick, int lo, int n,
                                void* const* windows, int64_t p_offset, int rank, int rows_local, int T, int slots,
                                int D, void* step, void* stream) {
  TFB_REQUIRE(y && wts && pick && windows && step, "combine_push: null pointer");
  TFB_REQUIRE(D > 0 && D % 4 == 0 && slots >= 1 && rows_local >= 1 && T >= rows_local && T % rows_local == 0,
              "combine_push: D %% 4 == 0 and T a multiple of the rows a rank");
  TFB_REQUIRE(p_offset % 16 == 0, "combine_push: 16-byte units");
  return check_cuda(launch(combine_push_kernel, dim3(T, (D + 1023) / 1024), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), y, wts, pick, lo, n,
                           reinterpret_cast<uint8_t* const*>(windows), p_offset, rank, rows_local, slots, D,
                           static_cast<uint32_t*>(step)),
                    "combine_push");
}

extern "C" int tfb_peer_push(const float* partial, void* const* windows, int64_t p_offset, int rank, int rows_local,
                             int T, int D, void* step, void* stream) {
  TFB_REQUIRE(partial && windows && step, "peer_push: null pointer");
  TFB_REQUIRE(D > 0 && D % 4 == 0 && rows_local >= 1 && T >= rows_local && T % rows_local == 0 && aligned16(partial),
              "peer_push: D %% 4 == 0, T a multiple of the rows a rank, 16-byte aligned rows");
  TFB_REQUIRE(p_offset % 16 == 0, "peer_push: 16-byte units");
  return check_cuda(launch(peer_push_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           reinterpret_cast<const float4*>(partial), reinterpret_cast<uint8_t* const*>(windows),
                           p_offset, rank, rows_local, D, static_cast<uint32_t*>(step)),
                    "peer_push");
}

extern "C" int tfb_window_picks(const int32_t* pick, const float* wts, int lo, int n, int32_t* pick_out,
                                float* wts_out, int count, void* stream) {
  TFB_REQUIRE(pick && wts && pick_out && wts_out, "window_picks: null pointer");
  TFB_REQUIRE(n >= 1 && lo >= 0 && count >= 0, "window_picks: bad sizes");
  if (count == 0) return TFB_OK;
  return check_cuda(launch(window_picks_kernel, dim3((count + 255) / 256), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), pick, wts, lo, n, pick_out, wts_out, count),
                    "window_picks");
}

extern "C" int tfb_peer_sum(void* const* windows, int rank, int64_t p_offset, int world, int rows_local, int D,
                            void* out, int out_f32, const float* extra, const float* extra_w, int extra_w_stride,
                            const void* residual, const void* step, void* stream) {
  TFB_REQUIRE(windows && out && step, "peer_sum: null pointer");
  TFB_REQUIRE(world >= 1 && world <= 32 && rank >= 0 && rank < world, "peer_sum: rank %d of %d", rank, world);
  TFB_REQUIRE(D > 0 && D % 4 == 0 && rows_local >= 1, "peer_sum: bad sizes");
  TFB_REQUIRE((extra == nullptr) == (extra_w == nullptr), "peer_sum: extra and its weights come together");
  TFB_REQUIRE(extra == nullptr || (aligned16(extra) && extra_w_stride >= 1), "peer_sum: extra rows 16-byte aligned");
  TFB_REQUIRE(aligned16(residual) && residual != out, "peer_sum: the residual rows are 16-byte aligned and not the output");
  auto* res = static_cast<const __nv_bfloat16*>(residual);
  const int64_t n4 = (int64_t)rows_local * D / 4;
  const int grid = (int)((n4 + 255) / 256 < 592 ? (n4 + 255) / 256 : 592);
  auto st = static_cast<cudaStream_t>(stream);
  auto wins = reinterpret_cast<uint8_t* const*>(windows);
  auto stp = static_cast<const uint32_t*>(step);
  if (out_f32)
    return check_cuda(launch(peer_sum_kernel<float>, dim3(grid), dim3(256), 0, st, wins, rank, p_offset, world,
                             rows_local, D, static_cast<float*>(out), extra, extra_w, extra_w_stride, res, stp,
                             wait_limit_ns()),
                      "peer_sum");
  return check_cuda(launch(peer_sum_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, wins, rank, p_offset, world,
                           rows_local, D, static_cast<__nv_bfloat16*>(out), extra, extra_w, extra_w_stride, res, stp,
                           wait_limit_ns()),
                    "peer_sum");
}
