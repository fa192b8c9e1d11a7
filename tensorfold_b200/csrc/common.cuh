// Shared device helpers and the packed expert-block geometry for the sm_100a routed-expert kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfb {

// ---- packed affine 4-bit block (group of 64 inputs x 32 output columns, one matrix) ----------------------------
// 288 int32 = 1152 bytes:
//   bytes [0, 512)    column tile 0 (block columns 0..15): 32 lanes x 16 bytes, the lane's mma A fragments
//   bytes [512, 1024) column tile 1 (block columns 16..31)
//   bytes [1024,1152) 32 (scale, bias) pairs, entry (c % 8) * 4 + c / 8 for block column c: scale in the low half
// Lane l = 4 * gq + t of a tile holds, for columns gq and gq + 8 of the tile, the 16 inputs 16 t .. 16 t + 15 of the
// group: uint4 = (col gq inputs 0..7, col gq inputs 8..15, col gq+8 inputs 0..7, col gq+8 inputs 8..15), each word
// with its nibbles stored as (i0, i2, i4, i6 | i1, i3, i5, i7) so that (w >> 4 m) & 0x000F000F is the pair
// (input 2 m, input 2 m + 1) in the two 16-bit halves.
constexpr int GS = 64;                 // inputs a group
constexpr int COLS = 32;               // output columns a block
constexpr int BLOCK_WORDS = 288;       // int32 a block
constexpr int BLOCK_BYTES = BLOCK_WORDS * 4;
constexpr int TILE_BYTES = 512;
constexpr int SB_OFFSET = 1024;

constexpr uint32_t NIB_MASK = 0x000F000Fu;
constexpr uint32_t BF16_128 = 0x43004300u;   // the bf16 pair (128, 128): 128 + q is exact for q in 0..15

enum ScaleType : int { SB_BF16 = 0, SB_FP16 = 1 };

// Position inside the 128-byte scale/bias area of block column c (uint32 index).
__host__ __device__ __forceinline__ int sb_slot(int c) { return (c & 7) * 4 + (c >> 3); }

// MLX nibble order (i0 .. i7 at bits 0, 4, .. 28) -> (i0, i2, i4, i6, i1, i3, i5, i7)
__host__ __device__ __forceinline__ uint32_t nib_shuffle(uint32_t w) {
  uint32_t even = w & 0x0F0F0F0Fu, odd = (w >> 4) & 0x0F0F0F0Fu;   // even: i0,i2,i4,i6 in bytes; odd: i1,i3,i5,i7
  even = (even | (even >> 4)) & 0x00FF00FFu;
  even = (even | (even >> 8)) & 0x0000FFFFu;
  odd = (odd | (odd >> 4)) & 0x00FF00FFu;
  odd = (odd | (odd >> 8)) & 0x0000FFFFu;
  return even | (odd << 16);
}

// nib_shuffle's inverse
__host__ __device__ __forceinline__ uint32_t nib_unshuffle(uint32_t v) {
  uint32_t out = 0;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    out |= ((v >> (4 * m)) & 0xFu) << (8 * m);
    out |= ((v >> (16 + 4 * m)) & 0xFu) << (8 * m + 4);
  }
  return out;
}

// Where MLX word (block column c, word j of the group's 8) lives inside the block, as a uint32 index.
__host__ __device__ __forceinline__ int word_slot(int c, int j) {
  const int tile = c >> 4, cc = c & 15, gq = cc & 7, hi = cc >> 3, t = j >> 1, half = j & 1;
  return tile * 128 + (gq * 4 + t) * 4 + hi * 2 + half;
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int SB>
__device__ __forceinline__ float sb_to_float(uint32_t half_bits) {
  if constexpr (SB == SB_FP16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(half_bits & 0xFFFFu)));
  } else {
    return __uint_as_float(half_bits << 16);
  }
}

// the bf16 pair (128 + q0, 128 + q1) of the nibbles at bits sh and sh + 16: one shift, one lop3 ((a & b) | c)
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int sh) {
  uint32_t t = w, r;
  if (sh) asm("shr.u32 %0, %1, %2;\n" : "=r"(t) : "r"(w), "r"(sh));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(t), "r"(NIB_MASK), "r"(BF16_128));
  return r;
}

// (scale, bias) of one column, stored as two 16-bit halves of a word, as fp32
template <int SB>
__device__ __forceinline__ float2 sb_pair(uint32_t v) {
  if constexpr (SB == SB_FP16) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
  } else {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
  }
}

// ---- device status word -----------------------------------------------------------------------------------------
// Kernels never trap: a wait that runs out records a word here and the kernel returns; the host reads it.
// Word = code | where << 8 | rank << 16.  code: 1 a bounded wait ran out, 2 a table held an index no kernel exists
// for.  where (time-outs): 0 a kernel's own copy pipeline (mbarrier), 1 the tokens barrier of an expert-parallel step,
// 2 its results barrier.  rank (barriers): the lowest rank whose flag had not arrived.  The first failure stays until
// the host reads the word (tfb_kernel_status), which clears it.
enum KernelStatus : int { ST_OK = 0, ST_WAIT_TIMEOUT = 1, ST_BAD_INDEX = 2 };
__host__ __device__ constexpr int status_word(int code, int where, int rank) { return code | (where << 8) | (rank << 16); }
static __device__ int g_kernel_status = 0;   // one copy: the library is built as a single translation unit

// ---- mbarrier / bulk copy (non-multicast) -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Two fp32 fused multiply-adds in one instruction (fma.rn.f32x2): each half is the same IEEE operation as fmaf.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  uint64_t ra, rb, rc, rd;
  float2 d;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
  return t;
}

// Bounded wait: false once `limit_ns` has passed (nothing is recorded).
__device__ __forceinline__ bool mbar_wait_for(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  uint64_t start = 0;
  for (uint32_t spin = 0; spin < (1u << 30); ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u) {
      const uint64_t now = global_ns();
      if (start == 0) start = now;
      else if (now - start > limit_ns) break;
    }
  }
  return false;
}

// Bounded wait: gives up after about a second, records ST_WAIT_TIMEOUT and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_wait_for(bar, parity, 1000000000ull)) return true;
  atomicCAS(&g_kernel_status, 0, ST_WAIT_TIMEOUT);
  return false;
}

// The same for a whole warp (every lane calls it): one answer for all lanes, so the branch on it never splits a warp
// in front of a warp-wide instruction.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

// global -> shared bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned), completion on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

__device__ __forceinline__ uint4 ldg_nc(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t comp(const uint4& v, int c) {
  return c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w;
}

// Programmatic dependent launch: a kernel launched with the attribute may start early and must wait here before it
// reads what the previous kernel in the stream wrote; without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// pdl_wait for a kernel's inputs: every pointer through which the kernel reads what earlier kernels wrote is passed
// through an empty volatile asm right behind the wait, so no load through it can be scheduled ahead of the wait (a
// const __restrict__ pointer otherwise invites the read-only path, whose loads count as invariant and may be hoisted
// over the wait - where they would read what the previous step left behind).
template <typename P>
__device__ __forceinline__ void after_wait(P& p) {     // P: a pointer type, restrict-qualified or not
  asm volatile("" : "+l"(p)::"memory");
}
template <typename P, typename... Rest>
__device__ __forceinline__ void after_wait(P& p, Rest&... rest) {
  after_wait(p);
  after_wait(rest...);
}

// A word that the kernel before this one in the stream wrote (a plan table, a count): loaded by a volatile asm, which
// the compiler keeps behind the volatile asm of pdl_wait.  The read-only path (__ldg, or a const __restrict__ pointer)
// must not be used for such data: those loads count as invariant and may be moved ahead of the wait, where they read
// what the previous step left behind.
__device__ __forceinline__ int ld_dep(const int* p) {
  int v;
  asm volatile("ld.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// ---- "whoever comes last finishes the work" -----------------------------------------------------------------------
// A CTA that has stored its part calls __syncthreads() and then ONE thread counts the CTA in with this atomic: the
// release half publishes, at GPU scope, everything the CTA's threads stored before the barrier (release is cumulative
// over what the barrier ordered before it); the acquire half lets the CTA that sees the last count read the other
// CTAs' parts after its next __syncthreads().  No per-thread fence is needed.
__device__ __forceinline__ int4 ld_dep4(const int* p) {   // 16-byte aligned
  int4 v;
  asm volatile("ld.global.v4.s32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int arrive_count(int* counter) {
  int seen;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(seen) : "l"(counter) : "memory");
  return seen;
}

// ---- activation epilogues (src/tensorfold/cuda/experts.cuh:57-75 states the roundings) -------------------------
// SwiGLU on bf16-rounded gate and up: bf16(silu(g)) * u, clipped first when limit > 0; the caller rounds to bf16.
__device__ __forceinline__ float swiglu(float g, float u, float limit) {
  float gv = round_bf16(g), uv = round_bf16(u);
  if (limit > 0.f) {
    gv = fminf(gv, limit);
    uv = fminf(fmaxf(uv, -limit), limit);
  }
  return round_bf16(gv / (1.f + expf(-gv))) * uv;
}

// The same with the hardware exponential and reciprocal (the prefill epilogue, where it sits on every output):
// silu differs from the exact one by a few fp32 ulps before its rounding to bf16.
__device__ __forceinline__ float swiglu_fast(float g, float u, float limit) {
  float gv = round_bf16(g), uv = round_bf16(u);
  if (limit > 0.f) {
    gv = fminf(gv, limit);
    uv = fminf(fmaxf(uv, -limit), limit);
  }
  return round_bf16(__fdividef(gv, 1.f + __expf(-gv))) * uv;
}

__device__ __forceinline__ float relu2(float a) {
  const float u = fmaxf(round_bf16(a), 0.f);
  return u * u;
}

enum Epilogue : int { EPI_F32 = 0, EPI_RELU2 = 1, EPI_SWIGLU = 2, EPI_BF16 = 3, EPI_SLICES = 4 };

}  // namespace tfb
