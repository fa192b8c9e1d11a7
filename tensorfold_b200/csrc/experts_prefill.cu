// Prefill form of the grouped 4-bit experts: a grouped GEMM on the tcgen05 tensor cores.
//
// A CTA owns one unit = (plan item of <= 192 pairs, 128 output columns).  The roles are swapped against the usual
// GEMM: the WEIGHTS are the MMA's A operand (M = 128 columns), the item's PAIRS the B operand (N = pairs rounded up to
// 16, <= 192), so an expert with 140 pairs costs 144 / 128 of a full tile instead of two, and every weight is
// dequantised exactly once.  Per group of 64 inputs (one pipeline stage):
//   warp 13 (a lane)   bulk-copies the packed blocks (4 column blocks x M matrices) into a deep staging ring;
//   warps 8-11         gather the pairs' input rows with 16-byte cp.async into the 128-byte-swizzled B tile;
//   warps 0-7          turn nibbles into the prefill form's bf16 weights (w = bf16(q * s + b), one rounding) and
//                      store them as the K-major, 128-byte-swizzled A tiles;
//   warp 12 (a lane)   issues tcgen05.mma (cta_group::1, kind::f16, M = 128, K = 16) into fp32 accumulators in tensor
//                      memory (gate at column 0, up at column 256), and commits each stage back to the producer.
// After the last group warps 0-11 read the accumulators (tcgen05.ld), apply the epilogue and store rows by pair id.
// One fp32 chain over K in group order: a pair's bits do not depend on its item, its chunk or the call.
// (Replaces src/tensorfold/cuda/experts_prefill.cu:31-195: prefill_kernel and its launch.)

#include "api.h"
#include "common.cuh"

namespace tfb {

constexpr int PF_COLS = 128;            // output columns a unit (MMA M)
constexpr int PF_MAXP = 192;            // pairs an item may hold (MMA N)
constexpr int PF_CB = PF_COLS / COLS;   // packed column blocks a unit
constexpr int PF_DQ_WARPS = 8;          // warps 0-7: dequantise, then the epilogue
constexpr int PF_GA_WARPS = 4;          // warps 8-11: gather the pairs' input rows
constexpr int PF_MMA_WARP = 12, PF_COPY_WARP = 13;
constexpr int PF_THREADS = 14 * 32;
constexpr int PF_GA_PER_THREAD = PF_MAXP * 8 / (PF_GA_WARPS * 32);   // 16-byte chunks a gather thread a stage

// Two rings: operand tiles (A per matrix and B) with SA stages, and the packed blocks as they come from HBM with SP
// stages (deeper: it hides the HBM latency, and a stage is free again as soon as it has been dequantised).
template <int M>
struct PrefillSmem {
  static constexpr int SA = M == 2 ? 3 : 4;
  static constexpr int SP = M == 2 ? 6 : 8;
  static constexpr int A_BYTES = PF_COLS * 128;                 // one matrix: 128 rows of 64 bf16
  static constexpr int B_BYTES = PF_MAXP * 128;
  static constexpr int AB_BYTES = M * A_BYTES + B_BYTES;        // a multiple of 1024
  static constexpr int PACKED_BYTES = PF_CB * M * BLOCK_BYTES;
  static constexpr int PACKED_OFFSET = SA * AB_BYTES;
  static constexpr int TABLE_OFFSET = PACKED_OFFSET + SP * PACKED_BYTES;   // int out_row[PF_MAXP]
  static constexpr int BAR_OFFSET = (TABLE_OFFSET + PF_MAXP * 4 + 15) / 16 * 16;
  static constexpr int NBARS = 2 * SP + 3 * SA + 1;
  static constexpr int TMEM_OFFSET = BAR_OFFSET + NBARS * 8;
  static constexpr int TOTAL = TMEM_OFFSET + 16 + 1024;         // + slack to align the tiles to 1024 bytes
};

// ---- tcgen05 wrappers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(dst_smem)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// K-major operand tile of rows x 64 bf16 (128 bytes a row), 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);            // start address
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset: the next 8-row group
  d |= (uint64_t)1 << 46;                              // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
  return d;
}
// kind::f16: D fp32, A and B bf16, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(PF_COLS >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// The prefill form's weight pair from the bf16 pair (128 + q0, 128 + q1) and the column's (scale, bias) word.
// bf16 scales: bf16(q * s + b) with one rounding (a bf16 fma), as src/tensorfold/cuda/experts_prefill.cu:25-29;
// fp16 scales: the fp32 fma rounded to bf16.
template <int SB>
__device__ __forceinline__ uint32_t prefill_pair(uint32_t v, uint32_t sb) {
  if constexpr (SB == SB_BF16) {
    const uint32_t k128 = BF16_128, s2 = __byte_perm(sb, sb, 0x1010), b2 = __byte_perm(sb, sb, 0x3232);
    __nv_bfloat162 q = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v),
                               *reinterpret_cast<const __nv_bfloat162*>(&k128));
    __nv_bfloat162 r = __hfma2(q, *reinterpret_cast<const __nv_bfloat162*>(&s2),
                               *reinterpret_cast<const __nv_bfloat162*>(&b2));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    const float2 f = sb_pair<SB>(sb);
    const float w0 = fmaf(f.x, bf16_lo(v) - 128.f, f.y), w1 = fmaf(f.x, bf16_hi(v) - 128.f, f.y);
    __nv_bfloat162 r = __floats2bfloat162_rn(w0, w1);
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

template <int M, int EPI, int SB>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_stride, int slots, const uint8_t* __restrict__ W, int KG,
               int NB, const int* __restrict__ items, const int* __restrict__ counts, const int* __restrict__ members,
               void* __restrict__ out, int N, float limit) {
  using SM = PrefillSmem<M>;
  constexpr int SA = SM::SA, SP = SM::SP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int* out_row = reinterpret_cast<int*>(smem + SM::TABLE_OFFSET);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFFSET);
  uint64_t* packed_full = bars;                  // [SP] the bulk copy landed
  uint64_t* packed_free = bars + SP;             // [SP] the eight dequantising warps have read it
  uint64_t* a_ready = bars + 2 * SP;             // [SA] the eight dequantising warps wrote their tiles
  uint64_t* b_ready = a_ready + SA;              // [SA] the pairs' input rows landed
  uint64_t* ab_free = b_ready + SA;              // [SA] the MMAs that read the stage retired
  uint64_t* acc_ready = ab_free + SA;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::TMEM_OFFSET);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nct = (NB + PF_CB - 1) / PF_CB;
  const int it = blockIdx.x / nct, ct = blockIdx.x - it * nct;

  if (tid == 0) {
    for (int s = 0; s < SP; ++s) {
      mbar_init(packed_full + s, 1);
      mbar_init(packed_free + s, PF_DQ_WARPS);
    }
    for (int s = 0; s < SA; ++s) {
      mbar_init(a_ready + s, PF_DQ_WARPS);
      mbar_init(b_ready + s, PF_GA_WARPS * 32);
      mbar_init(ab_free + s, 1);
    }
    mbar_init(acc_ready, 1);
    mbar_fence_init();
    fence_async_smem();
  }
  pdl_wait();
  after_wait(X, items, counts, members);
  const bool live = it < ld_dep(counts);          // uniform over the CTA
  constexpr uint32_t TMEM_COLS = 512;
  if (live && warp == PF_MMA_WARP) tmem_alloc(tmem_slot, TMEM_COLS);
  int e = 0, first = 0, cnt = 0;
  if (live) {
    e = ld_dep(items + 3 * it);
    first = ld_dep(items + 3 * it + 1);
    cnt = min(ld_dep(items + 3 * it + 2), PF_MAXP);
    for (int i = tid; i < PF_MAXP; i += PF_THREADS) out_row[i] = i < cnt ? ld_dep(members + first + i) : -1;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (!live) return;
  const uint32_t tmem_base = *tmem_slot;
  const int nmma = max(16, (cnt + 15) & ~15);
  const int cb0 = ct * PF_CB, ncb = min(PF_CB, NB - cb0);        // packed column blocks of this unit
  bool ok = true;

  if (warp == PF_COPY_WARP) {
    // ---------------- packed weights: HBM -> the packed ring, as far ahead as the ring allows ----------------
    if (lane == 0) {
      const uint8_t* wsrc = W + ((size_t)e * NB + cb0) * KG * (size_t)(M * BLOCK_BYTES);
      const size_t cb_stride = (size_t)KG * (M * BLOCK_BYTES);
      for (int g = 0; g < KG && ok; ++g) {
        const int s = g % SP, round = g / SP;
        if (round > 0) ok = mbar_wait(packed_free + s, (round - 1) & 1);
        if (!ok) break;
        uint8_t* dst = smem + SM::PACKED_OFFSET + s * SM::PACKED_BYTES;
        mbar_expect_tx(packed_full + s, (uint32_t)ncb * (M * BLOCK_BYTES));
        for (int j = 0; j < ncb; ++j)
          bulk_g2s(dst + j * (M * BLOCK_BYTES), wsrc + j * cb_stride + (size_t)g * (M * BLOCK_BYTES), M * BLOCK_BYTES,
                   packed_full + s);
      }
    }
    __syncwarp();
  } else if (warp == PF_MMA_WARP) {
    // ---------------- MMA issue: one lane ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(nmma);
      for (int g = 0; g < KG && ok; ++g) {
        const int s = g % SA, ph = (g / SA) & 1;
        ok = mbar_wait(a_ready + s, ph) && mbar_wait(b_ready + s, ph);
        if (!ok) break;
        tc_fence_after();
        const uint32_t abase = smem_addr(smem + s * SM::AB_BYTES), bbase = abase + M * SM::A_BYTES;
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma(tmem_base + m * 256, umma_desc(abase + m * SM::A_BYTES + ks * 32), umma_desc(bbase + ks * 32), idesc,
                 (g | ks) ? 1u : 0u);
        umma_commit(ab_free + s);
      }
      if (ok) umma_commit(acc_ready);
    }
    __syncwarp();
  } else if (warp >= PF_DQ_WARPS) {
    // ---------------- warps 8-11: gather the pairs' input rows into the swizzled B tiles ----------------
    // thread -> chunk c of rows r0, r0 + 16, ...: the row pointers stay in registers for the whole K loop
    const int gt = tid - PF_DQ_WARPS * 32, c = gt & 7, r0 = gt >> 3;
    const __nv_bfloat16* rowp[PF_GA_PER_THREAD];
#pragma unroll
    for (int j = 0; j < PF_GA_PER_THREAD; ++j) {
      const int r = r0 + 16 * j;
      const int p = r < cnt ? out_row[r] : -1;
      rowp[j] = p < 0 ? nullptr : X + (size_t)(slots ? p / slots : p) * x_stride + c * 8;
    }
    const uint32_t boff = (uint32_t)(r0 * 128 + ((c ^ (r0 & 7)) << 4));      // rows 16 apart share r & 7
    for (int g = 0; g < KG && ok; ++g) {
      const int s = g % SA, round = g / SA;
      if (round > 0) ok = mbar_wait_warp(ab_free + s, (round - 1) & 1);
      if (!ok) break;
      uint8_t* btile = smem + s * SM::AB_BYTES + M * SM::A_BYTES + boff;
#pragma unroll
      for (int j = 0; j < PF_GA_PER_THREAD; ++j)
        if (rowp[j]) cp_async16(btile + j * (16 * 128), rowp[j] + g * GS);
      cp_async_commit();
      if (g > 0) {                                   // the stage before this one has landed: publish it
        cp_async_wait<1>();
        fence_async_smem();
        mbar_arrive(b_ready + (g - 1) % SA);
      }
    }
    cp_async_wait<0>();
    fence_async_smem();
    if (ok) mbar_arrive(b_ready + (KG - 1) % SA);
  } else {
    // ---------------- warps 0-7: dequantise into the A tiles ----------------
    // warp -> packed column block cbw = warp & 3 and its 16-column tile tt = warp >> 2, for every matrix
    const int gq = lane >> 2, t = lane & 3, cbw = warp & 3, tt = warp >> 2;
    for (int g = 0; g < KG && ok; ++g) {
      const int sp = g % SP, sa = g % SA;
      ok = mbar_wait_warp(packed_full + sp, (g / SP) & 1);
      if (ok && g >= SA) ok = mbar_wait_warp(ab_free + sa, (g / SA - 1) & 1);
      if (!ok) break;
      if (cbw < ncb) {
        const uint8_t* blk = smem + SM::PACKED_OFFSET + sp * SM::PACKED_BYTES + cbw * (M * BLOCK_BYTES);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 sbv = *reinterpret_cast<const uint4*>(blk + m * BLOCK_BYTES + SB_OFFSET + gq * 16);
          const uint4 w = *reinterpret_cast<const uint4*>(blk + m * BLOCK_BYTES + tt * TILE_BYTES + lane * 16);
          const uint32_t sb_lo = comp(sbv, 2 * tt), sb_hi = comp(sbv, 2 * tt + 1);
          // rows of the A tile: column cbw * 32 + tt * 16 + gq (and + 8); chunks 2 t and 2 t + 1 of the row
          uint8_t* row = smem + sa * SM::AB_BYTES + m * SM::A_BYTES + (cbw * 32 + tt * 16 + gq) * 128;
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const uint32_t word = comp(w, h);
            const uint32_t sb = (h & 2) ? sb_hi : sb_lo;
            uint4 o;
            o.x = prefill_pair<SB>(nib_pair(word, 0), sb);
            o.y = prefill_pair<SB>(nib_pair(word, 4), sb);
            o.z = prefill_pair<SB>(nib_pair(word, 8), sb);
            o.w = prefill_pair<SB>(nib_pair(word, 12), sb);
            const int chunk = 2 * t + (h & 1);
            *reinterpret_cast<uint4*>(row + (h & 2) * 512 + ((chunk ^ gq) << 4)) = o;
          }
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(packed_free + sp);
        mbar_arrive(a_ready + sa);
      }
    }
  }
  // ---------------- epilogue: the twelve dequantising and gathering warps ----------------
  // TMEM lane quarter warp & 3 (output column (warp & 3) * 32 + lane of the unit); the three warps of a quarter take
  // a third of the pairs each, 16 pairs a load
  if (warp < PF_DQ_WARPS + PF_GA_WARPS) {
    if (ok) ok = mbar_wait_warp(acc_ready, 0);
    if (ok) {
      tc_fence_after();
      const int q = warp & 3, part = warp >> 2, col = ct * PF_COLS + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
      const int blocks = nmma / 16, per = (blocks + 2) / 3;
      const int jb = min(blocks, part * per) * 16, je = min(blocks, (part + 1) * per) * 16;
      for (int j0 = jb; j0 < je; j0 += 16) {
        uint32_t a[16], b[16];
        tmem_ld16(taddr + j0, a);
        if constexpr (M == 2) tmem_ld16(taddr + 256 + j0, b);
        tmem_ld_wait();
        if (col < N) {
          // the sixteen values first (independent chains the compiler can interleave: one after the other, each
          // behind its own row lookup and branch, they took 2 us a block), then their rows and the stores
          float r[16];
          int rows[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float v = __uint_as_float(a[j]);
            rows[j] = out_row[j0 + j];
            if constexpr (EPI == EPI_RELU2) {
              r[j] = relu2(v);
            } else if constexpr (EPI == EPI_SWIGLU) {
              r[j] = swiglu_fast(v, __uint_as_float(b[j]), limit);
            } else {
              r[j] = v;
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (rows[j] < 0) continue;
            const size_t at = (size_t)rows[j] * N + col;
            if constexpr (EPI == EPI_F32) {
              static_cast<float*>(out)[at] = r[j];
            } else {
              static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(r[j]);
            }
          }
        }
      }
    }
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (warp == PF_MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int M, int EPI, int SB>
int launch_prefill(const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb, const int* items,
                   const int* counts, const int* members, void* out, int n, float limit, int64_t max_items,
                   cudaStream_t stream) {
  using SM = PrefillSmem<M>;
  auto* kern = prefill_kernel<M, EPI, SB>;
  static bool configured[64] = {false};
  int dev = 0;
  TFB_CUDA(cudaGetDevice(&dev), "experts_prefill: cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(TFB_ERR_ARG, "experts_prefill: device index %d out of range", dev);
  if (!configured[dev]) {
    TFB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL),
             "experts_prefill: shared memory opt-in");
    configured[dev] = true;
  }
  const int64_t grid = max_items * ((nb + PF_CB - 1) / PF_CB);
  if (grid >= (int64_t(1) << 31)) return fail(TFB_ERR_ARG, "experts_prefill: too many units");
  return check_cuda(launch(kern, dim3((unsigned)grid), dim3(PF_THREADS), (size_t)SM::TOTAL, stream,
                           static_cast<const __nv_bfloat16*>(x), x_stride, slots, static_cast<const uint8_t*>(w), kg,
                           nb, items, counts, members, out, n, limit),
                    "experts_prefill");
}

}  // namespace tfb

using namespace tfb;

// Grouped 4-bit expert matmul, prefill form, over a plan whose items hold at most 192 pairs.  Arguments as the
// reference extension's `prefill` (src/tensorfold/cuda/experts.cpp:50-56); max_items = an upper bound of the items.
extern "C" int tfb_experts_prefill(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg,
                                   int nb, const int32_t* items, const int32_t* counts, const int32_t* members,
                                   void* out, int n, float limit, int64_t max_items, int sb_type, void* stream) {
  TFB_REQUIRE(gs == GS, "experts_prefill: groups of %d inputs only, not %d", GS, gs);
  TFB_REQUIRE(x && w && items && counts && members && out, "experts_prefill: null pointer");
  TFB_REQUIRE(kg >= 1 && nb >= 1 && n == nb * COLS, "experts_prefill: n must be the column blocks times %d", COLS);
  TFB_REQUIRE(aligned16(x) && x_stride % 8 == 0 && x_stride >= (int64_t)kg * GS,
              "experts_prefill: x rows of K = groups * group size inputs, 16-byte aligned");
  TFB_REQUIRE(aligned16(w), "experts_prefill: w must be 16-byte aligned");
  TFB_REQUIRE(slots >= 0 && max_items >= 0, "experts_prefill: bad slots or item count");
  TFB_REQUIRE(sb_type == SB_BF16 || sb_type == SB_FP16, "experts_prefill: scales are bf16 (0) or fp16 (1), not %d",
              sb_type);
  if (max_items == 0) return TFB_OK;
  auto st = static_cast<cudaStream_t>(stream);
#define TFB_PRE(EPI_, M_)                                                                                           \
  if (epi == EPI_)                                                                                                  \
    return sb_type == SB_BF16                                                                                       \
               ? launch_prefill<M_, EPI_, SB_BF16>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n,   \
                                                   limit, max_items, st)                                            \
               : launch_prefill<M_, EPI_, SB_FP16>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n,   \
                                                   limit, max_items, st);
  TFB_PRE(EPI_F32, 1) TFB_PRE(EPI_RELU2, 1) TFB_PRE(EPI_SWIGLU, 2) TFB_PRE(EPI_BF16, 1)
#undef TFB_PRE
  return fail(TFB_ERR_ARG, "experts_prefill: no kernel for epilogue %d", epi);
}
