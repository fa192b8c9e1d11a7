// Decode form of the grouped 4-bit experts: a memory-bound grouped GEMV.
//
// A CTA owns one unit = (plan item of <= 16 pairs, 32-column block).  The unit's packed weights are one contiguous
// run of KG * M blocks in HBM; the CTA's four warps split it by K (a fixed split, by shape only), each warp pulling its
// run through a private shared-memory ring with bulk async copies (one elected lane issues, an mbarrier a stage), so
// many kilobytes a warp are in flight while the lanes compute.  The weights are the mma A operand (16 columns x 16
// inputs a fragment, read from shared memory as one 128-bit word a lane), the pairs' inputs the B operand (8 pairs a
// tile).  Nibbles become the exact bf16 values 128 + q with one shift and one lop3; the 128 is taken out again per
// group in fp32: acc += s * sum((128 + q) x) + (b - 128 s) * sum(x), with sum(x) from an all-ones mma.  The four
// warps' sums meet in shared memory in warp order, so a pair's bits depend on nothing but its own row.
// (Replaces src/tensorfold/cuda/experts.cu:13-155,287-351: expert_kernel and its launch.)

#include "api.h"
#include "common.cuh"

namespace tfb {

constexpr int DEC_WARPS = 4;
constexpr int DEC_PAIRS = 16;          // pairs an item may hold in this form
constexpr int RED_STRIDE = COLS + 1;

template <int M, int STAGES, int GPS>
struct DecodeSmem {
  static constexpr int STAGE_BYTES = GPS * M * BLOCK_BYTES;
  static constexpr int RING_BYTES = DEC_WARPS * STAGES * STAGE_BYTES;
  static constexpr int RED_BYTES = DEC_WARPS * M * DEC_PAIRS * RED_STRIDE * 4;
  static constexpr int DATA_BYTES = RING_BYTES > RED_BYTES ? RING_BYTES : RED_BYTES;
  static constexpr int BAR_OFFSET = (DATA_BYTES + 15) / 16 * 16;
  static constexpr int TOTAL = BAR_OFFSET + DEC_WARPS * STAGES * 8;
};

template <int M, int EPI, int SB, int STAGES, int GPS>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_stride, int slots, const uint8_t* __restrict__ W, int KG,
              int NB, const int* __restrict__ items, const int* __restrict__ counts, const int* __restrict__ members,
              void* __restrict__ out, int N, float limit) {
  using SM = DecodeSmem<M, STAGES, GPS>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int pair_id[DEC_PAIRS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, t = lane & 3;
  const int it = blockIdx.x / NB, cb = blockIdx.x - it * NB;

  uint8_t* ring = smem + warp * (STAGES * SM::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFFSET) + warp * STAGES;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s, 1);
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncwarp();

  pdl_wait();                                         // the plan (and the inputs) come from the kernels before
  if (it >= __ldg(counts)) return;
  const int e = __ldg(items + 3 * it), first = __ldg(items + 3 * it + 1);
  const int cnt = min(__ldg(items + 3 * it + 2), DEC_PAIRS);

  // this warp's K run: groups [g0, g1)
  const int kgw = (KG + DEC_WARPS - 1) / DEC_WARPS;
  const int g0 = min(KG, warp * kgw), g1 = min(KG, g0 + kgw), ng = g1 - g0;
  const int nchunks = (ng + GPS - 1) / GPS;
  const uint8_t* src = W + (((size_t)e * NB + cb) * KG + g0) * (size_t)(M * BLOCK_BYTES);

  auto issue = [&](int c) {
    const int n = min(GPS, ng - c * GPS);
    const uint32_t bytes = (uint32_t)n * (M * BLOCK_BYTES);
    uint64_t* bar = bars + (c % STAGES);
    mbar_expect_tx(bar, bytes);
    bulk_g2s(ring + (c % STAGES) * SM::STAGE_BYTES, src + (size_t)c * SM::STAGE_BYTES, bytes, bar);
  };
  if (lane == 0)
    for (int c = 0; c < STAGES && c < nchunks; ++c) issue(c);

  if (tid < DEC_PAIRS) pair_id[tid] = tid < cnt ? __ldg(members + first + tid) : -1;

  // the lane's two pairs (tile 0: pair gq, tile 1: pair 8 + gq) and their input rows
  const bool two = cnt > 8;
  const bool v0 = gq < cnt, v1 = gq + 8 < cnt;
  const int p0 = v0 ? __ldg(members + first + gq) : 0, p1 = v1 ? __ldg(members + first + gq + 8) : 0;
  const __nv_bfloat16* x0 = X + (size_t)(slots ? p0 / slots : p0) * x_stride + 16 * t;
  const __nv_bfloat16* x1 = X + (size_t)(slots ? p1 / slots : p1) * x_stride + 16 * t;

  float acc[M][2][2][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int tt = 0; tt < 2; ++tt)
#pragma unroll
      for (int pt = 0; pt < 2; ++pt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][tt][pt][i] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const uint32_t ONES = 0x3F803F80u;                  // the bf16 pair (1, 1)
  bool ok = true;
  for (int c = 0; c < nchunks && ok; ++c) {
    const int s = c % STAGES;
    ok = mbar_wait(bars + s, (c / STAGES) & 1);
    if (!ok) break;
    const int n = min(GPS, ng - c * GPS);
    for (int gi = 0; gi < n; ++gi) {
      const int k0 = (g0 + c * GPS + gi) * GS;
      uint4 xa[2], xb[2];
      xa[0] = v0 ? ldg_nc(x0 + k0) : zero;
      xa[1] = v0 ? ldg_nc(x0 + k0 + 8) : zero;
      xb[0] = v1 ? ldg_nc(x1 + k0) : zero;
      xb[1] = v1 ? ldg_nc(x1 + k0 + 8) : zero;
      // sum of the group's inputs for pairs 2t and 2t + 1 of each tile (all-ones A)
      float xs[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        mma_bf16(xs[0], ONES, ONES, ONES, ONES, comp(xa[ks >> 1], 2 * (ks & 1)), comp(xa[ks >> 1], 2 * (ks & 1) + 1));
        if (two)
          mma_bf16(xs[1], ONES, ONES, ONES, ONES, comp(xb[ks >> 1], 2 * (ks & 1)),
                   comp(xb[ks >> 1], 2 * (ks & 1) + 1));
      }
      const uint8_t* blk = ring + s * SM::STAGE_BYTES + gi * (M * BLOCK_BYTES);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const uint4 sbv = *reinterpret_cast<const uint4*>(blk + m * BLOCK_BYTES + SB_OFFSET + gq * 16);
#pragma unroll
        for (int tt = 0; tt < 2; ++tt) {
          const uint4 w = *reinterpret_cast<const uint4*>(blk + m * BLOCK_BYTES + tt * TILE_BYTES + lane * 16);
          uint32_t a[4][4];
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t lo = ks < 2 ? w.x : w.y, hi = ks < 2 ? w.z : w.w;
            const int sh = 8 * (ks & 1);
            a[ks][0] = ((lo >> sh) & NIB_MASK) | BF16_128;
            a[ks][1] = ((hi >> sh) & NIB_MASK) | BF16_128;
            a[ks][2] = ((lo >> (sh + 4)) & NIB_MASK) | BF16_128;
            a[ks][3] = ((hi >> (sh + 4)) & NIB_MASK) | BF16_128;
          }
          const uint32_t sb_lo = comp(sbv, 2 * tt), sb_hi = comp(sbv, 2 * tt + 1);
          const float s_lo = sb_to_float<SB>(sb_lo & 0xFFFFu), s_hi = sb_to_float<SB>(sb_hi & 0xFFFFu);
          const float b_lo = fmaf(-128.f, s_lo, sb_to_float<SB>(sb_lo >> 16));
          const float b_hi = fmaf(-128.f, s_hi, sb_to_float<SB>(sb_hi >> 16));
#pragma unroll
          for (int pt = 0; pt < 2; ++pt) {
            if (pt == 1 && !two) break;
            const uint4* xv = pt ? xb : xa;
            float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(p, a[ks][0], a[ks][1], a[ks][2], a[ks][3], comp(xv[ks >> 1], 2 * (ks & 1)),
                       comp(xv[ks >> 1], 2 * (ks & 1) + 1));
            float(&d)[4] = acc[m][tt][pt];
            d[0] = fmaf(xs[pt][0], b_lo, fmaf(p[0], s_lo, d[0]));
            d[1] = fmaf(xs[pt][1], b_lo, fmaf(p[1], s_lo, d[1]));
            d[2] = fmaf(xs[pt][0], b_hi, fmaf(p[2], s_hi, d[2]));
            d[3] = fmaf(xs[pt][1], b_hi, fmaf(p[3], s_hi, d[3]));
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0 && c + STAGES < nchunks) issue(c + STAGES);
  }
  pdl_launch_dependents();

  // the four warps' sums meet in warp order (the ring's memory is free once every warp is past its loop)
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem);
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int tt = 0; tt < 2; ++tt)
#pragma unroll
      for (int pt = 0; pt < 2; ++pt) {
        float* base = red + ((warp * M + m) * DEC_PAIRS + pt * 8 + 2 * t) * RED_STRIDE + tt * 16 + gq;
        base[0] = acc[m][tt][pt][0];
        base[RED_STRIDE] = acc[m][tt][pt][1];
        base[8] = acc[m][tt][pt][2];
        base[RED_STRIDE + 8] = acc[m][tt][pt][3];
      }
  __syncthreads();
  const int col = tid & 31;
  for (int pi = tid >> 5; pi < cnt; pi += DEC_WARPS) {
    float v[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float sum = red[((0 * M + m) * DEC_PAIRS + pi) * RED_STRIDE + col];
#pragma unroll
      for (int w = 1; w < DEC_WARPS; ++w) sum += red[((w * M + m) * DEC_PAIRS + pi) * RED_STRIDE + col];
      v[m] = sum;
    }
    const size_t at = (size_t)pair_id[pi] * N + cb * COLS + col;
    if constexpr (EPI == EPI_F32) {
      static_cast<float*>(out)[at] = v[0];
    } else if constexpr (EPI == EPI_RELU2) {
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(relu2(v[0]));
    } else if constexpr (EPI == EPI_SWIGLU) {
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(swiglu(v[0], v[M - 1], limit));
    } else {
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(v[0]);
    }
  }
}

template <int M, int EPI, int SB>
int launch_decode(const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb, const int* items,
                  const int* counts, const int* members, void* out, int n, float limit, int64_t max_units,
                  cudaStream_t stream) {
  constexpr int STAGES = 4, GPS = 1;
  using SM = DecodeSmem<M, STAGES, GPS>;
  auto* kern = decode_kernel<M, EPI, SB, STAGES, GPS>;
  if (SM::TOTAL > 48 * 1024) {
    static bool configured[64] = {false};
    int dev = 0;
    TFB_CUDA(cudaGetDevice(&dev), "experts_run: cudaGetDevice");
    if (dev < 64 && !configured[dev]) {
      TFB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL),
               "experts_run: shared memory opt-in");
      configured[dev] = true;
    }
  }
  return check_cuda(launch(kern, dim3((unsigned)max_units), dim3(DEC_WARPS * 32), (size_t)SM::TOTAL, stream,
                           static_cast<const __nv_bfloat16*>(x), x_stride, slots, static_cast<const uint8_t*>(w), kg,
                           nb, items, counts, members, out, n, limit),
                    "experts_run");
}

}  // namespace tfb

using namespace tfb;

// Grouped 4-bit expert matmul, decode form.  Arguments as the reference extension's `run`
// (src/tensorfold/cuda/experts.cpp:43-48): epi 0 fp32 out, 1 relu^2, 2 SwiGLU over (gate, up), 3 bf16 out.
extern "C" int tfb_experts_run(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg,
                               int nb, const int32_t* items, const int32_t* counts, const int32_t* members, void* out,
                               int n, float limit, int64_t max_units, int sb_type, void* stream) {
  TFB_REQUIRE(gs == GS, "experts_run: groups of %d inputs only, not %d", GS, gs);
  TFB_REQUIRE(x && w && items && counts && members && out, "experts_run: null pointer");
  TFB_REQUIRE(kg >= 1 && nb >= 1 && n == nb * COLS, "experts_run: n must be the column blocks times %d", COLS);
  TFB_REQUIRE(aligned16(x) && x_stride % 8 == 0 && x_stride >= (int64_t)kg * GS,
              "experts_run: x rows of K = groups * group size inputs, 16-byte aligned");
  TFB_REQUIRE(aligned16(w), "experts_run: w must be 16-byte aligned");
  TFB_REQUIRE(slots >= 0 && max_units >= 0 && max_units < (int64_t(1) << 31), "experts_run: bad slots or unit count");
  TFB_REQUIRE(sb_type == SB_BF16 || sb_type == SB_FP16, "experts_run: scales are bf16 (0) or fp16 (1), not %d", sb_type);
  if (max_units == 0) return TFB_OK;
  auto st = static_cast<cudaStream_t>(stream);
#define TFB_RUN(EPI_, M_)                                                                                          \
  if (epi == EPI_)                                                                                                 \
    return sb_type == SB_BF16                                                                                      \
               ? launch_decode<M_, EPI_, SB_BF16>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n,   \
                                                  limit, max_units, st)                                            \
               : launch_decode<M_, EPI_, SB_FP16>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n,   \
                                                  limit, max_units, st);
  TFB_RUN(EPI_F32, 1) TFB_RUN(EPI_RELU2, 1) TFB_RUN(EPI_SWIGLU, 2) TFB_RUN(EPI_BF16, 1)
#undef TFB_RUN
  return fail(TFB_ERR_ARG, "experts_run: no kernel for epilogue %d", epi);
}
