// Decode form of the grouped 4-bit experts: a memory-bound grouped GEMV.
//
// A CTA of four warps owns one unit = (plan item of <= 8 pairs - 16 with PT = 2 - and CBC consecutive 32-column
// blocks).  A column block's packed weights for one expert are one contiguous run of KG * M blocks in HBM.  The four
// warps are KW K-slices times CBC = 4 / KW column blocks (KW is a function of the shape only); each warp pulls its run
// through a private shared-memory ring with bulk async copies (one elected lane issues; a slot holds G groups fetched
// by one copy a column block, an mbarrier a slot), so many kilobytes a warp are in flight while the lanes compute.
// The weights are the mma A operand (16 columns x 16 inputs a fragment, read from shared memory as one 128-bit word a
// lane), the pairs' inputs the B operand (8 pairs).  Nibbles become the
// exact bf16 values 128 + q with a shift and one lop3; the 128 is taken out again per group in fp32:
// acc += s * sum((128 + q) x) + (b - 128 s) * sum(x), with sum(x) from an all-ones mma.  K-slices meet in shared
// memory in slice order, so a pair's bits depend on nothing but its own row.
// (Replaces src/tensorfold/cuda/experts.cu:13-155,287-351: expert_kernel and its launch.)

#include "api.h"
#include <cstring>

#include "common.cuh"

namespace tfb {

constexpr int DEC_WARPS = 4;
constexpr int DEC_PAIRS = 16;          // pairs an item may hold at most in this form: PT mma tiles of 8 (PT = 1 or 2)
constexpr int RED_STRIDE = COLS + 1;

// Q = blocks a warp takes a group: M matrices (gate, up: adjacent in memory) or NCB column blocks of one matrix.
// A ring slot holds G consecutive groups, fetched by one bulk copy a column block: copies of 4.6 KB stream at the
// full HBM rate where copies of 2.3 KB reach 0.8 of it and 1.2 KB 0.63 (measured with the arithmetic taken out).
template <int Q, int G, int SLOTS>
struct DecodeSmem {
  static constexpr int STAGE_BYTES = G * Q * BLOCK_BYTES;                  // G groups a slot
  static constexpr int STAGES = SLOTS;
  static constexpr int RING_BYTES = DEC_WARPS * STAGES * STAGE_BYTES;
  static constexpr int RED_BYTES = DEC_WARPS * Q * DEC_PAIRS * RED_STRIDE * 4;
  static constexpr int DATA_BYTES = RING_BYTES > RED_BYTES ? RING_BYTES : RED_BYTES;
  static constexpr int BAR_OFFSET = (DATA_BYTES + 15) / 16 * 16;
  static constexpr int TOTAL = BAR_OFFSET + DEC_WARPS * STAGES * 8;
};

__device__ __forceinline__ void mma_bf16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %10, %10, %10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// The weighted combine folded into the down projection (COMBINE): every pair p = token * slots + slot of the call is
// in the plan; after a CTA has stored its pairs' fp32 rows it counts, per (token, column group), the slots that are
// done; the CTA that completes a token's last slot adds that token's rows in slot order (an fp32 fma chain from 0,
// the combine kernel's arithmetic) and stores the result row - so the layer needs no combine launch.
struct CombineArgs {
  const float* wts;      // [T, slots] fp32
  void* out;             // [T, N] bf16, or fp32 when out_f32
  int* arrive;           // [T, NB] ints, zero between launches (the kernel leaves them zero)
  int slots, out_f32;
};

template <int M, int NCB, int EPI, int SB, int KW, int G, int STAGES, int PT, bool COMBINE = false>
__global__ void __launch_bounds__(DEC_WARPS * 32, PT == 2 ? (M == 2 ? 4 : 1) : 5)
decode_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_stride, int slots, const uint8_t* __restrict__ W, int KG,
              int NB, const int* __restrict__ items, const int* __restrict__ counts, const int* __restrict__ members,
              void* __restrict__ out, int N, float limit, CombineArgs cmb) {
  static_assert(M == 1 || NCB == 1, "a warp takes two matrices of one column block, or column blocks of one matrix");
  constexpr int Q = M * NCB;
  using SM = DecodeSmem<Q, G, STAGES>;
  constexpr int CBC = DEC_WARPS / KW * NCB;           // column blocks a CTA
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int pair_id[DEC_PAIRS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, t = lane & 3;
  const int nbt = (NB + CBC - 1) / CBC;
  const int it = blockIdx.x / nbt, cbt = blockIdx.x - it * nbt;
  const int kslice = warp % KW, cbw = warp / KW, cb = cbt * CBC + cbw * NCB;   // the warp's first column block

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
  after_wait(X, items, counts, members);
  // the item is read together with the count that says whether it exists (its slot is always inside the table)
  const int n_items = ld_dep(counts);
  const int e = ld_dep(items + 3 * it), first = ld_dep(items + 3 * it + 1);
  constexpr int PAIRS = 8 * PT;
  const int cnt = min(ld_dep(items + 3 * it + 2), PAIRS);
  if (it >= n_items) return;

  // this warp's K run: groups [g0, g1) of column block cb
  const int kgw = (KG + KW - 1) / KW;
  const int g0 = min(KG, kslice * kgw), g1 = min(KG, g0 + kgw);
  const int ncb = max(0, min(NCB, NB - cb));          // column blocks of this warp that exist
  const int ng = ncb > 0 ? g1 - g0 : 0;
  const size_t cb_stride = (size_t)KG * (M * BLOCK_BYTES);
  const uint8_t* src = W + (((size_t)e * NB + min(cb, NB - 1)) * KG + g0) * (size_t)(M * BLOCK_BYTES);

  const int nslot = (ng + G - 1) / G;                 // slot fills of this warp's run
  auto issue = [&](int c) {                           // groups [c G, c G + G) of every column block of the warp
    uint64_t* bar = bars + (c % STAGES);
    uint8_t* dst = ring + (c % STAGES) * SM::STAGE_BYTES;
    const uint32_t bytes = (uint32_t)min(G, ng - c * G) * (M * BLOCK_BYTES);
    mbar_expect_tx(bar, (uint32_t)ncb * bytes);
#pragma unroll
    for (int j = 0; j < NCB; ++j)
      if (j < ncb)
        bulk_g2s(dst + j * (G * M * BLOCK_BYTES), src + j * cb_stride + (size_t)c * (G * M * BLOCK_BYTES), bytes, bar);
  };
  if (lane == 0)
    for (int c = 0; c < STAGES && c < nslot; ++c) issue(c);

  if (tid < DEC_PAIRS) pair_id[tid] = tid < cnt ? ld_dep(members + first + tid) : -1;

  // the lane's pairs (B operand column gq of each tile of 8) and their input rows
  // (lanes past the item's last pair read its first pair's row: an mma column depends on its own inputs only, and
  // those columns are never stored)
  const __nv_bfloat16* xrow[PT];
#pragma unroll
  for (int pt = 0; pt < PT; ++pt) {
    const int pr = ld_dep(members + first + (8 * pt + gq < cnt ? 8 * pt + gq : 0));
    xrow[pt] = X + (size_t)(slots ? pr / slots : pr) * x_stride + 16 * t + (size_t)g0 * GS;
  }

  float acc[Q][2][PT][4];
#pragma unroll
  for (int m = 0; m < Q; ++m)
#pragma unroll
    for (int tt = 0; tt < 2; ++tt)
#pragma unroll
      for (int pt = 0; pt < PT; ++pt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][tt][pt][i] = 0.f;

  const uint32_t ONES = 0x3F803F80u;                  // the bf16 pair (1, 1)
  // an item of a 16-pair plan that holds at most 8 pairs skips its second tile's loads and arithmetic (the same for
  // every thread of the CTA), so such a plan costs little where experts have few pairs
  const bool two = PT == 2 && cnt > 8;
  uint4 xn[PT][2];
#pragma unroll
  for (int pt = 0; pt < PT; ++pt) {
    xn[pt][0] = xn[pt][1] = make_uint4(0u, 0u, 0u, 0u);
    if (ng > 0 && (pt == 0 || two)) {
      xn[pt][0] = ldg_nc(xrow[pt]);
      xn[pt][1] = ldg_nc(xrow[pt] + 8);
    }
  }
  bool failed = false;
  for (int c = 0; c < ng; ++c) {
    const int fill = c / G, gi = c - fill * G, s = fill % STAGES;
    uint32_t xb[PT][8];
    float xs[PT][4];                                  // sum of the group's inputs for pairs 2t and 2t + 1 of each tile
#pragma unroll
    for (int pt = 0; pt < PT; ++pt) {
      if (pt == 1 && !two) continue;
      const uint4 x0 = xn[pt][0], x1 = xn[pt][1];
      if (c + 1 < ng) {                               // the next group's inputs travel while this one computes
        xn[pt][0] = ldg_nc(xrow[pt] + (c + 1) * GS);
        xn[pt][1] = ldg_nc(xrow[pt] + (c + 1) * GS + 8);
      }
      xb[pt][0] = x0.x; xb[pt][1] = x0.y; xb[pt][2] = x0.z; xb[pt][3] = x0.w;
      xb[pt][4] = x1.x; xb[pt][5] = x1.y; xb[pt][6] = x1.z; xb[pt][7] = x1.w;
      mma_bf16_zero(xs[pt], ONES, ONES, ONES, ONES, xb[pt][0], xb[pt][1]);
#pragma unroll
      for (int ks = 1; ks < 4; ++ks) mma_bf16(xs[pt], ONES, ONES, ONES, ONES, xb[pt][2 * ks], xb[pt][2 * ks + 1]);
    }
    if (gi == 0 && !mbar_wait_warp(bars + s, (fill / STAGES) & 1)) {
      // the copy never landed (recorded in the status word): give the other copies this warp issued a short while to
      // land, then the whole CTA leaves without storing anything
      for (int f = fill + 1; f < nslot && f < fill + STAGES; ++f) mbar_wait_for(bars + f % STAGES, (f / STAGES) & 1, 10000000ull);
      failed = true;
      break;
    }
    // group gi of the slot: matrices of a group are adjacent; column blocks are G groups apart
    const uint8_t* blk = ring + s * SM::STAGE_BYTES + gi * (M * BLOCK_BYTES);
#pragma unroll
    for (int m = 0; m < Q; ++m) {
      const uint8_t* bm = blk + (M == 1 ? m * (G * BLOCK_BYTES) : m * BLOCK_BYTES);
      const uint4 sbv = *reinterpret_cast<const uint4*>(bm + SB_OFFSET + gq * 16);
#pragma unroll
      for (int tt = 0; tt < 2; ++tt) {
        const uint4 w = *reinterpret_cast<const uint4*>(bm + tt * TILE_BYTES + lane * 16);
        float p[PT][4];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint32_t lo = ks < 2 ? w.x : w.y, hi = ks < 2 ? w.z : w.w;
          const int sh = 8 * (ks & 1);
          const uint32_t a0 = nib_pair(lo, sh), a1 = nib_pair(hi, sh);
          const uint32_t a2 = nib_pair(lo, sh + 4), a3 = nib_pair(hi, sh + 4);
#pragma unroll
          for (int pt = 0; pt < PT; ++pt) {           // the fragment is dequantised once for every tile of pairs
            if (pt == 1 && !two) continue;
            if (ks == 0)
              mma_bf16_zero(p[pt], a0, a1, a2, a3, xb[pt][0], xb[pt][1]);
            else
              mma_bf16(p[pt], a0, a1, a2, a3, xb[pt][2 * ks], xb[pt][2 * ks + 1]);
          }
        }
        const float2 sb_lo = sb_pair<SB>(comp(sbv, 2 * tt)), sb_hi = sb_pair<SB>(comp(sbv, 2 * tt + 1));
        const float s_lo = sb_lo.x, s_hi = sb_hi.x;
        const float b_lo = fmaf(-128.f, s_lo, sb_lo.y), b_hi = fmaf(-128.f, s_hi, sb_hi.y);
#pragma unroll
        for (int pt = 0; pt < PT; ++pt) {
          if (pt == 1 && !two) continue;
          float(&d)[4] = acc[m][tt][pt];
          // two fp32 fmas an instruction; each half rounds like fmaf
          const float2 xs2 = make_float2(xs[pt][0], xs[pt][1]);
          const float2 lo2 = ffma2(xs2, make_float2(b_lo, b_lo),
                                   ffma2(make_float2(p[pt][0], p[pt][1]), make_float2(s_lo, s_lo), make_float2(d[0], d[1])));
          const float2 hi2 = ffma2(xs2, make_float2(b_hi, b_hi),
                                   ffma2(make_float2(p[pt][2], p[pt][3]), make_float2(s_hi, s_hi), make_float2(d[2], d[3])));
          d[0] = lo2.x; d[1] = lo2.y; d[2] = hi2.x; d[3] = hi2.y;
        }
      }
    }
    __syncwarp();
    if (lane == 0 && (gi == G - 1 || c == ng - 1) && fill + STAGES < nslot) issue(fill + STAGES);
  }
  pdl_launch_dependents();

  // K-slices meet in slice order (the ring's memory is free once every warp is past its loop)
  if (__syncthreads_or(failed ? 1 : 0)) return;
  float* red = reinterpret_cast<float*>(smem);
#pragma unroll
  for (int m = 0; m < Q; ++m)
#pragma unroll
    for (int tt = 0; tt < 2; ++tt)
#pragma unroll
      for (int pt = 0; pt < PT; ++pt) {
        float* base = red + ((warp * Q + m) * DEC_PAIRS + 8 * pt + 2 * t) * RED_STRIDE + tt * 16 + gq;
        base[0] = acc[m][tt][pt][0];
        base[RED_STRIDE] = acc[m][tt][pt][1];
        base[8] = acc[m][tt][pt][2];
        base[RED_STRIDE + 8] = acc[m][tt][pt][3];
      }
  __syncthreads();
  // thread -> (column block cbo of the CTA, pair, column): CBC * PAIRS * 32 outputs over 128 threads
  for (int o = tid; o < CBC * PAIRS * COLS; o += DEC_WARPS * 32) {
    const int col = o & 31, pi = (o >> 5) % PAIRS, cbo = o / (PAIRS * COLS);
    const int cbi = cbt * CBC + cbo;
    if (pi >= cnt || cbi >= NB) continue;
    const int w0 = (cbo / NCB) * KW, q0 = (cbo % NCB) * M;      // first K-slice warp and block of this column block
    if constexpr (EPI == EPI_SLICES) {                 // the K slices as they are: [KW, rows, N], `limit` holds rows
      const size_t rows = (size_t)__float_as_int(limit);
#pragma unroll
      for (int k = 0; k < KW; ++k)
        static_cast<float*>(out)[(k * rows + pair_id[pi]) * N + cbi * COLS + col] =
            red[(((w0 + k) * Q + q0) * DEC_PAIRS + pi) * RED_STRIDE + col];
      continue;
    }
    float v[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float sum = red[((w0 * Q + q0 + m) * DEC_PAIRS + pi) * RED_STRIDE + col];
#pragma unroll
      for (int k = 1; k < KW; ++k) sum += red[(((w0 + k) * Q + q0 + m) * DEC_PAIRS + pi) * RED_STRIDE + col];
      v[m] = sum;
    }
    const size_t at = (size_t)pair_id[pi] * N + cbi * COLS + col;
    if constexpr (EPI == EPI_F32 || EPI == EPI_SLICES) {
      static_cast<float*>(out)[at] = v[0];
    } else if constexpr (EPI == EPI_RELU2) {
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(relu2(v[0]));
    } else if constexpr (EPI == EPI_SWIGLU) {
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(swiglu(v[0], v[M - 1], limit));
    } else {
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(v[0]);
    }
  }
  if constexpr (COMBINE) {
    static_assert(EPI == EPI_F32 && M == 1, "the combine follows the fp32 down projection");
    __shared__ int done[DEC_PAIRS];
    __syncthreads();                                  // this CTA's rows before its counts
    if (tid < PAIRS) {
      int mine = 0;
      if (tid < cnt) {
        int* ctr = cmb.arrive + (size_t)(pair_id[tid] / cmb.slots) * NB + cbt;
        const int seen = arrive_count(ctr);
        if (seen == cmb.slots - 1) {
          *ctr = 0;                                   // nobody else touches it before the next launch
          mine = 1;
        }
      }
      done[tid] = mine;
    }
    __syncthreads();
    const float* y = static_cast<const float*>(out);
    for (int pi = 0; pi < cnt; ++pi) {
      if (!done[pi]) continue;                        // the same for every thread of the CTA
      const int token = pair_id[pi] / cmb.slots;
      for (int o = tid; o < CBC * COLS; o += DEC_WARPS * 32) {
        const int col = cbt * (CBC * COLS) + o;
        if (col >= N) continue;
        const float* rows = y + (size_t)token * cmb.slots * N + col;
        const float* w = cmb.wts + (size_t)token * cmb.slots;
        float acc = 0.f;
        for (int s0 = 0; s0 < cmb.slots; s0 += 8) {   // eight rows in flight, then their fma chain in slot order
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = s0 + j < cmb.slots ? __ldcg(rows + (size_t)(s0 + j) * N) : 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (s0 + j < cmb.slots) acc = fmaf(w[s0 + j], v[j], acc);
        }
        if (cmb.out_f32)
          static_cast<float*>(cmb.out)[(size_t)token * N + col] = acc;
        else
          static_cast<__nv_bfloat16*>(cmb.out)[(size_t)token * N + col] = __float2bfloat16_rn(acc);
      }
    }
  }
}

// SMs of the current device (looked up once a device)
inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// K-slices a CTA for a projection of kg groups: the shape's alone, so a pair's bits never depend on the call.
__host__ __device__ inline int decode_kslices(int kg) { return kg >= 32 ? 4 : kg >= 8 ? 2 : 1; }

// DEEP: a grid of at most three CTAs an SM (a few tokens) is bound by the latency of a warp's own stream, not by how
// many CTAs share an SM: four slots put a K slice of eight groups in flight at once.
template <int M, int EPI, int SB, int KW, int PT, bool DEEP, bool COMBINE>
int launch_decode_kw(const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb, const int* items,
                     const int* counts, const int* members, void* out, int n, float limit, int64_t max_items,
                     cudaStream_t stream, CombineArgs cmb) {
  // two groups a slot, two slots a warp (9.2 KB); gate/up items of 16 pairs keep more registers a thread, so fewer
  // CTAs share an SM (4, by the launch bounds) and each gets a third slot
  constexpr int G = 2;
  constexpr int STAGES = DEEP ? 4 : M == 2 && PT == 2 ? 3 : 2;
  constexpr int NCB = M == 1 ? 2 : 1;                 // one matrix: a warp shares its inputs between two column blocks
  using SM = DecodeSmem<M * NCB, G, STAGES>;
  auto* kern = decode_kernel<M, NCB, EPI, SB, KW, G, STAGES, PT, COMBINE>;
  static_assert(SM::TOTAL <= (DEEP ? 75 : M == 2 && PT == 2 ? 56 : 48) * 1024, "the decode kernel's shared memory lets 3, 4 or 5 CTAs share an SM");
  if constexpr (SM::TOTAL > 48 * 1024) {
    static bool configured[64] = {false};
    int dev = 0;
    TFB_CUDA(cudaGetDevice(&dev), "experts_run: cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(TFB_ERR_ARG, "experts_run: device index %d out of range", dev);
    if (!configured[dev]) {
      TFB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL),
               "experts_run: shared memory opt-in");
      configured[dev] = true;
    }
  }
  constexpr int CBC = DEC_WARPS / KW * NCB;
  const int64_t grid = max_items * ((nb + CBC - 1) / CBC);
  if (grid >= (int64_t(1) << 31)) return fail(TFB_ERR_ARG, "experts_run: too many units");
  return check_cuda(launch(kern, dim3((unsigned)grid), dim3(DEC_WARPS * 32), (size_t)SM::TOTAL, stream,
                           static_cast<const __nv_bfloat16*>(x), x_stride, slots, static_cast<const uint8_t*>(w), kg,
                           nb, items, counts, members, out, n, limit, cmb),
                    "experts_run");
}

template <int M, int EPI, int SB, int PT, bool COMBINE = false>
int launch_decode(const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb, const int* items,
                  const int* counts, const int* members, void* out, int n, float limit, int64_t max_items,
                  cudaStream_t stream, CombineArgs cmb = CombineArgs{nullptr, nullptr, nullptr, 0, 0}) {
  const int kw = decode_kslices(kg);
  if constexpr (PT == 1) {
    const int cbc = DEC_WARPS / kw * (M == 1 ? 2 : 1);
    if (max_items * ((nb + cbc - 1) / cbc) <= 3 * sm_count()) {
      switch (kw) {
        case 4:
          return launch_decode_kw<M, EPI, SB, 4, PT, true, COMBINE>(x, x_stride, slots, w, kg, nb, items, counts, members, out,
                                                           n, limit, max_items, stream, cmb);
        case 2:
          return launch_decode_kw<M, EPI, SB, 2, PT, true, COMBINE>(x, x_stride, slots, w, kg, nb, items, counts, members, out,
                                                           n, limit, max_items, stream, cmb);
        default:
          return launch_decode_kw<M, EPI, SB, 1, PT, true, COMBINE>(x, x_stride, slots, w, kg, nb, items, counts, members, out,
                                                           n, limit, max_items, stream, cmb);
      }
    }
  }
  switch (kw) {
    case 4:
      return launch_decode_kw<M, EPI, SB, 4, PT, false, COMBINE>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n,
                                                        limit, max_items, stream, cmb);
    case 2:
      return launch_decode_kw<M, EPI, SB, 2, PT, false, COMBINE>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n,
                                                        limit, max_items, stream, cmb);
    default:
      return launch_decode_kw<M, EPI, SB, 1, PT, false, COMBINE>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n,
                                                        limit, max_items, stream, cmb);
  }
}

}  // namespace tfb

using namespace tfb;

static int experts_run(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb,
                       const int32_t* items, const int32_t* counts, const int32_t* members, void* out, int n,
                       float limit, int64_t max_units, int sb_type, int tile, void* stream) {
  TFB_REQUIRE(gs == GS, "experts_run: groups of %d inputs only, not %d", GS, gs);
  TFB_REQUIRE(x && w && items && counts && members && out, "experts_run: null pointer");
  TFB_REQUIRE(kg >= 1 && nb >= 1 && n == nb * COLS, "experts_run: n must be the column blocks times %d", COLS);
  TFB_REQUIRE(aligned16(x) && x_stride % 8 == 0 && x_stride >= (int64_t)kg * GS,
              "experts_run: x rows of K = groups * group size inputs, 16-byte aligned");
  TFB_REQUIRE(aligned16(w), "experts_run: w must be 16-byte aligned");
  TFB_REQUIRE(slots >= 0 && max_units >= 0 && max_units < (int64_t(1) << 31), "experts_run: bad slots or unit count");
  TFB_REQUIRE(sb_type == SB_BF16 || sb_type == SB_FP16, "experts_run: scales are bf16 (0) or fp16 (1), not %d", sb_type);
  TFB_REQUIRE(tile == 8 || tile == 16, "experts_run: items of 8 or 16 pairs, not %d", tile);
  const int64_t max_items = (max_units + nb - 1) / nb;
  if (max_items == 0) return TFB_OK;
  auto st = static_cast<cudaStream_t>(stream);
#define TFB_RUN3(EPI_, M_, SB_)                                                                                    \
  return tile == 8 ? launch_decode<M_, EPI_, SB_, 1>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n, \
                                                     limit, max_items, st)                                         \
                   : launch_decode<M_, EPI_, SB_, 2>(x, x_stride, slots, w, kg, nb, items, counts, members, out, n, \
                                                     limit, max_items, st)
#define TFB_RUN(EPI_, M_)                              \
  if (epi == EPI_) {                                   \
    if (sb_type == SB_BF16) TFB_RUN3(EPI_, M_, SB_BF16); \
    TFB_RUN3(EPI_, M_, SB_FP16);                       \
  }
  TFB_RUN(EPI_F32, 1) TFB_RUN(EPI_RELU2, 1) TFB_RUN(EPI_SWIGLU, 2) TFB_RUN(EPI_BF16, 1) TFB_RUN(EPI_SLICES, 1)
#undef TFB_RUN
#undef TFB_RUN3
  return fail(TFB_ERR_ARG, "experts_run: no kernel for epilogue %d", epi);
}

// Grouped 4-bit expert matmul, decode form.  Arguments as the reference extension's `run`
// (src/tensorfold/cuda/experts.cpp:43-48): epi 0 fp32 out, 1 relu^2, 2 SwiGLU over (gate, up), 3 bf16 out.
// max_units = an upper bound of items * nb, as the reference passes it.  Items hold at most 8 pairs.
extern "C" int tfb_experts_run(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg,
                               int nb, const int32_t* items, const int32_t* counts, const int32_t* members, void* out,
                               int n, float limit, int64_t max_units, int sb_type, void* stream) {
  TFB_REQUIRE(epi >= EPI_F32 && epi <= EPI_BF16, "experts_run: no kernel for epilogue %d", epi);
  return experts_run(gs, epi, x, x_stride, slots, w, kg, nb, items, counts, members, out, n, limit, max_units, sb_type,
                     8, stream);
}

// The same over a plan whose items hold up to `tile` = 8 or 16 pairs: with 16 a weight fragment is dequantised once
// for two mma tiles of pairs, which pays when experts see 9 or more pairs each (expert-parallel ranks, larger decode
// batches).  A pair's bits do not depend on the tile.
extern "C" int tfb_experts_run_tile(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg,
                                    int nb, const int32_t* items, const int32_t* counts, const int32_t* members,
                                    void* out, int n, float limit, int64_t max_units, int sb_type, int tile,
                                    void* stream) {
  TFB_REQUIRE(epi >= EPI_F32 && epi <= EPI_BF16, "experts_run: no kernel for epilogue %d", epi);
  return experts_run(gs, epi, x, x_stride, slots, w, kg, nb, items, counts, members, out, n, limit, max_units, sb_type,
                     tile, stream);
}

// The decode form with its K slices left apart: part [tfb_decode_kslices(kg), rows, n] fp32, slice k of pair p at
// part[k, p, :]; adding the slices in order k = 0, 1, .. gives epilogue 0's bits.  For a caller that folds the sum into
// its next kernel.  (src/tensorfold/cuda/kernels/qmm.py:156-177 `matmul(reduce=False, part=)`)
extern "C" int tfb_experts_run_slices(int gs, const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb,
                                      const int32_t* items, const int32_t* counts, const int32_t* members, float* part,
                                      int n, int rows, int64_t max_units, int sb_type, int tile, void* stream) {
  TFB_REQUIRE(rows >= 0, "experts_run_slices: bad row count %d", rows);
  float carried;
  static_assert(sizeof(carried) == sizeof(rows), "the row count rides in the limit's four bytes");
  memcpy(&carried, &rows, sizeof(carried));
  return experts_run(gs, EPI_SLICES, x, x_stride, slots, w, kg, nb, items, counts, members, part, n, carried, max_units,
                     sb_type, tile, stream);
}

// K slices the decode form cuts a projection of kg groups into (a function of the shape alone).
extern "C" int tfb_decode_kslices(int kg) { return decode_kslices(kg); }

// The down projection and the weighted combine in one launch: y [P, n] fp32 per pair as tfb_experts_run_tile with
// epilogue 0 (x = act [P, K] bf16, one row a pair), and out [T, n] (bf16, or fp32 when out_f32) = sum over a token's
// slots in slot order of wts[t, s] * y[t * slots + s, :], formed by the CTA that stores the token's last row.  Every
// pair t * slots + s of the T tokens must be in the plan.  arrive: int scratch [T, nb], zero before the first call (a
// call leaves it zero).  (src/tensorfold/cuda/experts.py:141-150 `down` then src/tensorfold/cuda/moe.py:131-151 `combine`)
extern "C" int tfb_experts_down_combine(int gs, const void* x, int64_t x_stride, const void* w, int kg, int nb,
                                        const int32_t* items, const int32_t* counts, const int32_t* members, float* y,
                                        int n, int64_t max_units, int sb_type, int tile, const float* wts, int slots,
                                        void* out, int out_f32, int32_t* arrive, void* stream) {
  TFB_REQUIRE(gs == GS, "experts_down_combine: groups of %d inputs only, not %d", GS, gs);
  TFB_REQUIRE(x && w && items && counts && members && y && wts && out && arrive, "experts_down_combine: null pointer");
  TFB_REQUIRE(kg >= 1 && nb >= 1 && n == nb * COLS, "experts_down_combine: n must be the column blocks times %d", COLS);
  TFB_REQUIRE(aligned16(x) && x_stride % 8 == 0 && x_stride >= (int64_t)kg * GS,
              "experts_down_combine: x rows of K = groups * group size inputs, 16-byte aligned");
  TFB_REQUIRE(aligned16(w), "experts_down_combine: w must be 16-byte aligned");
  TFB_REQUIRE(slots >= 1 && max_units >= 0 && max_units < (int64_t(1) << 31), "experts_down_combine: bad slots or unit count");
  TFB_REQUIRE(sb_type == SB_BF16 || sb_type == SB_FP16, "experts_down_combine: scales are bf16 (0) or fp16 (1), not %d",
              sb_type);
  TFB_REQUIRE(tile == 8 || tile == 16, "experts_down_combine: items of 8 or 16 pairs, not %d", tile);
  const int64_t max_items = (max_units + nb - 1) / nb;
  if (max_items == 0) return TFB_OK;
  auto st = static_cast<cudaStream_t>(stream);
  const CombineArgs cmb{wts, out, arrive, slots, out_f32 ? 1 : 0};
#define TFB_DC(SB_)                                                                                                  \
  return tile == 8 ? launch_decode<1, EPI_F32, SB_, 1, true>(x, x_stride, 0, w, kg, nb, items, counts, members, y, n, \
                                                             0.f, max_items, st, cmb)                                \
                   : launch_decode<1, EPI_F32, SB_, 2, true>(x, x_stride, 0, w, kg, nb, items, counts, members, y, n, \
                                                             0.f, max_items, st, cmb)
  if (sb_type == SB_BF16) TFB_DC(SB_BF16);
  TFB_DC(SB_FP16);
#undef TFB_DC
}
