// Router logits, top-k selection with softmax renormalisation, the expert plan (token sort) and the weighted
// combine. Every result is a function of its own row only, so a row's bits never depend on the call's other rows.

#include <cooperative_groups.h>

#include "api.h"
#include "common.cuh"

namespace tfb {

// ================================================================================================================
// Router: logits[r, e] = sum_k x[r, k] * w[e, k] in fp32, in ONE documented order so a CPU restatement can follow it
// bit for bit: lane l of 32 walks k = 256 c + 8 l + j (c ascending, j = 0..7) with acc = fma(x, w, acc), then the 32
// lane sums meet in a butterfly (xor 16, 8, 4, 2, 1).  (Reference: src/tensorfold/cuda/moe.py:23-55 leaves the
// order to Triton's tl.dot.)
// ================================================================================================================
constexpr int R_WARPS = 4, R_ET = 4, R_RT = 8;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

__global__ void __launch_bounds__(R_WARPS * 32)
router_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_stride, const __nv_bfloat16* __restrict__ W,
              float* __restrict__ out, int T, int D, int NE) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e0 = (blockIdx.y * R_WARPS + warp) * R_ET;
  const int r0 = blockIdx.x * R_RT;
  if (e0 >= NE) return;
  const int nr = min(R_RT, T - r0), ne = min(R_ET, NE - e0);
  float acc[R_RT][R_ET];
#pragma unroll
  for (int r = 0; r < R_RT; ++r)
#pragma unroll
    for (int e = 0; e < R_ET; ++e) acc[r][e] = 0.f;
  pdl_wait();
  after_wait(X);
  // the next chunk's twelve 16-byte loads travel while this chunk's 256 fmas run
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 wn[R_ET], xn[R_RT];
  auto fetch = [&](int k) {
#pragma unroll
    for (int e = 0; e < R_ET; ++e) wn[e] = (e < ne && k < D) ? ldg_nc(W + (size_t)(e0 + e) * D + k) : zero;
#pragma unroll
    for (int r = 0; r < R_RT; ++r) xn[r] = (r < nr && k < D) ? ldg_nc(X + (size_t)(r0 + r) * x_stride + k) : zero;
  };
  fetch(8 * lane);
  for (int k = 8 * lane; k < D; k += 256) {
    float wv[R_ET][8];
    uint4 xc[R_RT];
#pragma unroll
    for (int e = 0; e < R_ET; ++e) unpack8(wn[e], wv[e]);
#pragma unroll
    for (int r = 0; r < R_RT; ++r) xc[r] = xn[r];
    fetch(k + 256);
    // two rows an instruction (fma.rn.f32x2: each half is the fmaf of its own row, in the same k order); rows past
    // the last were fetched as zeros and are never stored
#pragma unroll
    for (int r = 0; r < R_RT; r += 2) {
      float xa[8], xb[8];
      unpack8(xc[r], xa);
      unpack8(xc[r + 1], xb);
#pragma unroll
      for (int e = 0; e < R_ET; ++e)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 d = ffma2(make_float2(xa[j], xb[j]), make_float2(wv[e][j], wv[e][j]),
                                 make_float2(acc[r][e], acc[r + 1][e]));
          acc[r][e] = d.x;
          acc[r + 1][e] = d.y;
        }
    }
  }
  pdl_launch_dependents();
#pragma unroll
  for (int r = 0; r < R_RT; ++r)
#pragma unroll
    for (int e = 0; e < R_ET; ++e) {
      float a = acc[r][e];
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) a = a + __shfl_xor_sync(0xffffffffu, a, m);
      if (lane == 0 && r < nr && e < ne) out[(size_t)(r0 + r) * NE + e0 + e] = a;
    }
}

// The same arithmetic for few rows: a CTA an expert and eight rows, a warp a row, every chunk of the row's inputs and
// of the expert's weights in flight at once (two memory round trips in all).  Bits equal router_kernel's.
constexpr int RR_WARPS = 8, RR_ROWS = 8, RR_CH = 8;

__global__ void __launch_bounds__(RR_WARPS * 32)
router_rows_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_stride, const __nv_bfloat16* __restrict__ W,
                   float* __restrict__ out, int T, int D, int NE) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = blockIdx.x, rbase = blockIdx.y * RR_ROWS;
  constexpr int RPW = RR_ROWS / RR_WARPS;
  float acc[RPW];
#pragma unroll
  for (int i = 0; i < RPW; ++i) acc[i] = 0.f;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  pdl_wait();
  after_wait(X);
  for (int kb = 0; kb < D; kb += 256 * RR_CH) {
    float wv[RR_CH][8];
#pragma unroll
    for (int c = 0; c < RR_CH; ++c) {
      const int k = kb + 256 * c + 8 * lane;
      unpack8(k < D ? ldg_nc(W + (size_t)e * D + k) : zero, wv[c]);
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const int r = rbase + warp + RR_WARPS * i;
      if (r >= T) break;
      uint4 xv[RR_CH];
#pragma unroll
      for (int c = 0; c < RR_CH; ++c) {
        const int k = kb + 256 * c + 8 * lane;
        xv[c] = k < D ? ldg_nc(X + (size_t)r * x_stride + k) : zero;
      }
#pragma unroll
      for (int c = 0; c < RR_CH; ++c) {
        if (kb + 256 * c + 8 * lane < D) {
          float xf[8];
          unpack8(xv[c], xf);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i] = fmaf(xf[j], wv[c][j], acc[i]);
        }
      }
    }
  }
  pdl_launch_dependents();
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int r = rbase + warp + RR_WARPS * i;
    float a = acc[i];
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) a = a + __shfl_xor_sync(0xffffffffu, a, m);
    if (lane == 0 && r < T) out[(size_t)r * NE + e] = a;
  }
}

// ================================================================================================================
// The router for prompts, on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 accumulate).  A CTA of eight warps owns
// 64 rows x 32 experts: four row tiles times two halves of the inputs, the halves added in order (first + second).
// Per block of 32 inputs a lane loads 8 consecutive inputs of its rows and of its experts' rows as one 16-byte word
// each; the two mma steps of a block take inputs (0, 1 | 2, 3) and (4, 5 | 6, 7) of every lane's word - A and B are
// permuted alike, so the products pair up correctly.  Two blocks are in flight while two are multiplied.  The order
// of the sum is fixed: a row's logits do not depend on the other rows of the call.  The last bits differ from the
// fp32-fma router's (the reference's Triton router changes its blocking with the row count in the same way,
// src/tensorfold/cuda/moe.py:23-55).
// ================================================================================================================
constexpr int RT_ROWT = 4, RT_KH = 2, RT_NT = 4;     // row tiles and input halves a CTA; n-tiles of 8 experts a warp

__global__ void __launch_bounds__(RT_ROWT * RT_KH * 32)
router_mma_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_stride, const __nv_bfloat16* __restrict__ W,
                  float* __restrict__ out, int T, int D, int NE) {
  __shared__ float part[RT_ROWT][RT_NT * 4][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int rt = warp % RT_ROWT, kh = warp / RT_ROWT;
  const int r0 = (blockIdx.x * RT_ROWT + rt) * 16, e0 = blockIdx.y * (8 * RT_NT);
  pdl_wait();
  after_wait(X);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  // rows past the last and experts past the last are read as zeros and never stored
  const bool row_lo = r0 + g < T, row_hi = r0 + g + 8 < T;
  const int blocks = D / 32, half = (blocks + RT_KH - 1) / RT_KH;
  const int kb0 = min(blocks, kh * half), kb1 = min(blocks, kb0 + half);
  const __nv_bfloat16* xa = X + (size_t)(row_lo ? r0 + g : 0) * x_stride + 8 * t;
  const __nv_bfloat16* xb = X + (size_t)(row_hi ? r0 + g + 8 : 0) * x_stride + 8 * t;
  const __nv_bfloat16* wr[RT_NT];
  bool live[RT_NT];
#pragma unroll
  for (int j = 0; j < RT_NT; ++j) {
    live[j] = e0 + 8 * j + g < NE;
    wr[j] = W + (size_t)(live[j] ? e0 + 8 * j + g : 0) * D + 8 * t;
  }
  float acc[RT_NT][4];
#pragma unroll
  for (int j = 0; j < RT_NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  uint4 an[2][2], bn[2][RT_NT];                       // the two blocks in flight
  auto fetch = [&](int kb) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const bool in = kb + u < kb1;
      const int k = (kb + u) * 32;
      an[u][0] = in && row_lo ? ldg_nc(xa + k) : zero;
      an[u][1] = in && row_hi ? ldg_nc(xb + k) : zero;
#pragma unroll
      for (int j = 0; j < RT_NT; ++j) bn[u][j] = in && live[j] ? ldg_nc(wr[j] + k) : zero;
    }
  };
  fetch(kb0);
  for (int kb = kb0; kb < kb1; kb += 2) {
    uint4 a[2][2], b[2][RT_NT];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      a[u][0] = an[u][0];
      a[u][1] = an[u][1];
#pragma unroll
      for (int j = 0; j < RT_NT; ++j) b[u][j] = bn[u][j];
    }
    fetch(kb + 2);                                    // past the end: zeros, no loads
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int j = 0; j < RT_NT; ++j) {
        mma_bf16(acc[j], a[u][0].x, a[u][1].x, a[u][0].y, a[u][1].y, b[u][j].x, b[u][j].y);
        mma_bf16(acc[j], a[u][0].z, a[u][1].z, a[u][0].w, a[u][1].w, b[u][j].z, b[u][j].w);
      }
  }
  pdl_launch_dependents();
  if (kh == 1) {
#pragma unroll
    for (int j = 0; j < RT_NT; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) part[rt][4 * j + i][lane] = acc[j][i];
  }
  __syncthreads();
  if (kh != 0) return;
  // acc[j]: (row g, expert 2t), (row g, 2t + 1), (row g + 8, 2t), (row g + 8, 2t + 1) of n-tile j
#pragma unroll
  for (int j = 0; j < RT_NT; ++j) {
    const int e = e0 + 8 * j + 2 * t;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = acc[j][i] + part[rt][4 * j + i][lane];
    if (row_lo) {
      if (e < NE) out[(size_t)(r0 + g) * NE + e] = v[0];
      if (e + 1 < NE) out[(size_t)(r0 + g) * NE + e + 1] = v[1];
    }
    if (row_hi) {
      if (e < NE) out[(size_t)(r0 + g + 8) * NE + e] = v[2];
      if (e + 1 < NE) out[(size_t)(r0 + g + 8) * NE + e + 1] = v[3];
    }
  }
}

// ================================================================================================================
// Selection: a warp a row.  TOPK rounds of (largest fp32 logit, the lower id among equals), weight
// bf16(exp(l_k - l_0) / sum_k exp(l_k - l_0)); with a shared expert, slot TOPK = id E with weight
// bf16(sigmoid(bf16(logit E))).  (src/tensorfold/cuda/moe.py:58-85)
// ================================================================================================================
constexpr int S_WARPS = 4;

// One row by one warp: writes the row's slots of pick / wts; returns this lane's pick (lanes < slots) for callers
// that keep the picks on chip.
// fp32 -> uint32 that orders the same way (both zeros share a key, as they compare equal), and back
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = f == 0.f ? 0u : __float_as_uint(f);
  return u ^ (static_cast<uint32_t>(static_cast<int32_t>(u) >> 31) | 0x80000000u);
}
__device__ __forceinline__ float order_value(uint32_t k) {
  return __uint_as_float(k ^ ((k & 0x80000000u) ? 0x80000000u : 0xFFFFFFFFu));
}

template <int VPL>
__device__ __forceinline__ int select_row(const float* __restrict__ Lr, int E, int top_k, int shared, int lane,
                                          int* __restrict__ pick_row, float* __restrict__ wts_row) {
  // keys order like the logits; 0 (below every real key) marks a taken or missing entry
  uint32_t key[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = i * 32 + lane;
    key[i] = e < E ? order_key(__ldcg(Lr + e)) : 0u;      // L2: another CTA of this launch may have written it
  }
  float top = 0.f, total = 0.f, my_ex = 0.f;
  int my_pick = -1;
  for (int k = 0; k < top_k; ++k) {
    uint32_t bk = key[0];
    uint32_t bi = lane;
#pragma unroll
    for (int i = 1; i < VPL; ++i)
      if (key[i] > bk) {
        bk = key[i];
        bi = i * 32 + lane;
      }
    const uint32_t mx = __reduce_max_sync(0xffffffffu, bk);
    const uint32_t idx = __reduce_min_sync(0xffffffffu, bk == mx ? bi : 0xFFFFFFFFu);   // the lower id among equals
    const float val = order_value(mx);
    if (k == 0) top = val;
    const float ex = expf(val - top);
    total += ex;
    if (lane == k) {
      my_pick = (int)idx;
      my_ex = ex;
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (i * 32 + lane == (int)idx) key[i] = 0u;
  }
  if (lane < top_k) {
    pick_row[lane] = my_pick;
    wts_row[lane] = round_bf16(my_ex / total);
  } else if (lane == top_k && shared) {
    const float sg = round_bf16(__ldcg(Lr + E));
    my_pick = E;
    pick_row[lane] = E;
    wts_row[lane] = round_bf16(1.f / (1.f + expf(-sg)));
  }
  return my_pick;
}

template <int VPL>
__global__ void __launch_bounds__(S_WARPS * 32)
select_kernel(const float* __restrict__ L, int NL, int* __restrict__ pick, float* __restrict__ wts, int T, int E,
              int top_k, int shared) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * S_WARPS + (threadIdx.x >> 5);
  if (r >= T) return;
  pdl_wait();
  after_wait(L);
  const int slots = top_k + (shared ? 1 : 0);
  select_row<VPL>(L + (size_t)r * NL, E, top_k, shared, lane, pick + (size_t)r * slots, wts + (size_t)r * slots);
  pdl_launch_dependents();
}

// Sigmoid-plus-bias selection (the GLM and Nemotron routers): score = sigmoid(logit); the TOPK experts with the
// largest score + bias (the lower id among equals); weights = the picked scores, divided by their sum in pick order
// when `norm` (sum + 1e-20), times `scale`; then `shared` slots with ids E, E + 1, .. and weight 1.
// (src/tensorfold/families/glm5_next/cuda/glue.py:351-390; src/tensorfold/families/nemotron_h/cuda/glue.py:50-100)
template <int VPL>
__global__ void __launch_bounds__(S_WARPS * 32)
select_sigmoid_kernel(const float* __restrict__ L, int NL, const float* __restrict__ bias, int* __restrict__ pick,
                      float* __restrict__ wts, int T, int E, int top_k, int shared, float scale, int norm) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * S_WARPS + (threadIdx.x >> 5);
  if (r >= T) return;
  pdl_wait();
  after_wait(L);
  const int slots = top_k + shared;
  const float* Lr = L + (size_t)r * NL;
  uint32_t key[VPL];
  float score[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = i * 32 + lane;
    score[i] = e < E ? 1.f / (1.f + expf(-Lr[e])) : 0.f;
    key[i] = e < E ? order_key(score[i] + bias[e]) : 0u;
    if (e < E && key[i] == 0u) key[i] = 1u;           // -inf / NaN choices still rank above "taken"
  }
  float total = 0.f, my_score = 0.f;
  int my_pick = -1;
  for (int k = 0; k < top_k; ++k) {
    uint32_t bk = key[0];
    uint32_t bi = lane;
    float bs = score[0];
#pragma unroll
    for (int i = 1; i < VPL; ++i)
      if (key[i] > bk) {
        bk = key[i];
        bi = i * 32 + lane;
        bs = score[i];
      }
    const uint32_t mx = __reduce_max_sync(0xffffffffu, bk);
    const uint32_t idx = __reduce_min_sync(0xffffffffu, bk == mx ? bi : 0xFFFFFFFFu);
    const float sk = __shfl_sync(0xffffffffu, bs, idx & 31u);      // the owner lane's best is this entry
    total += sk;
    if (lane == k) {
      my_pick = (int)idx;
      my_score = sk;
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (i * 32 + lane == (int)idx) key[i] = 0u;
  }
  int* pick_row = pick + (size_t)r * slots;
  float* wts_row = wts + (size_t)r * slots;
  if (lane < top_k) {
    float w = my_score;
    if (norm) w = w / (total + 1e-20f);
    pick_row[lane] = my_pick;
    wts_row[lane] = w * scale;
  } else if (lane < slots) {
    pick_row[lane] = E + (lane - top_k);
    wts_row[lane] = 1.f;
  }
  pdl_launch_dependents();
}

// ================================================================================================================
// Plan: pairs p = row * slots + slot grouped by ascending expert, pair order kept inside an expert (a stable counting
// sort); items (expert, first, count <= tile) in expert order then chunk order; counts = (items, distinct experts).
// One block: each of the 32 warps owns a contiguous run of pairs, counts them per expert, a scan over warps and over
// experts gives every (warp, expert) its first slot, and a second walk scatters.  Ids outside [0, E) are left out.
// (Semantics of src/tensorfold/cuda/experts.cu:157-285, pinned by tests/cuda/test_experts.py:107-134.)
// ================================================================================================================
constexpr int PLAN_THREADS = 1024, PLAN_EMAX = 1024, PLAN_BATCH = 8;

// A split plan: experts with at least `hot` pairs get their items (of Tb pairs) in a second table, for the prompt-form
// kernel; the others stay in the first (items of T pairs).  hot = INT_MAX (and no second table): the plain plan.
struct PlanSplit {
  int hot, Tb;
  int* items;        // second table [., 3], or null
  int* counts;       // [2]: its items, its distinct experts
};

// Exclusive prefix over the NT threads of a block, of two packed 64-bit values a thread; sum_* = the block's totals.
// tot: [2][NT / 32] in shared memory.  Every thread of the block calls it.
template <int NT>
__device__ __forceinline__ void block_prefix2(uint64_t& a, uint64_t& b, uint64_t (*tot)[NT / 32], uint64_t& sum_a,
                                              uint64_t& sum_b) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t ia = a, ib = b;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint64_t ua = __shfl_up_sync(0xffffffffu, ia, o), ub = __shfl_up_sync(0xffffffffu, ib, o);
    if (lane >= o) {
      ia += ua;
      ib += ub;
    }
  }
  if (lane == 31) {
    tot[0][warp] = ia;
    tot[1][warp] = ib;
  }
  __syncthreads();
  if (warp == 0) {                                   // the warps' totals become their inclusive prefix, in place
    uint64_t ta = lane < NT / 32 ? tot[0][lane] : 0, tb = lane < NT / 32 ? tot[1][lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint64_t ua = __shfl_up_sync(0xffffffffu, ta, o), ub = __shfl_up_sync(0xffffffffu, tb, o);
      if (lane >= o) {
        ta += ua;
        tb += ub;
      }
    }
    if (lane < NT / 32) {
      tot[0][lane] = ta;
      tot[1][lane] = tb;
    }
  }
  __syncthreads();
  const uint64_t base_a = warp ? tot[0][warp - 1] : 0, base_b = warp ? tot[1][warp - 1] : 0;
  sum_a = tot[0][NT / 32 - 1];
  sum_b = tot[1][NT / 32 - 1];
  a = base_a + ia - a;
  b = base_b + ib - b;
  __syncthreads();                                   // tot is free again
}

// The lanes of the warp whose key equals this lane's (keys < 2^nbits; lanes with ok == false match nobody): one ballot
// a key bit.  (match.any does the same but walks the distinct keys one by one, ~30 of them in a warp of random picks.)
__device__ __forceinline__ unsigned same_key_lanes(int e, bool ok, int nbits) {
  unsigned m = __ballot_sync(0xffffffffu, ok);
  for (int b = 0; b < nbits; ++b) {
    const bool bit = (e >> b) & 1;
    const unsigned bal = __ballot_sync(0xffffffffu, bit);
    m &= bit ? bal : ~bal;
  }
  return ok ? m : 0u;
}

template <bool CG>
__device__ __forceinline__ int load_pick(const int* p) {
  if constexpr (CG) return __ldcg(p);                // written by other CTAs of this launch: read it in L2
  else return *p;
}

// The whole block of NT threads: `picks` may live in global or shared memory (CG: global, written earlier in the same
// launch).  Each of the NT / 32 warps owns a contiguous run of pairs, counts them per expert (whist [NT / 32][E]), a
// prefix over the warps and over the experts (in turns of NT experts) gives every (warp, expert) its first slot, and
// a second walk scatters.  first: [E]; tot2: [2][NT / 32]; all in shared memory.
// With `ctot` (a cluster launch: `nparts` blocks, this one `part`; E <= NT) the pairs are cut into nparts * NT / 32
// runs; each block counts its runs, the blocks read one another's per-expert totals through distributed shared memory,
// and each scatters its own runs.  The tables are the same as one block's.
template <int NT, bool CG = false>
__device__ void plan_block(const int* picks, int P, int E, int T, int* __restrict__ members, int* __restrict__ items,
                           int* __restrict__ counts, int* whist, int* first, uint64_t (*tot2)[NT / 32], int lo = 0,
                           PlanSplit sp = PlanSplit{0x7FFFFFFF, 1, nullptr, nullptr}, int* ctot = nullptr,
                           int part = 0, int nparts = 1) {
  constexpr int NWARP = NT / 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < NWARP * E; i += NT) whist[i] = 0;
  const int runs = NWARP * nparts;
  const int seg = (((P + runs - 1) / runs + 31) / 32) * 32;
  const int p0 = (int)min((int64_t)P, (int64_t)(part * NWARP + warp) * seg), p1 = min(P, p0 + seg);
  int* mine = whist + warp * E;
  const int nbits = 32 - __clz(max(E - 1, 0));
  __syncthreads();
  for (int base0 = p0; base0 < p1; base0 += 32 * PLAN_BATCH) {
    int ev[PLAN_BATCH];                              // the loads of a batch are independent: all in flight at once
#pragma unroll
    for (int i = 0; i < PLAN_BATCH; ++i) {
      const int p = base0 + 32 * i + lane;
      ev[i] = p < p1 ? load_pick<CG>(picks + p) - lo : -1;
    }
#pragma unroll
    for (int i = 0; i < PLAN_BATCH; ++i) {
      if (base0 + 32 * i >= p1) break;
      const int e = ev[i];
      const bool ok = e >= 0 && e < E;
      const unsigned peers = same_key_lanes(e, ok, nbits);
      if (ok && lane == __ffs(peers) - 1) mine[e] += __popc(peers);
      __syncwarp();
    }
  }
  __syncthreads();
  // experts in turns of NT: an expert's pairs, items and (for a split plan) hot items get their first slots from a
  // prefix over the experts; two packed words: A = pairs | items << 32, B = experts in use | hot items << 16 | hot
  // experts << 48
  uint64_t carry_a = 0, carry_b = 0;
  for (int e0 = 0; e0 < E; e0 += NT) {
    const int e = e0 + tid;
    const bool live = e < E;
    int c = 0;
    if (live)
      for (int w = 0; w < NWARP; ++w) {
        const int v = whist[w * E + e];
        whist[w * E + e] = c;
        c += v;
      }
    int before = 0;                                  // pairs of this expert in the blocks before this one
    if (ctot != nullptr) {
      namespace cg = cooperative_groups;
      cg::cluster_group cluster = cg::this_cluster();
      if (live) ctot[e] = c;
      cluster.sync();
      if (live) {
        c = 0;
        for (int r = 0; r < nparts; ++r) {
          const int v = cluster.map_shared_rank(ctot, r)[e];
          if (r < part) before += v;
          c += v;
        }
      }
    }
    const bool hot = c >= sp.hot;
    const int n_items = hot ? 0 : (c + T - 1) / T, n_hot = hot ? (c + sp.Tb - 1) / sp.Tb : 0;
    uint64_t a = (uint64_t)(uint32_t)c | ((uint64_t)(uint32_t)n_items << 32);
    uint64_t b = (uint64_t)(c > 0 && !hot ? 1u : 0u) | ((uint64_t)(uint32_t)n_hot << 16) | ((uint64_t)(hot ? 1u : 0u) << 48);
    uint64_t sum_a, sum_b;
    block_prefix2<NT>(a, b, tot2, sum_a, sum_b);
    a += carry_a;
    b += carry_b;
    if (live) {
      const int at = (int)(uint32_t)a, item0 = (int)(a >> 32), hot0 = (int)((b >> 16) & 0xFFFFFFFFu);
      first[e] = at + before;                        // every block of a cluster writes the same tables
      for (int j = 0; j < n_items; ++j) {
        int* it = items + 3 * (item0 + j);
        it[0] = e;
        it[1] = at + T * j;
        it[2] = min(T, c - T * j);
      }
      for (int j = 0; j < n_hot; ++j) {
        int* it = sp.items + 3 * (hot0 + j);
        it[0] = e;
        it[1] = at + sp.Tb * j;
        it[2] = min(sp.Tb, c - sp.Tb * j);
      }
    }
    carry_a += sum_a;
    carry_b += sum_b;
  }
  if (tid == 0) {
    counts[0] = (int)(carry_a >> 32);
    counts[1] = (int)(carry_b & 0xFFFFu);
    if (sp.counts != nullptr) {
      sp.counts[0] = (int)((carry_b >> 16) & 0xFFFFFFFFu);
      sp.counts[1] = (int)(carry_b >> 48);
    }
  }
  __syncthreads();
  for (int base0 = p0; base0 < p1; base0 += 32 * PLAN_BATCH) {
    int ev[PLAN_BATCH];
#pragma unroll
    for (int i = 0; i < PLAN_BATCH; ++i) {
      const int p = base0 + 32 * i + lane;
      ev[i] = p < p1 ? load_pick<CG>(picks + p) - lo : -1;
    }
#pragma unroll
    for (int i = 0; i < PLAN_BATCH; ++i) {
      if (base0 + 32 * i >= p1) break;
      const int p = base0 + 32 * i + lane, e = ev[i];
      const bool ok = e >= 0 && e < E;
      const unsigned peers = same_key_lanes(e, ok, nbits);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int b = ok ? mine[e] : 0;
      if (ok) members[first[e] + b + rank] = p;
      __syncwarp();
      if (ok && rank == 0) mine[e] = b + __popc(peers);
      __syncwarp();
    }
  }
}

__global__ void __launch_bounds__(PLAN_THREADS)
plan_kernel(const int* __restrict__ picks, int P, int E, int T, int* __restrict__ members, int* __restrict__ items,
            int* __restrict__ counts, int lo, PlanSplit sp) {
  extern __shared__ int whist[];                 // [32][E]: pairs of expert e in warp w's run, then their first slot
  __shared__ int first[PLAN_EMAX];
  __shared__ uint64_t tot2[2][PLAN_THREADS / 32];
  pdl_wait();
  after_wait(picks);
  plan_block<PLAN_THREADS>(picks, P, E, T, members, items, counts, whist, first, tot2, lo, sp);
  pdl_launch_dependents();
}

// The plan on a cluster of PLAN_CLUSTER blocks (many pairs: a prompt, or all ranks' tokens of an expert-parallel step).
constexpr int PLAN_CLUSTER = 8;

__global__ void __launch_bounds__(PLAN_THREADS)
plan_cluster_kernel(const int* __restrict__ picks, int P, int E, int T, int* __restrict__ members,
                    int* __restrict__ items, int* __restrict__ counts, int lo, PlanSplit sp) {
  extern __shared__ int whist[];
  __shared__ int first[PLAN_EMAX];
  __shared__ int tot[PLAN_EMAX];
  __shared__ uint64_t tot2[2][PLAN_THREADS / 32];
  pdl_wait();
  after_wait(picks);
  plan_block<PLAN_THREADS>(picks, P, E, T, members, items, counts, whist, first, tot2, lo, sp, tot, (int)blockIdx.x,
                           PLAN_CLUSTER);
  cooperative_groups::this_cluster().sync();          // no block leaves while another may still read its totals
  pdl_launch_dependents();
}

// Selection and plan of a small call in one block of NT threads: the warps take rows in turn, the picks stay in shared
// memory for the plan.  NP = E + (shared != 0) plan experts.  Results equal select_kernel's followed by plan_kernel's
// at any NT; a few rows take a block of four warps (its barriers and its histogram are a fraction of the full
// block's: 6.4 -> about 3 us at one row).
template <int VPL, int NT>
__global__ void __launch_bounds__(NT)
select_plan_kernel(const float* __restrict__ L, int NL, int* __restrict__ pick, float* __restrict__ wts, int T, int E,
                   int top_k, int shared, int tile, int* __restrict__ members, int* __restrict__ items,
                   int* __restrict__ counts, int plan_lo, int plan_n) {
  extern __shared__ int dyn[];                   // whist [NT / 32][NP], then the picks [T * slots]
  __shared__ int first[PLAN_EMAX];
  __shared__ uint64_t tot2[2][NT / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = top_k + (shared ? 1 : 0);
  int* picks_sh = dyn + (NT / 32) * plan_n;
  pdl_wait();
  after_wait(L);
  for (int r = warp; r < T; r += NT / 32) {
    const int mine = select_row<VPL>(L + (size_t)r * NL, E, top_k, shared, lane, pick + (size_t)r * slots,
                                     wts + (size_t)r * slots);
    if (lane < slots) picks_sh[r * slots + lane] = mine;
  }
  __syncthreads();
  plan_block<NT>(picks_sh, T * slots, plan_n, tile, members, items, counts, dyn, first, tot2, plan_lo);
  pdl_launch_dependents();
}

// ================================================================================================================
// A few rows: router, selection and plan in ONE launch.  CTA (expert, eight rows) computes its logits exactly as
// router_rows_kernel does; the CTA that completes a group of eight rows (counted with an atomic) selects those rows,
// a warp a row; the CTA that completes the last group makes the plan.  Results equal the three kernels' bit for bit.
// arrive: [1 + row groups] ints, zero between launches (the kernel leaves them zero).
// ================================================================================================================
constexpr int ROUTE_THREADS = RR_WARPS * 32;

template <int VPL>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_stride, const __nv_bfloat16* __restrict__ W,
             float* __restrict__ logits, int T, int D, int NE, int E, int top_k, int shared, int* __restrict__ pick,
             float* __restrict__ wts, int tile, int* __restrict__ members, int* __restrict__ items,
             int* __restrict__ counts, int plan_lo, int plan_n, int* __restrict__ arrive) {
  static_assert(RR_ROWS == RR_WARPS, "a warp a row, in the router and in the selection");
  extern __shared__ int dyn[];                       // the plan's: whist [RR_WARPS][plan_n], first [plan_n]
  __shared__ uint64_t tot2[2][ROUTE_THREADS / 32];
  __shared__ int last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int e = blockIdx.x, group = blockIdx.y, r = group * RR_ROWS + warp;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  pdl_wait();
  after_wait(X);
  float acc = 0.f;
  for (int kb = 0; kb < D; kb += 256 * RR_CH) {
    float wv[RR_CH][8];
    uint4 xv[RR_CH];
#pragma unroll
    for (int c = 0; c < RR_CH; ++c) {
      const int k = kb + 256 * c + 8 * lane;
      unpack8(k < D ? ldg_nc(W + (size_t)e * D + k) : zero, wv[c]);
      xv[c] = (k < D && r < T) ? ldg_nc(X + (size_t)r * x_stride + k) : zero;
    }
#pragma unroll
    for (int c = 0; c < RR_CH; ++c) {
      if (kb + 256 * c + 8 * lane < D) {
        float xf[8];
        unpack8(xv[c], xf);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(xf[j], wv[c][j], acc);
      }
    }
  }
  pdl_launch_dependents();
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) acc = acc + __shfl_xor_sync(0xffffffffu, acc, m);
  if (lane == 0 && r < T) logits[(size_t)r * NE + e] = acc;
  // ---- the CTA that finishes a row group selects its rows ----
  __syncthreads();
  if (tid == 0) {
    const int seen = arrive_count(arrive + 1 + group);
    last = seen == NE - 1;
    if (seen == NE - 1) arrive[1 + group] = 0;
  }
  __syncthreads();
  if (!last) return;
  const int slots = top_k + (shared ? 1 : 0);
  if (r < T) select_row<VPL>(logits + (size_t)r * NE, E, top_k, shared, lane, pick + (size_t)r * slots, wts + (size_t)r * slots);
  // ---- the CTA that finishes the last row group plans ----
  __syncthreads();
  if (tid == 0) {
    const int seen = arrive_count(arrive);
    last = seen == (int)gridDim.y - 1;
    if (seen == (int)gridDim.y - 1) arrive[0] = 0;
  }
  __syncthreads();
  if (!last) return;
  plan_block<ROUTE_THREADS, true>(pick, T * slots, plan_n, tile, members, items, counts, dyn, dyn + RR_WARPS * plan_n,
                                  tot2, plan_lo);
}

// ================================================================================================================
// Combine: out[r, d] = sum over slots in slot order of wts[r, s] * y[r, s, d] (fp32 fma chain from 0), rounded once.
// (src/tensorfold/cuda/moe.py:131-151; src/tensorfold/cuda/exl3/experts.cu:181-190 for the fp32-out form.)
// ================================================================================================================
// With `pick`: only slots whose expert id lies in [lo, lo + n) take part (the others' rows are not read).
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
combine_kernel(const TY* __restrict__ y, const float* __restrict__ wts, TO* __restrict__ out, int S, int D,
               const int* __restrict__ pick, int lo, int n) {
  const int r = blockIdx.x;
  const int d = (blockIdx.y * 256 + threadIdx.x) * 4;
  if (d >= D) return;
  pdl_wait();
  after_wait(y, wts);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < S; ++s) {
    if (pick != nullptr) {
      const int e = pick[(size_t)r * S + s] - lo;
      if (e < 0 || e >= n) continue;
    }
    const float w = wts[(size_t)r * S + s];
    const TY* src = y + ((size_t)r * S + s) * D + d;
    float v[4];
    if constexpr (sizeof(TY) == 4) {
      const float4 f = *reinterpret_cast<const float4*>(src);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      const uint2 u = *reinterpret_cast<const uint2*>(src);
      v[0] = bf16_lo(u.x); v[1] = bf16_hi(u.x); v[2] = bf16_lo(u.y); v[3] = bf16_hi(u.y);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = fmaf(w, v[j], acc[j]);
  }
  pdl_launch_dependents();
  TO* dst = out + (size_t)r * D + d;
  if constexpr (sizeof(TO) == 4) {
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(acc[0], acc[1]), b = __floats2bfloat162_rn(acc[2], acc[3]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst) = u;
  }
}

// ================================================================================================================
// Combine, residual add and RMSNorm in one pass over a row (the Nemotron family's step behind its MoE block):
// delta = bf16(sum over the routed slots of wt * y, an fp32 fma chain in slot order, + the shared slots' y in slot
// order); hn = bf16(h + delta); out = bf16(hn * rsqrt(mean(hn^2) + eps) * w); xs = the sums of out over groups of 64.
// (src/tensorfold/families/nemotron_h/cuda/glue.py:104-141: _add_moe_norm, add_moe_norm)
// ================================================================================================================
constexpr int AMN_THREADS = 256, AMN_MAX_PER_THREAD = 8;   // rows of up to 256 * 4 * 8 = 8192 columns

template <typename TY>
__global__ void __launch_bounds__(AMN_THREADS)
add_moe_norm_kernel(const __nv_bfloat16* __restrict__ h, const TY* __restrict__ y, const float* __restrict__ wt,
                    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ hn, __nv_bfloat16* __restrict__ out,
                    float* __restrict__ xs, int D, int slots, int routed, float eps) {
  __shared__ float warp_sq[AMN_THREADS / 32];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  pdl_wait();
  after_wait(h, y, wt);
  float hv[AMN_MAX_PER_THREAD][4];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < AMN_MAX_PER_THREAD; ++i) {
    const int d = (i * AMN_THREADS + tid) * 4;
    if (d >= D) break;
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, sh[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < slots; ++s) {
      const TY* src = y + ((size_t)r * slots + s) * D + d;
      float v[4];
      if constexpr (sizeof(TY) == 4) {
        const float4 f = *reinterpret_cast<const float4*>(src);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      } else {
        const uint2 u = *reinterpret_cast<const uint2*>(src);
        v[0] = bf16_lo(u.x); v[1] = bf16_hi(u.x); v[2] = bf16_lo(u.y); v[3] = bf16_hi(u.y);
      }
      if (s < routed) {
        const float ws = wt[(size_t)r * slots + s];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = fmaf(ws, v[j], acc[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) sh[j] += v[j];
      }
    }
    const uint2 hx = *reinterpret_cast<const uint2*>(h + (size_t)r * D + d);
    const float x4[4] = {bf16_lo(hx.x), bf16_hi(hx.x), bf16_lo(hx.y), bf16_hi(hx.y)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      hv[i][j] = round_bf16(x4[j] + round_bf16(acc[j] + sh[j]));
      sq = fmaf(hv[i][j], hv[i][j], sq);
    }
    __nv_bfloat162 a = __floats2bfloat162_rn(hv[i][0], hv[i][1]), b = __floats2bfloat162_rn(hv[i][2], hv[i][3]);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(hn + (size_t)r * D + d) = o;
  }
  pdl_launch_dependents();
  // the row's sum of squares: lanes (butterfly), then the warps in warp order
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, m);
  if (lane == 0) warp_sq[tid >> 5] = sq;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < AMN_THREADS / 32; ++i) total += warp_sq[i];
  const float inv = 1.f / sqrtf(total / (float)D + eps);
#pragma unroll
  for (int i = 0; i < AMN_MAX_PER_THREAD; ++i) {
    const int d = (i * AMN_THREADS + tid) * 4;
    if (d >= D) break;                                 // D is a multiple of 64: a warp's lanes leave in groups of 16
    const uint2 wx = *reinterpret_cast<const uint2*>(w + d);
    const float w4[4] = {bf16_lo(wx.x), bf16_hi(wx.x), bf16_lo(wx.y), bf16_hi(wx.y)};
    float o4[4], gs = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o4[j] = round_bf16(hv[i][j] * inv * w4[j]);
      gs += o4[j];
    }
    __nv_bfloat162 a = __floats2bfloat162_rn(o4[0], o4[1]), b = __floats2bfloat162_rn(o4[2], o4[3]);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(out + (size_t)r * D + d) = o;
    // 16 lanes hold a group of 64 columns
    const unsigned half_mask = 0xFFFFu << (lane & 16);
#pragma unroll
    for (int m = 8; m >= 1; m >>= 1) gs += __shfl_xor_sync(half_mask, gs, m);
    if ((lane & 15) == 0) xs[(size_t)r * (D / 64) + d / 64] = gs;
  }
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_router(const void* x, int64_t x_stride, const void* rows, float* logits, int T, int D, int NE,
                          void* stream) {
  TFB_REQUIRE(x && rows && logits, "router: null pointer");
  TFB_REQUIRE(T >= 0 && D > 0 && NE > 0, "router: bad sizes T=%d D=%d NE=%d", T, D, NE);
  TFB_REQUIRE(D % 8 == 0 && x_stride % 8 == 0 && x_stride >= D, "router: D and the row stride must be multiples of 8");
  TFB_REQUIRE(aligned16(x) && aligned16(rows), "router: x and rows must be 16-byte aligned");
  if (T == 0) return TFB_OK;
  // few rows: the row-form kernel (latency of two round trips); measured faster up to 64 rows x 128 experts and
  // 32 rows x 257 experts, slower from twice that on (it re-reads the rows once an expert); the bits are the same
  if ((int64_t)T * NE <= 8704) {
    const dim3 rgrid(NE, (T + RR_ROWS - 1) / RR_ROWS);
    return check_cuda(launch(router_rows_kernel, rgrid, dim3(RR_WARPS * 32), 0, static_cast<cudaStream_t>(stream),
                             static_cast<const __nv_bfloat16*>(x), x_stride,
                             static_cast<const __nv_bfloat16*>(rows), logits, T, D, NE),
                      "router");
  }
  const dim3 grid((T + R_RT - 1) / R_RT, (NE + R_WARPS * R_ET - 1) / (R_WARPS * R_ET));
  return check_cuda(launch(router_kernel, grid, dim3(R_WARPS * 32), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(x), x_stride, static_cast<const __nv_bfloat16*>(rows),
                           logits, T, D, NE),
                    "router");
}

// tfb_router for prompts: the same logits up to the last bits, on the tensor cores (a fixed summation order of its
// own; a row's bits do not depend on the call's other rows).  D a multiple of 32.
extern "C" int tfb_router_prompt(const void* x, int64_t x_stride, const void* rows, float* logits, int T, int D, int NE,
                                 void* stream) {
  TFB_REQUIRE(x && rows && logits, "router_prompt: null pointer");
  TFB_REQUIRE(T >= 0 && D > 0 && NE > 0, "router_prompt: bad sizes T=%d D=%d NE=%d", T, D, NE);
  TFB_REQUIRE(D % 32 == 0 && x_stride % 8 == 0 && x_stride >= D,
              "router_prompt: D must be a multiple of 32 and the row stride of 8");
  TFB_REQUIRE(aligned16(x) && aligned16(rows), "router_prompt: x and rows must be 16-byte aligned");
  if (T == 0) return TFB_OK;
  const dim3 grid((T + 16 * RT_ROWT - 1) / (16 * RT_ROWT), (NE + 8 * RT_NT - 1) / (8 * RT_NT));
  return check_cuda(launch(router_mma_kernel, grid, dim3(RT_ROWT * RT_KH * 32), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(x), x_stride, static_cast<const __nv_bfloat16*>(rows),
                           logits, T, D, NE),
                    "router_prompt");
}

extern "C" int tfb_select_rows(const float* logits, int NL, int32_t* pick, float* wts, int T, int E, int top_k,
                               int shared, void* stream) {
  TFB_REQUIRE(logits && pick && wts, "select_rows: null pointer");
  TFB_REQUIRE(E >= 1 && E <= 1024, "select_rows: 1..1024 experts, not %d", E);
  TFB_REQUIRE(top_k >= 1 && top_k <= E && top_k <= 31, "select_rows: top_k=%d must be 1..min(E, 31)", top_k);
  TFB_REQUIRE(NL >= E + (shared ? 1 : 0), "select_rows: %d logits a row cannot hold %d experts%s", NL, E,
              shared ? " and the shared gate" : "");
  if (T <= 0) return TFB_OK;
  const int grid = (T + S_WARPS - 1) / S_WARPS;
  auto st = static_cast<cudaStream_t>(stream);
  const int vpl = (E + 31) / 32;
#define TFB_SEL(V)                                                                                            \
  return check_cuda(launch(select_kernel<V>, dim3(grid), dim3(S_WARPS * 32), 0, st, logits, NL, pick, wts, T, E, \
                           top_k, shared ? 1 : 0),                                                              \
                    "select_rows")
  if (vpl <= 4) TFB_SEL(4);
  if (vpl <= 8) TFB_SEL(8);
  if (vpl <= 16) TFB_SEL(16);
  TFB_SEL(32);
#undef TFB_SEL
}

// from here on the plan runs on a cluster of blocks (measured: 8.7 -> 6.7 us at 4096 pairs, 24.6 -> 10.4 us at 16384;
// break-even near 2048)
constexpr int64_t PLAN_CLUSTER_PAIRS = 4096;

static int plan_launch(const int32_t* picks, int64_t pairs, int lo, int experts, int tile, int32_t* members,
                       int32_t* items, int32_t* counts, void* stream,
                       PlanSplit sp = PlanSplit{0x7FFFFFFF, 1, nullptr, nullptr}) {
  TFB_REQUIRE(picks && members && items && counts, "plan: null pointer");
  TFB_REQUIRE(experts >= 1 && experts <= PLAN_EMAX, "plan: at most %d experts, not %d", PLAN_EMAX, experts);
  TFB_REQUIRE(tile >= 1, "plan: items hold at least one pair");
  TFB_REQUIRE(pairs >= 0 && pairs < (int64_t(1) << 30), "plan: bad pair count");
  const size_t smem = sizeof(int) * 32 * (size_t)experts;
  static int configured[64] = {0};
  int dev = 0;
  TFB_CUDA(cudaGetDevice(&dev), "plan: cudaGetDevice");
  if (dev < 64 && !configured[dev]) {
    TFB_CUDA(cudaFuncSetAttribute(plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)(sizeof(int) * 32 * PLAN_EMAX)),
             "plan: shared memory opt-in");
    configured[dev] = 1;
  }
  if (pairs >= PLAN_CLUSTER_PAIRS) {
    static int cluster_ok[64] = {0};
    if (dev < 64 && !cluster_ok[dev]) {
      TFB_CUDA(cudaFuncSetAttribute(plan_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)(sizeof(int) * 32 * PLAN_EMAX)),
               "plan: shared memory opt-in");
      cluster_ok[dev] = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(PLAN_CLUSTER);
    cfg.blockDim = dim3(PLAN_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PLAN_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 2 : 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, plan_cluster_kernel, picks, (int)pairs, experts, tile, members, items,
                                         counts, lo, sp),
                      "plan");
  }
  return check_cuda(launch(plan_kernel, dim3(1), dim3(PLAN_THREADS), smem, static_cast<cudaStream_t>(stream), picks,
                           (int)pairs, experts, tile, members, items, counts, lo, sp),
                    "plan");
}

extern "C" int tfb_select_sigmoid(const float* logits, int NL, const float* bias, int32_t* pick, float* wts, int T,
                                  int E, int top_k, int shared_slots, float scale, int norm, void* stream) {
  TFB_REQUIRE(logits && bias && pick && wts, "select_sigmoid: null pointer");
  TFB_REQUIRE(E >= 1 && E <= 1024, "select_sigmoid: 1..1024 experts, not %d", E);
  TFB_REQUIRE(top_k >= 1 && top_k <= E && shared_slots >= 0 && top_k + shared_slots <= 32,
              "select_sigmoid: top_k=%d and %d shared slots must fit 32 slots", top_k, shared_slots);
  TFB_REQUIRE(NL >= E, "select_sigmoid: %d logits a row cannot hold %d experts", NL, E);
  if (T <= 0) return TFB_OK;
  const int grid = (T + S_WARPS - 1) / S_WARPS;
  auto st = static_cast<cudaStream_t>(stream);
  const int vpl = (E + 31) / 32;
#define TFB_SEL(V)                                                                                             \
  return check_cuda(launch(select_sigmoid_kernel<V>, dim3(grid), dim3(S_WARPS * 32), 0, st, logits, NL, bias,  \
                           pick, wts, T, E, top_k, shared_slots, scale, norm ? 1 : 0),                          \
                    "select_sigmoid")
  if (vpl <= 4) TFB_SEL(4);
  if (vpl <= 8) TFB_SEL(8);
  if (vpl <= 16) TFB_SEL(16);
  TFB_SEL(32);
#undef TFB_SEL
}

extern "C" int tfb_plan(const int32_t* picks, int64_t pairs, int experts, int tile, int32_t* members, int32_t* items,
                        int32_t* counts, void* stream) {
  return plan_launch(picks, pairs, 0, experts, tile, members, items, counts, stream);
}

// The plan of the ids in [lo, lo + experts) only, renumbered from 0: an expert-parallel rank's share of the pairs.
extern "C" int tfb_plan_window(const int32_t* picks, int64_t pairs, int lo, int experts, int tile, int32_t* members,
                               int32_t* items, int32_t* counts, void* stream) {
  TFB_REQUIRE(lo >= 0, "plan_window: the window starts at a non-negative id");
  return plan_launch(picks, pairs, lo, experts, tile, members, items, counts, stream);
}

extern "C" int tfb_plan_split(const int32_t* picks, int64_t pairs, int lo, int experts, int tile, int big_tile, int hot,
                              int32_t* members, int32_t* items, int32_t* counts, int32_t* big_items,
                              int32_t* big_counts, void* stream) {
  TFB_REQUIRE(lo >= 0, "plan_split: the window starts at a non-negative id");
  TFB_REQUIRE(big_items && big_counts, "plan_split: null pointer");
  TFB_REQUIRE(big_tile >= 1 && hot >= 1 && pairs < (1 << 20), "plan_split: bad tile, threshold or pair count");
  return plan_launch(picks, pairs, lo, experts, tile, members, items, counts, stream,
                     PlanSplit{hot, big_tile, big_items, big_counts});
}

// Rows the fused selection + plan kernel takes (one block); larger calls use tfb_select_rows then tfb_plan.
extern "C" int tfb_select_plan_max_rows(void) { return 128; }

static int select_plan_launch(const float* logits, int NL, int32_t* pick, float* wts, int T, int E, int top_k,
                              int shared, int tile, int plan_lo, int plan_n, int32_t* members, int32_t* items,
                              int32_t* counts, void* stream) {
  TFB_REQUIRE(logits && pick && wts && members && items && counts, "select_plan: null pointer");
  const int NP = E + (shared ? 1 : 0);
  TFB_REQUIRE(plan_lo >= 0 && plan_n >= 1 && plan_lo + plan_n <= NP, "select_plan: the plan window [%d, %d) leaves "
              "the %d experts", plan_lo, plan_lo + plan_n, NP);
  TFB_REQUIRE(E >= 1 && NP <= PLAN_EMAX, "select_plan: at most %d experts, not %d", PLAN_EMAX, NP);
  TFB_REQUIRE(top_k >= 1 && top_k <= E && top_k <= 31, "select_plan: top_k=%d must be 1..min(E, 31)", top_k);
  TFB_REQUIRE(NL >= NP, "select_plan: %d logits a row cannot hold %d experts%s", NL, E,
              shared ? " and the shared gate" : "");
  TFB_REQUIRE(T >= 0 && T <= tfb_select_plan_max_rows(), "select_plan: at most %d rows, not %d",
              tfb_select_plan_max_rows(), T);
  TFB_REQUIRE(tile >= 1, "select_plan: items hold at least one pair");
  const int slots = top_k + (shared ? 1 : 0);
  auto st = static_cast<cudaStream_t>(stream);
  const int vpl = (E + 31) / 32;
  int dev = 0;
  TFB_CUDA(cudaGetDevice(&dev), "select_plan: cudaGetDevice");
  constexpr int SMALL_THREADS = 128, SMALL_ROWS = 4;      // a row a warp
#define TFB_SP(V)                                                                                                  \
  do {                                                                                                             \
    if (T <= SMALL_ROWS) {                                                                                         \
      const size_t smem = sizeof(int) * ((SMALL_THREADS / 32) * (size_t)plan_n + (size_t)T * slots);              \
      return check_cuda(launch(select_plan_kernel<V, SMALL_THREADS>, dim3(1), dim3(SMALL_THREADS), smem, st, logits, \
                               NL, pick, wts, T, E, top_k, shared ? 1 : 0, tile, members, items, counts, plan_lo,  \
                               plan_n),                                                                            \
                        "select_plan");                                                                            \
    }                                                                                                              \
    const size_t smem = sizeof(int) * (32 * (size_t)plan_n + (size_t)T * slots);                                   \
    static int configured[64] = {0};                                                                               \
    if (dev < 64 && !configured[dev]) {                                                                            \
      TFB_CUDA(cudaFuncSetAttribute(select_plan_kernel<V, PLAN_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                    (int)(sizeof(int) * (32 * PLAN_EMAX + 128 * 32))),                             \
               "select_plan: shared memory opt-in");                                                               \
      configured[dev] = 1;                                                                                         \
    }                                                                                                              \
    return check_cuda(launch(select_plan_kernel<V, PLAN_THREADS>, dim3(1), dim3(PLAN_THREADS), smem, st, logits, NL, \
                             pick, wts, T, E, top_k, shared ? 1 : 0, tile, members, items, counts, plan_lo, plan_n), \
                      "select_plan");                                                                              \
  } while (0)
  if (vpl <= 4) TFB_SP(4);
  if (vpl <= 8) TFB_SP(8);
  if (vpl <= 16) TFB_SP(16);
  TFB_SP(32);
#undef TFB_SP
}

extern "C" int tfb_select_plan(const float* logits, int NL, int32_t* pick, float* wts, int T, int E, int top_k,
                               int shared, int tile, int32_t* members, int32_t* items, int32_t* counts, void* stream) {
  return select_plan_launch(logits, NL, pick, wts, T, E, top_k, shared, tile, 0, E + (shared ? 1 : 0), members, items,
                            counts, stream);
}

// tfb_select_plan whose plan covers only the ids in [plan_lo, plan_lo + plan_n), renumbered from 0 (pick and wts still
// hold every slot): what an expert-parallel rank needs for the tokens of all ranks.
extern "C" int tfb_select_plan_window(const float* logits, int NL, int32_t* pick, float* wts, int T, int E, int top_k,
                                      int shared, int tile, int plan_lo, int plan_n, int32_t* members, int32_t* items,
                                      int32_t* counts, void* stream) {
  return select_plan_launch(logits, NL, pick, wts, T, E, top_k, shared, tile, plan_lo, plan_n, members, items, counts,
                            stream);
}

// Rows the one-launch router + selection + plan takes: the row-form router's range (rows x router rows <= 8704).
extern "C" int tfb_route_max_rows(int NE) { return NE >= 1 ? (8704 / NE < 256 ? 8704 / NE : 256) : 0; }

// tfb_router, tfb_select_rows and tfb_plan_window of a few rows in one launch (the same bits): logits [T, NE] fp32 from
// x [T, D] and rows [NE, D] (NE = E + 1 with the shared expert's gate row), pick / wts [T, slots], and the plan of the
// ids in [plan_lo, plan_lo + plan_n).  arrive: int scratch [1 + (T + 7) / 8], zero before the first call (a call leaves
// it zero).  T <= tfb_route_max_rows(NE).
extern "C" int tfb_route(const void* x, int64_t x_stride, const void* rows, float* logits, int T, int D, int NE, int E,
                         int top_k, int shared, int32_t* pick, float* wts, int tile, int plan_lo, int plan_n,
                         int32_t* members, int32_t* items, int32_t* counts, int32_t* arrive, void* stream) {
  TFB_REQUIRE(x && rows && logits && pick && wts && members && items && counts && arrive, "route: null pointer");
  TFB_REQUIRE(D > 0 && D % 8 == 0 && x_stride % 8 == 0 && x_stride >= D, "route: D and the row stride must be multiples of 8");
  TFB_REQUIRE(aligned16(x) && aligned16(rows), "route: x and rows must be 16-byte aligned");
  const int NP = E + (shared ? 1 : 0);
  TFB_REQUIRE(E >= 1 && NP <= PLAN_EMAX && NE >= NP, "route: %d router rows cannot hold %d experts%s", NE, E,
              shared ? " and the shared gate" : "");
  TFB_REQUIRE(top_k >= 1 && top_k <= E && top_k <= 31, "route: top_k=%d must be 1..min(E, 31)", top_k);
  TFB_REQUIRE(plan_lo >= 0 && plan_n >= 1 && plan_lo + plan_n <= NP, "route: the plan window [%d, %d) leaves the %d experts",
              plan_lo, plan_lo + plan_n, NP);
  TFB_REQUIRE(tile >= 1, "route: items hold at least one pair");
  TFB_REQUIRE(T >= 0 && T <= tfb_route_max_rows(NE), "route: at most %d rows of %d router rows, not %d",
              tfb_route_max_rows(NE), NE, T);
  if (T == 0) return TFB_OK;
  const dim3 grid(NE, (T + RR_ROWS - 1) / RR_ROWS);
  const size_t smem = sizeof(int) * (size_t)(RR_WARPS + 1) * plan_n;
  auto st = static_cast<cudaStream_t>(stream);
  const int vpl = (E + 31) / 32;
#define TFB_ROUTE(V)                                                                                              \
  return check_cuda(launch(route_kernel<V>, grid, dim3(ROUTE_THREADS), smem, st, static_cast<const __nv_bfloat16*>(x), \
                           x_stride, static_cast<const __nv_bfloat16*>(rows), logits, T, D, NE, E, top_k,           \
                           shared ? 1 : 0, pick, wts, tile, members, items, counts, plan_lo, plan_n, arrive),     \
                    "route")
  if (vpl <= 4) TFB_ROUTE(4);
  if (vpl <= 8) TFB_ROUTE(8);
  if (vpl <= 16) TFB_ROUTE(16);
  TFB_ROUTE(32);
#undef TFB_ROUTE
}

static int combine_launch(const void* y, int y_bf16, const float* wts, void* out, int out_f32, int T, int slots, int D,
                          const int32_t* pick, int lo, int n, void* stream) {
  TFB_REQUIRE(y && wts && out, "combine: null pointer");
  TFB_REQUIRE(D > 0 && D % 4 == 0 && slots >= 1, "combine: D must be a multiple of 4 and slots >= 1");
  TFB_REQUIRE(aligned16(y) && aligned16(out), "combine: y and out must be 16-byte aligned");
  if (T <= 0) return TFB_OK;
  const dim3 grid(T, (D + 1023) / 1024);
  auto st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (y_bf16 && out_f32)
    e = launch(combine_kernel<__nv_bfloat16, float>, grid, dim3(256), 0, st, static_cast<const __nv_bfloat16*>(y), wts,
               static_cast<float*>(out), slots, D, pick, lo, n);
  else if (y_bf16)
    e = launch(combine_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, st,
               static_cast<const __nv_bfloat16*>(y), wts, static_cast<__nv_bfloat16*>(out), slots, D, pick, lo, n);
  else if (out_f32)
    e = launch(combine_kernel<float, float>, grid, dim3(256), 0, st, static_cast<const float*>(y), wts,
               static_cast<float*>(out), slots, D, pick, lo, n);
  else
    e = launch(combine_kernel<float, __nv_bfloat16>, grid, dim3(256), 0, st, static_cast<const float*>(y), wts,
               static_cast<__nv_bfloat16*>(out), slots, D, pick, lo, n);
  return check_cuda(e, "combine");
}

extern "C" int tfb_combine(const void* y, int y_bf16, const float* wts, void* out, int out_f32, int T, int slots,
                           int D, void* stream) {
  return combine_launch(y, y_bf16, wts, out, out_f32, T, slots, D, nullptr, 0, 0, stream);
}

// tfb_combine over the slots whose expert id pick[T, slots] lies in [lo, lo + n): an expert-parallel rank's partial
// sum of each token (rows of other ranks' pairs are never read, so y needs no clearing).
extern "C" int tfb_combine_window(const void* y, int y_bf16, const float* wts, const int32_t* pick, int lo, int n,
                                  void* out, int out_f32, int T, int slots, int D, void* stream) {
  TFB_REQUIRE(pick, "combine_window: null pointer");
  TFB_REQUIRE(lo >= 0 && n >= 1, "combine_window: bad window");
  return combine_launch(y, y_bf16, wts, out, out_f32, T, slots, D, pick, lo, n, stream);
}

// hn [R, D] bf16 = h + the layer's combined output, out [R, D] bf16 = its RMSNorm times w, xs [R, D / 64] fp32 = the
// sums of out over groups of 64: the combine (routed slots weighted, shared slots added), the residual add and the norm
// in one pass.  y [R, slots, D] fp32 (or bf16: the prompt form), wt [R, slots] fp32; the first `routed` slots are the
// routed ones.  D a multiple of 64, at most 8192.
// (src/tensorfold/families/nemotron_h/cuda/glue.py:128-141 `add_moe_norm`)
extern "C" int tfb_add_moe_norm(const void* h, const void* y, int y_bf16, const float* wt, const void* w, void* hn,
                                void* out, float* xs, int R, int D, int slots, int routed, float eps, void* stream) {
  TFB_REQUIRE(h && y && wt && w && hn && out && xs, "add_moe_norm: null pointer");
  TFB_REQUIRE(D > 0 && D % 64 == 0 && D <= AMN_THREADS * 4 * AMN_MAX_PER_THREAD,
              "add_moe_norm: D must be a multiple of 64, at most %d", AMN_THREADS * 4 * AMN_MAX_PER_THREAD);
  TFB_REQUIRE(slots >= 1 && routed >= 0 && routed <= slots, "add_moe_norm: %d routed of %d slots", routed, slots);
  TFB_REQUIRE(aligned16(h) && aligned16(y) && aligned16(w) && aligned16(hn) && aligned16(out),
              "add_moe_norm: rows must be 16-byte aligned");
  if (R <= 0) return TFB_OK;
  auto st = static_cast<cudaStream_t>(stream);
  auto* hb = static_cast<const __nv_bfloat16*>(h);
  auto* wb = static_cast<const __nv_bfloat16*>(w);
  cudaError_t e;
  if (y_bf16)
    e = launch(add_moe_norm_kernel<__nv_bfloat16>, dim3(R), dim3(AMN_THREADS), 0, st, hb,
               static_cast<const __nv_bfloat16*>(y), wt, wb, static_cast<__nv_bfloat16*>(hn),
               static_cast<__nv_bfloat16*>(out), xs, D, slots, routed, eps);
  else
    e = launch(add_moe_norm_kernel<float>, dim3(R), dim3(AMN_THREADS), 0, st, hb, static_cast<const float*>(y), wt, wb,
               static_cast<__nv_bfloat16*>(hn), static_cast<__nv_bfloat16*>(out), xs, D, slots, routed, eps);
  return check_cuda(e, "add_moe_norm");
}
