// Routed experts on EXL3 trellis-coded weights (ExLlamaV3's format), any codebook, a width per expert matrix.
//
// A 16 x 16 tile is a circular MSB-first bitstream of 256 values; value p's 16-bit state is the window ending at
// E(p) = (p >> 1) K2 + (p odd ? K2 : K2 >> 1) (K2 = half-bits a value); a codebook turns a state into an fp16 value;
// value p sits at row 2 (l % 4) + (j & 1) + 8 ((j >> 1) & 1), column l / 4 + 8 (j >> 2) of its tile (l = p / 8,
// j = p % 8) - so lane l's eight values are exactly its mma.m16n8k16 fragment of the tile.  Here the tile
// (transposed) is the A operand (16 output columns x 16 inputs) and eight pairs' rotated inputs the B operand.
// The layer is y = (((x * suh) H) W_q) H * svh per 128-block, H = 128-point Hadamard / sqrt(128).
// Fixed-order reductions everywhere: a pair's bits never depend on the other rows of the call.
// (Replaces src/tensorfold/cuda/exl3/experts.cu and experts_grouped.cuh; the trellises are read in place.)

#include "api.h"
#include "common.cuh"

namespace tfb {
namespace exl3 {

constexpr float HAD_SCALE = 0.08838834764831845f;   // 1 / sqrt(128)
constexpr int GR_WARPS = 4;                         // K slices a CTA of the grouped kernel (part of the arithmetic)
constexpr int GR_NTB_MAX = 4;                       // 16-column tiles a CTA at most (no effect on the arithmetic)
constexpr int GR_PAIRS = 8;                         // pairs a CTA (one mma B tile)

// ---- codebooks: two states -> two fp16 values (src/tensorfold/cuda/exl3/format.py:31-48) ------------------------
template <int CB>
__device__ __forceinline__ uint32_t cb_pair(uint32_t s0, uint32_t s1) {
  if constexpr (CB == 2) {                            // mul1: fma(1024 + sum of the bytes of s * M, scale, bias) in fp16
    const uint32_t h0 = __dp4a(s0 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t h1 = __dp4a(s1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t hv = __byte_perm(h0, h1, 0x5410);
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&hv), __half2half2(__ushort_as_half(0x1EEE)),
                              __half2half2(__ushort_as_half(0xC931)));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {                                            // 3inst / mcg: the two fp16 halves of the masked product, added
    uint32_t x0 = CB == 1 ? s0 * 0xCBAC1FEDu : s0 * 89226354u + 64248484u;
    uint32_t x1 = CB == 1 ? s1 * 0xCBAC1FEDu : s1 * 89226354u + 64248484u;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;\n" : "=r"(x0) : "r"(x0), "r"(0x8FFF8FFFu), "r"(0x3B603B60u));   // (x & M) ^ F
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;\n" : "=r"(x1) : "r"(x1), "r"(0x8FFF8FFFu), "r"(0x3B603B60u));
    const __half2 h0 = *reinterpret_cast<const __half2*>(&x0), h1 = *reinterpret_cast<const __half2*>(&x1);
    const __half2 r = __halves2half2(__hadd(__low2half(h0), __high2half(h0)), __hadd(__low2half(h1), __high2half(h1)));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

// ---- a lane's eight states of a tile ----------------------------------------------------------------------------
// delta(j): first bit of value 8 l + j's window relative to value 8 l's (the same for every lane)
template <int K2>
__host__ __device__ constexpr int delta(int j) {
  return ((j + 1) * K2 - ((K2 & 1) ? ((j + 1) & 1) : 0)) / 2 - (K2 >> 1);
}
template <int K2>
struct Win {
  static constexpr int TW = 4 * K2;                                 // 32-bit words a tile
  static constexpr int SPAN = delta<K2>(7) + 16;                    // stream bits a lane's windows cover
  static constexpr int NW = K2 == 8 ? 2 : (31 + SPAN + 31) / 32;    // words a lane reads (worst offset; <= 4)
  static constexpr int NV = (SPAN + 31) / 32;                       // 32-bit chunks of the lane's span
};

// The words of a tile a lane needs: NW consecutive words (cyclically) from the one holding the first bit of value
// 8 lane's window.  4 bits a value (K2 = 8): exactly words lane - 1 and lane.
template <int K2>
__device__ __forceinline__ void lane_words(const uint32_t* __restrict__ tile, int lane, uint32_t (&w)[Win<K2>::NW]) {
  constexpr int TW = Win<K2>::TW, NW = Win<K2>::NW;
  const int first = 4 * lane * K2 + (K2 >> 1) - 16 + 32 * TW;       // E(8 lane) - 16, made non-negative
  int wi = (first >> 5) % TW;
#pragma unroll
  for (int i = 0; i < NW; ++i) {
    w[i] = __ldg(tile + wi);
    wi = wi + 1 == TW ? 0 : wi + 1;
  }
}

// st[j] = state of value 8 lane + j from the lane's words.
template <int K2>
__device__ __forceinline__ void lane_states(const uint32_t (&w)[Win<K2>::NW], int lane, uint32_t (&st)[8]) {
  constexpr int NW = Win<K2>::NW, NV = Win<K2>::NV;
  if constexpr (K2 == 8) {
    // windows of 16 bits ending at bit 4 (j + 1) of the lane's own word: three reach back into the word before
    const uint32_t q = __funnelshift_r(w[1], w[0], 20);
    st[0] = (q >> 8) & 0xFFFFu;
    st[1] = (q >> 4) & 0xFFFFu;
    st[2] = q & 0xFFFFu;
    st[3] = w[1] >> 16;
    st[4] = (w[1] >> 12) & 0xFFFFu;
    st[5] = (w[1] >> 8) & 0xFFFFu;
    st[6] = (w[1] >> 4) & 0xFFFFu;
    st[7] = w[1] & 0xFFFFu;
  } else {
    const int off = (4 * lane * K2 + (K2 >> 1) - 16 + 32 * Win<K2>::TW) & 31;
    uint32_t v[NV];                                   // v[i] = stream bits [first + 32 i, first + 32 i + 32)
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = __funnelshift_l(i + 1 < NW ? w[i + 1] : 0u, w[i], off);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = delta<K2>(j), i = d >> 5, o = d & 31;
      if (o <= 16) {
        st[j] = (v[i] >> (16 - o)) & 0xFFFFu;
      } else {                                        // the window runs into the next chunk (d + 16 <= SPAN: it exists)
        st[j] = __funnelshift_l(v[i + 1 < NV ? i + 1 : i], v[i], o) >> 16;
      }
    }
  }
}

// The lane's tile values as the mma A fragment of the transposed tile (rows = output columns, k = inputs):
// a0 = (col g, k 2t, 2t+1) = values 0, 1; a1 = (col g + 8, same k) = values 4, 5; a2 = (col g, k + 8) = values 2, 3;
// a3 = (col g + 8, k + 8) = values 6, 7.
template <int CB, int K2>
__device__ __forceinline__ void decode_words(const uint32_t (&w)[Win<K2>::NW], int lane, uint32_t (&a)[4]) {
  uint32_t st[8];
  lane_states<K2>(w, lane, st);
  a[0] = cb_pair<CB>(st[0], st[1]);
  a[2] = cb_pair<CB>(st[2], st[3]);
  a[1] = cb_pair<CB>(st[4], st[5]);
  a[3] = cb_pair<CB>(st[6], st[7]);
}

template <int CB, int K2>
__device__ __forceinline__ void decode_tile(const uint32_t* __restrict__ tile, int lane, uint32_t (&a)[4]) {
  uint32_t w[Win<K2>::NW];
  lane_words<K2>(tile, lane, w);
  decode_words<CB, K2>(w, lane, a);
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One warp's k tiles [kt0, kt0 + nkt) of GR_NTB column tiles into acc; the next row of tiles' words and inputs are
// loaded before this row is decoded.
template <int CB, int K2, int GR_NTB>
__device__ __forceinline__ void warp_tiles(const uint32_t* __restrict__ T, int ntiles, int kt0, int nkt, int nt0,
                                           const __half* __restrict__ x, int lane, float (&acc)[GR_NTB][4]) {
  constexpr int TW = Win<K2>::TW, NW = Win<K2>::NW;
  const int t = lane & 3;
  uint32_t wn[GR_NTB][NW], bn0, bn1;
  auto fetch = [&](int kt) {
    bn0 = *reinterpret_cast<const uint32_t*>(x + kt * 16 + 2 * t);
    bn1 = *reinterpret_cast<const uint32_t*>(x + kt * 16 + 2 * t + 8);
    const uint32_t* row = T + ((size_t)kt * ntiles + nt0) * TW;
#pragma unroll
    for (int i = 0; i < GR_NTB; ++i) lane_words<K2>(row + i * TW, lane, wn[i]);
  };
  if (nkt > 0) fetch(kt0);
  for (int it = 0; it < nkt; ++it) {
    uint32_t wc[GR_NTB][NW];
    const uint32_t b0 = bn0, b1 = bn1;
#pragma unroll
    for (int i = 0; i < GR_NTB; ++i)
#pragma unroll
      for (int j = 0; j < NW; ++j) wc[i][j] = wn[i][j];
    if (it + 1 < nkt) fetch(kt0 + it + 1);
#pragma unroll
    for (int i = 0; i < GR_NTB; ++i) {
      uint32_t a[4];
      decode_words<CB, K2>(wc[i], lane, a);
      mma_f16(acc[i], a, b0, b1);
    }
  }
}

// Program (routed expert u, 64 columns, matrix x pair tile): up to 8 members times W_q; the four warps split K and
// meet in warp order.  Z[mat][pair][n] fp32.
template <int CB, int GR_NTB>
__global__ void __launch_bounds__(GR_WARPS * 32)
grouped_kernel(const __half* __restrict__ X0, const __half* __restrict__ X1, const int64_t* __restrict__ TP0,
               const int64_t* __restrict__ TP1, const int* __restrict__ K2_0, const int* __restrict__ K2_1,
               const int* __restrict__ uids, const int* __restrict__ ucount, const int* __restrict__ members,
               float* __restrict__ Z, int K, int N, int P, int maxm, int slots, int mtiles) {
  __shared__ int rows_sh[GR_PAIRS];
  __shared__ float red[GR_WARPS][GR_PAIRS][GR_NTB * 16 + 1];
  pdl_wait();
  const int u = blockIdx.x;
  const int mtile = blockIdx.z % mtiles, mat = blockIdx.z / mtiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // the count and the tile's members are read together (row u exists in the table for every u of the grid): most
  // CTAs of a grid sized for the worst case find nothing and leave after one round trip, not two
  const int n_u = ucount[0];
  if (threadIdx.x < GR_PAIRS) {
    const int m = mtile * GR_PAIRS + threadIdx.x;
    const int code = m < maxm ? members[(size_t)u * maxm + m] : -1;
    rows_sh[threadIdx.x] = code >= 0 ? (code >> 5) * slots + (code & 31) : -1;
  }
  if (u >= n_u) return;
  __syncthreads();
  if (rows_sh[0] < 0) return;                         // members come first: this pair tile is empty
  const int e = uids[u];
  const uint32_t* T = reinterpret_cast<const uint32_t*>(mat ? TP1[e] : TP0[e]);
  const int k2 = mat ? K2_1[e] : K2_0[e];
  const __half* X = mat ? X1 : X0;
  // lanes past the last member read the first member's row: an mma column depends on its own inputs only
  const int r = rows_sh[g] >= 0 ? rows_sh[g] : rows_sh[0];
  const __half* x = X + (size_t)r * K;
  const int KT = K >> 4, ntiles = N >> 4, per_warp = KT / GR_WARPS;
  const int kt0 = warp * per_warp, nt0 = blockIdx.y * GR_NTB;
  float acc[GR_NTB][4];
#pragma unroll
  for (int i = 0; i < GR_NTB; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  switch (k2) {
#define TFB_K2(K2_)                                                          \
  case K2_:                                                                  \
    warp_tiles<CB, K2_, GR_NTB>(T, ntiles, kt0, per_warp, nt0, x, lane, acc); \
    break;
    TFB_K2(2) TFB_K2(3) TFB_K2(4) TFB_K2(5) TFB_K2(6) TFB_K2(7) TFB_K2(8) TFB_K2(9) TFB_K2(10) TFB_K2(11) TFB_K2(12)
    TFB_K2(13) TFB_K2(14) TFB_K2(15) TFB_K2(16)
#undef TFB_K2
    default:
      atomicCAS(&g_kernel_status, 0, ST_BAD_INDEX);    // a width the host should have refused
      break;
  }
  pdl_launch_dependents();
  // acc[i]: d0 = (col g, pair 2t), d1 = (col g, pair 2t + 1), d2 = (col g + 8, pair 2t), d3 = (col g + 8, pair 2t + 1)
#pragma unroll
  for (int i = 0; i < GR_NTB; ++i) {
    red[warp][2 * t][i * 16 + g] = acc[i][0];
    red[warp][2 * t + 1][i * 16 + g] = acc[i][1];
    red[warp][2 * t][i * 16 + g + 8] = acc[i][2];
    red[warp][2 * t + 1][i * 16 + g + 8] = acc[i][3];
  }
  __syncthreads();
  for (int o = threadIdx.x; o < GR_PAIRS * GR_NTB * 16; o += GR_WARPS * 32) {
    const int pi = o / (GR_NTB * 16), col = o % (GR_NTB * 16);
    const int row = rows_sh[pi];
    if (row < 0) continue;
    float s = red[0][pi][col];
#pragma unroll
    for (int w = 1; w < GR_WARPS; ++w) s += red[w][pi][col];
    Z[((size_t)mat * P + row) * N + nt0 * 16 + col] = s;
  }
}

// W_q [K, N] fp16 of one matrix through the same lane decode (the bit-exactness hook).
template <int CB, int K2>
__global__ void dequant_kernel(const uint32_t* __restrict__ T, __half* __restrict__ out, int K, int N) {
  const int kt = blockIdx.x, nt = blockIdx.y, lane = threadIdx.x, g = lane >> 2, t = lane & 3;
  uint32_t a[4];
  decode_tile<CB, K2>(T + ((size_t)kt * (N >> 4) + nt) * Win<K2>::TW, lane, a);
  // a0 = (col g, k 2t, 2t+1), a1 = (col g + 8, ...), a2 = (col g, k 2t + 8, ..), a3 = (col g + 8, k 2t + 8, ..)
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const __half2 h = *reinterpret_cast<const __half2*>(&a[q]);
    const int col = nt * 16 + g + 8 * (q & 1), row = kt * 16 + 2 * t + 8 * (q >> 1);
    out[(size_t)row * N + col] = __low2half(h);
    out[(size_t)(row + 1) * N + col] = __high2half(h);
  }
}

// ---- 128-point Walsh-Hadamard transform, 4 values a lane: strides 1, 2 in registers, 4 .. 64 across lanes ---------
__device__ __forceinline__ void fwht128(float (&v)[4], int lane) {
  const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c;
  v[1] = b + d;
  v[2] = a - c;
  v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = (lane & m) ? o - v[j] : v[j] + o;
    }
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

// Program (pair, 128-block of K, matrix): xh = fp16(((x * suh) H)) for gate and up of every routed slot.
template <typename TIN>
__global__ void __launch_bounds__(32)
rot_in_kernel(const TIN* __restrict__ x, int64_t x_stride, const int* __restrict__ pick,
              const __half* __restrict__ suh0, const __half* __restrict__ suh1, __half* __restrict__ out0,
              __half* __restrict__ out1, int K, int slots, int E) {
  pdl_wait();
  const int p = blockIdx.x, blk = blockIdx.y, mat = blockIdx.z, lane = threadIdx.x;
  const int e = pick[p];
  if (e < 0 || e >= E) return;
  const __half* suh = (mat ? suh1 : suh0) + (size_t)e * K + blk * 128 + 4 * lane;
  const TIN* xr = x + (size_t)(p / slots) * x_stride + blk * 128 + 4 * lane;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = to_float<TIN>(xr[j]) * __half2float(suh[j]);
  fwht128(v, lane);
  __half* o = (mat ? out1 : out0) + (size_t)p * K + blk * 128 + 4 * lane;
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = __float2half_rn(v[j] * HAD_SCALE);
  pdl_launch_dependents();
}

// Program (pair, 128-block of the width): rotate gate and up, * svh, SwiGLU (act_mode 0: bf16 roundings as the GLM
// family; 1: fp32), * suh_d, rotate, fp16.
__global__ void __launch_bounds__(32)
gateup_epilogue_kernel(const float* __restrict__ Z, const int* __restrict__ pick, const __half* __restrict__ svh_g,
                       const __half* __restrict__ svh_u, const __half* __restrict__ suh_d, __half* __restrict__ xd,
                       int P, int N, int E, float limit, int act_mode) {
  pdl_wait();
  const int p = blockIdx.x, blk = blockIdx.y, lane = threadIdx.x;
  const int e = pick[p];
  if (e < 0 || e >= E) return;
  const int n = blk * 128 + 4 * lane;
  float gv[4], uv[4], v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    gv[j] = Z[(size_t)p * N + n + j];
    uv[j] = Z[((size_t)P + p) * N + n + j];
  }
  fwht128(gv, lane);
  fwht128(uv, lane);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float sg = __half2float(svh_g[(size_t)e * N + n + j]), su = __half2float(svh_u[(size_t)e * N + n + j]);
    float act;
    if (act_mode == 0) {
      const float gg = fminf(round_bf16(gv[j] * HAD_SCALE * sg), limit);
      const float uu = fminf(fmaxf(round_bf16(uv[j] * HAD_SCALE * su), -limit), limit);
      act = round_bf16(round_bf16(gg / (1.f + expf(-gg))) * uu);
    } else {
      const float gg = fminf(gv[j] * HAD_SCALE * sg, limit);
      const float uu = fminf(fmaxf(uv[j] * HAD_SCALE * su, -limit), limit);
      act = gg / (1.f + expf(-gg)) * uu;
    }
    v[j] = act * __half2float(suh_d[(size_t)e * N + n + j]);
  }
  fwht128(v, lane);
  __half* o = xd + (size_t)p * N + n;
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = __float2half_rn(v[j] * HAD_SCALE);
  pdl_launch_dependents();
}

// Program (row, 128-block of the model width), a warp a slot: y = (Z H) * svh_d per slot (fp32, also stored), then,
// when `out` is given, out = sum over slots in slot order of wts * y (an fma chain from 0).  Slots that are not routed
// experts keep the y the caller put there.
__global__ void down_epilogue_kernel(const float* __restrict__ Z, const int* __restrict__ pick,
                                     const __half* __restrict__ svh_d, float* __restrict__ y,
                                     const float* __restrict__ wts, float* __restrict__ out, int D, int E,
                                     int slots) {
  __shared__ float4 part[32][32];                     // [slot][lane]
  pdl_wait();
  const int r = blockIdx.x, blk = blockIdx.y, k = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blk * 128 + 4 * lane, p = r * slots + k;
  const int e = pick[p];
  float o[4];
  if (e >= 0 && e < E) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = Z[(size_t)p * D + n + j];
    fwht128(v, lane);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j] = v[j] * HAD_SCALE * __half2float(svh_d[(size_t)e * D + n + j]);
      y[(size_t)p * D + n + j] = o[j];
    }
  } else if (out != nullptr) {
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = y[(size_t)p * D + n + j];
  }
  if (out == nullptr) return;
  part[k][lane] = make_float4(o[0], o[1], o[2], o[3]);
  __syncthreads();
  if (k != 0) return;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int q = 0; q < slots; ++q) {
    const float w = wts[r * slots + q];
    const float4 s = part[q][lane];
    acc[0] = fmaf(w, s.x, acc[0]);
    acc[1] = fmaf(w, s.y, acc[1]);
    acc[2] = fmaf(w, s.z, acc[2]);
    acc[3] = fmaf(w, s.w, acc[3]);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) out[(size_t)r * D + n + j] = acc[j];
  pdl_launch_dependents();
}

}  // namespace exl3

// Grouping for the EXL3 kernels in one block: the plan's stable sort (one item an expert), then the reference's
// tables: uids = distinct routed experts (< E) ascending, members[u][<= maxm] = row * 32 + slot in row order, -1 after
// the last.  (src/tensorfold/cuda/exl3/experts.cu:19-72)
__global__ void __launch_bounds__(PLAN_THREADS)
exl3_group_kernel(const int* __restrict__ picks, int P, int E, int slots, int* __restrict__ tmp_members,
                  int* __restrict__ tmp_items, int* __restrict__ tmp_counts, int* __restrict__ uids,
                  int* __restrict__ ucount, int* __restrict__ members, int maxm, int maxu) {
  extern __shared__ int whist[];
  __shared__ int first[PLAN_EMAX];
  __shared__ int wsum[4][32];
  pdl_wait();
  plan_block(picks, P, E, P + 1, tmp_members, tmp_items, tmp_counts, whist, first, wsum);
  __threadfence_block();
  __syncthreads();
  const int n = min(tmp_counts[0], maxu);
  if (threadIdx.x == 0) ucount[0] = n;
  for (int u = threadIdx.x; u < n; u += PLAN_THREADS) uids[u] = tmp_items[3 * u];
  for (int64_t i = threadIdx.x; i < (int64_t)n * maxm; i += PLAN_THREADS) {
    const int u = (int)(i / maxm), j = (int)(i - (int64_t)u * maxm);
    const int f = tmp_items[3 * u + 1], c = tmp_items[3 * u + 2];
    int code = -1;
    if (j < c) {
      const int p = tmp_members[f + j];
      code = (p / slots) * 32 + p % slots;
    }
    members[i] = code;
  }
  pdl_launch_dependents();
}

}  // namespace tfb

using namespace tfb;

static int exl3_check_k2(const char* who, int k2) {
  TFB_REQUIRE(k2 >= 2 && k2 <= 16, "%s: half-bit width %d outside 2..16", who, k2);
  return TFB_OK;
}

// W_q [K, N] fp16 of one trellis [K/16, N/16, 8 * k2] int16.  (exl3/experts.py:205-213 `dequant`)
extern "C" int tfb_exl3_dequant(const void* trellis, void* out, int K, int N, int k2, int cb, void* stream) {
  TFB_REQUIRE(trellis && out, "exl3_dequant: null pointer");
  TFB_REQUIRE(K > 0 && N > 0 && K % 16 == 0 && N % 16 == 0, "exl3_dequant: K and N must be multiples of 16");
  TFB_REQUIRE(cb >= 0 && cb <= 2, "exl3_dequant: codebook must be 0 (3inst), 1 (mcg) or 2 (mul1)");
  if (int rc = exl3_check_k2("exl3_dequant", k2)) return rc;
  const dim3 grid(K / 16, N / 16);
  auto st = static_cast<cudaStream_t>(stream);
  auto* t = static_cast<const uint32_t*>(trellis);
  auto* o = static_cast<__half*>(out);
#define TFB_DQ(CB_, K2_)                                               \
  case K2_:                                                            \
    exl3::dequant_kernel<CB_, K2_><<<grid, 32, 0, st>>>(t, o, K, N);   \
    break;
#define TFB_DQ_ALL(CB_)                                                                                          \
  switch (k2) {                                                                                                  \
    TFB_DQ(CB_, 2) TFB_DQ(CB_, 3) TFB_DQ(CB_, 4) TFB_DQ(CB_, 5) TFB_DQ(CB_, 6) TFB_DQ(CB_, 7) TFB_DQ(CB_, 8)     \
    TFB_DQ(CB_, 9) TFB_DQ(CB_, 10) TFB_DQ(CB_, 11) TFB_DQ(CB_, 12) TFB_DQ(CB_, 13) TFB_DQ(CB_, 14)               \
    TFB_DQ(CB_, 15) TFB_DQ(CB_, 16)                                                                              \
  }
  if (cb == 0) { TFB_DQ_ALL(0) } else if (cb == 1) { TFB_DQ_ALL(1) } else { TFB_DQ_ALL(2) }
#undef TFB_DQ_ALL
#undef TFB_DQ
  return check_launch("exl3_dequant");
}

// pick [R, slots] -> uids [maxu], ucount [1], members [maxu, maxm]; tmp_members [R * slots], tmp_items
// [3 * min(R * slots, E)], tmp_counts [2] are caller scratch.  (exl3/experts.cpp `group`)
extern "C" int tfb_exl3_group(const int32_t* pick, int32_t* uids, int32_t* ucount, int32_t* members,
                              int32_t* tmp_members, int32_t* tmp_items, int32_t* tmp_counts, int R, int slots, int E,
                              int maxu, int maxm, void* stream) {
  TFB_REQUIRE(pick && uids && ucount && members && tmp_members && tmp_items && tmp_counts, "exl3_group: null pointer");
  TFB_REQUIRE(E >= 1 && E <= PLAN_EMAX, "exl3_group: at most %d experts, not %d", PLAN_EMAX, E);
  TFB_REQUIRE(slots >= 1 && slots <= 32, "exl3_group: 1..32 slots, not %d", slots);
  TFB_REQUIRE(R >= 0 && maxu >= 0 && maxm >= 0, "exl3_group: bad sizes");
  static int configured[64] = {0};
  int dev = 0;
  TFB_CUDA(cudaGetDevice(&dev), "exl3_group: cudaGetDevice");
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    TFB_CUDA(cudaFuncSetAttribute(exl3_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)(sizeof(int) * 32 * PLAN_EMAX)),
             "exl3_group: shared memory opt-in");
    configured[dev] = 1;
  }
  return check_cuda(launch(exl3_group_kernel, dim3(1), dim3(PLAN_THREADS), sizeof(int) * 32 * (size_t)E,
                           static_cast<cudaStream_t>(stream), pick, R * slots, E, slots, tmp_members, tmp_items,
                           tmp_counts, uids, ucount, members, maxm, maxu),
                    "exl3_group");
}

// xg / xu [R * slots, K] fp16 = rotated, suh-scaled inputs of every routed pair.  (exl3/experts.cpp `rot_in`)
extern "C" int tfb_exl3_rot_in(const void* x, int64_t x_stride, int x_is_fp16, const int32_t* pick, const void* suh0,
                               const void* suh1, void* out0, void* out1, int R, int K, int slots, int E,
                               void* stream) {
  TFB_REQUIRE(x && pick && suh0 && suh1 && out0 && out1, "exl3_rot_in: null pointer");
  TFB_REQUIRE(K > 0 && K % 128 == 0, "exl3_rot_in: K must be a multiple of 128");
  TFB_REQUIRE(slots >= 1 && slots <= 32 && x_stride >= K, "exl3_rot_in: bad slots or stride");
  if (R <= 0) return TFB_OK;
  const dim3 grid(R * slots, K / 128, 2);
  auto st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (x_is_fp16)
    e = launch(exl3::rot_in_kernel<__half>, grid, dim3(32), 0, st, static_cast<const __half*>(x), x_stride, pick,
               static_cast<const __half*>(suh0), static_cast<const __half*>(suh1), static_cast<__half*>(out0),
               static_cast<__half*>(out1), K, slots, E);
  else
    e = launch(exl3::rot_in_kernel<__nv_bfloat16>, grid, dim3(32), 0, st, static_cast<const __nv_bfloat16*>(x),
               x_stride, pick, static_cast<const __half*>(suh0), static_cast<const __half*>(suh1),
               static_cast<__half*>(out0), static_cast<__half*>(out1), K, slots, E);
  return check_cuda(e, "exl3_rot_in");
}

// Z [mats, P, N] fp32 = rotated inputs times W_q for every routed pair.  tp*: int64 trellis pointers [E]; k2_*: int32
// half-bit widths [E].  (exl3/experts.cpp `grouped`)
extern "C" int tfb_exl3_grouped(const void* x0, const void* x1, const int64_t* tp0, const int64_t* tp1,
                                const int32_t* k2_0, const int32_t* k2_1, const int32_t* uids, const int32_t* ucount,
                                const int32_t* members, float* z, int mats, int K, int N, int P, int slots, int cb,
                                int maxm, int maxu, void* stream) {
  TFB_REQUIRE(x0 && x1 && tp0 && tp1 && k2_0 && k2_1 && uids && ucount && members && z, "exl3_grouped: null pointer");
  TFB_REQUIRE(mats == 1 || mats == 2, "exl3_grouped: one or two matrices");
  TFB_REQUIRE(K > 0 && N > 0 && K % (16 * exl3::GR_WARPS) == 0 && N % (16 * exl3::GR_NTB_MAX) == 0,
              "exl3_grouped: K must be a multiple of %d and N of %d", 16 * exl3::GR_WARPS, 16 * exl3::GR_NTB_MAX);
  TFB_REQUIRE(cb >= 0 && cb <= 2, "exl3_grouped: codebook must be 0 (3inst), 1 (mcg) or 2 (mul1)");
  TFB_REQUIRE(slots >= 1 && slots <= 32 && maxm >= 0 && maxu >= 0, "exl3_grouped: bad sizes");
  if (maxu == 0 || maxm == 0) return TFB_OK;
  const int mtiles = (maxm + exl3::GR_PAIRS - 1) / exl3::GR_PAIRS;
  TFB_REQUIRE((int64_t)mats * mtiles <= 65535, "exl3_grouped: too many pair tiles for one launch");
  // column tiles a CTA: fewer when the call is small, so that every SM gets work (columns are independent: no effect
  // on any result)
  const int64_t units4 = (int64_t)maxu * (N / 64) * mats * mtiles;
  const int ntb = units4 >= 1184 ? 4 : units4 >= 592 ? 2 : 1;
  const dim3 grid(maxu, N / (16 * ntb), mats * mtiles);
  auto st = static_cast<cudaStream_t>(stream);
  auto* h0 = static_cast<const __half*>(x0);
  auto* h1 = static_cast<const __half*>(x1);
  cudaError_t e = cudaSuccess;
#define TFB_GR(CB_, NTB_)                                                                                          \
  e = launch(exl3::grouped_kernel<CB_, NTB_>, grid, dim3(exl3::GR_WARPS * 32), 0, st, h0, h1, tp0, tp1, k2_0, k2_1, \
             uids, ucount, members, z, K, N, P, maxm, slots, mtiles)
#define TFB_GR_CB(CB_)                  \
  if (ntb == 4) TFB_GR(CB_, 4);         \
  else if (ntb == 2) TFB_GR(CB_, 2);    \
  else TFB_GR(CB_, 1)
  if (cb == 0) { TFB_GR_CB(0); } else if (cb == 1) { TFB_GR_CB(1); } else { TFB_GR_CB(2); }
#undef TFB_GR_CB
#undef TFB_GR
  return check_cuda(e, "exl3_grouped");
}

// xd [P, N] fp16 from Z [2, P, N].  (exl3/experts.cpp `gateup_epilogue`)
extern "C" int tfb_exl3_gateup_epilogue(const float* z, const int32_t* pick, const void* svh_g, const void* svh_u,
                                        const void* suh_d, void* xd, int P, int N, int E, float limit, int act_mode,
                                        void* stream) {
  TFB_REQUIRE(z && pick && svh_g && svh_u && suh_d && xd, "exl3_gateup_epilogue: null pointer");
  TFB_REQUIRE(N > 0 && N % 128 == 0, "exl3_gateup_epilogue: N must be a multiple of 128");
  TFB_REQUIRE(act_mode == 0 || act_mode == 1, "exl3_gateup_epilogue: act_mode 0 (bf16 roundings) or 1 (fp32)");
  if (P <= 0) return TFB_OK;
  return check_cuda(launch(exl3::gateup_epilogue_kernel, dim3(P, N / 128), dim3(32), 0,
                           static_cast<cudaStream_t>(stream), z, pick, static_cast<const __half*>(svh_g),
                           static_cast<const __half*>(svh_u), static_cast<const __half*>(suh_d),
                           static_cast<__half*>(xd), P, N, E, limit, act_mode),
                    "exl3_gateup_epilogue");
}

// y [R * slots, D] fp32 from Z [R * slots, D]; with wts and out also out [R, D] = the slot-order weighted sum.
// (exl3/experts.cpp `down_epilogue`, `combine`, `down_combine`)
extern "C" int tfb_exl3_down_epilogue(const float* z, const int32_t* pick, const void* svh_d, float* y,
                                      const float* wts, float* out, int R, int D, int E, int slots, void* stream) {
  TFB_REQUIRE(z && pick && svh_d && y, "exl3_down_epilogue: null pointer");
  TFB_REQUIRE((wts == nullptr) == (out == nullptr), "exl3_down_epilogue: wts and out come together");
  TFB_REQUIRE(D > 0 && D % 128 == 0 && slots >= 1 && slots <= 32, "exl3_down_epilogue: D % 128 == 0, 1..32 slots");
  if (R <= 0) return TFB_OK;
  return check_cuda(launch(exl3::down_epilogue_kernel, dim3(R, D / 128), dim3(32 * slots), 0,
                           static_cast<cudaStream_t>(stream), z, pick, static_cast<const __half*>(svh_d), y, wts, out,
                           D, E, slots),
                    "exl3_down_epilogue");
}

// ---- grouping without caller scratch ---------------------------------------------------------------------------
// For hosts that cannot give this library device memory at call time: a serving process that handed every free byte
// of HBM to its own pools at start-up (so a later cudaMalloc fails), or a decode loop where allocation calls are
// banned because they stall the whole device.  The sort's temporaries live in the array below, which every GPU that
// loads the library carries until the process ends (about 140 KB).
constexpr int GROUP_STATIC_MAX_PAIRS = 32768;         // R * slots a call may sort
constexpr int GROUP_STATIC_WORDS = GROUP_STATIC_MAX_PAIRS + 3 * tfb::PLAN_EMAX + 64;
static __device__ __align__(256) int g_group_scratch[GROUP_STATIC_WORDS];
static int* g_group_scratch_ptr[64] = {nullptr};      // the array's device address, per device (host code cannot use the symbol itself)

// Same result as tfb_exl3_group, with no scratch arguments.  Limits: R * slots <= 32768, E <= 1024, slots <= 32.
// The first call on a device looks up the array's device address (cudaGetSymbolAddress) and opts the kernel into its
// shared-memory size; make that first call before starting any stream capture.  All calls on a device share the one
// array: two calls whose kernels may run at the same time on that GPU (different streams) would corrupt each other -
// keep them on one stream or order them with events.  Nothing in the array has to start at zero; a call overwrites
// what it reads.  Calls no allocating routine.
extern "C" int tfb_exl3_group_static(const int32_t* pick, int32_t* uids, int32_t* ucount, int32_t* members, int R,
                                     int slots, int E, int maxu, int maxm, void* stream) {
  TFB_REQUIRE(pick && uids && ucount && members, "exl3_group_static: null pointer");
  TFB_REQUIRE(E >= 1 && E <= PLAN_EMAX, "exl3_group_static: at most %d experts, not %d", PLAN_EMAX, E);
  TFB_REQUIRE(slots >= 1 && slots <= 32, "exl3_group_static: 1..32 slots, not %d", slots);
  TFB_REQUIRE(R >= 0 && maxu >= 0 && maxm >= 0, "exl3_group_static: bad sizes");
  TFB_REQUIRE((int64_t)R * slots <= GROUP_STATIC_MAX_PAIRS,
              "exl3_group_static: %lld pairs exceed the built-in scratch (%d pairs); use tfb_exl3_group with caller "
              "scratch", (long long)R * slots, GROUP_STATIC_MAX_PAIRS);
  int dev = 0;
  TFB_CUDA(cudaGetDevice(&dev), "exl3_group_static: cudaGetDevice");
  TFB_REQUIRE(dev >= 0 && dev < 64, "exl3_group_static: device index %d out of range", dev);
  if (g_group_scratch_ptr[dev] == nullptr) {
    int* ptr = nullptr;
    TFB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_group_scratch),
             "exl3_group_static: cudaGetSymbolAddress");
    TFB_CUDA(cudaFuncSetAttribute(exl3_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)(sizeof(int) * 32 * PLAN_EMAX)),
             "exl3_group_static: shared memory opt-in");
    g_group_scratch_ptr[dev] = ptr;
  }
  int* base = g_group_scratch_ptr[dev];
  int* tmp_counts = base;                             // [2] (+ padding to keep the next arrays 256-byte aligned)
  int* tmp_items = base + 64;                         // [3 * min(pairs, E)]
  int* tmp_members = base + 64 + 3 * PLAN_EMAX;       // [pairs]
  return check_cuda(launch(exl3_group_kernel, dim3(1), dim3(PLAN_THREADS), sizeof(int) * 32 * (size_t)E,
                           static_cast<cudaStream_t>(stream), pick, R * slots, E, slots, tmp_members, tmp_items,
                           tmp_counts, uids, ucount, members, maxm, maxu),
                    "exl3_group_static");
}
