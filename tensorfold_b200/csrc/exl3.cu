// Routed experts on EXL3 trellis-coded weights (ExLlamaV3's format), any codebook, a width per expert matrix.
//
// A 16 x 16 tile is a circular MSB-first bitstream of 256 values; value p's 16-bit state is the window ending at
// E(p) = (p >> 1) K2 + (p odd ? K2 : K2 >> 1) (K2 = half-bits a value); a codebook turns a state into an fp16 value;
// value p sits at row 2 (l % 4) + (j & 1) + 8 ((j >> 1) & 1), column l / 4 + 8 (j >> 2) of its tile (l = p / 8,
// j = p % 8) - so lane l's eight values are exactly its mma.m16n8k16 fragment of the tile.  Here the tile
// (transposed) is the A operand (16 output columns x 16 inputs) and the pairs' rotated inputs the B operand.
// The layer is y = (((x * suh) H) W_q) H * svh per 128-block, H = 128-point Hadamard / sqrt(128).
//
// Three launches a layer call (src/tensorfold/cuda/exl3/experts.py:173-202 needs seven):
//   prologue  one block sorts the (row, slot) pairs by expert into items of <= 16 pairs (the affine plan's sort), the
//             others rotate every routed pair's input for gate and up (x * suh, 128-point transform, fp16);
//   gate/up   CTA = (item, 64 columns, matrix): the four warps split K, each pulls its rows of tiles through a private
//             shared-memory ring with bulk async copies, decodes from shared memory and multiplies; the K slices meet
//             in warp order; the LAST of the four CTAs that share (item, 128 columns) - counted with an atomic - runs
//             the epilogue (rotate, svh, SwiGLU, suh_d, rotate) for the block and stores the down projection's input;
//   down      the same kernel with the output rotation (and svh) as its epilogue; y fp32 per pair.
// Fixed-order reductions everywhere: a pair's bits never depend on the other rows of the call.
// (Replaces src/tensorfold/cuda/exl3/experts.cu and experts_grouped.cuh; the trellises are read in place.)

#include <type_traits>

#include "api.h"
#include "common.cuh"

namespace tfb {
namespace exl3 {

constexpr float HAD_SCALE = 0.08838834764831845f;   // 1 / sqrt(128)
constexpr int GR_WARPS = 4;                         // K slices a CTA (part of the arithmetic: they meet in warp order)
constexpr int GR_NTB = 4;                           // 16-column tiles a CTA: 64 columns (2: the narrow CTAs, 32 columns)
constexpr int GR_NARROW_NTB = 2;
constexpr int GR_PT = 2;                            // mma tiles of 8 pairs an item: 16 pairs (4: the wide items, 32 pairs)
constexpr int GR_PAIRS = 8 * GR_PT;
constexpr int GR_WIDE_PT = 4;
constexpr int GR_SLOT_BYTES = 2048;                 // a ring slot: whole rows of the CTA's four tiles
constexpr int GR_STAGES = 3;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }

// ---- codebooks: two states -> two fp16 values (src/tensorfold/cuda/exl3/format.py:31-48) ------------------------
template <int CB>
__device__ __forceinline__ uint32_t cb_pair(uint32_t s0, uint32_t s1) {
  if constexpr (CB == 2) {                            // mul1: fma(1024 + sum of the bytes of s * M, scale, bias) in fp16
    const uint32_t h0 = __dp4a(s0 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t h1 = __dp4a(s1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t hv = prmt(h0, h1, 0x5410);
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&hv), __half2half2(__ushort_as_half(0x1EEE)),
                              __half2half2(__ushort_as_half(0xC931)));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {                                            // 3inst / mcg: the two fp16 halves of the masked product, added
    uint32_t x0 = CB == 1 ? s0 * 0xCBAC1FEDu : s0 * 89226354u + 64248484u;
    uint32_t x1 = CB == 1 ? s1 * 0xCBAC1FEDu : s1 * 89226354u + 64248484u;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;\n" : "=r"(x0) : "r"(x0), "r"(0x8FFF8FFFu), "r"(0x3B603B60u));   // (x & M) ^ F
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;\n" : "=r"(x1) : "r"(x1), "r"(0x8FFF8FFFu), "r"(0x3B603B60u));
    // each value = low half + high half of its own word: the fp16 adds take the halves straight from the register
    // (no permute), one permute packs the two results
    uint32_t r;
    asm("{\n.reg .b16 a, b, c, d;\n"
        "mov.b32 {a, b}, %1;\n"
        "mov.b32 {c, d}, %2;\n"
        "add.rn.f16 a, a, b;\n"
        "add.rn.f16 c, c, d;\n"
        "mov.b32 %0, {a, c};\n}\n"
        : "=r"(r)
        : "r"(x0), "r"(x1));
    return r;
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
// 8 lane's window.  4 bits a value (K2 = 8): exactly words lane - 1 and lane.  GLOBAL: the tile is in global memory
// (read-only path); else in shared memory.
template <int K2, bool GLOBAL>
__device__ __forceinline__ void lane_words(const uint32_t* __restrict__ tile, int lane, uint32_t (&w)[Win<K2>::NW]) {
  constexpr int TW = Win<K2>::TW, NW = Win<K2>::NW;
  const int first = 4 * lane * K2 + (K2 >> 1) - 16 + 32 * TW;       // E(8 lane) - 16, made non-negative
  int wi = (first >> 5) % TW;
#pragma unroll
  for (int i = 0; i < NW; ++i) {
    w[i] = GLOBAL ? __ldg(tile + wi) : tile[wi];
    wi = wi + 1 == TW ? 0 : wi + 1;
  }
}

// st[j] = state of value 8 lane + j from the lane's words.
template <int K2>
__device__ __forceinline__ void lane_states(const uint32_t (&w)[Win<K2>::NW], int lane, uint32_t (&st)[8]) {
  constexpr int NW = Win<K2>::NW, NV = Win<K2>::NV;
  if constexpr (K2 == 8) {
    // 16-bit windows ending 4 (j + 1) bits into the lane's own word w[1], the stream running on from w[0].  Three
    // funnel shifts line the windows up on byte boundaries; a byte permute then cuts each one out, zero-extended.
    const uint32_t q16 = __funnelshift_r(w[1], w[0], 16);           // stream bits -16 .. 16 of the own word
    const uint32_t q20 = __funnelshift_r(w[1], w[0], 20);           // -20 .. 12
    const uint32_t q4 = __funnelshift_r(w[1], w[0], 4);             // -4 .. 28
    st[0] = prmt(q20, 0u, 0x4421);                                  // bits -12 .. 4
    st[1] = prmt(q16, 0u, 0x4421);                                  // -8 .. 8
    st[2] = prmt(q20, 0u, 0x4410);                                  // -4 .. 12
    st[3] = prmt(q16, 0u, 0x4410);                                  // 0 .. 16
    st[4] = prmt(q4, 0u, 0x4421);                                   // 4 .. 20
    st[5] = prmt(w[1], 0u, 0x4421);                                 // 8 .. 24
    st[6] = prmt(q4, 0u, 0x4410);                                   // 12 .. 28
    st[7] = prmt(w[1], 0u, 0x4410);                                 // 16 .. 32
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

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One warp's k-tile rows [kt0, kt0 + nkt) of the CTA's four column tiles into acc.  The rows travel through the warp's
// ring: a slot holds ROWS whole rows (one bulk copy a row: the four tiles of a row are contiguous in the trellis), the
// elected lane refills a slot as soon as the warp has decoded it.  The rows of a slot are unrolled in blocks of up to
// four, whose inputs are loaded before the block's tiles are decoded.  x[pt]: the lane's pair (B column lane / 4 of
// tile pt) at input 16 kt0 + 2 (lane % 4).  NPT: the mma tiles of eight pairs that are live (one decode feeds them all).
// Returns false when a copy never landed.
template <int CB, int K2, int PT, int NPT, int NTB, bool COMPACT>
__device__ __forceinline__ bool warp_rows(const uint8_t* __restrict__ T, int ntiles, int kt0, int nkt, int nt0,
                                          const __half* const (&x)[PT], uint8_t* ring, uint64_t* bars, int lane,
                                          float (&acc)[NTB][PT][4]) {
  constexpr int TW = Win<K2>::TW, NW = Win<K2>::NW;
  constexpr int TILE_B = 16 * K2, SEG = NTB * TILE_B;                 // bytes a tile / a row of the CTA's tiles
  constexpr int ROWS = GR_SLOT_BYTES / SEG < 1 ? 1 : (GR_SLOT_BYTES / SEG > 16 ? 16 : GR_SLOT_BYTES / SEG);
  // rows a block (their inputs sit in registers; 4 was 3 % slower).  COMPACT: one row a block and the blocks of a slot
  // walked by a loop - a fifth of the code, for layers of mixed widths, where blocks that decode different widths
  // share an SM and the unrolled loops of five or seven widths miss the instruction cache all the time
  constexpr int RBMAX = COMPACT ? 1 : 2;
  constexpr int RB = ROWS < RBMAX ? ROWS : RBMAX;
  static_assert(ROWS * SEG <= GR_SLOT_BYTES, "a slot holds whole rows");
  const int nslot = (nkt + ROWS - 1) / ROWS;
  const uint8_t* src = T + ((size_t)kt0 * ntiles + nt0) * TILE_B;
  const size_t row_stride = (size_t)ntiles * TILE_B;
  auto issue = [&](int f) {
    const int rows = min(ROWS, nkt - f * ROWS);
    uint64_t* bar = bars + f % GR_STAGES;
    uint8_t* dst = ring + (f % GR_STAGES) * GR_SLOT_BYTES;
    mbar_expect_tx(bar, (uint32_t)(rows * SEG));
    for (int r = 0; r < rows; ++r) bulk_g2s(dst + r * SEG, src + (size_t)(f * ROWS + r) * row_stride, SEG, bar);
  };
  if (lane == 0)
    for (int f = 0; f < GR_STAGES && f < nslot; ++f) issue(f);
  // where the lane's words sit inside a tile: NW consecutive words (cyclically) from the one that holds the first bit
  // of value 8 lane's window
  int word[NW];
  {
    int wi = ((4 * lane * K2 + (K2 >> 1) - 16 + 32 * TW) >> 5) % TW;
#pragma unroll
    for (int j = 0; j < NW; ++j) {
      word[j] = wi;
      wi = wi + 1 == TW ? 0 : wi + 1;
    }
  }
  const __half* xp[PT];
#pragma unroll
  for (int pt = 0; pt < PT; ++pt) xp[pt] = x[pt];
  int stage = 0;
  uint32_t phase = 0;
  for (int f = 0; f < nslot; ++f) {
    const int rows = min(ROWS, nkt - f * ROWS);
    const uint32_t* slot = reinterpret_cast<const uint32_t*>(ring + stage * GR_SLOT_BYTES);
#pragma unroll(COMPACT ? 1 : 16)
    for (int r0 = 0; r0 < ROWS; r0 += RB) {
      if (r0 < rows) {
        uint32_t b[RB][NPT][2];
#pragma unroll
        for (int r = 0; r < RB; ++r)
#pragma unroll
          for (int pt = 0; pt < NPT; ++pt) {
            b[r][pt][0] = b[r][pt][1] = 0u;
            if (r0 + r < rows) {
              b[r][pt][0] = *reinterpret_cast<const uint32_t*>(xp[pt] + (r0 + r) * 16);
              b[r][pt][1] = *reinterpret_cast<const uint32_t*>(xp[pt] + (r0 + r) * 16 + 8);
            }
          }
        if (r0 == 0 && !mbar_wait_warp(bars + stage, phase)) {
          for (int g = f + 1; g < nslot && g < f + GR_STAGES; ++g)    // give the other copies in flight a while to land
            mbar_wait_for(bars + g % GR_STAGES, (g / GR_STAGES) & 1, 10000000ull);
          return false;
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) {
          if (r0 + r < rows) {
#pragma unroll
            for (int i = 0; i < NTB; ++i) {
              const uint32_t* tile = slot + (r0 + r) * (SEG / 4) + i * TW;
              uint32_t w[NW], a[4];
#pragma unroll
              for (int j = 0; j < NW; ++j) w[j] = tile[word[j]];
              decode_words<CB, K2>(w, lane, a);
#pragma unroll
              for (int pt = 0; pt < NPT; ++pt) mma_f16(acc[i][pt], a, b[r][pt][0], b[r][pt][1]);   // one decode, every pair tile
            }
          }
        }
      }
    }
#pragma unroll
    for (int pt = 0; pt < PT; ++pt) xp[pt] += ROWS * 16;
    __syncwarp();
    if (lane == 0 && f + GR_STAGES < nslot) issue(f + GR_STAGES);
    if (++stage == GR_STAGES) {
      stage = 0;
      phase ^= 1u;
    }
  }
  return true;
}

// ---- 128-point Walsh-Hadamard transform by 16 lanes, 8 consecutive values a lane ---------------------------------
// Strides 1, 2, 4 inside the lane, 8 .. 64 across the 16 lanes of a half warp (sub = lane % 16); a warp transforms two
// blocks at once.  Not scaled.
__device__ __forceinline__ void hadamard128(float (&v)[8], int sub) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1)
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if ((i & h) == 0) {
        const float a = v[i], b = v[i + h];
        v[i] = a + b;
        v[i + h] = a - b;
      }
#pragma unroll
  for (int m = 1; m < 16; m <<= 1)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (sub & m) ? o - v[i] : v[i] + o;
    }
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z); f[5] = bf16_hi(u.z); f[6] = bf16_lo(u.w); f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ void load8(const __half* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {   // another CTA of this launch wrote it: L2
  const float4 a = __ldcg(reinterpret_cast<const float4*>(p)), b = __ldcg(reinterpret_cast<const float4*>(p) + 1);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void store8(__half* p, const float (&f)[8], float scale) {
  uint4 u;
  __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i] * scale, f[2 * i + 1] * scale);
  *reinterpret_cast<uint4*>(p) = u;
}

// ---- epilogues of one pair and one 128-block, by a half warp ------------------------------------------------------
// gate/up: rotate both, * svh, SwiGLU (act_mode 0: the GLM family's bf16 roundings; 1: fp32), * suh_d, rotate, fp16.
// (arithmetic of src/tensorfold/cuda/exl3/experts.cu:116-158)
__device__ __forceinline__ void gateup_block(const float* zg, const float* zu, const __half* svh_g, const __half* svh_u,
                                             const __half* suh_d, __half* xd, int sub, float limit, int act_mode,
                                             bool store) {
  float g[8], u[8], sg[8], su[8], sd[8];
  load8(zg + 8 * sub, g);
  load8(zu + 8 * sub, u);
  load8(svh_g + 8 * sub, sg);
  load8(svh_u + 8 * sub, su);
  load8(suh_d + 8 * sub, sd);
  hadamard128(g, sub);
  hadamard128(u, sub);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float act;
    if (act_mode == 0) {
      const float gv = fminf(round_bf16(g[i] * HAD_SCALE * sg[i]), limit);
      const float uv = fminf(fmaxf(round_bf16(u[i] * HAD_SCALE * su[i]), -limit), limit);
      act = round_bf16(round_bf16(gv / (1.f + expf(-gv))) * uv);
    } else {
      const float gv = fminf(g[i] * HAD_SCALE * sg[i], limit);
      const float uv = fminf(fmaxf(u[i] * HAD_SCALE * su[i], -limit), limit);
      act = gv / (1.f + expf(-gv)) * uv;
    }
    g[i] = act * sd[i];
  }
  hadamard128(g, sub);
  if (store) store8(xd + 8 * sub, g, HAD_SCALE);
}

// down: y = rotate(z) * svh, fp32.  (src/tensorfold/cuda/exl3/experts.cu:161-180)
__device__ __forceinline__ void down_block(const float* z, const __half* svh, float* y, int sub, bool store) {
  float v[8], s[8];
  load8(z + 8 * sub, v);
  load8(svh + 8 * sub, s);
  hadamard128(v, sub);
  if (!store) return;
  float4 a, b;
  a.x = v[0] * HAD_SCALE * s[0]; a.y = v[1] * HAD_SCALE * s[1]; a.z = v[2] * HAD_SCALE * s[2]; a.w = v[3] * HAD_SCALE * s[3];
  b.x = v[4] * HAD_SCALE * s[4]; b.y = v[5] * HAD_SCALE * s[5]; b.z = v[6] * HAD_SCALE * s[6]; b.w = v[7] * HAD_SCALE * s[7];
  reinterpret_cast<float4*>(y + 8 * sub)[0] = a;
  reinterpret_cast<float4*>(y + 8 * sub)[1] = b;
}

// What the prologue needs to lay the items out by width: the three matrices' width tables [E] and the table it fills,
// [3, stride, 4] (gate, up, down order).
struct WidthOrder {
  const int* k2[3];
  int* sorted;
  int stride;
};

struct GroupedArgs {
  const __half* x[2];            // rotated inputs [P, K] fp16 of matrix 0 / 1
  const int64_t* tp[2];          // trellis pointers [E]
  const int* k2[2];              // half-bit widths [E]
  const int* items;              // [., 3] (expert, first, count <= 16)
  const int* sorted[2];          // or null: the items in the order their CTAs should run, [., 4] = (expert, first, count, index)
  const int* counts;             // [0] = items
  const int* members;            // pair ids p = row * slots + slot, grouped by expert
  float* z;                      // [mats, P, N] fp32
  int* arrive;                   // [max items * N / 128] zero between launches
  const __half* sv[2];           // svh [E, N] of matrix 0 / 1
  const __half* suh_next;        // gate/up: suh of the down projection [E, N]
  void* out;                     // gate/up: xd [P, N] fp16; down: y [P, N] fp32
  int K, N, P, mats, epi, act_mode;
  float limit;
};

enum GroupedEpilogue : int { GE_NONE = 0, GE_GATEUP = 1, GE_DOWN = 2 };

// CTA (item, 64 columns, matrix).  PT: mma tiles of eight pairs an item may hold (2: items of 16 pairs; 4: items of 32,
// for calls with many pairs an expert - every weight tile is then decoded once for up to 32 pairs).
// K2F: 0, or the one width every tensor of the launch has (the host knows it): the kernel then holds that width's loop
// alone - a tenth of the code, which matters where a CTA's life is short (one token: the dominant stall of the
// all-widths kernel was the instruction fetch).
// NTB: 16-column tiles a CTA (4, or 2 where the launch would otherwise have too few CTAs to fill the GPU).
template <int CB, int PT, int K2F, int NTB, bool COMPACT>
__global__ void __launch_bounds__(GR_WARPS * 32)
grouped_kernel(const GroupedArgs a) {
  constexpr int PAIRS = 8 * PT, GR_RED_STRIDE = NTB * 16 + 1;
  constexpr int RING_BYTES = GR_WARPS * GR_STAGES * GR_SLOT_BYTES, RED_BYTES = GR_WARPS * PAIRS * GR_RED_STRIDE * 4;
  // the K slices meet in the ring's memory (free by then)
  __shared__ __align__(128) uint8_t ring[RING_BYTES > RED_BYTES ? RING_BYTES : RED_BYTES];
  __shared__ uint64_t bars[GR_WARPS * GR_STAGES];
  __shared__ int pair_sh[PAIRS];
  __shared__ int last_sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int nt0 = blockIdx.x * NTB, mat = blockIdx.z;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < GR_STAGES; ++s) mbar_init(bars + warp * GR_STAGES + s, 1);
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncwarp();
  pdl_wait();
  const int *items = a.items, *counts = a.counts, *members = a.members, *sorted = a.sorted[mat];
  const __half* xin = a.x[mat];
  after_wait(items, counts, members, xin, sorted);
  // the item is read together with the count that says whether it exists (its slot is always inside the table)
  const int n_items = ld_dep(counts);
  int it = blockIdx.y, e, first, cnt;
  if (sorted != nullptr) {                            // the CTA's place in the launch is not the item's index
    const int4 s4 = ld_dep4(sorted + 4 * blockIdx.y);
    e = s4.x, first = s4.y, cnt = min(s4.z, PAIRS), it = s4.w;
  } else {
    e = ld_dep(items + 3 * it), first = ld_dep(items + 3 * it + 1), cnt = min(ld_dep(items + 3 * it + 2), PAIRS);
  }
  if ((int)blockIdx.y >= n_items) return;
  if (tid < PAIRS) pair_sh[tid] = tid < cnt ? ld_dep(members + first + tid) : -1;
  const uint8_t* T = reinterpret_cast<const uint8_t*>(a.tp[mat][e]);
  const int k2 = a.k2[mat][e];
  const int live = (cnt + 7) >> 3;                   // mma tiles of pairs in use
  // lanes past the item's last pair read its first pair's row: an mma column depends on its own inputs only
  const int KT = a.K >> 4, per_warp = (KT + GR_WARPS - 1) / GR_WARPS;
  const int kt0 = min(KT, warp * per_warp), nkt = min(KT, kt0 + per_warp) - kt0;
  const __half* x[PT];
#pragma unroll
  for (int pt = 0; pt < PT; ++pt) {
    const int p = ld_dep(members + first + (8 * pt + g < cnt ? 8 * pt + g : 0));
    x[pt] = xin + (size_t)p * a.K + kt0 * 16 + 2 * t;
  }
  float acc[NTB][PT][4];
#pragma unroll
  for (int i = 0; i < NTB; ++i)
#pragma unroll
    for (int pt = 0; pt < PT; ++pt) acc[i][pt][0] = acc[i][pt][1] = acc[i][pt][2] = acc[i][pt][3] = 0.f;
  bool ok = true;
  uint8_t* my_ring = ring + warp * (GR_STAGES * GR_SLOT_BYTES);
  uint64_t* my_bars = bars + warp * GR_STAGES;
#define TFB_K2_BODY(K2_)                                                                                  \
    if constexpr (PT == 2)                                                                                \
      ok = live > 1 ? warp_rows<CB, K2_, 2, 2, NTB, COMPACT>(T, a.N >> 4, kt0, nkt, nt0, x, my_ring, my_bars, lane, acc)  \
                    : warp_rows<CB, K2_, 2, 1, NTB, COMPACT>(T, a.N >> 4, kt0, nkt, nt0, x, my_ring, my_bars, lane, acc); \
    else                                                                                                  \
      ok = live > 2 ? warp_rows<CB, K2_, 4, 4, NTB, COMPACT>(T, a.N >> 4, kt0, nkt, nt0, x, my_ring, my_bars, lane, acc)  \
                    : warp_rows<CB, K2_, 4, 2, NTB, COMPACT>(T, a.N >> 4, kt0, nkt, nt0, x, my_ring, my_bars, lane, acc);
#define TFB_K2(K2_) \
  case K2_:         \
    TFB_K2_BODY(K2_) \
    break;
  if constexpr (K2F != 0) {
    if (k2 == K2F) {
      TFB_K2_BODY(K2F)
    } else {
      atomicCAS(&g_kernel_status, 0, ST_BAD_INDEX);   // not the width the host promised
      ok = false;
    }
  } else {
    switch (k2) {
      TFB_K2(2) TFB_K2(3) TFB_K2(4) TFB_K2(5) TFB_K2(6) TFB_K2(7) TFB_K2(8) TFB_K2(9) TFB_K2(10) TFB_K2(11) TFB_K2(12)
      TFB_K2(13) TFB_K2(14) TFB_K2(15) TFB_K2(16)
      default:
        atomicCAS(&g_kernel_status, 0, ST_BAD_INDEX);   // a width the host should have refused
        ok = false;
        break;
    }
  }
#undef TFB_K2
#undef TFB_K2_BODY
  pdl_launch_dependents();
  if (__syncthreads_or(ok ? 0 : 1)) return;           // a copy never landed (recorded): store nothing
  // the K slices meet in warp order (the ring's memory is free: every warp is past its loop)
  // acc[i][pt]: d0 = (col g, pair 2t), d1 = (col g, pair 2t + 1), d2 = (col g + 8, pair 2t), d3 = (col g + 8, 2t + 1)
  float* red = reinterpret_cast<float*>(ring);
#pragma unroll
  for (int i = 0; i < NTB; ++i)
#pragma unroll
    for (int pt = 0; pt < PT; ++pt) {
      float* base = red + (warp * PAIRS + 8 * pt + 2 * t) * GR_RED_STRIDE + i * 16 + g;
      base[0] = acc[i][pt][0];
      base[GR_RED_STRIDE] = acc[i][pt][1];
      base[8] = acc[i][pt][2];
      base[GR_RED_STRIDE + 8] = acc[i][pt][3];
    }
  __syncthreads();
  for (int o = tid; o < PAIRS * NTB * 16; o += GR_WARPS * 32) {
    const int pi = o / (NTB * 16), col = o % (NTB * 16);
    const int p = pair_sh[pi];
    if (p < 0) continue;
    float s = red[pi * GR_RED_STRIDE + col];
#pragma unroll
    for (int w = 1; w < GR_WARPS; ++w) s += red[(w * PAIRS + pi) * GR_RED_STRIDE + col];
    a.z[((size_t)mat * a.P + p) * a.N + nt0 * 16 + col] = s;
  }
  if (a.epi == GE_NONE) return;
  // Whoever finishes last among the CTAs that share (item, 128 columns) - two column halves, times the matrices -
  // finds every part of the block in z and runs the block's epilogue.
  constexpr int PER_BLOCK = 128 / (16 * NTB);          // CTAs that share a 128-column block of one matrix
  const int blk = blockIdx.x / PER_BLOCK;
  int* counter = a.arrive + (size_t)it * (a.N >> 7) + blk;
  __syncthreads();
  if (tid == 0) {
    const int need = PER_BLOCK * a.mats;
    const int seen = arrive_count(counter);
    last_sh = seen == need - 1;
    if (seen == need - 1) *counter = 0;               // nobody else touches it before the next launch
  }
  __syncthreads();
  if (!last_sh) return;
  // a half warp a pair (the transform's shuffles need every lane of the warp: a half without a pair repeats the item's
  // first pair and stores nothing); pairs fill an item from the front, so a warp whose first pair is missing is done
  const int sub = lane & 15, half = lane >> 4;
  for (int p0 = 2 * warp; p0 < PAIRS && pair_sh[p0] >= 0; p0 += 2 * GR_WARPS) {
    const int p = pair_sh[p0 + half];
    const int q = p < 0 ? pair_sh[0] : p;
    const size_t at = (size_t)q * a.N + blk * 128, sc = (size_t)e * a.N + blk * 128;
    if (a.epi == GE_GATEUP)
      gateup_block(a.z + at, a.z + (size_t)a.P * a.N + at, a.sv[0] + sc, a.sv[1] + sc, a.suh_next + sc,
                   static_cast<__half*>(a.out) + at, sub, a.limit, a.act_mode, p >= 0);
    else
      down_block(a.z + at, a.sv[0] + sc, static_cast<float*>(a.out) + at, sub, p >= 0);
  }
}

}  // namespace exl3
}  // namespace tfb

namespace tfb {
namespace exl3 {

// W_q [K, N] fp16 of one matrix through the same lane decode (the bit-exactness hook).
template <int CB, int K2>
__global__ void dequant_kernel(const uint32_t* __restrict__ T, __half* __restrict__ out, int K, int N) {
  const int kt = blockIdx.x, nt = blockIdx.y, lane = threadIdx.x, g = lane >> 2, t = lane & 3;
  uint32_t w[Win<K2>::NW], a[4];
  lane_words<K2, true>(T + ((size_t)kt * (N >> 4) + nt) * Win<K2>::TW, lane, w);
  decode_words<CB, K2>(w, lane, a);
  // a0 = (col g, k 2t, 2t+1), a1 = (col g + 8, ...), a2 = (col g, k 2t + 8, ..), a3 = (col g + 8, k 2t + 8, ..)
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const __half2 h = *reinterpret_cast<const __half2*>(&a[q]);
    const int col = nt * 16 + g + 8 * (q & 1), row = kt * 16 + 2 * t + 8 * (q >> 1);
    out[(size_t)row * N + col] = __low2half(h);
    out[(size_t)(row + 1) * N + col] = __high2half(h);
  }
}

}  // namespace exl3

// The first launch of a layer call.  Block 0 (when `sort`): the plan's stable sort of the pairs by expert, items of at
// most 16 pairs (ids outside [0, E) are left out), and the number of distinct experts into ucount.  The other blocks:
// out_m[p, :] = fp16(((x[row of p] * suh_m[expert of p]) H) / sqrt(128)) for every routed pair and 128-block, a half
// warp a block, both matrices from one read of x.  suh1 == nullptr: one matrix.
// (src/tensorfold/cuda/exl3/experts.cu:19-111: `group` and `rot_in`)
template <typename TIN>
__global__ void __launch_bounds__(PLAN_THREADS)
exl3_prologue_kernel(const int* __restrict__ picks, int P, int E, int slots, int sort, int* __restrict__ members,
                     int* __restrict__ items, int* __restrict__ counts, int* __restrict__ ucount,
                     const TIN* __restrict__ x, int64_t x_stride, const __half* __restrict__ suh0,
                     const __half* __restrict__ suh1, __half* __restrict__ out0, __half* __restrict__ out1, int K,
                     exl3::WidthOrder wo) {
  extern __shared__ int whist[];
  __shared__ int first[PLAN_EMAX];
  __shared__ uint64_t tot2[2][PLAN_THREADS / 32];
  __shared__ int bucket[3][16];
  pdl_wait();
  after_wait(picks, x);
  if (blockIdx.x == 0) {
    if (sort) {
      plan_block<PLAN_THREADS>(picks, P, E, sort, members, items, counts, whist, first, tot2);
      if (threadIdx.x == 0) ucount[0] = counts[1];    // written by this thread inside plan_block
      if (wo.sorted != nullptr) {
        // The items once more for each matrix, widest trellis first: blocks that run at the same time then decode the
        // same width, i.e. run the same code (every width is its own unrolled loop; seven of them at once on an SM
        // miss the instruction cache all the time).  The order inside a width is whatever the atomics give: no
        // result depends on it.
        if (threadIdx.x < 48) bucket[threadIdx.x / 16][threadIdx.x % 16] = 0;
        __threadfence_block();
        __syncthreads();
        const int n = counts[0];
        for (int i = threadIdx.x; i < n; i += PLAN_THREADS) {
          const int e = items[3 * i];
#pragma unroll
          for (int m = 0; m < 3; ++m) atomicAdd(&bucket[m][16 - min(max(wo.k2[m][e], 1), 16)], 1);
        }
        __syncthreads();
        if (threadIdx.x < 3) {
          int run = 0;
          for (int b = 0; b < 16; ++b) {
            const int c = bucket[threadIdx.x][b];
            bucket[threadIdx.x][b] = run;
            run += c;
          }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += PLAN_THREADS) {
          const int4 item = make_int4(items[3 * i], items[3 * i + 1], items[3 * i + 2], i);
#pragma unroll
          for (int m = 0; m < 3; ++m) {
            const int at = atomicAdd(&bucket[m][16 - min(max(wo.k2[m][item.x], 1), 16)], 1);
            reinterpret_cast<int4*>(wo.sorted + (size_t)m * wo.stride * 4)[at] = item;
          }
        }
      }
    }
    pdl_launch_dependents();
    return;
  }
  const int lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
  const int nblk = K >> 7;
  const int64_t units = (int64_t)P * nblk;
  const int64_t warps = (int64_t)(gridDim.x - 1) * (PLAN_THREADS / 32);
  for (int64_t u0 = 2 * ((int64_t)(blockIdx.x - 1) * (PLAN_THREADS / 32) + (threadIdx.x >> 5)); u0 < units;
       u0 += 2 * warps) {
    const bool have = u0 + half < units;              // the transform's shuffles need every lane: an idle half repeats u0
    const int64_t u = have ? u0 + half : u0;
    const int p = (int)(u / nblk), blk = (int)(u - (int64_t)p * nblk);
    const int e = picks[p];
    const bool routed = have && e >= 0 && e < E;
    const int es = routed ? e : 0;
    float xv[8];
    exl3::load8(x + (size_t)(p / slots) * x_stride + blk * 128 + 8 * sub, xv);
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const __half* suh = m ? suh1 : suh0;
      if (suh == nullptr) continue;
      float s[8], v[8];
      exl3::load8(suh + (size_t)es * K + blk * 128 + 8 * sub, s);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = xv[i] * s[i];
      exl3::hadamard128(v, sub);
      if (routed) exl3::store8((m ? out1 : out0) + (size_t)p * K + blk * 128 + 8 * sub, v, exl3::HAD_SCALE);
    }
  }
  pdl_launch_dependents();
}

// The prompt form's epilogue: out[m, block] = rotate(z[m, block]) / sqrt(128) * svh + bias for every row and
// 128-column block of a product z [M, N] fp32, a half warp a block.
// (the epilogue of src/tensorfold/cuda/exl3/prefill.py:15-44 `_gemm`)
template <typename TOUT>
__global__ void __launch_bounds__(256)
exl3_rot_out_kernel(const float* __restrict__ z, const __half* __restrict__ svh, const __half* __restrict__ bias,
                    TOUT* __restrict__ out, int64_t out_stride, int M, int N) {
  const int lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
  const int nblk = N >> 7;
  const int64_t units = (int64_t)M * nblk;
  const int64_t warps = (int64_t)gridDim.x * 8;
  pdl_wait();
  after_wait(z);
  for (int64_t u0 = 2 * ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)); u0 < units; u0 += 2 * warps) {
    const bool have = u0 + half < units;              // the transform's shuffles need every lane: an idle half repeats u0
    const int64_t u = have ? u0 + half : u0;
    const int m = (int)(u / nblk), blk = (int)(u - (int64_t)m * nblk);
    float v[8], s[8], b[8];
    const float4* src = reinterpret_cast<const float4*>(z + (size_t)m * N + blk * 128 + 8 * sub);
    const float4 lo = src[0], hi = src[1];
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    exl3::load8(svh + blk * 128 + 8 * sub, s);
#pragma unroll
    for (int i = 0; i < 8; ++i) b[i] = 0.f;
    if (bias != nullptr) exl3::load8(bias + blk * 128 + 8 * sub, b);
    exl3::hadamard128(v, sub);
    if (!have) continue;
    TOUT* dst = out + (size_t)m * out_stride + blk * 128 + 8 * sub;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float y = fmaf(v[i] * exl3::HAD_SCALE, s[i], b[i]);
      if constexpr (sizeof(TOUT) == 4) dst[i] = y;
      else if constexpr (std::is_same<TOUT, __half>::value) dst[i] = __float2half_rn(y);
      else dst[i] = __float2bfloat16_rn(y);
    }
  }
  pdl_launch_dependents();
}

// Grouping for callers of the `group` operator, in one block: the plan's stable sort (one item an expert), then the
// reference's tables: uids = distinct routed experts (< E) ascending, members[u][<= maxm] = row * 32 + slot in row
// order, -1 after the last.  (src/tensorfold/cuda/exl3/experts.cu:19-72)
__global__ void __launch_bounds__(PLAN_THREADS)
exl3_group_kernel(const int* __restrict__ picks, int P, int E, int slots, int* __restrict__ tmp_members,
                  int* __restrict__ tmp_items, int* __restrict__ tmp_counts, int* __restrict__ uids,
                  int* __restrict__ ucount, int* __restrict__ members, int maxm, int maxu) {
  extern __shared__ int whist[];
  __shared__ int first[PLAN_EMAX];
  __shared__ uint64_t tot2[2][PLAN_THREADS / 32];
  pdl_wait();
  after_wait(picks);
  plan_block<PLAN_THREADS>(picks, P, E, P + 1, tmp_members, tmp_items, tmp_counts, whist, first, tot2);
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

// Opts a plan-sized kernel into the dynamic shared memory of PLAN_EMAX experts, once a device.
template <typename Kernel>
static int plan_smem_opt_in(Kernel kernel, int* configured, const char* what) {
  int dev = 0;
  TFB_CUDA(cudaGetDevice(&dev), what);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    TFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)(sizeof(int) * 32 * PLAN_EMAX)),
             what);
    configured[dev] = 1;
  }
  return TFB_OK;
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
  if (int rc = plan_smem_opt_in(exl3_group_kernel, configured, "exl3_group: shared memory opt-in")) return rc;
  return check_cuda(launch(exl3_group_kernel, dim3(1), dim3(PLAN_THREADS), sizeof(int) * 32 * (size_t)E,
                           static_cast<cudaStream_t>(stream), pick, R * slots, E, slots, tmp_members, tmp_items,
                           tmp_counts, uids, ucount, members, maxm, maxu),
                    "exl3_group");
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

// The first launch of a routed call: sorts the pairs by expert (when `sort`, which is then the pairs an item holds, 16
// or 32: members [R * slots], items [(min(R * slots, E) + R * slots / sort), 3] = (expert, first, count <= sort),
// counts [2], ucount [1] = distinct experts)
// and rotates the inputs: out0 / out1 [R * slots, K] fp16 for the two matrices (suh1 / out1 null: one matrix).
// sorted (or null): int32 [3, sorted_stride, 4], filled with the items as (expert, first, count, index), once in the
// order of each matrix's widths k2_g / k2_u / k2_d [E] (widest first), for tfb_exl3_gateup / tfb_exl3_down of a layer
// whose tensors differ in width; sorted_stride >= the sort's items.
extern "C" int tfb_exl3_prologue(const void* x, int64_t x_stride, int x_is_fp16, const int32_t* pick, const void* suh0,
                                 const void* suh1, void* out0, void* out1, int R, int K, int slots, int E, int sort,
                                 int32_t* members, int32_t* items, int32_t* counts, int32_t* ucount,
                                 const int32_t* k2_g, const int32_t* k2_u, const int32_t* k2_d, int32_t* sorted,
                                 int sorted_stride, void* stream) {
  TFB_REQUIRE(x && pick && suh0 && out0, "exl3_prologue: null pointer");
  TFB_REQUIRE(sorted == nullptr || (sort && k2_g && k2_u && k2_d && sorted_stride >= 1 && aligned16(sorted)),
              "exl3_prologue: the width order needs the sort, the three width tables and a 16-byte aligned table");
  const exl3::WidthOrder wo = {{k2_g, k2_u, k2_d}, sorted, sorted_stride};
  TFB_REQUIRE((suh1 == nullptr) == (out1 == nullptr), "exl3_prologue: the second matrix's scales and output come together");
  TFB_REQUIRE(!sort || (members && items && counts && ucount), "exl3_prologue: null sort table");
  TFB_REQUIRE(sort == 0 || sort == 8 * exl3::GR_PT || sort == 8 * exl3::GR_WIDE_PT,
              "exl3_prologue: sort is 0 (the caller sorted), %d or %d (pairs an item)", 8 * exl3::GR_PT, 8 * exl3::GR_WIDE_PT);
  TFB_REQUIRE(K > 0 && K % 128 == 0, "exl3_prologue: K must be a multiple of 128");
  TFB_REQUIRE(slots >= 1 && slots <= 32 && x_stride >= K && x_stride % 8 == 0, "exl3_prologue: bad slots or stride");
  TFB_REQUIRE(aligned16(x) && aligned16(suh0) && aligned16(out0) && aligned16(suh1) && aligned16(out1),
              "exl3_prologue: 16-byte aligned rows");
  TFB_REQUIRE(E >= 1 && E <= PLAN_EMAX, "exl3_prologue: at most %d experts, not %d", PLAN_EMAX, E);
  if (R <= 0) return TFB_OK;
  const int64_t units = (int64_t)R * slots * (K / 128);
  const int64_t want = (units + 2 * (PLAN_THREADS / 32) - 1) / (2 * (PLAN_THREADS / 32));
  const int rot_blocks = (int)(want < 2 * sm_count() ? want : 2 * sm_count());
  const dim3 grid(1 + rot_blocks);
  const size_t smem = sort ? sizeof(int) * 32 * (size_t)E : 0;
  auto st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (x_is_fp16) {
    static int configured[64] = {0};
    if (int rc = plan_smem_opt_in(exl3_prologue_kernel<__half>, configured, "exl3_prologue: shared memory opt-in")) return rc;
    e = launch(exl3_prologue_kernel<__half>, grid, dim3(PLAN_THREADS), smem, st, pick, R * slots, E, slots, sort, members,
               items, counts, ucount, static_cast<const __half*>(x), x_stride, static_cast<const __half*>(suh0),
               static_cast<const __half*>(suh1), static_cast<__half*>(out0), static_cast<__half*>(out1), K, wo);
  } else {
    static int configured[64] = {0};
    if (int rc = plan_smem_opt_in(exl3_prologue_kernel<__nv_bfloat16>, configured, "exl3_prologue: shared memory opt-in"))
      return rc;
    e = launch(exl3_prologue_kernel<__nv_bfloat16>, grid, dim3(PLAN_THREADS), smem, st, pick, R * slots, E, slots, sort,
               members, items, counts, ucount, static_cast<const __nv_bfloat16*>(x), x_stride,
               static_cast<const __half*>(suh0), static_cast<const __half*>(suh1), static_cast<__half*>(out0),
               static_cast<__half*>(out1), K, wo);
  }
  return check_cuda(e, "exl3_prologue");
}

static int exl3_grouped_launch(const char* who, const exl3::GroupedArgs& a, int cb, int max_items, int item_pairs,
                               int k2_all, int col_tiles, void* stream) {
  TFB_REQUIRE(col_tiles == exl3::GR_NTB || col_tiles == exl3::GR_NARROW_NTB, "%s: %d or %d column tiles a block, not %d",
              who, exl3::GR_NTB, exl3::GR_NARROW_NTB, col_tiles);
  TFB_REQUIRE(k2_all == 0 || k2_all == -1 || (k2_all >= 2 && k2_all <= 16),
              "%s: k2_all is 0, -1 (the widths differ) or the one width of every tensor", who);
  TFB_REQUIRE(k2_all == 8 || col_tiles == exl3::GR_NTB, "%s: only a launch of 4.00-bit tensors (k2_all 8) takes blocks of %d "
              "column tiles", who, exl3::GR_NARROW_NTB);
  TFB_REQUIRE(item_pairs == 8 * exl3::GR_PT || item_pairs == 8 * exl3::GR_WIDE_PT, "%s: items of %d or %d pairs, not %d",
              who, 8 * exl3::GR_PT, 8 * exl3::GR_WIDE_PT, item_pairs);
  TFB_REQUIRE(a.K > 0 && a.N > 0 && a.K % 128 == 0 && a.N % 128 == 0, "%s: K and N must be multiples of 128", who);
  TFB_REQUIRE(cb >= 0 && cb <= 2, "%s: codebook must be 0 (3inst), 1 (mcg) or 2 (mul1)", who);
  TFB_REQUIRE(max_items >= 0 && a.P >= 0, "%s: bad sizes", who);
  if (max_items == 0 || a.P == 0) return TFB_OK;
  TFB_REQUIRE(max_items <= 65535, "%s: too many items for one launch", who);
  const dim3 grid(a.N / (16 * col_tiles), max_items, a.mats);          // an item's column blocks run together
  auto st = static_cast<cudaStream_t>(stream);
  const dim3 block(exl3::GR_WARPS * 32);
  const bool wide = item_pairs == 8 * exl3::GR_WIDE_PT;
  const bool four = k2_all == 8;                      // the one width with a kernel of its own (4.00 bits a weight)
  const bool narrow = col_tiles == exl3::GR_NARROW_NTB;
  cudaError_t e;
#define TFB_GR4(CB_, PT_, K2F_) launch(exl3::grouped_kernel<CB_, PT_, K2F_, exl3::GR_NTB, false>, grid, block, 0, st, a)
#define TFB_GRN(CB_, PT_) launch(exl3::grouped_kernel<CB_, PT_, 8, exl3::GR_NARROW_NTB, false>, grid, block, 0, st, a)
#define TFB_GRC(CB_, PT_) launch(exl3::grouped_kernel<CB_, PT_, 0, exl3::GR_NTB, true>, grid, block, 0, st, a)
#define TFB_GR(CB_)                                                                                     \
  e = k2_all == -1 ? (wide ? TFB_GRC(CB_, exl3::GR_WIDE_PT) : TFB_GRC(CB_, exl3::GR_PT))                 \
      : narrow     ? (wide ? TFB_GRN(CB_, exl3::GR_WIDE_PT) : TFB_GRN(CB_, exl3::GR_PT))                 \
      : four       ? (wide ? TFB_GR4(CB_, exl3::GR_WIDE_PT, 8) : TFB_GR4(CB_, exl3::GR_PT, 8))           \
                   : (wide ? TFB_GR4(CB_, exl3::GR_WIDE_PT, 0) : TFB_GR4(CB_, exl3::GR_PT, 0))
  if (cb == 0) {
    TFB_GR(0);
  } else if (cb == 1) {
    TFB_GR(1);
  } else {
    TFB_GR(2);
  }
#undef TFB_GRC
#undef TFB_GRN
#undef TFB_GR4
#undef TFB_GR
  return check_cuda(e, who);
}

// xd [P, N] fp16 = the down projection's rotated input of every routed pair: gate and up (trellis GEMV over the rotated
// inputs xg, xu [P, K] fp16), output rotation, svh, SwiGLU (act_mode 0: bf16 roundings, 1: fp32; clipped at limit),
// suh_d, rotation - one launch.  tp_*: int64 trellis pointers [E] (16-byte aligned trellises), k2_*: int32 [E];
// items / counts / members: the prologue's sort; z: fp32 scratch [2, P, N]; arrive: int scratch
// [max_items * N / 128], zero before the first call (every call leaves it zero); max_items >= the sort's items.
// sorted_g / sorted_u (or null): the prologue's width orders of the two matrices ([., 4] each).  item_pairs: 16 or 32,
// the most pairs an item of the sort holds (32: one decode of a weight tile serves up to 32 pairs, at more registers
// a thread - for calls with many pairs an expert); a pair's bits do not depend on it.  k2_all: 0, or the width that
// every k2_g and k2_u entry has (a promise: the launch may then use a kernel built for that width alone; a tensor of
// another width sets the status word and stores nothing); -1: the widths differ (a build of the kernel with short
// loops: blocks of different widths then share an SM's instruction cache).  col_tiles: 4 or 2, the 16-column tiles a block takes - 2
// doubles the blocks of a launch that would otherwise not fill the GPU (few experts in use; built for k2_all = 8 only);
// no result depends on it.
// (exl3/experts.cpp `grouped` + `gateup_epilogue`: src/tensorfold/cuda/exl3/experts_grouped.cuh:190-284,
// src/tensorfold/cuda/exl3/experts.cu:116-158)
extern "C" int tfb_exl3_gateup(const void* xg, const void* xu, const int64_t* tp_g, const int64_t* tp_u,
                               const int32_t* k2_g, const int32_t* k2_u, const int32_t* items, const int32_t* counts,
                               const int32_t* members, float* z, int32_t* arrive, const void* svh_g, const void* svh_u,
                               const void* suh_d, void* xd, int K, int N, int P, int cb, int max_items, float limit,
                               int act_mode, const int32_t* sorted_g, const int32_t* sorted_u, int item_pairs,
                               int k2_all, int col_tiles, void* stream) {
  TFB_REQUIRE((sorted_g == nullptr) == (sorted_u == nullptr) && aligned16(sorted_g) && aligned16(sorted_u),
              "exl3_gateup: the two width orders come together, 16-byte aligned");
  TFB_REQUIRE(xg && xu && tp_g && tp_u && k2_g && k2_u && items && counts && members && z && arrive && svh_g && svh_u &&
                  suh_d && xd,
              "exl3_gateup: null pointer");
  TFB_REQUIRE(act_mode == 0 || act_mode == 1, "exl3_gateup: act_mode 0 (bf16 roundings) or 1 (fp32)");
  TFB_REQUIRE(aligned16(z) && aligned16(svh_g) && aligned16(svh_u) && aligned16(suh_d) && aligned16(xd),
              "exl3_gateup: 16-byte aligned rows");
  exl3::GroupedArgs a = {};
  a.x[0] = static_cast<const __half*>(xg);
  a.x[1] = static_cast<const __half*>(xu);
  a.tp[0] = tp_g;
  a.tp[1] = tp_u;
  a.k2[0] = k2_g;
  a.k2[1] = k2_u;
  a.items = items;
  a.sorted[0] = sorted_g;
  a.sorted[1] = sorted_u;
  a.counts = counts;
  a.members = members;
  a.z = z;
  a.arrive = arrive;
  a.sv[0] = static_cast<const __half*>(svh_g);
  a.sv[1] = static_cast<const __half*>(svh_u);
  a.suh_next = static_cast<const __half*>(suh_d);
  a.out = xd;
  a.K = K;
  a.N = N;
  a.P = P;
  a.mats = 2;
  a.epi = exl3::GE_GATEUP;
  a.act_mode = act_mode;
  a.limit = limit;
  return exl3_grouped_launch("exl3_gateup", a, cb, max_items, item_pairs, k2_all, col_tiles, stream);
}

// y [P, N] fp32 = rotate(x [P, K] fp16 times W_q of each pair's expert) * svh of every routed pair (rows of other
// pairs are left as they are) - one launch; z: fp32 scratch [P, N]; the other arguments as tfb_exl3_gateup
// (sorted: the prologue's width order of the down matrices, or null).
// (exl3/experts.cpp `grouped` + `down_epilogue`: src/tensorfold/cuda/exl3/experts.cu:161-180)
extern "C" int tfb_exl3_down(const void* x, const int64_t* tp, const int32_t* k2, const int32_t* items,
                             const int32_t* counts, const int32_t* members, float* z, int32_t* arrive, const void* svh,
                             float* y, int K, int N, int P, int cb, int max_items, const int32_t* sorted,
                             int item_pairs, int k2_all, int col_tiles, void* stream) {
  TFB_REQUIRE(x && tp && k2 && items && counts && members && z && arrive && svh && y, "exl3_down: null pointer");
  TFB_REQUIRE(aligned16(sorted), "exl3_down: the width order must be 16-byte aligned");
  TFB_REQUIRE(aligned16(z) && aligned16(svh) && aligned16(y), "exl3_down: 16-byte aligned rows");
  exl3::GroupedArgs a = {};
  a.x[0] = a.x[1] = static_cast<const __half*>(x);
  a.tp[0] = a.tp[1] = tp;
  a.k2[0] = a.k2[1] = k2;
  a.items = items;
  a.sorted[0] = a.sorted[1] = sorted;
  a.counts = counts;
  a.members = members;
  a.z = z;
  a.arrive = arrive;
  a.sv[0] = a.sv[1] = static_cast<const __half*>(svh);
  a.suh_next = nullptr;
  a.out = y;
  a.K = K;
  a.N = N;
  a.P = P;
  a.mats = 1;
  a.epi = exl3::GE_DOWN;
  a.act_mode = 1;
  a.limit = 0.f;
  return exl3_grouped_launch("exl3_down", a, cb, max_items, item_pairs, k2_all, col_tiles, stream);
}

// out [M, N] (fp32: out_type 0, fp16: 1, bf16: 2; rows out_stride elements apart) = rotate(z) / sqrt(128) * svh + bias
// for every 128-column block of z [M, N] fp32 (bias fp16 [N] or null): the output side of an EXL3 product formed
// elsewhere (a dense GEMM over the decoded W_q for prompts).
// (src/tensorfold/cuda/exl3/prefill.py:15-44: the rotation epilogue of `_gemm`)
extern "C" int tfb_exl3_rot_out(const float* z, const void* svh, const void* bias, void* out, int64_t out_stride,
                                int out_type, int M, int N, void* stream) {
  TFB_REQUIRE(z && svh && out, "exl3_rot_out: null pointer");
  TFB_REQUIRE(N > 0 && N % 128 == 0 && out_stride >= N, "exl3_rot_out: N must be a multiple of 128, rows at least N apart");
  TFB_REQUIRE(out_type >= 0 && out_type <= 2, "exl3_rot_out: out_type 0 (fp32), 1 (fp16) or 2 (bf16)");
  TFB_REQUIRE(aligned16(z) && aligned16(svh) && aligned16(bias), "exl3_rot_out: 16-byte aligned rows");
  if (M <= 0) return TFB_OK;
  const int64_t units = (int64_t)M * (N / 128);
  const int64_t want = (units + 15) / 16;
  const dim3 grid((unsigned)(want < 8 * sm_count() ? want : 8 * sm_count()));
  auto st = static_cast<cudaStream_t>(stream);
  auto* sv = static_cast<const __half*>(svh);
  auto* bi = static_cast<const __half*>(bias);
  cudaError_t e;
  if (out_type == 0)
    e = launch(exl3_rot_out_kernel<float>, grid, dim3(256), 0, st, z, sv, bi, static_cast<float*>(out), out_stride, M, N);
  else if (out_type == 1)
    e = launch(exl3_rot_out_kernel<__half>, grid, dim3(256), 0, st, z, sv, bi, static_cast<__half*>(out), out_stride, M, N);
  else
    e = launch(exl3_rot_out_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, z, sv, bi, static_cast<__nv_bfloat16*>(out),
               out_stride, M, N);
  return check_cuda(e, "exl3_rot_out");
}
