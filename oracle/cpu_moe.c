/* TEST INFRASTRUCTURE, NOT PRODUCT: a CPU restatement of the reference's routed-expert MoE path in plain C.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may build, load or call
 * this file; the product (tensorfold_b200/) never does.  Every function names the reference lines it restates
 * (paths inside the bertholomus/TensorFold tree).
 *
 * Parity pins: the nibble extraction against the reference's own Metal header compiled as C++ (oracle/build_ref.py,
 * as tests/test_affine_rows.py:82-111 does), the plan against the semantics of tests/cuda/test_experts.py:107-134,
 * the routing indices against sorted(key = (-logit, id)) as tests/cuda/test_flashnext_kernels.py:119-122.
 */

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) { /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

static inline float fp16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int shift = 0;
      while (!(man & 0x400u)) {
        man <<= 1;
        ++shift;
      }
      man &= 0x3FFu;
      u = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7F800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline float sb_to_f32(uint16_t v, int sb_type) { return sb_type ? fp16_to_f32(v) : bf16_to_f32(v); }

/* code i of a row of 4-bit codes held little-endian in 32-bit words.
 * Restates code_at<4> of src/tensorfold/kernels/qwen/dense/v1/affine_rows.py:14-21. */
static inline uint32_t code_at4(const uint32_t* w, int i) { return (w[i >> 3] >> ((i & 7) * 4)) & 0xFu; }

uint32_t tfo_code_at(const uint32_t* words, int index, int bits) {
  const int bit = index * bits, word = bit >> 5, shift = bit & 31;
  uint32_t v = words[word] >> shift;
  if (shift + bits > 32) v |= words[word + 1] << (32 - shift);
  return v & ((1u << bits) - 1u);
}

/* ---------------------------------------------------------------------------------------------------------------
 * Router logits (src/tensorfold/cuda/moe.py:23-55: fp32 x . w over bf16 inputs).  The reference leaves the summation
 * order to Triton; this restatement and the CUDA kernel share one stated order: lane l of 32 walks
 * k = 256 c + 8 l + j (c ascending, j = 0..7) with acc = fma(x, w, acc); the 32 lane sums meet in a butterfly
 * (xor 16, 8, 4, 2, 1).
 * ------------------------------------------------------------------------------------------------------------- */
void tfo_router_logits(const uint16_t* x, int64_t x_stride, const uint16_t* w, float* out, int T, int D, int NE) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int r = 0; r < T; ++r)
    for (int e = 0; e < NE; ++e) {
      float lane[32];
      for (int l = 0; l < 32; ++l) {
        float acc = 0.f;
        for (int k = 8 * l; k < D; k += 256)
          for (int j = 0; j < 8; ++j)
            acc = fmaf(bf16_to_f32(x[(int64_t)r * x_stride + k + j]), bf16_to_f32(w[(int64_t)e * D + k + j]), acc);
        lane[l] = acc;
      }
      for (int m = 16; m >= 1; m >>= 1) {
        float nxt[32];
        for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ m];
        memcpy(lane, nxt, sizeof lane);
      }
      out[(int64_t)r * NE + e] = lane[0];
    }
}

/* ---------------------------------------------------------------------------------------------------------------
 * Top-k rows (src/tensorfold/cuda/moe.py:58-85): k rounds of (max, lowest index among equals, exp(m - top)),
 * weights bf16(ex / total); with a shared expert, slot k = id E, weight bf16(sigmoid(bf16(logit E))).
 * ------------------------------------------------------------------------------------------------------------- */
void tfo_topk_rows(const float* L, int NL, int32_t* pick, float* wts, int T, int E, int top_k, int shared) {
  const int slots = top_k + (shared ? 1 : 0);
#pragma omp parallel for schedule(static)
  for (int r = 0; r < T; ++r) {
    float* v = (float*)malloc(sizeof(float) * (size_t)E);
    float ex[64];
    memcpy(v, L + (int64_t)r * NL, sizeof(float) * (size_t)E);
    float top = -INFINITY, total = 0.f;
    for (int e = 0; e < E; ++e)
      if (v[e] > top) top = v[e];
    for (int k = 0; k < top_k; ++k) {
      float m = -INFINITY;
      int idx = 0;
      for (int e = 0; e < E; ++e)
        if (v[e] > m) {
          m = v[e];
          idx = e;
        }
      ex[k] = expf(m - top);
      total += ex[k];
      pick[(int64_t)r * slots + k] = idx;
      v[idx] = -INFINITY;
    }
    for (int k = 0; k < top_k; ++k) wts[(int64_t)r * slots + k] = round_bf16(ex[k] / total);
    if (shared) {
      const float sg = round_bf16(L[(int64_t)r * NL + E]);
      pick[(int64_t)r * slots + top_k] = E;
      wts[(int64_t)r * slots + top_k] = round_bf16(1.f / (1.f + expf(-sg)));
    }
    free(v);
  }
}

/* ---------------------------------------------------------------------------------------------------------------
 * Plan (src/tensorfold/cuda/experts.cu:157-285; golden semantics tests/cuda/test_experts.py:107-115): experts
 * ascending, an expert's pairs ascending, items of <= tile pairs.  Returns the item count.
 * ------------------------------------------------------------------------------------------------------------- */
int tfo_plan(const int32_t* picks, int P, int E, int tile, int32_t* members, int32_t* items, int32_t* counts) {
  int* cnt = (int*)calloc((size_t)E + 1, sizeof(int));
  for (int p = 0; p < P; ++p)
    if (picks[p] >= 0 && picks[p] < E) cnt[picks[p]]++;
  int* off = (int*)malloc(sizeof(int) * ((size_t)E + 1));
  int total = 0, n_items = 0, distinct = 0;
  for (int e = 0; e < E; ++e) {
    off[e] = total;
    for (int j = 0; j < cnt[e]; j += tile) {
      items[3 * n_items] = e;
      items[3 * n_items + 1] = total + j;
      items[3 * n_items + 2] = cnt[e] - j < tile ? cnt[e] - j : tile;
      ++n_items;
    }
    distinct += cnt[e] > 0;
    total += cnt[e];
  }
  for (int p = 0; p < P; ++p)
    if (picks[p] >= 0 && picks[p] < E) members[off[picks[p]]++] = p;
  counts[0] = n_items;
  counts[1] = distinct;
  free(cnt);
  free(off);
  return n_items;
}

/* ---------------------------------------------------------------------------------------------------------------
 * The CPU affine-row kernel: restates the shader body of src/tensorfold/kernels/qwen/dense/v1/affine_rows.py:26-94
 * for 4-bit codes.  Lane l of 32 takes the 32-code blocks l, l + 32, ... of an output row; each code is dequantised
 * once, w = fma(scale, q, bias) (:64), and folded into the row's own chain acc = fma(x, w, acc) (:79) in code
 * order; the 32 lane partials are then summed (simd_sum, :89 - Metal does not state its order; a butterfly
 * xor 16..1 is used here).  `wrow` holds the dequantised row so several input rows share one dequantisation, as the
 * shader's RT rows do.
 * ------------------------------------------------------------------------------------------------------------- */
static void dequant_row(const uint32_t* words, const uint16_t* scales, const uint16_t* biases, int sb_type, int K,
                        int gs, float* wrow) {
  for (int g = 0; g < K / gs; ++g) {
    const float s = sb_to_f32(scales[g], sb_type), b = sb_to_f32(biases[g], sb_type);
    for (int i = 0; i < gs; ++i) wrow[g * gs + i] = fmaf(s, (float)code_at4(words, g * gs + i), b);
  }
}

static float row_dot(const float* x, const float* wrow, int K) {
  const int blocks = K / 32;
  float lane[32];
  for (int l = 0; l < 32; ++l) {
    float acc = 0.f;
    for (int b = l; b < blocks; b += 32)
      for (int i = 0; i < 32; ++i) acc = fmaf(x[b * 32 + i], wrow[b * 32 + i], acc);
    lane[l] = acc;
  }
  for (int m = 16; m >= 1; m >>= 1) {
    float nxt[32];
    for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ m];
    memcpy(lane, nxt, sizeof lane);
  }
  return lane[0];
}

/* out[r, n] = x[r, :] . W[n, :] for R rows; out_bf16 != 0 rounds to bf16 as the shader's store does (:90). */
void tfo_affine_rows(const uint16_t* x, int R, const uint32_t* words, const uint16_t* scales, const uint16_t* biases,
                     int sb_type, int N, int K, int gs, float* out, int out_bf16) {
  float* xf = (float*)malloc(sizeof(float) * (size_t)R * K);
  for (int64_t i = 0; i < (int64_t)R * K; ++i) xf[i] = bf16_to_f32(x[i]);
#pragma omp parallel
  {
    float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
    for (int n = 0; n < N; ++n) {
      dequant_row(words + (int64_t)n * (K / 8), scales + (int64_t)n * (K / gs), biases + (int64_t)n * (K / gs),
                  sb_type, K, gs, wrow);
      for (int r = 0; r < R; ++r) {
        const float v = row_dot(xf + (int64_t)r * K, wrow, K);
        out[(int64_t)r * N + n] = out_bf16 ? round_bf16(v) : v;
      }
    }
    free(wrow);
  }
  free(xf);
}

/* Dequantised weights [N, K]: mode 0 fp32 fma(scale, q, bias) (affine_rows.py:64; the decode form of
 * src/tensorfold/cuda/experts.cu:94-106 applies the same scale and bias per group); mode 1 the prefill form's bf16
 * weight, src/tensorfold/cuda/experts_prefill.cu:25-29: for bf16 scales one rounding of the exact q * s + b (a bf16
 * fma), for fp16 scales the fp32 fma rounded to bf16.  Written as fp32 values either way. */
void tfo_dequant(const uint32_t* words, const uint16_t* scales, const uint16_t* biases, int sb_type, int64_t rows,
                 int K, int gs, int mode, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < rows; ++n)
    for (int k = 0; k < K; ++k) {
      const float s = sb_to_f32(scales[n * (K / gs) + k / gs], sb_type);
      const float b = sb_to_f32(biases[n * (K / gs) + k / gs], sb_type);
      const float q = (float)code_at4(words + n * (K / 8), k);
      float v;
      if (mode == 0) {
        v = fmaf(s, q, b);
      } else if (sb_type == 0) {
        /* exact in double (12-bit product, short addend), then one rounding to bf16's 8 significant bits */
        const double exact = (double)s * (double)q + (double)b;
        int ex;
        const double m = frexp(exact, &ex);
        v = (float)ldexp(nearbyint(m * 256.0), ex - 8);
      } else {
        v = round_bf16(fmaf(s, q, b));
      }
      out[n * K + k] = v;
    }
}

/* SwiGLU with the families' roundings (src/tensorfold/cuda/experts.cuh:57-65). */
static inline float swiglu(float g, float u, float limit) {
  float gv = round_bf16(g), uv = round_bf16(u);
  if (limit > 0.f) {
    gv = fminf(gv, limit);
    uv = fminf(fmaxf(uv, -limit), limit);
  }
  return round_bf16(round_bf16(gv / (1.f + expf(-gv))) * uv);
}

typedef struct {
  const uint32_t* words; /* [E, N, K/8] */
  const uint16_t* scales; /* [E, N, K/gs] */
  const uint16_t* biases;
} tfo_matrix;

/* ---------------------------------------------------------------------------------------------------------------
 * One MoE layer on the CPU: router -> top-k -> plan -> per expert gate/up rows -> SwiGLU -> down rows -> combine.
 * Orchestration of src/tensorfold/cuda/moe.py:119-128,131-151,176-186 with the affine-row kernel above as the
 * matmul.  act is bf16 (experts.cuh:57-65), y stays fp32 as the decode form's (experts.py:141-150), the combine is an
 * fp32 fma chain in slot order rounded once to bf16 (moe.py:131-142).  pick_out / wts_out / act_out / y_out may be
 * NULL.  Returns 0, or -1 when memory runs out.
 * ------------------------------------------------------------------------------------------------------------- */
int tfo_moe_layer(const uint16_t* x, int T, int D, const uint16_t* router_rows, int E, int top_k, int shared,
                  tfo_matrix gate, tfo_matrix up, tfo_matrix down, int NI, int gs, int sb_type, float limit,
                  uint16_t* out, int32_t* pick_out, float* wts_out, uint16_t* act_out, float* y_out) {
  const int NE = E + (shared ? 1 : 0), slots = top_k + (shared ? 1 : 0), P = T * slots;
  float* logits = (float*)malloc(sizeof(float) * (size_t)T * NE);
  int32_t* pick = (int32_t*)malloc(sizeof(int32_t) * (size_t)P);
  float* wts = (float*)malloc(sizeof(float) * (size_t)P);
  int32_t* members = (int32_t*)malloc(sizeof(int32_t) * (size_t)P);
  int32_t* items = (int32_t*)malloc(sizeof(int32_t) * 3 * ((size_t)P + NE));
  int32_t counts[2];
  float* xf = (float*)malloc(sizeof(float) * (size_t)T * D);
  float* act = (float*)malloc(sizeof(float) * (size_t)P * NI);
  float* y = (float*)malloc(sizeof(float) * (size_t)P * D);
  if (!logits || !pick || !wts || !members || !items || !xf || !act || !y) return -1;
  for (int64_t i = 0; i < (int64_t)T * D; ++i) xf[i] = bf16_to_f32(x[i]);
  tfo_router_logits(x, D, router_rows, logits, T, D, NE);
  tfo_topk_rows(logits, NE, pick, wts, T, E, top_k, shared);
  const int n_items = tfo_plan(pick, P, NE, P > 0 ? P : 1, members, items, counts); /* one item an expert */
#pragma omp parallel
  {
    float* wg = (float*)malloc(sizeof(float) * (size_t)(D > NI ? D : NI));
    float* wu = (float*)malloc(sizeof(float) * (size_t)D);
    /* gate and up: one (expert, column) at a time, every pair of the expert against the same dequantised rows */
#pragma omp for collapse(2) schedule(dynamic, 16)
    for (int it = 0; it < n_items; ++it)
      for (int n = 0; n < NI; ++n) {
        const int e = items[3 * it], first = items[3 * it + 1], cnt = items[3 * it + 2];
        const int64_t row = (int64_t)e * NI + n;
        dequant_row(gate.words + row * (D / 8), gate.scales + row * (D / gs), gate.biases + row * (D / gs), sb_type, D,
                    gs, wg);
        dequant_row(up.words + row * (D / 8), up.scales + row * (D / gs), up.biases + row * (D / gs), sb_type, D, gs,
                    wu);
        for (int i = 0; i < cnt; ++i) {
          const int p = members[first + i];
          const float* xr = xf + (int64_t)(p / slots) * D;
          act[(int64_t)p * NI + n] = swiglu(row_dot(xr, wg, D), row_dot(xr, wu, D), limit);
        }
      }
#pragma omp for collapse(2) schedule(dynamic, 16)
    for (int it = 0; it < n_items; ++it)
      for (int n = 0; n < D; ++n) {
        const int e = items[3 * it], first = items[3 * it + 1], cnt = items[3 * it + 2];
        const int64_t row = (int64_t)e * D + n;
        dequant_row(down.words + row * (NI / 8), down.scales + row * (NI / gs), down.biases + row * (NI / gs), sb_type,
                    NI, gs, wg);
        for (int i = 0; i < cnt; ++i) {
          const int p = members[first + i];
          y[(int64_t)p * D + n] = row_dot(act + (int64_t)p * NI, wg, NI);
        }
      }
    free(wg);
    free(wu);
  }
#pragma omp parallel for schedule(static)
  for (int r = 0; r < T; ++r)
    for (int d = 0; d < D; ++d) {
      float acc = 0.f;
      for (int s = 0; s < slots; ++s) acc = fmaf(wts[r * slots + s], y[((int64_t)r * slots + s) * D + d], acc);
      out[(int64_t)r * D + d] = f32_to_bf16(acc);
    }
  if (pick_out) memcpy(pick_out, pick, sizeof(int32_t) * (size_t)P);
  if (wts_out) memcpy(wts_out, wts, sizeof(float) * (size_t)P);
  if (act_out)
    for (int64_t i = 0; i < (int64_t)P * NI; ++i) act_out[i] = f32_to_bf16(act[i]);
  if (y_out) memcpy(y_out, y, sizeof(float) * (size_t)P * D);
  free(logits); free(pick); free(wts); free(members); free(items); free(xf); free(act); free(y);
  return 0;
}

int tfo_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void tfo_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
