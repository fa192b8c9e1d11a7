/* TEST INFRASTRUCTURE, NOT PRODUCT: a CPU restatement in plain C of the reference's EXL3 routed-expert path, used to
 * time that path on the host cores (bench.py's CPU-baseline legs) and checked against the numpy restatement
 * (oracle/exl3.py, itself pinned to the reference's format.py by tests/golden/).
 *
 * Follows src/tensorfold/cuda/exl3/format.py of the bertholomus/TensorFold tree: codebooks :31-48, window ends
 * :58-66, tile positions :69-77, states :95-116, unpack :119-132, rotation and layer :145-180; the routed wrapper is
 * the `_reference` of tests/cuda/test_exl3_experts.py:137-161 (SwiGLU between the projections, weighted sum over the
 * slots).  Arithmetic: weights exact fp16 values, everything else fp32.
 */

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float half_bits_to_f32(uint16_t h) {
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

/* double -> fp16 bits, round to nearest even, one rounding (finite inputs inside the fp16 range) */
static inline uint16_t f64_to_half_bits(double v) {
  const uint16_t sign = v < 0 || (v == 0 && 1.0 / v < 0) ? 0x8000u : 0;
  double a = fabs(v);
  if (a == 0) return sign;
  int e;
  double m = frexp(a, &e); /* a = m * 2^e, m in [0.5, 1) */
  int exp = e - 1;         /* a = (2 m) * 2^exp, 2 m in [1, 2) */
  if (exp < -14) {         /* subnormal: units of 2^-24 */
    const double q = nearbyint(ldexp(a, 24));
    return (uint16_t)(sign | (uint16_t)q); /* q == 1024 rolls into the smallest normal */
  }
  double frac = nearbyint(ldexp(2.0 * m - 1.0, 10)); /* 0 .. 1024, ties to even under the default rounding mode */
  if (frac == 1024.0) {
    frac = 0;
    ++exp;
  }
  if (exp > 15) return (uint16_t)(sign | 0x7C00u);
  return (uint16_t)(sign | ((uint16_t)(exp + 15) << 10) | (uint16_t)frac);
}

/* format.py:31-48 - the fp16 value (as bits) of a 16-bit state */
static inline uint16_t codebook_bits(uint32_t s, int cb) {
  if (cb == 2) {
    const uint32_t x = s * 0x83DCD12Du;
    const uint32_t h = 1024u + (x & 255u) + ((x >> 8) & 255u) + ((x >> 16) & 255u) + (x >> 24);
    return f64_to_half_bits((double)h * (double)half_bits_to_f32(0x1EEE) + (double)half_bits_to_f32(0xC931));
  }
  uint32_t x = cb == 1 ? s * 0xCBAC1FEDu : s * 89226354u + 64248484u;
  x = (x & 0x8FFF8FFFu) ^ 0x3B603B60u;
  return f64_to_half_bits((double)half_bits_to_f32((uint16_t)(x & 0xFFFFu)) + (double)half_bits_to_f32((uint16_t)(x >> 16)));
}

/* format.py:58-66 - one past the last stream bit of value p's window */
static inline int window_end(int p, int k2) { return (p >> 1) * k2 + ((p & 1) ? k2 : (k2 >> 1)); }

/* One 16 x 16 tile (4 * k2 little-endian 32-bit words, an MSB-first circular bit stream) into fp16 bits, tile[k][n]. */
static void decode_tile(const uint16_t* t16, int k2, const uint16_t* table, uint16_t tile[16][16]) {
  const int tw = 4 * k2;
  uint32_t w[64];
  for (int i = 0; i < tw; ++i) w[i] = (uint32_t)t16[2 * i] | ((uint32_t)t16[2 * i + 1] << 16);
  for (int p = 0; p < 256; ++p) {
    const int first = window_end(p, k2) - 16 + 32 * tw;
    const int i0 = (first / 32) % tw, off = first % 32;
    const uint64_t pair = ((uint64_t)w[i0] << 32) | (uint64_t)w[(i0 + 1) % tw];
    const uint32_t s = (uint32_t)((pair >> (48 - off)) & 0xFFFFu);
    const int lane = p >> 3, j = p & 7; /* format.py:69-77 */
    const int row = 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1), col = (lane >> 2) + 8 * (j >> 2);
    tile[row][col] = table[s];
  }
}

static uint16_t* g_tables[3] = {0, 0, 0};

static const uint16_t* table_of(int cb) {
  uint16_t* t = g_tables[cb];
  if (t) return t;
#pragma omp critical(tfo_exl3_table)
  {
    if (!g_tables[cb]) {
      uint16_t* n = (uint16_t*)malloc(65536 * sizeof(uint16_t));
      for (uint32_t s = 0; s < 65536u; ++s) n[s] = codebook_bits(s, cb);
      g_tables[cb] = n;
    }
  }
  return g_tables[cb];
}

/* W_q [K, N] as fp16 bits from a trellis int16 [K/16, N/16, 8 * k2] (format.py:119-132). */
void tfo_exl3_unpack(const uint16_t* trellis, int K, int N, int k2, int cb, uint16_t* out) {
  const uint16_t* table = table_of(cb);
  const int kt_n = K / 16, nt_n = N / 16;
#pragma omp parallel for collapse(2) schedule(static)
  for (int kt = 0; kt < kt_n; ++kt)
    for (int nt = 0; nt < nt_n; ++nt) {
      uint16_t tile[16][16];
      decode_tile(trellis + ((size_t)kt * nt_n + nt) * 8 * k2, k2, table, tile);
      for (int r = 0; r < 16; ++r)
        for (int c = 0; c < 16; ++c) out[(size_t)(kt * 16 + r) * N + nt * 16 + c] = tile[r][c];
    }
}

/* format.py:145-172 - the 128-point Hadamard transform / sqrt(128) on every block of 128, in place */
static void rotate128(float* v, int n) {
  for (int b = 0; b < n; b += 128) {
    float* x = v + b;
    for (int h = 1; h < 128; h <<= 1)
      for (int i = 0; i < 128; i += 2 * h)
        for (int j = i; j < i + h; ++j) {
          const float a = x[j], c = x[j + h];
          x[j] = a + c;
          x[j + h] = a - c;
        }
    for (int i = 0; i < 128; ++i) x[i] *= 0.08838834764831845f;
  }
}

/* z [m, N] += xr [m, K] . W_q, the tiles decoded once for all m rows */
static void matmul_rows(const float* xr, int m, const uint16_t* trellis, int K, int N, int k2, const uint16_t* table,
                        float* z) {
  const int kt_n = K / 16, nt_n = N / 16;
  memset(z, 0, (size_t)m * N * sizeof(float));
  for (int kt = 0; kt < kt_n; ++kt)
    for (int nt = 0; nt < nt_n; ++nt) {
      uint16_t tile[16][16];
      float w[16][16];
      decode_tile(trellis + ((size_t)kt * nt_n + nt) * 8 * k2, k2, table, tile);
      for (int r = 0; r < 16; ++r)
        for (int c = 0; c < 16; ++c) w[r][c] = half_bits_to_f32(tile[r][c]);
      for (int i = 0; i < m; ++i) {
        const float* x = xr + (size_t)i * K + kt * 16;
        float* o = z + (size_t)i * N + nt * 16;
        for (int r = 0; r < 16; ++r)
          for (int c = 0; c < 16; ++c) o[c] += x[r] * w[r][c];
      }
    }
}

typedef struct {
  const uint16_t* const* trellis; /* [E] */
  const int32_t* k2;              /* [E] */
  const uint16_t* const* suh;     /* [E] fp16 bits [K] */
  const uint16_t* const* svh;     /* [E] fp16 bits [N] */
} Exl3Matrices;

/* y [m, N] = rot(rot(x * suh) W_q) * svh (format.py:174-180) for the m rows of one expert */
static void linear_rows(const float* x, int m, const Exl3Matrices* mats, int e, int K, int N, const uint16_t* table,
                        float* xr, float* y) {
  for (int i = 0; i < m; ++i) {
    for (int k = 0; k < K; ++k) xr[(size_t)i * K + k] = x[(size_t)i * K + k] * half_bits_to_f32(mats->suh[e][k]);
    rotate128(xr + (size_t)i * K, K);
  }
  matmul_rows(xr, m, mats->trellis[e], K, N, mats->k2[e], table, y);
  for (int i = 0; i < m; ++i) {
    rotate128(y + (size_t)i * N, N);
    for (int n = 0; n < N; ++n) y[(size_t)i * N + n] *= half_bits_to_f32(mats->svh[e][n]);
  }
}

/* out [R, D] fp32 = sum over slots of wts * down_e(silu(gate_e(x)) * up_e(x)); picks outside [0, E) are skipped.
 * Experts in parallel (each decodes its three matrices once for all its rows); per-pair rows are added to `out` in
 * slot order afterwards, so the result does not depend on the thread count.  Returns 0, or -1 when out of memory. */
int tfo_exl3_routed(const float* x, const int32_t* pick, const float* wts, int R, int slots, int E, int D, int NI,
                    Exl3Matrices gate, Exl3Matrices up, Exl3Matrices down, int cb, float* out) {
  const uint16_t* table = table_of(cb);
  const int P = R * slots;
  float* ypair = (float*)calloc((size_t)P * D, sizeof(float));
  if (!ypair) return -1;
  int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int e = 0; e < E; ++e) {
    int m = 0;
    for (int p = 0; p < P; ++p) m += pick[p] == e;
    if (m == 0) continue;
    const int wide = D > NI ? D : NI;
    int* ids = (int*)malloc((size_t)m * sizeof(int));
    float* xs = (float*)malloc((size_t)m * wide * sizeof(float));
    float* xr = (float*)malloc((size_t)m * wide * sizeof(float));
    float* g = (float*)malloc((size_t)m * NI * sizeof(float));
    float* u = (float*)malloc((size_t)m * NI * sizeof(float));
    float* y = (float*)malloc((size_t)m * D * sizeof(float));
    if (!ids || !xs || !xr || !g || !u || !y) {
#pragma omp atomic write
      failed = 1;
    } else {
      int i = 0;
      for (int p = 0; p < P; ++p)
        if (pick[p] == e) {
          memcpy(xs + (size_t)i * D, x + (size_t)(p / slots) * D, (size_t)D * sizeof(float));
          ids[i++] = p;
        }
      linear_rows(xs, m, &gate, e, D, NI, table, xr, g);
      linear_rows(xs, m, &up, e, D, NI, table, xr, u);
      for (size_t q = 0; q < (size_t)m * NI; ++q) g[q] = g[q] / (1.0f + expf(-g[q])) * u[q];
      linear_rows(g, m, &down, e, NI, D, table, xr, y);
      for (i = 0; i < m; ++i) memcpy(ypair + (size_t)ids[i] * D, y + (size_t)i * D, (size_t)D * sizeof(float));
    }
    free(ids);
    free(xs);
    free(xr);
    free(g);
    free(u);
    free(y);
  }
  if (!failed) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < R; ++r) {
      float* o = out + (size_t)r * D;
      memset(o, 0, (size_t)D * sizeof(float));
      for (int s = 0; s < slots; ++s) {
        const int e = pick[r * slots + s];
        if (e < 0 || e >= E) continue;
        const float w = wts[r * slots + s];
        const float* yp = ypair + (size_t)(r * slots + s) * D;
        for (int d = 0; d < D; ++d) o[d] += w * yp[d];
      }
    }
  }
  free(ypair);
  return failed ? -1 : 0;
}
