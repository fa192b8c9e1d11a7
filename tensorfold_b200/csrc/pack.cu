// Load-time relayout of MLX affine 4-bit experts into the kernels' blocks, its inverse, and the dequantised weight
// values (the hook the bit-exactness checks use).  (src/tensorfold/cuda/experts.py:28-58, experts_pack.cu)

#include "api.h"
#include "common.cuh"

namespace tfb {

// One thread an output word of out [E, N/32, K/64, 288].
__global__ void __launch_bounds__(256)
pack_kernel(const uint32_t* __restrict__ words, const uint16_t* __restrict__ scales,
            const uint16_t* __restrict__ biases, uint32_t* __restrict__ out, int64_t total, int N, int K8, int KG,
            int NB) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  const int slot = (int)(i % BLOCK_WORDS);
  int64_t blk = i / BLOCK_WORDS;
  const int g = (int)(blk % KG);
  blk /= KG;
  const int b = (int)(blk % NB);
  const int64_t e = blk / NB;
  if (slot < 256) {
    const int tile = slot >> 7, lane = (slot & 127) >> 2, c4 = slot & 3;
    const int c = tile * 16 + (c4 >> 1) * 8 + (lane >> 2), j = 2 * (lane & 3) + (c4 & 1);
    out[i] = nib_shuffle(words[(e * N + b * COLS + c) * K8 + g * 8 + j]);
  } else {
    const int s = slot - 256;
    const int c = (s & 3) * 8 + (s >> 2);
    const int64_t at = (e * N + b * COLS + c) * KG + g;
    out[i] = (uint32_t)scales[at] | ((uint32_t)biases[at] << 16);
  }
}

// pack's inverse: one thread an MLX word, plus one a (scale, bias) pair.
__global__ void __launch_bounds__(256)
unpack_kernel(const uint32_t* __restrict__ blocks, uint32_t* __restrict__ words, uint16_t* __restrict__ scales,
              uint16_t* __restrict__ biases, int64_t nwords, int64_t nsb, int N, int K8, int KG, int NB) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i < nwords) {
    const int j8 = (int)(i % K8);
    const int64_t en = i / K8;
    const int n = (int)(en % N);
    const int64_t e = en / N;
    const int g = j8 >> 3, j = j8 & 7, b = n / COLS, c = n % COLS;
    const uint32_t* blk = blocks + ((e * NB + b) * KG + g) * BLOCK_WORDS;
    words[i] = nib_unshuffle(blk[word_slot(c, j)]);
  } else if (i < nwords + nsb) {
    const int64_t q = i - nwords;
    const int g = (int)(q % KG);
    const int64_t en = q / KG;
    const int n = (int)(en % N);
    const int64_t e = en / N;
    const int b = n / COLS, c = n % COLS;
    const uint32_t v = blocks[((e * NB + b) * KG + g) * BLOCK_WORDS + 256 + sb_slot(c)];
    scales[q] = (uint16_t)(v & 0xFFFFu);
    biases[q] = (uint16_t)(v >> 16);
  }
}

// The weight value the kernels multiply by.  mode 0 (decode form, and the CPU affine-row reference's
// src/tensorfold/kernels/qwen/dense/v1/affine_rows.py:64): fp32 fma(scale, q, bias).  mode 1 (prefill form,
// src/tensorfold/cuda/experts_prefill.cu:25-29): bf16 with one rounding for bf16 scales (a bf16 fma); for fp16
// scales the fp32 fma rounded to bf16.
template <int SB>
__device__ __forceinline__ __nv_bfloat16 prefill_weight(int q, uint32_t s_bits, uint32_t b_bits) {
  if constexpr (SB == SB_BF16) {
    const __nv_bfloat16 s = __ushort_as_bfloat16((unsigned short)s_bits), b = __ushort_as_bfloat16((unsigned short)b_bits);
    return __hfma(__int2bfloat16_rn(q), s, b);
  } else {
    return __float2bfloat16_rn(fmaf(sb_to_float<SB>(s_bits), (float)q, sb_to_float<SB>(b_bits)));
  }
}

template <int SB>
__global__ void __launch_bounds__(256)
dequant_kernel(const uint32_t* __restrict__ blocks, void* __restrict__ out, int mode, int64_t nwords, int N, int K8,
               int KG, int NB) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= nwords) return;
  const int j8 = (int)(i % K8);
  const int64_t en = i / K8;
  const int n = (int)(en % N);
  const int64_t e = en / N;
  const int g = j8 >> 3, j = j8 & 7, b = n / COLS, c = n % COLS;
  const uint32_t* blk = blocks + ((e * NB + b) * KG + g) * BLOCK_WORDS;
  const uint32_t w = nib_unshuffle(blk[word_slot(c, j)]);
  const uint32_t sbv = blk[256 + sb_slot(c)];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int q = (w >> (4 * k)) & 0xF;
    if (mode == 0) {
      static_cast<float*>(out)[i * 8 + k] = fmaf(sb_to_float<SB>(sbv & 0xFFFFu), (float)q, sb_to_float<SB>(sbv >> 16));
    } else {
      static_cast<__nv_bfloat16*>(out)[i * 8 + k] = prefill_weight<SB>(q, sbv & 0xFFFFu, sbv >> 16);
    }
  }
}

// Sums of each group of 64 inputs of a row, fp32: xs[m, g] (the quantity the matmuls fold the biases with;
// src/tensorfold/cuda/kernels/qmm.py:137-153).  One warp a (row, group): lane l adds inputs 2 l and 2 l + 1, then a
// butterfly 16..1 - one stated order.
__global__ void __launch_bounds__(128)
group_sums_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, float* __restrict__ xs, int M, int KG) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit < (int64_t)M * KG) {
    const int m = (int)(unit / KG), g = (int)(unit - (int64_t)m * KG);
    const uint32_t u = *reinterpret_cast<const uint32_t*>(x + (size_t)m * ldx + g * GS + 2 * lane);
    float v = bf16_lo(u) + bf16_hi(u);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) xs[unit] = v;
  }
  pdl_launch_dependents();
}

}  // namespace tfb

using namespace tfb;

static int check_shape(const char* who, int E, int N, int K, int gs) {
  TFB_REQUIRE(gs == GS, "%s: groups of %d inputs only, not %d", who, GS, gs);
  TFB_REQUIRE(E >= 1 && N >= COLS && K >= GS, "%s: bad shape E=%d N=%d K=%d", who, E, N, K);
  TFB_REQUIRE(N % COLS == 0 && K % GS == 0, "%s: N must be a multiple of %d and K of %d (N=%d, K=%d)", who, COLS, GS,
              N, K);
  return TFB_OK;
}

extern "C" int tfb_pack(const void* words, const void* scales, const void* biases, int gs, void* out, int E, int N,
                        int K, void* stream) {
  TFB_REQUIRE(words && scales && biases && out, "pack: null pointer");
  if (int rc = check_shape("pack", E, N, K, gs)) return rc;
  const int KG = K / GS, NB = N / COLS;
  const int64_t total = (int64_t)E * NB * KG * BLOCK_WORDS;
  pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(words), static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases),
      static_cast<uint32_t*>(out), total, N, K / 8, KG, NB);
  return check_launch("pack");
}

extern "C" int tfb_unpack(const void* blocks, int gs, void* words, void* scales, void* biases, int E, int N, int K,
                          void* stream) {
  TFB_REQUIRE(blocks && words && scales && biases, "unpack: null pointer");
  if (int rc = check_shape("unpack", E, N, K, gs)) return rc;
  const int KG = K / GS, NB = N / COLS;
  const int64_t nwords = (int64_t)E * N * (K / 8), nsb = (int64_t)E * N * KG;
  unpack_kernel<<<(unsigned)((nwords + nsb + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(blocks), static_cast<uint32_t*>(words), static_cast<uint16_t*>(scales),
      static_cast<uint16_t*>(biases), nwords, nsb, N, K / 8, KG, NB);
  return check_launch("unpack");
}

extern "C" int tfb_dequant(const void* blocks, int gs, int sb_type, int mode, void* out, int E, int N, int K,
                           void* stream) {
  TFB_REQUIRE(blocks && out, "dequant: null pointer");
  if (int rc = check_shape("dequant", E, N, K, gs)) return rc;
  TFB_REQUIRE(mode == 0 || mode == 1, "dequant: mode 0 (fp32 decode form) or 1 (bf16 prefill form), not %d", mode);
  TFB_REQUIRE(sb_type == SB_BF16 || sb_type == SB_FP16, "dequant: scales are bf16 (0) or fp16 (1), not %d", sb_type);
  const int KG = K / GS, NB = N / COLS;
  const int64_t nwords = (int64_t)E * N * (K / 8);
  const unsigned grid = (unsigned)((nwords + 255) / 256);
  auto st = static_cast<cudaStream_t>(stream);
  if (sb_type == SB_BF16)
    dequant_kernel<SB_BF16><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(blocks), out, mode, nwords, N, K / 8,
                                                  KG, NB);
  else
    dequant_kernel<SB_FP16><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(blocks), out, mode, nwords, N, K / 8,
                                                  KG, NB);
  return check_launch("dequant");
}

extern "C" int tfb_group_sums(const void* x, int64_t x_stride, float* xs, int M, int K, int gs, void* stream) {
  TFB_REQUIRE(x && xs, "group_sums: null pointer");
  TFB_REQUIRE(gs == GS && K > 0 && K % GS == 0 && x_stride >= K && x_stride % 2 == 0,
              "group_sums: groups of %d inputs, K a multiple of it", GS);
  TFB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 3u) == 0, "group_sums: x must be 4-byte aligned");
  if (M <= 0) return TFB_OK;
  const int64_t units = (int64_t)M * (K / GS);
  return check_cuda(launch(group_sums_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), 0,
                           static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), x_stride, xs, M,
                           K / GS),
                    "group_sums");
}
