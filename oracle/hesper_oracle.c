/*
 * hesper_oracle.c -- CPU restatement of Hesper's quantized-inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker and the timed CPU
 * baseline for the CUDA library; nothing in the shipped library links, loads or
 * calls it.  It restates, in plain C, the arithmetic the reference defines in
 * its Lean sources (the reference itself needs the Lean 4 toolchain and cannot
 * be compiled where this is built).  Every function cites the reference file
 * and lines it follows, as paths inside the Verilean/hesper repository.
 *
 * Pinning status:
 *   - i2_s decode/pack, BitLinear forward:   pinned by the reference's own
 *     known-answer tests (all-+1 KAT, code table, xorshift32 equivalence cases).
 *   - attention:                             pinned by the reference's literal
 *     2-head/3-position fixture and its online == three-step equivalence check.
 *   - int8 activation quantiser:             rule taken from the reference's
 *     Q8_1 quantiser; the reference holds no asserted vector for it
 *     (parity unpinned for the quantiser itself).
 *   - Q4_K / Q8_0 absolute values:           parity unpinned -- the formats come
 *     from ggml/llama.cpp, which the reference neither vendors nor pins; the
 *     restatement follows the format description in the reference's Lean files.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fopenmp -shared).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Host info                                                                  */
/* ------------------------------------------------------------------------- */

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* IEEE binary16 <-> binary32 (round-to-nearest-even), no hardware dependence */
/* ------------------------------------------------------------------------- */

/* f16 -> f32, exact.  Same value table as the arithmetic conversion in
 * Hesper/Quantization/Q4_K_M.lean:84-102 (normals, subnormals). */
ORC_API float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  uint32_t e = (h >> 10) & 0x1F;
  uint32_t m = h & 0x3FF;
  uint32_t bits;
  if (e == 0) {
    if (m == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int sh = 0;
      while (!(m & 0x400)) { m <<= 1; ++sh; }
      m &= 0x3FF;
      bits = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | (m << 13);
    }
  } else if (e == 31) {
    bits = sign | 0x7F800000u | (m << 13);
  } else {
    bits = sign | ((e + 127 - 15) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* f32 -> f16 with IEEE round-to-nearest-even (what cvt.rn.f16.f32 does).  The
 * reference's KV writers pack f32 -> f16 RN (Hesper/Layers/Attention.lean:701-979). */
ORC_API uint16_t orc_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7FFFFFFFu;
  if (ax >= 0x7F800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0));
  }
  if (ax >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (ax < 0x33000001u) { /* < 2^-25 (or exactly 2^-25 -> ties to even -> 0) */
    return (uint16_t)sign;
  }
  int e = (int)(ax >> 23) - 127;
  uint32_t m = (ax & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
  int shift;
  uint32_t he;
  if (e < -14) { /* subnormal half */
    shift = 13 + (-14 - e);
    he = 0;
  } else {
    shift = 13;
    he = (uint32_t)(e + 15);
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  uint32_t out;
  if (he == 0) {
    out = q; /* may carry into exponent 1: correct */
  } else {
    out = ((he - 1) << 10) + q; /* q includes the implicit bit (0x400) */
  }
  return (uint16_t)(sign | out);
}

/* bf16 helpers (embedding / LM-head table dtype of the BitNet-shaped model). */
ORC_API float orc_bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

ORC_API uint16_t orc_f32_to_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7FFFu + lsb;
  return (uint16_t)(x >> 16);
}

/* ------------------------------------------------------------------------- */
/* Seeded generators used by the reference's own tests                        */
/* ------------------------------------------------------------------------- */

/* xorshift32 step: Tests/BitLinearEquivalence.lean:49-59. */
static inline uint32_t xs32(uint32_t *s) {
  uint32_t x = *s;
  x ^= x << 13;
  x ^= x >> 17;
  x ^= x << 5;
  *s = x;
  return x;
}

/* One BitLinear equivalence case exactly as genCase builds it
 * (Tests/BitLinearEquivalence.lean:79-93): K*N ternary draws (u % 3 -> -1,0,+1),
 * then M*K floats u/2^32*2-1, then the scale u/2^32*0.1+0.01. */
ORC_API void orc_gen_bitlinear_case(uint32_t seed, int K, int N, int M,
                                    int8_t *ternary, float *x, float *scale) {
  uint32_t s = seed;
  for (long i = 0; i < (long)K * N; ++i) {
    uint32_t u = xs32(&s);
    ternary[i] = (int8_t)((int)(u % 3u) - 1);
  }
  for (long i = 0; i < (long)M * K; ++i) {
    uint32_t u = xs32(&s);
    x[i] = (float)(((double)u / 4294967296.0) * 2.0 - 1.0);
  }
  uint32_t u = xs32(&s);
  *scale = (float)(((double)u / 4294967296.0) * 0.1 + 0.01);
}

/* LCG array generator of Tests/CUDA/CUDAFlashAttnGoldenTest.lean:60-77:
 * s <- (s*1103515245 + 12345) mod 2^31, value s/2^31*2-1 snapped to f32.
 * Returns the state after n draws so arrays chain as the test chains them. */
ORC_API uint64_t orc_lcg_fill(uint64_t seed, long n, float *out) {
  uint64_t s = seed;
  for (long i = 0; i < n; ++i) {
    s = (s * 1103515245ull + 12345ull) % 2147483648ull;
    out[i] = (float)(((double)s / 2147483648.0) * 2.0 - 1.0);
  }
  return s;
}

/* ------------------------------------------------------------------------- */
/* i2_s ternary format                                                         */
/* ------------------------------------------------------------------------- */

/* Hesper/Layers/BitLinearSpec.lean:43-60 (decodeI2S): element `col` of the row
 * starting at `row_start` -> -1, 0, +1 (code 3 decodes to +2 by the formula). */
ORC_API int orc_i2s_decode(const uint8_t *packed, long nbytes, long row_start,
                           int col) {
  int group128 = col / 128;
  int c = col % 128;
  int byte_pos = c % 32;
  int shift_idx = c / 32;
  long off = row_start + (long)group128 * 32 + byte_pos;
  if (off >= nbytes) return 0;
  int shift = 6 - 2 * shift_idx;
  return (int)((packed[off] >> shift) & 3) - 1;
}

/* Hesper/Layers/BitLinearSpec.lean:120-143 (packI2S): -1/0/+1 -> codes 0/1/2. */
ORC_API void orc_i2s_pack(const int8_t *ternary, int K, int N, uint8_t *packed) {
  long bpr = K / 4;
  memset(packed, 0, (size_t)(bpr * N));
  for (int i = 0; i < N; ++i) {
    for (int j = 0; j < K; ++j) {
      int t = ternary[(long)i * K + j];
      uint8_t code = (t == -1) ? 0 : (t == 0 ? 1 : 2);
      int c = j % 128;
      long off = (long)i * bpr + (long)(j / 128) * 32 + (c % 32);
      int shift = 6 - 2 * (c / 32);
      packed[off] = (uint8_t)((packed[off] & ~(3u << shift)) | (code << shift));
    }
  }
}

/* Hesper/Layers/BitLinearSpec.lean:65-91 (forwardRow / forward):
 * y[m,n] = scale * sum_k w[n,k]*x[m,k], k ascending, scale applied last, all in
 * double as Lean's Float is binary64.  x is given as f32 and widened. */
ORC_API void orc_bitlinear_spec(const uint8_t *packed, float scale, int K, int N,
                                int M, const float *x, double *y) {
  long bpr = K / 4;
  long nbytes = bpr * N;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    for (int m = 0; m < M; ++m) {
      double acc = 0.0;
      for (int k = 0; k < K; ++k) {
        int w = orc_i2s_decode(packed, nbytes, (long)n * bpr, k);
        acc = acc + (double)w * (double)x[(long)m * K + k];
      }
      y[(long)m * N + n] = (double)scale * acc;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* RMSNorm and the per-token int8 activation quantiser                        */
/* ------------------------------------------------------------------------- */

/* Hesper/Training/VerifiedBackward.lean:95-99 (rmsNormForward), in double:
 * y = x / sqrt(mean(x^2) + eps) * gamma. */
ORC_API void orc_rmsnorm_f64(const float *x, const float *gamma, int K, double eps,
                             double *y) {
  double ss = 0.0;
  for (int k = 0; k < K; ++k) ss += (double)x[k] * (double)x[k];
  double rms = sqrt(ss / (double)K + eps);
  for (int k = 0; k < K; ++k) y[k] = (double)x[k] / rms * (double)gamma[k];
}

/* The f32 contract of the fused RMSNorm prologue: the sum of squares is taken
 * in double (so its summation order cannot show in the result), the reciprocal
 * root is rounded to f32 once, and each element is (x*rinv)*gamma with two f32
 * roundings.  Same formula as rmsNormForward above up to those roundings. */
ORC_API void orc_rmsnorm_f32(const float *x, const float *gamma, int K, float eps,
                             float *y) {
  double ss = 0.0;
  for (int k = 0; k < K; ++k) ss += (double)x[k] * (double)x[k];
  float rinv = (float)(1.0 / sqrt(ss / (double)K + (double)eps));
  for (int k = 0; k < K; ++k) {
    float t = x[k] * rinv;
    y[k] = gamma ? t * gamma[k] : t;
  }
}

/* Per-token absmax int8 quantiser.  Rule of the reference's Q8_1 quantiser
 * (Hesper/Layers/Linear.lean:1023-1048: d = amax/127, round to nearest even as
 * cvt.rni, Hesper/CUDA/PTX.lean:484; amax == 0 -> q = 0) applied to a whole token
 * instead of a 32-block, with the division by d carried out as one multiplication
 * by the f32 reciprocal scale:  d = amax/127,  inv = 127/amax (both IEEE f32
 * divisions),  q = rint_ties_even(x * inv).  |x*inv| <= 127*(1+2^-23), so no
 * clamp is needed.  Returns d, the scale the outputs are multiplied by. */
ORC_API float orc_quant_act_i8(const float *x, int K, int8_t *q) {
  float amax = 0.0f;
  for (int k = 0; k < K; ++k) {
    float a = fabsf(x[k]);
    if (a > amax) amax = a;
  }
  float d = amax / 127.0f;
  float inv = (amax == 0.0f) ? 0.0f : 127.0f / amax;
  for (int k = 0; k < K; ++k) {
    float v = x[k] * inv;
    q[k] = (int8_t)(int)rintf(v); /* default rounding mode = ties-to-even */
  }
  return d;
}

/* Integer BitLinear: acc[n] = sum_k t[n,k]*q[k] in int32.  This is
 * BitLinearSpec.forward (Hesper/Layers/BitLinearSpec.lean:65-77) evaluated on
 * integer-valued activations with scale 1: all partial sums are integers below
 * 2^24 for K up to 132 104, so the spec's arithmetic is exact. */
ORC_API void orc_bitlinear_i8(const uint8_t *packed, int K, int N, const int8_t *q,
                              int32_t *acc) {
  long bpr = K / 4;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint8_t *row = packed + (long)n * bpr;
    int32_t a = 0;
    for (int g = 0; g < K / 128; ++g) {
      const uint8_t *b = row + g * 32;
      const int8_t *xq = q + g * 128;
      for (int j = 0; j < 32; ++j) {
        uint8_t v = b[j];
        a += (((v >> 6) & 3) - 1) * xq[j];
        a += (((v >> 4) & 3) - 1) * xq[32 + j];
        a += (((v >> 2) & 3) - 1) * xq[64 + j];
        a += ((v & 3) - 1) * xq[96 + j];
      }
    }
    acc[n] = a;
  }
}

/* Full ternary x int8 forward for M tokens, the contract the CUDA path is held
 * to bit for bit:  optional RMSNorm prologue (orc_rmsnorm_f32), per-token
 * quantiser, int32 accumulate, y = ((float)acc * d) * s  [+ residual], each
 * operation one f32 rounding.  acc_out / d_out may be NULL. */
ORC_API void orc_bitlinear_forward(const uint8_t *packed, float scale, int K, int N,
                                   int M, const float *x, const float *gamma,
                                   float eps, const float *residual,
                                   int32_t *acc_out, float *d_out, float *y) {
  float *xn = (float *)malloc(sizeof(float) * (size_t)K);
  int8_t *q = (int8_t *)malloc((size_t)K);
  int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)N);
  for (int m = 0; m < M; ++m) {
    const float *xm = x + (long)m * K;
    if (gamma) {
      orc_rmsnorm_f32(xm, gamma, K, eps, xn);
      xm = xn;
    }
    float d = orc_quant_act_i8(xm, K, q);
    orc_bitlinear_i8(packed, K, N, q, acc);
    for (int n = 0; n < N; ++n) {
      float v = ((float)acc[n] * d) * scale;
      if (residual) v = v + residual[(long)m * N + n];
      y[(long)m * N + n] = v;
    }
    if (acc_out) memcpy(acc_out + (long)m * N, acc, sizeof(int32_t) * (size_t)N);
    if (d_out) d_out[m] = d;
  }
  free(xn);
  free(q);
  free(acc);
}

/* relu(s_g*g)^2 * (s_u*u): Hesper/Layers/BitLinear.lean:611-621.  Inputs are the
 * already scaled gate and up values; one f32 rounding per operation. */
static inline float relu2_mul(float g, float u) {
  float r = g > 0.0f ? g : 0.0f;
  return (r * r) * u;
}

/* Fused gate/up BitLinear pair with the ReLU^2 GLU epilogue
 * (Hesper/Layers/BitLinear.lean:553-621, API :1419). */
ORC_API void orc_bitlinear_gateup_relu2(const uint8_t *pg, float sg,
                                        const uint8_t *pu, float su, int K, int N,
                                        int M, const float *x, const float *gamma,
                                        float eps, float *y) {
  float *g = (float *)malloc(sizeof(float) * (size_t)M * N);
  float *u = (float *)malloc(sizeof(float) * (size_t)M * N);
  orc_bitlinear_forward(pg, sg, K, N, M, x, gamma, eps, NULL, NULL, NULL, g);
  orc_bitlinear_forward(pu, su, K, N, M, x, gamma, eps, NULL, NULL, NULL, u);
  for (long i = 0; i < (long)M * N; ++i) y[i] = relu2_mul(g[i], u[i]);
  free(g);
  free(u);
}

/* ------------------------------------------------------------------------- */
/* GGUF Q4_K and Q8_0                                                          */
/* ------------------------------------------------------------------------- */

/* getScaleMin: Hesper/Quantization/Q4_K_M.lean:120-144 (12 scale bytes ->
 * 6-bit scale and min of sub-block j). */
ORC_API void orc_q4k_scale_min(const uint8_t *scales, int j, int *sc, int *m) {
  if (j < 4) {
    *sc = scales[j] & 63;
    *m = scales[j + 4] & 63;
  } else {
    *sc = (scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4);
    *m = (scales[j + 4] >> 4) | ((scales[j] >> 6) << 4);
  }
}

/* Dequantise one 144-byte super-block to 256 f32 weights.  Layout and order:
 * Hesper/Quantization/Q4_K_M.lean:13-52; arithmetic as the reference's f32
 * kernel (Hesper/Layers/Linear.lean:146-190): d1 = d*sc, m1 = dmin*m,
 * w = d1*q - m1, each an f32 operation. */
ORC_API void orc_q4k_dequant_block(const uint8_t *blk, float *w) {
  uint16_t dh, mh;
  memcpy(&dh, blk, 2);
  memcpy(&mh, blk + 2, 2);
  float d = orc_f16_to_f32(dh), dmin = orc_f16_to_f32(mh);
  const uint8_t *scales = blk + 4;
  const uint8_t *qs = blk + 16;
  for (int c = 0; c < 4; ++c) {
    int sa, ma, sb, mb;
    orc_q4k_scale_min(scales, 2 * c, &sa, &ma);
    orc_q4k_scale_min(scales, 2 * c + 1, &sb, &mb);
    float d1 = d * (float)sa, m1 = dmin * (float)ma;
    float d2 = d * (float)sb, m2 = dmin * (float)mb;
    for (int l = 0; l < 32; ++l) {
      uint8_t b = qs[32 * c + l];
      w[64 * c + l] = d1 * (float)(b & 0xF) - m1;
      w[64 * c + 32 + l] = d2 * (float)(b >> 4) - m2;
    }
  }
}

/* Q4_K matvec / small-batch matmul, f32 weights as dequantised above, products
 * and the running sum in double (the accumulation the reference's own golden
 * dumper uses, scripts/llama_parity/dump_dg_q8mm_golden.cpp:28-43). */
ORC_API void orc_q4k_matvec(const uint8_t *blocks, int K, int N, int M,
                            const float *x, const float *residual, float *y) {
  int bpr = K / 256;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float w[256];
    double acc[64];
    for (int m0 = 0; m0 < M; m0 += 64) {
      int mb = (M - m0 < 64) ? (M - m0) : 64;
      for (int m = 0; m < mb; ++m) acc[m] = 0.0;
      for (int b = 0; b < bpr; ++b) {
        orc_q4k_dequant_block(blocks + ((long)n * bpr + b) * 144, w);
        for (int m = 0; m < mb; ++m) {
          const float *xm = x + (long)(m0 + m) * K + b * 256;
          double a = acc[m];
          for (int i = 0; i < 256; ++i) a += (double)w[i] * (double)xm[i];
          acc[m] = a;
        }
      }
      for (int m = 0; m < mb; ++m) {
        double v = acc[m];
        if (residual) v += (double)residual[(long)(m0 + m) * N + n];
        y[(long)(m0 + m) * N + n] = (float)v;
      }
    }
  }
}

/* Q8_0 matvec: 34-byte blocks, w = d*int8 in f32 (Hesper/Layers/Linear.lean:6207-6223),
 * double accumulate (scripts/llama_parity/dump_dg_q8mm_golden.cpp:28-43). */
ORC_API void orc_q8_0_matvec(const uint8_t *blocks, int K, int N, int M,
                             const float *x, const float *residual, float *y) {
  int bpr = K / 32;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    for (int m = 0; m < M; ++m) {
      const float *xm = x + (long)m * K;
      double acc = 0.0;
      for (int b = 0; b < bpr; ++b) {
        const uint8_t *blk = blocks + ((long)n * bpr + b) * 34;
        uint16_t dh;
        memcpy(&dh, blk, 2);
        float d = orc_f16_to_f32(dh);
        for (int i = 0; i < 32; ++i) {
          int8_t q = (int8_t)blk[2 + i];
          acc += (double)(d * (float)q) * (double)xm[b * 32 + i];
        }
      }
      if (residual) acc += (double)residual[(long)m * N + n];
      y[(long)m * N + n] = (float)acc;
    }
  }
}

/* GELU (tanh form): Hesper/Layers/FusedFFNSpec.lean:42-45. */
ORC_API double orc_gelu_tanh(double x) {
  const double c = 0.7978845608028654; /* sqrt(2/pi) */
  return 0.5 * x * (1.0 + tanh(c * (x + 0.044715 * x * x * x)));
}

/* gelu_tanh(x.Wg) * (x.Wu): Hesper/Layers/FusedFFNSpec.lean:117-122 over two
 * k-quant tensors (fmt 12 = Q4_K, 8 = Q8_0, the GGUF type ids). */
ORC_API void orc_kquant_gateup_gelu(const uint8_t *bg, const uint8_t *bu, int fmt,
                                    int K, int N, int M, const float *x, float *y) {
  float *g = (float *)malloc(sizeof(float) * (size_t)M * N);
  float *u = (float *)malloc(sizeof(float) * (size_t)M * N);
  if (fmt == 12) {
    orc_q4k_matvec(bg, K, N, M, x, NULL, g);
    orc_q4k_matvec(bu, K, N, M, x, NULL, u);
  } else {
    orc_q8_0_matvec(bg, K, N, M, x, NULL, g);
    orc_q8_0_matvec(bu, K, N, M, x, NULL, u);
  }
  for (long i = 0; i < (long)M * N; ++i)
    y[i] = (float)(orc_gelu_tanh((double)g[i]) * (double)u[i]);
  free(g);
  free(u);
}

/* ------------------------------------------------------------------------- */
/* Attention                                                                   */
/* ------------------------------------------------------------------------- */

/* Three-step single-head attention in double: scores, softmax, weighted sum.
 * Hesper/Training/VerifiedBackward.lean:134-142 (attentionForward) with
 * softmaxForward :33-37 (max starts at -1e30).  k, v are [L][D] row-major. */
ORC_API void orc_attention_head(const double *q, const double *k, const double *v,
                                int L, int D, double scale, double *out) {
  double *sc = (double *)malloc(sizeof(double) * (size_t)(L > 0 ? L : 1));
  double mx = -1e30;
  for (int s = 0; s < L; ++s) {
    double dot = 0.0;
    for (int d = 0; d < D; ++d) dot += q[d] * k[(long)s * D + d];
    sc[s] = scale * dot;
    if (sc[s] > mx) mx = sc[s];
  }
  double sum = 0.0;
  for (int s = 0; s < L; ++s) {
    sc[s] = exp(sc[s] - mx);
    sum += sc[s];
  }
  for (int d = 0; d < D; ++d) {
    double o = 0.0;
    for (int s = 0; s < L; ++s) o += (sc[s] / sum) * v[(long)s * D + d];
    out[d] = o;
  }
  free(sc);
}

/* Online-softmax form: Hesper/WGSL/FlashAttention.lean:60-90 (flashAttentionSpec),
 * statement for statement (running max -1e30, renormalised accumulator). */
ORC_API void orc_flash_attention_head(const double *q, const double *k,
                                      const double *v, int L, int D, double scale,
                                      double *out) {
  double mx = -1e30, sum = 0.0;
  for (int d = 0; d < D; ++d) out[d] = 0.0;
  for (int s = 0; s < L; ++s) {
    double score = 0.0;
    for (int d = 0; d < D; ++d) score += q[d] * k[(long)s * D + d];
    score *= scale;
    double nm = mx > score ? mx : score;
    double eo = exp(mx - nm), en = exp(score - nm);
    double ns = sum * eo + en;
    for (int d = 0; d < D; ++d)
      out[d] = out[d] * (sum * eo / ns) + v[(long)s * D + d] * (en / ns);
    mx = nm;
    sum = ns;
  }
}

/* GQA decode attention over an f16 KV cache for a batch of sequences.
 *   q      : [B][H][D]     f32 (q_is_f16 = 0) or f16 bits (q_is_f16 = 1)
 *   k, v   : [B][Hkv][max_seq][D]  f16 bits -- per sequence this is the cache
 *            layout of Hesper/WGSL/FlashAttention.lean:590-597 /
 *            Tests/CUDA/V11LauncherParityTest.lean:72-95
 *   seqlens: [B] number of valid positions (the query sits at position len-1,
 *            so every cached position is visible: causal at the last position)
 *   window : 0 = none; else only positions [len - window, len) contribute, the
 *            rule of flashAttentionSWAKernel (Hesper/WGSL/FlashAttention.lean:1621-1624)
 *   GQA map kvHead = h / (H/Hkv): Hesper/WGSL/FlashAttentionExperiments.lean:71-72.
 * Output f32 [B][H][D], arithmetic in double (three-step form). */
ORC_API void orc_attn_decode(const void *q, int q_is_f16, const uint16_t *k,
                             const uint16_t *v, const int32_t *seqlens, int B, int H,
                             int Hkv, int D, int max_seq, int window, float scale,
                             float *out) {
  int G = H / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    for (int h = 0; h < H; ++h) {
      int len = seqlens[b];
      int start = 0;
      if (window > 0 && len > window) start = len - window;
      int L = len - start;
      float *o = out + ((long)b * H + h) * D;
      if (L <= 0) {
        for (int d = 0; d < D; ++d) o[d] = 0.0f;
        continue;
      }
      int kvh = h / G;
      double *qd = (double *)malloc(sizeof(double) * (size_t)D);
      double *kd = (double *)malloc(sizeof(double) * (size_t)L * D);
      double *vd = (double *)malloc(sizeof(double) * (size_t)L * D);
      double *od = (double *)malloc(sizeof(double) * (size_t)D);
      for (int d = 0; d < D; ++d) {
        long qi = ((long)b * H + h) * D + d;
        qd[d] = q_is_f16 ? (double)orc_f16_to_f32(((const uint16_t *)q)[qi])
                         : (double)((const float *)q)[qi];
      }
      long base = (((long)b * Hkv + kvh) * max_seq + start) * D;
      for (long i = 0; i < (long)L * D; ++i) {
        kd[i] = (double)orc_f16_to_f32(k[base + i]);
        vd[i] = (double)orc_f16_to_f32(v[base + i]);
      }
      orc_attention_head(qd, kd, vd, L, D, (double)scale, od);
      for (int d = 0; d < D; ++d) o[d] = (float)od[d];
      free(qd);
      free(kd);
      free(vd);
      free(od);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Decode-step glue                                                            */
/* ------------------------------------------------------------------------- */

/* NeoX split-half RoPE on one head vector, pairs (d, d + D/2), angle
 * pos * base^(-2i/D): Hesper/Layers/RoPE.lean:90-97,189-247.  In place, f32
 * data, trigonometry in double then one rounding per output element. */
ORC_API void orc_rope_neox(float *x, int D, int pos, double base) {
  int half = D / 2;
  for (int i = 0; i < half; ++i) {
    double theta = (double)pos * pow(base, -2.0 * (double)i / (double)D);
    double c = cos(theta), s = sin(theta);
    double x0 = x[i], x1 = x[i + half];
    x[i] = (float)(x0 * c - x1 * s);
    x[i + half] = (float)(x0 * s + x1 * c);
  }
}

/* Greedy argmax, first strict maximum: Hesper/Models/BitNet.lean:474-479,
 * Hesper/Inference/Sampling.lean:74. */
ORC_API int orc_argmax(const float *x, long n) {
  long best = 0;
  float bv = x[0];
  for (long i = 1; i < n; ++i)
    if (x[i] > bv) {
      bv = x[i];
      best = i;
    }
  return (int)best;
}

/* LM head over a bf16 table [V][K] (tied embedding of the BitNet-shaped model;
 * the reference uses an f16 table, Hesper/Models/BitNet.lean:437-445):
 * logits[v] = sum_k table[v,k]*x[k], double accumulate. */
ORC_API void orc_lmhead_bf16(const uint16_t *table, long V, int K, const float *x,
                             float *logits) {
#pragma omp parallel for schedule(static)
  for (long v = 0; v < V; ++v) {
    const uint16_t *row = table + v * K;
    double acc = 0.0;
    for (int k = 0; k < K; ++k) acc += (double)orc_bf16_to_f32(row[k]) * (double)x[k];
    logits[v] = (float)acc;
  }
}

/* ------------------------------------------------------------------------- */
/* Whole decode step of a BitNet-b1.58-shaped model                            */
/* ------------------------------------------------------------------------- */

/* Layer order of TransformerBlock.forwardWithCache (Hesper/Layers/TransformerBlock.lean:439-485)
 * and Attention.forwardWithCache (Hesper/Layers/Attention.lean:1171-1248):
 *   attn_norm -> wq,wk,wv -> RoPE(q,k) -> KV append -> attention -> attn_sub_norm ->
 *   wo + residual -> ffn_norm -> relu(gate)^2*up -> ffn_sub_norm -> down + residual,
 * then final norm, tied LM head (Hesper/Models/BitNet.lean:431-445) and greedy argmax.
 * Linear layers follow orc_bitlinear_forward (int8 activations), the KV cache is f16,
 * the embedding / LM-head table is bf16. */
typedef struct orc_bitnet_layer {
  const float *attn_norm, *attn_sub_norm, *ffn_norm, *ffn_sub_norm;
  const uint8_t *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
  float sq, sk, sv, so, sgate, sup, sdown;
} orc_bitnet_layer;

typedef struct orc_bitnet {
  int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq;
  double rope_base;
  float eps;
  const orc_bitnet_layer *layers;
  const uint16_t *embed; /* bf16 [vocab][hidden] */
  const float *final_norm;
  uint16_t *kcache, *vcache; /* [layer][kv_head][max_seq][head_dim] f16 */
  int exact_attention;       /* 1: attention by orc_attn_decode_exact (mirror of the library) */
} orc_bitnet;

ORC_API void orc_attn_decode_exact(const void *q, int q_is_f16, const uint16_t *k,
                                   const uint16_t *v, const int32_t *seqlens, int B, int H,
                                   int Hkv, int D, int max_seq, int window, float scale_log2,
                                   float *out);

ORC_API void orc_bitnet_set_exact_attention(orc_bitnet *m, int on) { m->exact_attention = on; }

ORC_API orc_bitnet *orc_bitnet_create(int n_layers, int hidden, int n_heads, int n_kv_heads,
                                      int head_dim, int ffn, int vocab, int max_seq,
                                      double rope_base, float eps, const orc_bitnet_layer *layers,
                                      const uint16_t *embed, const float *final_norm) {
  orc_bitnet *m = (orc_bitnet *)calloc(1, sizeof(orc_bitnet));
  m->n_layers = n_layers; m->hidden = hidden; m->n_heads = n_heads; m->n_kv_heads = n_kv_heads;
  m->head_dim = head_dim; m->ffn = ffn; m->vocab = vocab; m->max_seq = max_seq;
  m->rope_base = rope_base; m->eps = eps; m->layers = layers; m->embed = embed;
  m->final_norm = final_norm;
  size_t n = (size_t)n_layers * n_kv_heads * max_seq * head_dim;
  m->kcache = (uint16_t *)calloc(n, 2);
  m->vcache = (uint16_t *)calloc(n, 2);
  return m;
}

ORC_API void orc_bitnet_destroy(orc_bitnet *m) {
  if (!m) return;
  free(m->kcache);
  free(m->vcache);
  free(m);
}

/* One token at position `pos`: fills logits[vocab] and returns the greedy token. */
ORC_API int orc_bitnet_step(orc_bitnet *m, int token, int pos, float *logits) {
  const int Hd = m->hidden, H = m->n_heads, Hkv = m->n_kv_heads, D = m->head_dim, F = m->ffn;
  const int qdim = H * D, kvdim = Hkv * D;
  float *x = (float *)malloc(sizeof(float) * Hd), *x1 = (float *)malloc(sizeof(float) * Hd);
  float *q = (float *)malloc(sizeof(float) * qdim), *k = (float *)malloc(sizeof(float) * kvdim);
  float *v = (float *)malloc(sizeof(float) * kvdim), *att = (float *)malloc(sizeof(float) * qdim);
  float *h = (float *)malloc(sizeof(float) * F);
  for (int i = 0; i < Hd; ++i) x[i] = orc_bf16_to_f32(m->embed[(size_t)token * Hd + i]);
  int32_t len = pos + 1;
  for (int l = 0; l < m->n_layers; ++l) {
    const orc_bitnet_layer *L = &m->layers[l];
    orc_bitlinear_forward(L->wq, L->sq, Hd, qdim, 1, x, L->attn_norm, m->eps, NULL, NULL, NULL, q);
    orc_bitlinear_forward(L->wk, L->sk, Hd, kvdim, 1, x, L->attn_norm, m->eps, NULL, NULL, NULL, k);
    orc_bitlinear_forward(L->wv, L->sv, Hd, kvdim, 1, x, L->attn_norm, m->eps, NULL, NULL, NULL, v);
    for (int hh = 0; hh < H; ++hh) orc_rope_neox(q + hh * D, D, pos, m->rope_base);
    for (int hh = 0; hh < Hkv; ++hh) orc_rope_neox(k + hh * D, D, pos, m->rope_base);
    uint16_t *kc = m->kcache + (size_t)l * Hkv * m->max_seq * D;
    uint16_t *vc = m->vcache + (size_t)l * Hkv * m->max_seq * D;
    for (int hh = 0; hh < Hkv; ++hh)
      for (int d = 0; d < D; ++d) {
        kc[((size_t)hh * m->max_seq + pos) * D + d] = orc_f32_to_f16(k[hh * D + d]);
        vc[((size_t)hh * m->max_seq + pos) * D + d] = orc_f32_to_f16(v[hh * D + d]);
      }
    {
      /* scale exactly as the decode engine forms it: f32 operations */
      const float scale = 1.0f / sqrtf((float)D);
      if (m->exact_attention)
        orc_attn_decode_exact(q, 0, kc, vc, &len, 1, H, Hkv, D, m->max_seq, 0,
                              scale * 1.4426950408889634f, att);
      else
        orc_attn_decode(q, 0, kc, vc, &len, 1, H, Hkv, D, m->max_seq, 0, scale, att);
    }
    orc_bitlinear_forward(L->wo, L->so, qdim, Hd, 1, att, L->attn_sub_norm, m->eps, x, NULL, NULL, x1);
    orc_bitlinear_gateup_relu2(L->wgate, L->sgate, L->wup, L->sup, Hd, F, 1, x1, L->ffn_norm, m->eps, h);
    orc_bitlinear_forward(L->wdown, L->sdown, F, Hd, 1, h, L->ffn_sub_norm, m->eps, x1, NULL, NULL, x);
  }
  float *xn = (float *)malloc(sizeof(float) * Hd);
  orc_rmsnorm_f32(x, m->final_norm, Hd, m->eps, xn);
  orc_lmhead_bf16(m->embed, m->vocab, Hd, xn, logits);
  int tok = orc_argmax(logits, m->vocab);
  free(x); free(x1); free(q); free(k); free(v); free(att); free(h); free(xn);
  return tok;
}

/* ------------------------------------------------------------------------- */
/* Operation-for-operation mirror of the CUDA library's EXACT attention mode   */
/* ------------------------------------------------------------------------- */

/* 2^x for x <= 0 from IEEE f32 operations only; same constants and order as the kernel. */
static float orc_exp2_det(float x) {
  if (!(x > -120.0f)) return 0.0f;
  const float n = rintf(x);
  const float f = x - n;
  float p = 1.5403530e-4f;
  p = fmaf(p, f, 1.3398874e-3f);
  p = fmaf(p, f, 9.6184370e-3f);
  p = fmaf(p, f, 5.5503324e-2f);
  p = fmaf(p, f, 2.4022648e-1f);
  p = fmaf(p, f, 6.9314720e-1f);
  p = fmaf(p, f, 1.0f);
  return ldexpf(p, (int)n);
}

/* Same inputs, outputs and head mapping as orc_attn_decode, but every f32 operation in
 * the order the library's bit-reproducible kernel fixes: 32 "lanes" each own D/32
 * consecutive dims, partial dot products by fma with d ascending, the 32 partials combined
 * by the xor-butterfly 16,8,4,2,1, online softmax in the exp2 domain with orc_exp2_det,
 * acc = fma(p, v, acc*alpha), l = fma(l, alpha, p), out = acc / l.  Not a restatement of a
 * reference function: it exists so that a whole-model run can be compared token for token
 * (see orc_bitnet_step with exact_attention = 1); orc_attn_decode remains the definition. */
ORC_API void orc_attn_decode_exact(const void *q, int q_is_f16, const uint16_t *k,
                                   const uint16_t *v, const int32_t *seqlens, int B, int H,
                                   int Hkv, int D, int max_seq, int window, float scale_log2,
                                   float *out) {
  const int G = H / Hkv, DL = D / 32;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    for (int h = 0; h < H; ++h) {
      int len = seqlens[b];
      if (len < 0) len = 0;
      if (len > max_seq) len = max_seq;
      int start = 0;
      if (window > 0 && len > window) start = len - window;
      const int kvh = h / G;
      float qf[256], acc[256];
      for (int d = 0; d < D; ++d) {
        long qi = ((long)b * H + h) * D + d;
        qf[d] = q_is_f16 ? orc_f16_to_f32(((const uint16_t *)q)[qi]) : ((const float *)q)[qi];
        acc[d] = 0.0f;
      }
      const uint16_t *kb = k + ((long)b * Hkv + kvh) * (long)max_seq * D;
      const uint16_t *vb = v + ((long)b * Hkv + kvh) * (long)max_seq * D;
      float m = -INFINITY, l = 0.0f;
      for (int s = start; s < len; ++s) {
        float part[32], tmp[32];
        for (int lane = 0; lane < 32; ++lane) {
          float pp = 0.0f;
          for (int j = 0; j < DL; ++j) {
            int d = lane * DL + j;
            pp = fmaf(qf[d], orc_f16_to_f32(kb[(long)s * D + d]), pp);
          }
          part[lane] = pp;
        }
        for (int o = 16; o > 0; o >>= 1) {
          for (int lane = 0; lane < 32; ++lane) tmp[lane] = part[lane] + part[lane ^ o];
          memcpy(part, tmp, sizeof(part));
        }
        const float sc = part[0] * scale_log2;
        const float mn = (m > sc) ? m : sc;
        const float alpha = orc_exp2_det(m - mn);
        const float pw = orc_exp2_det(sc - mn);
        l = fmaf(l, alpha, pw);
        for (int d = 0; d < D; ++d)
          acc[d] = fmaf(pw, orc_f16_to_f32(vb[(long)s * D + d]), acc[d] * alpha);
        m = mn;
      }
      float *o = out + ((long)b * H + h) * D;
      for (int d = 0; d < D; ++d) o[d] = l > 0.0f ? acc[d] / l : 0.0f;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Whole decode step of a Gemma-4-E4B-shaped model (Q4_K weights)              */
/* ------------------------------------------------------------------------- */

/* Block order of Gemma4.forwardBlock (Hesper/Models/Gemma4.lean:485): norm -> q/k/v ->
 * RoPE -> f16 KV append -> attention -> o_proj -> post-attention norm then add -> norm ->
 * gelu_tanh(gate)*up -> down_proj -> post-FFN norm then add (forwardNormThenAdd); final norm,
 * Q4_K LM head, greedy argmax.  Sliding-window layers attend to the last `window` positions
 * (the rule of flashAttentionSWAKernel, Hesper/WGSL/FlashAttention.lean:1621-1624); layer l is
 * global when (l+1) % global_every == 0.  Unsharded: the tensor-parallel run must reproduce it. */
typedef struct orc_gemma_layer {
  const float *attn_norm, *post_attn_norm, *ffn_norm, *post_ffn_norm;
  const uint8_t *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
} orc_gemma_layer;

typedef struct orc_gemma {
  int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq, window, global_every;
  double rope_base;
  float eps, attn_scale, embed_scale;
  const orc_gemma_layer *layers;
  const uint16_t *embed; /* bf16 */
  const uint8_t *lm_head;
  const float *final_norm;
  uint16_t *kcache, *vcache;
} orc_gemma;

ORC_API orc_gemma *orc_gemma_create(int n_layers, int hidden, int n_heads, int n_kv_heads,
                                    int head_dim, int ffn, int vocab, int max_seq, int window,
                                    int global_every, double rope_base, float eps,
                                    float attn_scale, float embed_scale,
                                    const orc_gemma_layer *layers, const uint16_t *embed,
                                    const uint8_t *lm_head, const float *final_norm) {
  orc_gemma *m = (orc_gemma *)calloc(1, sizeof(orc_gemma));
  m->n_layers = n_layers; m->hidden = hidden; m->n_heads = n_heads; m->n_kv_heads = n_kv_heads;
  m->head_dim = head_dim; m->ffn = ffn; m->vocab = vocab; m->max_seq = max_seq;
  m->window = window; m->global_every = global_every; m->rope_base = rope_base; m->eps = eps;
  m->attn_scale = attn_scale; m->embed_scale = embed_scale; m->layers = layers;
  m->embed = embed; m->lm_head = lm_head; m->final_norm = final_norm;
  size_t n = (size_t)n_layers * n_kv_heads * max_seq * head_dim;
  m->kcache = (uint16_t *)calloc(n, 2);
  m->vcache = (uint16_t *)calloc(n, 2);
  return m;
}

ORC_API void orc_gemma_destroy(orc_gemma *m) {
  if (!m) return;
  free(m->kcache);
  free(m->vcache);
  free(m);
}

ORC_API int orc_gemma_step(orc_gemma *m, int token, int pos, float *logits) {
  const int Hd = m->hidden, H = m->n_heads, Hkv = m->n_kv_heads, D = m->head_dim, F = m->ffn;
  const int qdim = H * D, kvdim = Hkv * D;
  float *x = (float *)malloc(sizeof(float) * Hd), *x1 = (float *)malloc(sizeof(float) * Hd);
  float *xn = (float *)malloc(sizeof(float) * Hd), *o = (float *)malloc(sizeof(float) * Hd);
  float *q = (float *)malloc(sizeof(float) * qdim), *k = (float *)malloc(sizeof(float) * kvdim);
  float *v = (float *)malloc(sizeof(float) * kvdim), *att = (float *)malloc(sizeof(float) * qdim);
  float *h = (float *)malloc(sizeof(float) * F);
  for (int i = 0; i < Hd; ++i)
    x[i] = orc_bf16_to_f32(m->embed[(size_t)token * Hd + i]) * m->embed_scale;
  int32_t len = pos + 1;
  for (int l = 0; l < m->n_layers; ++l) {
    const orc_gemma_layer *L = &m->layers[l];
    const int global = m->global_every > 0 && (l + 1) % m->global_every == 0;
    orc_rmsnorm_f32(x, L->attn_norm, Hd, m->eps, xn);
    orc_q4k_matvec(L->wq, Hd, qdim, 1, xn, NULL, q);
    orc_q4k_matvec(L->wk, Hd, kvdim, 1, xn, NULL, k);
    orc_q4k_matvec(L->wv, Hd, kvdim, 1, xn, NULL, v);
    for (int hh = 0; hh < H; ++hh) orc_rope_neox(q + hh * D, D, pos, m->rope_base);
    for (int hh = 0; hh < Hkv; ++hh) orc_rope_neox(k + hh * D, D, pos, m->rope_base);
    uint16_t *kc = m->kcache + (size_t)l * Hkv * m->max_seq * D;
    uint16_t *vc = m->vcache + (size_t)l * Hkv * m->max_seq * D;
    for (int hh = 0; hh < Hkv; ++hh)
      for (int d = 0; d < D; ++d) {
        kc[((size_t)hh * m->max_seq + pos) * D + d] = orc_f32_to_f16(k[hh * D + d]);
        vc[((size_t)hh * m->max_seq + pos) * D + d] = orc_f32_to_f16(v[hh * D + d]);
      }
    orc_attn_decode(q, 0, kc, vc, &len, 1, H, Hkv, D, m->max_seq, global ? 0 : m->window,
                    m->attn_scale, att);
    orc_q4k_matvec(L->wo, qdim, Hd, 1, att, NULL, o);
    orc_rmsnorm_f32(o, L->post_attn_norm, Hd, m->eps, xn);
    for (int i = 0; i < Hd; ++i) x1[i] = x[i] + xn[i];
    orc_rmsnorm_f32(x1, L->ffn_norm, Hd, m->eps, xn);
    orc_kquant_gateup_gelu(L->wgate, L->wup, 12, Hd, F, 1, xn, h);
    orc_q4k_matvec(L->wdown, F, Hd, 1, h, NULL, o);
    orc_rmsnorm_f32(o, L->post_ffn_norm, Hd, m->eps, xn);
    for (int i = 0; i < Hd; ++i) x[i] = x1[i] + xn[i];
  }
  orc_rmsnorm_f32(x, m->final_norm, Hd, m->eps, xn);
  orc_q4k_matvec(m->lm_head, Hd, m->vocab, 1, xn, NULL, logits);
  int tok = orc_argmax(logits, m->vocab);
  free(x); free(x1); free(xn); free(o); free(q); free(k); free(v); free(att); free(h);
  return tok;
}
