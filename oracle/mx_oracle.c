/*
 * CPU oracle for the MixedGemm hot path.  TEST INFRASTRUCTURE ONLY: this file is the
 * checker used by tests/, by the smoke entry and by the CPU-baseline leg of the bench.
 * It is never linked into, imported by or called from the CUDA product path.
 *
 * It restates, in plain C with the reference's literal float expression chain, what
 * the reference computes on its hot path (paths are relative to the MixedGemm project):
 *   - src/reorder.cu:94-269   reorder_bf16_mixed_kernel   (activations -> FP4 / FP6 / FP8)
 *   - src/reorder.cu:271-432  reorder_bf16_fp4_kernel     (weights -> FP4 in three K segments)
 *   - include/reorder.cuh:119-124 + src/reorder.cu:181-208 scale-factor coordinates
 *   - src/gemm.cu:22-47, src/fp4.cu / fp6.cu / fp8.cu      block-scaled GEMM semantics
 *
 * The float -> E2M1 / E3M2 / E4M3 / UE8M0 / bf16 conversions that the reference delegates
 * to CUTLASS's NumericConverter (round-to-nearest-even, saturating) are restated here as
 * one generic ExMy encoder.  Parity pin: tests/golden/cutlass_tables.json holds the tables
 * produced by CUTLASS's own host converters (generator committed beside it) and the
 * CPU tests check this file against them; on a GPU box the compiled reference kernel
 * (oracle/_ref) is compared as well.
 *
 * Build: see oracle/build_oracle.py (gcc -O2 -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define FP4_MAX 6.0f   /* src/reorder.cu:17 */
#define FP6_MAX 28.0f  /* src/reorder.cu:18 */
#define FP8_MAX 448.0f /* src/reorder.cu:19 */

enum { FMT_E2M1 = 0, FMT_E3M2 = 1, FMT_E4M3 = 2 };

/* ------------------------------------------------------------------ bf16 helpers */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* float -> bf16, round to nearest even (NumericConverter<bfloat16_t,float>). */
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/* ------------------------------------------------------------------ ExMy encoder
 * Round-to-nearest-even conversion of a finite float into a sign/exponent/mantissa
 * code with `ebits` exponent bits (bias 2^(ebits-1)-1) and `mbits` mantissa bits, with
 * subnormals, saturating at `maxv` (the formats here have no infinities). */
static uint8_t encode_exmy(float f, int ebits, int mbits, float maxv) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint8_t sign = (uint8_t)((u >> 31) << (ebits + mbits));
  float a = fabsf(f);
  if (a == 0.0f) return sign;
  if (a > maxv) a = maxv;
  int bias = (1 << (ebits - 1)) - 1;
  int emin = 1 - bias; /* exponent of the smallest normal */
  int e;
  (void)frexpf(a, &e);
  e -= 1; /* a = m * 2^e, m in [1,2) */
  if (e < emin) e = emin;
  /* number of mantissa steps of size 2^(e-mbits) */
  float steps = ldexpf(a, mbits - e); /* exact: power-of-two scaling */
  float q = rintf(steps);             /* default rounding mode = nearest even */
  int qi = (int)q;                    /* in [0, 2^(mbits+1)] */
  int code;
  if (e == emin && qi < (1 << mbits)) {
    code = qi; /* subnormal (exponent field 0) */
  } else {
    /* qi in [2^mbits, 2^(mbits+1)]; the carry into the exponent is the encoding's own */
    code = ((e + bias) << mbits) + (qi - (1 << mbits));
  }
  return (uint8_t)(sign | (uint8_t)code);
}

uint8_t orc_encode(float f, int fmt) {
  switch (fmt) {
    case FMT_E2M1: return encode_exmy(f, 2, 1, FP4_MAX);
    case FMT_E3M2: return encode_exmy(f, 3, 2, FP6_MAX);
    default:       return encode_exmy(f, 4, 3, FP8_MAX);
  }
}

/* code -> float for the three element formats (E4M3 here never holds NaN codes). */
float orc_decode(uint8_t code, int fmt) {
  int ebits = fmt == FMT_E2M1 ? 2 : fmt == FMT_E3M2 ? 3 : 4;
  int mbits = fmt == FMT_E2M1 ? 1 : fmt == FMT_E3M2 ? 2 : 3;
  int bias = (1 << (ebits - 1)) - 1;
  int s = (code >> (ebits + mbits)) & 1;
  int e = (code >> mbits) & ((1 << ebits) - 1);
  int m = code & ((1 << mbits) - 1);
  float v = e == 0 ? ldexpf((float)m, 1 - bias - mbits)
                   : ldexpf((float)((1 << mbits) + m), e - bias - mbits);
  return s ? -v : v;
}

/* float power of two -> UE8M0 byte (NumericConverter<float_ue8m0_t,float>): the biased
 * exponent; the reference only ever feeds exact powers of two (src/reorder.cu:180-185). */
static inline uint8_t f32_to_ue8m0(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t e = (u >> 23) & 0xff;
  if (u & 0x7fffffu) e += 1; /* round up a non-power-of-two (never hit here) */
  return (uint8_t)e;
}

/* ------------------------------------------------------------------ scale-factor layout
 * Byte offset of the scale of (row r, 32-block kb) inside one segment's scale buffer:
 * CUTLASS Sm1xx block-scaled layout, atom ((32,4),(32,4)):((16,4),(0,1)) tiled K-first
 * (include/reorder.cuh:119-124; coordinates built at src/reorder.cu:181-185). */
size_t orc_sf_offset(int r, int kb, int kseg) {
  size_t katoms = (size_t)((kseg + 127) / 128);
  return (size_t)(r % 32) * 16 + (size_t)((r / 32) % 4) * 4 + (size_t)(kb % 4) +
         (size_t)(kb / 4) * 512 + (size_t)(r / 128) * 512 * katoms;
}

size_t orc_sf_bytes(int rows, int kseg) {
  return (size_t)((rows + 127) / 128) * (size_t)((kseg + 127) / 128) * 512;
}

/* ------------------------------------------------------------------ one 32-group
 * src/reorder.cu:160-248 for one (row, group): scale, then quantise the 32 values. */
static uint8_t quantise_group(const float* v, float fmax, int fmt, uint8_t* codes) {
  float maxv = 0.0f;
  for (int i = 0; i < 32; ++i) { /* mymax over |x| (src/reorder.cu:81-91,166-169) */
    float a = fabsf(v[i]);
    maxv = maxv > a ? maxv : a;
  }
  float scale;
  if (maxv == 0.0f) scale = 0.5f; /* src/reorder.cu:179 */
  else scale = bf16_to_f32(f32_to_bf16_rne(ldexpf(1.0f, (int)ceilf(log2f(maxv / fmax)))));
  uint8_t sf = f32_to_ue8m0(scale);
  float r_scale = (float)(1.0 / (double)scale); /* src/reorder.cu:212 */
  for (int i = 0; i < 32; ++i) {
    float t = roundf(v[i] * r_scale); /* half away from zero */
    t = fmaxf(-fmax, fminf(fmax, t)); /* clamp (src/reorder.cu:41) */
    float b = bf16_to_f32(f32_to_bf16_rne(t)); /* converterScale: float -> bf16 */
    codes[i] = orc_encode(b, fmt);
  }
  return sf;
}

/* ------------------------------------------------------------------ activations
 * X[M,K] bf16 bits; idx[K]; outputs as in src/bindings.cpp:88-93. */
void orc_reorder_quantize_x(const uint16_t* X, int M, int K, const int16_t* idx, int KN,
                            int KS, int KO, uint8_t* AN, uint8_t* AS, uint8_t* AO,
                            uint8_t* SFAN, uint8_t* SFAS, uint8_t* SFAO) {
  int gN = KN / 32, gS = KS / 32;
  int G = K / 32;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < M; ++r) {
    const uint16_t* x = X + (size_t)r * K;
    for (int g = 0; g < G; ++g) {
      float v[32];
      uint8_t c[32];
      for (int i = 0; i < 32; ++i) v[i] = bf16_to_f32(x[(uint16_t)idx[g * 32 + i]]);
      if (g < gN) { /* FP4: low nibble = even element (src/reorder.cu:30-33,243-246) */
        uint8_t sf = quantise_group(v, FP4_MAX, FMT_E2M1, c);
        SFAN[orc_sf_offset(r, g, KN)] = sf;
        uint8_t* o = AN + (size_t)r * (KN / 2) + (size_t)g * 16;
        for (int i = 0; i < 16; ++i) o[i] = (uint8_t)((c[2 * i] & 0xF) | (c[2 * i + 1] << 4));
      } else if (g < gN + gS) { /* FP6: 4 codes in 3 bytes (src/reorder.cu:54-63) */
        int gs = g - gN;
        uint8_t sf = quantise_group(v, FP6_MAX, FMT_E3M2, c);
        SFAS[orc_sf_offset(r, gs, KS)] = sf;
        uint8_t* o = AS + (size_t)r * (KS / 4 * 3) + (size_t)gs * 24;
        for (int i = 0; i < 8; ++i) {
          uint8_t v0 = c[4 * i] & 0x3F, v1 = c[4 * i + 1] & 0x3F, v2 = c[4 * i + 2] & 0x3F,
                  v3 = c[4 * i + 3] & 0x3F;
          o[3 * i + 0] = (uint8_t)(v0 | ((v1 & 0x03) << 6));
          o[3 * i + 1] = (uint8_t)((v1 >> 2) | ((v2 & 0x0F) << 4));
          o[3 * i + 2] = (uint8_t)((v2 >> 4) | (v3 << 2));
        }
      } else { /* FP8: one byte per element (src/reorder.cu:228-231) */
        int go = g - gN - gS;
        uint8_t sf = quantise_group(v, FP8_MAX, FMT_E4M3, c);
        SFAO[orc_sf_offset(r, go, KO)] = sf;
        memcpy(AO + (size_t)r * KO + (size_t)go * 32, c, 32);
      }
    }
  }
}

/* ------------------------------------------------------------------ weights
 * W[N,K] bf16 bits -> three all-E2M1 segments (src/reorder.cu:271-432). */
void orc_reorder_quantize_w(const uint16_t* W, int N, int K, const int16_t* idx, int KN,
                            int KS, int KO, uint8_t* BN, uint8_t* BS, uint8_t* BO,
                            uint8_t* SFBN, uint8_t* SFBS, uint8_t* SFBO) {
  int gN = KN / 32, gS = KS / 32;
  int G = K / 32;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < N; ++r) {
    const uint16_t* x = W + (size_t)r * K;
    for (int g = 0; g < G; ++g) {
      float v[32];
      uint8_t c[32];
      for (int i = 0; i < 32; ++i) v[i] = bf16_to_f32(x[(uint16_t)idx[g * 32 + i]]);
      uint8_t sf = quantise_group(v, FP4_MAX, FMT_E2M1, c);
      uint8_t* o;
      if (g < gN) {
        SFBN[orc_sf_offset(r, g, KN)] = sf;
        o = BN + (size_t)r * (KN / 2) + (size_t)g * 16;
      } else if (g < gN + gS) {
        SFBS[orc_sf_offset(r, g - gN, KS)] = sf;
        o = BS + (size_t)r * (KS / 2) + (size_t)(g - gN) * 16;
      } else {
        SFBO[orc_sf_offset(r, g - gN - gS, KO)] = sf;
        o = BO + (size_t)r * (KO / 2) + (size_t)(g - gN - gS) * 16;
      }
      for (int i = 0; i < 16; ++i) o[i] = (uint8_t)((c[2 * i] & 0xF) | (c[2 * i + 1] << 4));
    }
  }
}

/* ------------------------------------------------------------------ dequantise
 * Expand one packed segment to float32 [rows, kseg]: code value * 2^(sf-127).
 * fmt: FMT_E2M1 (nibbles), FMT_E3M2 (6-bit stream), FMT_E4M3 (bytes). */
void orc_dequantize(const uint8_t* codes, const uint8_t* sf, int rows, int kseg, int fmt,
                    float* out) {
  size_t pitch = fmt == FMT_E2M1 ? (size_t)kseg / 2 : fmt == FMT_E3M2 ? (size_t)kseg / 4 * 3
                                                                      : (size_t)kseg;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const uint8_t* p = codes + (size_t)r * pitch;
    for (int k = 0; k < kseg; ++k) {
      uint8_t c;
      if (fmt == FMT_E2M1) c = (p[k / 2] >> ((k & 1) * 4)) & 0xF;
      else if (fmt == FMT_E3M2) {
        size_t bit = (size_t)k * 6;
        uint32_t w = p[bit / 8] | ((bit / 8 + 1 < pitch ? p[bit / 8 + 1] : 0u) << 8);
        c = (w >> (bit % 8)) & 0x3F;
      } else c = p[k];
      int e = (int)sf[orc_sf_offset(r, k / 32, kseg)] - 127;
      out[(size_t)r * kseg + k] = ldexpf(orc_decode(c, fmt), e);
    }
  }
}

/* ------------------------------------------------------------------ GEMM semantics
 * Y[m,n] = sum_k A[m,k] * B[n,k] in double over already-dequantised operands
 * (src/gemm.cu:44-46 summed without the reference's intermediate bf16 roundings). */
void orc_gemm_f64(const float* A, const float* B, int M, int N, int K, double* Y) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const float* a = A + (size_t)m * K;
      const float* b = B + (size_t)n * K;
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)a[k] * (double)b[k];
      Y[(size_t)m * N + n] = acc;
    }
}

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
