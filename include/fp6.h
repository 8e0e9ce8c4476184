/*
 * fp6.h - the MXFP6 (E3M2) segment: packed layout helpers and the single-format GEMM
 * entry.  Replaces MixedGemm's include/fp6.h (matmul_host6, include/fp6.h:46-56,
 * src/fp6.cu:35-194).
 */
#ifndef MIXEDGEMM_FP6_H
#define MIXEDGEMM_FP6_H
#include "mxdtype.h"
#ifdef __cplusplus
extern "C" {
#endif

/* E3M2 code (sign bit 0x20) of element k: bits [6k, 6k+6) of the row's byte stream
 * (src/reorder.cu:54-63). */
static inline uint8_t mg_fp6_get(const uint8_t* row, int k) {
  size_t bit = (size_t)k * 6, b = bit >> 3;
  unsigned w = row[b] | ((bit & 7) > 2 ? (unsigned)row[b + 1] << 8 : 0u);
  return (uint8_t)((w >> (bit & 7)) & 0x3F);
}
/* Pack four codes into three bytes. */
static inline void mg_fp6_pack4(uint8_t v0, uint8_t v1, uint8_t v2, uint8_t v3, uint8_t out[3]) {
  unsigned w = (v0 & 0x3Fu) | ((v1 & 0x3Fu) << 6) | ((v2 & 0x3Fu) << 12) | ((v3 & 0x3Fu) << 18);
  out[0] = (uint8_t)w; out[1] = (uint8_t)(w >> 8); out[2] = (uint8_t)(w >> 16);
}
/* Value of an E3M2 code: bias 3, subnormal step 1/16, largest magnitude 28. */
static inline float mg_fp6_value(uint8_t code) {
  int e = (code >> 2) & 7, m = code & 3;
  float v = e ? (float)(4 + m) * (float)(1 << e) / 32.f : (float)m / 16.f;
  return (code & 0x20) ? -v : v;
}

/*
 * D = bf16( A6[M,K] * B4[N,K]^T (+ C) ): A MXFP6 E3M2, B MXFP4 (matmul_host6 computes
 * this with C = D).  K must be a multiple of 128 on this entry.
 */
int mg_matmul_fp6(const uint8_t* A, const uint8_t* B, int M, int N, int K, const void* C_bf16,
                  void* D_bf16, const uint8_t* SFA, const uint8_t* SFB, void* stream);

#ifdef __cplusplus
}
#endif
#endif
