/*
 * fp8.h - the MXFP8 (E4M3) segment: layout helpers and the single-format GEMM entry.
 * Replaces MixedGemm's include/fp8.h (matmul_host8, include/fp8.h:46-56,
 * src/fp8.cu:35-194).
 */
#ifndef MIXEDGEMM_FP8_H
#define MIXEDGEMM_FP8_H
#include "mxdtype.h"
#ifdef __cplusplus
extern "C" {
#endif

/* Value of an E4M3 code (finite-only variant: bias 7, largest magnitude 448, 0x7F = NaN). */
static inline float mg_fp8_value(uint8_t code) {
  int e = (code >> 3) & 15, m = code & 7;
  float v = e ? (float)(8 + m) : (float)m;
  int sh = (e ? e : 1) - 10; /* v * 2^(e-7-3) */
  v = sh >= 0 ? v * (float)(1 << sh) : v / (float)(1 << -sh);
  return (code & 0x80) ? -v : v;
}

/*
 * D = bf16( A8[M,K] * B4[N,K]^T (+ C) ): A MXFP8 E4M3, B MXFP4 (matmul_host8 computes
 * this with C = D).  K must be a multiple of 128 on this entry.
 */
int mg_matmul_fp8(const uint8_t* A, const uint8_t* B, int M, int N, int K, const void* C_bf16,
                  void* D_bf16, const uint8_t* SFA, const uint8_t* SFB, void* stream);

#ifdef __cplusplus
}
#endif
#endif
