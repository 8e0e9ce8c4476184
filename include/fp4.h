/*
 * fp4.h - the MXFP4 (E2M1) segment: packed layout helpers and the single-format GEMM
 * entry.  Replaces MixedGemm's include/fp4.h, whose one prototype is
 * matmul_host4 (include/fp4.h:46-56, defined at src/fp4.cu:35-192).
 */
#ifndef MIXEDGEMM_FP4_H
#define MIXEDGEMM_FP4_H
#include "mxdtype.h"
#ifdef __cplusplus
extern "C" {
#endif

/* E2M1 code (sign bit 0x8) of element k of a packed row. */
static inline uint8_t mg_fp4_get(const uint8_t* row, int k) { return (row[k >> 1] >> ((k & 1) * 4)) & 0xF; }
static inline void mg_fp4_set(uint8_t* row, int k, uint8_t code) {
  int s = (k & 1) * 4;
  row[k >> 1] = (uint8_t)((row[k >> 1] & ~(0xF << s)) | ((code & 0xF) << s));
}
/* Value of an E2M1 code: magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6. */
static inline float mg_fp4_value(uint8_t code) {
  static const float mag[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  return (code & 8) ? -mag[code & 7] : mag[code & 7];
}

/*
 * D[M,N] = bf16( A[M,K] * B[N,K]^T  (+ C[M,N] when C != NULL) ), A and B both MXFP4.
 * Same operands as matmul_host4 (src/fp4.cu:35-45); device pointers; runs on `stream`.
 * Returns an MG_* status (mixedgemm_c.h).
 */
int mg_matmul_fp4(const uint8_t* A, const uint8_t* B, int M, int N, int K, const void* C_bf16,
                  void* D_bf16, const uint8_t* SFA, const uint8_t* SFB, void* stream);

#ifdef __cplusplus
}
#endif
#endif
