/*
 * mxdtype.h - plain-C description of the packed MX operand formats that cross the
 * library boundary.  It takes the place of MixedGemm's include/mxdtype.h (a CUTLASS
 * sub-byte accessor whose symbols nothing in the reference uses) and of the type
 * aliases in include/reorder.cuh:36-40; the formats themselves are defined by what
 * src/reorder.cu writes (PackFp4 :30-33, pack_4_fp6_to_3_bytes :54-63, stores :250-268).
 *
 * Every operand is split along K into three segments, in this order:
 *   "normal"    KN elements   FP4  E2M1   2 per byte, even element in the low nibble
 *   "sensitive" KS elements   FP6  E3M2   4 per 3 bytes, little-endian bit stream
 *   "outlier"   KO elements   FP8  E4M3   1 per byte
 * (weights use E2M1 in all three).  One UE8M0 scale byte (biased exponent, bias 127)
 * covers 32 consecutive elements of a row; element value = code value * 2^(scale-127).
 * KN, KS and KO are multiples of 32.
 */
#ifndef MIXEDGEMM_MXDTYPE_H
#define MIXEDGEMM_MXDTYPE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MG_GROUP 32 /* elements per scale factor */

/* elements per storage vector, as in the reference's kElementsPerVector* constants */
#define MG_ELEMS_PER_BYTE_FP4 2
#define MG_ELEMS_PER_3BYTES_FP6 4
#define MG_ELEMS_PER_BYTE_FP8 1

/* Largest magnitudes (src/reorder.cu:17-19). */
#define MG_FP4_MAX 6
#define MG_FP6_MAX 28
#define MG_FP8_MAX 448

/* Row pitches in bytes of the packed code buffers. */
static inline size_t mg_pitch_fp4(int k) { return (size_t)k / 2; }
static inline size_t mg_pitch_fp6(int k) { return (size_t)k / 4 * 3; }
static inline size_t mg_pitch_fp8(int k) { return (size_t)k; }

/*
 * Scale-factor layout of one segment: rows are tiled in blocks of 128 and K in blocks
 * of 128 elements (4 scales); each 128 x 4 block is a 512-byte atom in which
 * row r, scale kb sits at (r%32)*16 + (r/32)*4 + kb.  Atoms of one row block are
 * consecutive along K.  This is the layout the reference obtains from CUTLASS
 * (include/reorder.cuh:119-124) and addresses at src/reorder.cu:181-185; an atom can be
 * copied unchanged into tensor memory for a block-scaled tcgen05.mma.
 */
static inline size_t mg_sf_offset(int row, int kb, int kseg) {
  size_t katoms = (size_t)((kseg + 127) / 128);
  return (size_t)(row % 32) * 16 + (size_t)((row / 32) % 4) * 4 + (size_t)(kb % 4) +
         (size_t)(kb / 4) * 512 + (size_t)(row / 128) * 512 * katoms;
}

#ifdef __cplusplus
}
#endif
#endif
