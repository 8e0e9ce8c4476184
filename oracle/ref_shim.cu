/*
 * C entry points around the reference's own launchers, so that tests can run the
 * reference reorder kernels on the GPU and compare bytes.  TEST INFRASTRUCTURE ONLY.
 *
 * Only declarations appear here: the definitions (and the explicit instantiations for
 * K in {4096, 3584, 5120, 14336, 18944, 12288, 13824}, src/reorder.cu:508-576) come from
 * the reference's src/reorder.cu, compiled where it lies by oracle/build_oracle.py.
 * The reference's GEMM sources are never built: they target sm_120 and trap elsewhere.
 */
#include <cstdint>
#include <cuda_runtime.h>
#include "cutlass/numeric_types.h"

typedef cutlass::float_ue8m0_t sf_t;
typedef cutlass::bfloat16_t bf16_t;

/* include/reorder.cuh:295-323 */
template <int group_size, int hidden_dim>
void run_reorder_bf16_mixed(bf16_t*, int, int, int16_t*, uint8_t*, uint8_t*, uint8_t*, sf_t*, sf_t*,
                            sf_t*, int, int, int);
template <int group_size, int hidden_dim>
void run_reorder_bf16_fp4(bf16_t*, int, int, int16_t*, uint8_t*, uint8_t*, uint8_t*, sf_t*, sf_t*,
                          sf_t*, int, int, int);

#define DISPATCH_K(FN)                                                                 \
  switch (K) {                                                                         \
    case 4096:  FN<32, 4096>(ARGS);  break;                                            \
    case 3584:  FN<32, 3584>(ARGS);  break;                                            \
    case 5120:  FN<32, 5120>(ARGS);  break;                                            \
    case 14336: FN<32, 14336>(ARGS); break;                                            \
    case 18944: FN<32, 18944>(ARGS); break;                                            \
    case 12288: FN<32, 12288>(ARGS); break;                                            \
    case 13824: FN<32, 13824>(ARGS); break;                                            \
    default: return -1;                                                                \
  }

#define ARGS (bf16_t*)X, rows_m, rows_n, idx, o4, o6, o8, (sf_t*)s4, (sf_t*)s6, (sf_t*)s8, KN, KS, KO

extern "C" int ref_supports_k(int K) {
  return K == 4096 || K == 3584 || K == 5120 || K == 14336 || K == 18944 || K == 12288 || K == 13824;
}

/* Device pointers in, device buffers out; returns 0, -1 (K not instantiated) or a cudaError. */
extern "C" int ref_reorder_quantize_x(void* X, int rows_m, int rows_n, int K, int16_t* idx, int KN,
                                      int KS, int KO, uint8_t* o4, uint8_t* o6, uint8_t* o8,
                                      uint8_t* s4, uint8_t* s6, uint8_t* s8) {
  DISPATCH_K(run_reorder_bf16_mixed)
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaDeviceSynchronize();
}

extern "C" int ref_reorder_quantize_w(void* X, int rows_m, int rows_n, int K, int16_t* idx, int KN,
                                      int KS, int KO, uint8_t* o4, uint8_t* o6, uint8_t* o8,
                                      uint8_t* s4, uint8_t* s6, uint8_t* s8) {
  DISPATCH_K(run_reorder_bf16_fp4)
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaDeviceSynchronize();
}
