/* Stand-in for CUTLASS's examples/common/helper.h, which the reference's headers include
 * (include/reorder.cuh:33) but which is absent from the header trees of this image.
 * The reference uses nothing from it on the reorder path. */
#pragma once
#include <cstdio>
#include <cuda_runtime.h>
#define CUDA_CHECK(status)                                                         \
  do {                                                                             \
    cudaError_t e_ = (status);                                                     \
    if (e_ != cudaSuccess) std::fprintf(stderr, "CUDA: %s\n", cudaGetErrorString(e_)); \
  } while (0)
