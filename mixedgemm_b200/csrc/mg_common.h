// Internal helpers shared by the translation units of libmixedgemm_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "mixedgemm_c.h"

namespace mg {

// Records the failing cudaError_t for mg_last_cuda_error() and maps it to MG_ERR_CUDA.
int note_cuda_error(cudaError_t e);

#define MG_CUDA_TRY(expr)                                   \
  do {                                                      \
    cudaError_t mg_e_ = (expr);                             \
    if (mg_e_ != cudaSuccess) return mg::note_cuda_error(mg_e_); \
  } while (0)

// Number of SMs and opt-in shared memory of the current device (cached per device).
struct DeviceInfo {
  int sm_count;
  int smem_optin;
  int cc_major;
};
int device_info(DeviceInfo* out);

// Address of the device-side error word (one per device, set by kernels whose bounded
// waits expire).  Resolved with cudaGetSymbolAddress in capi.cu.
int device_status_word(int** dev_ptr);

static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace mg
