// Internal helpers shared by the translation units of libmixedgemm_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

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

// True unless MG_PDL=0: kernels are launched with programmatic stream serialisation, so that a
// kernel's prologue (barrier set-up, TMEM allocation, descriptor prefetch) overlaps the tail of
// the kernel before it; every kernel waits (griddepcontrol.wait) before it touches global memory.
bool pdl_enabled();

// <<<grid, block, smem, stream>>> with the programmatic-dependent-launch attribute when enabled.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace mg
