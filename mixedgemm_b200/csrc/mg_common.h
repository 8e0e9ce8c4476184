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

// Switches that choose between kernels or turn a mode off (mg_set_option / mg_get_option).  Each is
// read from the environment (MG_<NAME>) once, when the library is first used, and can be changed at
// run time through the C ABI; -1 stands for "let the library decide".
struct Options {
  int gemm_bn;        // GEMM_BN: 128 / 256 forces the tile width of the single-CTA kernel
  int gemm_2cta;      // GEMM_2CTA: 0 / 1 forces the CTA-pair kernel off / on where it applies
  int gemm_csplit;    // GEMM_CSPLIT: 0 turns the cluster split-K form off
  int gemm_splitk;    // GEMM_SPLITK: 0 turns split-K through the workspace off, n > 0 forces n splits
  int gemm_swap;      // GEMM_SWAP: 0 / 1 forces the decode form (weights as the 128-row operand) off / on
  int gemm_sched;     // GEMM_SCHED: 0 deals the CTA-pair kernel's tiles out round-robin instead of by cost
  int gemm_max_clusters;  // GEMM_MAX_CLUSTERS: n > 0 caps the SM pairs the CTA-pair kernel uses
  int pdl;            // PDL: 0 launches without programmatic dependent launch
  int reorder_ctas;   // REORDER_CTAS: n > 0 caps the quantiser's grid (to share the GPU with another kernel)
  int fault_skip_load;  // FAULT_SKIP_LOAD: n > 0 makes the GEMM's first CTA withhold its n-th stage load
                        // (host-side fault injection for the bounded-wait test; the kernel then gives up
                        // after the wait limit and returns normally)
};
Options options();

// True unless the PDL option is 0: kernels are launched with programmatic stream serialisation, so
// that a kernel's prologue (barrier set-up, TMEM allocation, descriptor prefetch) overlaps the tail
// of the kernel before it; every kernel waits (griddepcontrol.wait) before it touches global memory.
bool pdl_enabled();

// Limit of every bounded wait inside the kernels, in SM clock cycles (about one second unless
// mg_set_wait_limit_us changed it).
long long wait_limit_cycles();

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
