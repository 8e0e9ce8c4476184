// Reorder-index calibration: per-channel absmax over the rows of X, then the stable ascending
// argsort of those maxima as int16 - the index MixedGemm's quantisers take.  The reference
// computes it outside its module, in torch (main.py:31-33, commented out there and with an
// unstable sort); here it is two small kernels with no scratch memory.
//
//   column_absmax_kernel  one CTA per 128 channels, 16 x 16 threads: a thread reads 8 channels
//                         (16 bytes) of every 16th row and keeps the largest magnitude bits
//                         (for non-negative bf16, integer order of the bits is numeric order)
//   stable_rank_kernel    every CTA holds all K keys in shared memory; thread i counts the keys
//                         smaller than key_i plus the equal keys left of i: that count is the
//                         position of channel i in the stable ascending order
#include "mg_common.h"
#include "ptx_sm100.cuh"

namespace {

constexpr int kColsPerCta = 128;

__global__ void __launch_bounds__(256) column_absmax_kernel(const uint16_t* __restrict__ X, int M, int K,
                                                            uint16_t* __restrict__ keys) {
  ptx::grid_dep_launch_dependents();
  ptx::grid_dep_wait();
  __shared__ uint32_t red[16][64];  // [row lane][channel pair]
  const int cx = threadIdx.x & 15, ry = threadIdx.x >> 4;
  const int col0 = blockIdx.x * kColsPerCta + cx * 8;
  uint32_t m[4] = {0, 0, 0, 0};  // two 15-bit magnitudes per word
  if (col0 < K) {
    for (int r = ry; r < M; r += 16) {
      const uint4 v = *reinterpret_cast<const uint4*>(X + (size_t)r * K + col0);
      const uint32_t w[4] = {v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu, v.z & 0x7FFF7FFFu, v.w & 0x7FFF7FFFu};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = max(m[i] & 0xFFFFu, w[i] & 0xFFFFu), hi = max(m[i] >> 16, w[i] >> 16);
        m[i] = lo | (hi << 16);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) red[ry][cx * 4 + i] = m[i];
  __syncthreads();
  if (threadIdx.x < 64) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const uint32_t w = red[r][threadIdx.x];
      lo = max(lo, w & 0xFFFFu);
      hi = max(hi, w >> 16);
    }
    const int c = blockIdx.x * kColsPerCta + threadIdx.x * 2;
    if (c < K) *reinterpret_cast<uint32_t*>(keys + c) = lo | (hi << 16);
  }
}

__global__ void __launch_bounds__(256) stable_rank_kernel(const uint16_t* __restrict__ keys, int K,
                                                          int16_t* __restrict__ idx) {
  extern __shared__ uint16_t sk[];
  ptx::grid_dep_launch_dependents();
  ptx::grid_dep_wait();
  for (int j = threadIdx.x; j < K; j += blockDim.x) sk[j] = keys[j];
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= K) return;
  const uint32_t ki = sk[i];
  int rank = 0;
  for (int j = 0; j < i; ++j) rank += sk[j] <= ki;  // equal keys left of i come first
  for (int j = i + 1; j < K; ++j) rank += sk[j] < ki;
  idx[rank] = (int16_t)i;
}

}  // namespace

// absmax_bits receives the per-channel maxima (bf16 bit patterns, sign cleared); it is an
// output in its own right and the sort's input, so no scratch memory is involved.
extern "C" int mg_reorder_index(const void* X, int M, int K, int16_t* idx, uint16_t* absmax_bits, void* stream) {
  if (M <= 0 || K <= 0 || K % 8 || K > 32736) return MG_ERR_SHAPE;
  if (!X || !idx || !absmax_bits) return MG_ERR_NULL;
  if (!mg::aligned(X, 16) || !mg::aligned(absmax_bits, 4)) return MG_ERR_ALIGN;
  mg::DeviceInfo di;
  int rc = mg::device_info(&di);
  if (rc != MG_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ctas = (K + kColsPerCta - 1) / kColsPerCta;
  MG_CUDA_TRY(mg::launch_kernel(column_absmax_kernel, dim3(ctas), dim3(256), 0, st, static_cast<const uint16_t*>(X), M, K,
                                absmax_bits));
  const size_t smem = (size_t)K * 2;
  if (smem > 48 * 1024)
    MG_CUDA_TRY(cudaFuncSetAttribute(stable_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MG_CUDA_TRY(mg::launch_kernel(stable_rank_kernel, dim3((K + 255) / 256), dim3(256), smem, st,
                                static_cast<const uint16_t*>(absmax_bits), K, idx));
  return MG_OK;
}
