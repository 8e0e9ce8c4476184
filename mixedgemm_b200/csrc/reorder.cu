// Reorder-and-quantise kernels for sm_100a.
//
// One kernel template serves activations (FP4 / FP6 / FP8 by K segment) and weights
// (FP4 in all three segments).  It produces byte-for-byte what MixedGemm's
// reorder_bf16_mixed_kernel / reorder_bf16_fp4_kernel write (src/reorder.cu:94-432 of that
// project), but is organised for an HBM-bound B200:
//   * a CTA stages R whole rows in shared memory with 128-bit coalesced loads and keeps
//     the reorder index there, pre-multiplied to byte offsets, for all its row tiles;
//   * a thread owns one (row, 32-element group): lanes of a warp walk R rows of the same
//     group, and rows are skewed by 16 bytes, so the channel gather hits distinct banks;
//   * the group maximum, the E8M0 scale (exponent arithmetic, no log2) and the codes are
//     computed in registers; codes leave as 16/8-byte vector stores;
//   * float -> E2M1/E3M2/E4M3 uses the sm_100 cvt.rn.satfinite.*x2 instructions.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp6.h>
#include <cuda_fp8.h>

#include "mg_common.h"

namespace {

constexpr int kThreads = 256;
constexpr int kRowSkew = 16;  // bytes added to the shared-memory row pitch

struct SegOut {
  uint8_t* codes;  // packed codes of this segment
  uint8_t* sf;     // swizzled scale bytes
  int katoms;      // ceil(kseg / 128)
  int pitch;       // bytes per row of `codes`
};

struct ReorderParams {
  const uint16_t* X;
  const int16_t* idx;
  int rows, K;
  int g4, g46;  // groups in segment 0, in segments 0+1
  SegOut seg[3];
  int num_tiles;
};

__device__ __forceinline__ int4 ld_stream16(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Integer nearest, halves away from zero, sign kept on zero: roundf() for |t| < 2^22.
__device__ __forceinline__ float round_half_away(float t) {
  float h = __uint_as_float((__float_as_uint(t) & 0x80000000u) | 0x3f000000u);
  return truncf(t + h);
}

// E8M0 byte of the smallest power of two 2^e with maxv <= fmt_max * 2^e, from the bf16
// bit pattern of maxv (fmt_max = 1.5 * 2^2, 1.75 * 2^4, 1.75 * 2^8).
__device__ __forceinline__ int scale_byte(float maxv, int fmt) {
  unsigned a = __float_as_uint(maxv) >> 16;
  int E = (int)(a >> 7), m = (int)(a & 0x7F);
  int sh = fmt == 0 ? 2 : fmt == 1 ? 4 : 8;
  int thr = fmt == 0 ? 64 : 96;
  int sf = E - sh + (m > thr ? 1 : 0);
  sf = max(0, min(254, sf));
  return a == 0 ? 126 : sf;
}

template <int R, bool WEIGHTS>
__global__ void __launch_bounds__(kThreads) reorder_quantize_kernel(const ReorderParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = p.K;
  const int tid = threadIdx.x;
  uint16_t* idx2 = reinterpret_cast<uint16_t*>(smem);
  uint8_t* tile = smem + ((2 * K + 15) & ~15);
  const int pitch = 2 * K + kRowSkew;

  for (int i = tid; i < K; i += kThreads) {
    unsigned v = (uint16_t)p.idx[i];
    v = min(v, (unsigned)(K - 1));
    idx2[i] = (uint16_t)(v * 2);
  }

  const int G = K >> 5;
  const int chunks = K >> 3;  // 16-byte chunks per row

  for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
    const int row0 = t * R;
    __syncthreads();  // the previous tile has been consumed (and idx2 is written)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool live = row0 + r < p.rows;
      const uint16_t* src = p.X + (size_t)(row0 + r) * K;
#pragma unroll 2
      for (int c = tid; c < chunks; c += kThreads) {
        int4 v = make_int4(0, 0, 0, 0);
        if (live) v = ld_stream16(src + c * 8);
        *reinterpret_cast<int4*>(tile + r * pitch + c * 16) = v;
      }
    }
    __syncthreads();

    for (int w = tid; w < R * G; w += kThreads) {
      const int r = w % R, g = w / R;
      const int row = row0 + r;
      if (row >= p.rows) continue;
      const uint8_t* rowp = tile + r * pitch;
      const uint4* ip = reinterpret_cast<const uint4*>(idx2 + g * 32);

      float x[32];
      float maxv = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 iv = ip[q];
        const unsigned o[4] = {iv.x, iv.y, iv.z, iv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          unsigned lo = *reinterpret_cast<const uint16_t*>(rowp + (o[j] & 0xFFFFu));
          unsigned hi = *reinterpret_cast<const uint16_t*>(rowp + (o[j] >> 16));
          x[q * 8 + j * 2] = __uint_as_float(lo << 16);
          x[q * 8 + j * 2 + 1] = __uint_as_float(hi << 16);
          maxv = fmaxf(maxv, fmaxf(fabsf(x[q * 8 + j * 2]), fabsf(x[q * 8 + j * 2 + 1])));
        }
      }

      const int seg = g < p.g4 ? 0 : (g < p.g46 ? 1 : 2);
      const int gs = g - (seg == 0 ? 0 : (seg == 1 ? p.g4 : p.g46));
      const int fmt = WEIGHTS ? 0 : seg;
      const SegOut so = seg == 0 ? p.seg[0] : (seg == 1 ? p.seg[1] : p.seg[2]);

      const int sf = scale_byte(maxv, fmt);
      so.sf[(size_t)(row & 31) * 16 + (size_t)((row >> 5) & 3) * 4 + (gs & 3) + (size_t)(gs >> 2) * 512 +
            (size_t)(row >> 7) * 512 * so.katoms] = (uint8_t)sf;
      const float rs = __uint_as_float((unsigned)(254 - sf) << 23);  // 2^(127-sf)

#pragma unroll
      for (int i = 0; i < 32; ++i) x[i] = round_half_away(x[i] * rs);

      uint8_t* out = so.codes + (size_t)row * so.pitch;
      if (fmt == 0) {
        unsigned wds[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          unsigned wd = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            unsigned b = __nv_cvt_float2_to_fp4x2(make_float2(x[q * 8 + j * 2], x[q * 8 + j * 2 + 1]),
                                                  __NV_E2M1, cudaRoundNearest);
            wd |= (b & 0xFFu) << (8 * j);
          }
          wds[q] = wd;
        }
        *reinterpret_cast<uint4*>(out + (size_t)gs * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
      } else if (fmt == 1) {
        unsigned w24[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          unsigned p01 = __nv_cvt_float2_to_fp6x2(make_float2(x[q * 4], x[q * 4 + 1]), __NV_E3M2, cudaRoundNearest);
          unsigned p23 = __nv_cvt_float2_to_fp6x2(make_float2(x[q * 4 + 2], x[q * 4 + 3]), __NV_E3M2, cudaRoundNearest);
          w24[q] = (p01 & 0x3Fu) | ((p01 >> 2) & 0xFC0u) | ((p23 & 0x3Fu) << 12) | ((p23 & 0x3F00u) << 10);
        }
        unsigned ow[6];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const unsigned a = w24[h * 4], b = w24[h * 4 + 1], c = w24[h * 4 + 2], d = w24[h * 4 + 3];
          ow[h * 3] = a | (b << 24);
          ow[h * 3 + 1] = (b >> 8) | (c << 16);
          ow[h * 3 + 2] = (c >> 16) | (d << 8);
        }
        uint2* o8 = reinterpret_cast<uint2*>(out + (size_t)gs * 24);
        o8[0] = make_uint2(ow[0], ow[1]);
        o8[1] = make_uint2(ow[2], ow[3]);
        o8[2] = make_uint2(ow[4], ow[5]);
      } else {
        unsigned wds[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          unsigned wd = 0;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            // the reference rounds the integer to bf16 before the E4M3 conversion
            float a = __bfloat162float(__float2bfloat16_rn(x[q * 4 + j * 2]));
            float b = __bfloat162float(__float2bfloat16_rn(x[q * 4 + j * 2 + 1]));
            unsigned h = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
            wd |= (h & 0xFFFFu) << (16 * j);
          }
          wds[q] = wd;
        }
        uint4* o16 = reinterpret_cast<uint4*>(out + (size_t)gs * 32);
        o16[0] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
        o16[1] = make_uint4(wds[4], wds[5], wds[6], wds[7]);
      }
    }
  }
}

size_t smem_bytes(int K, int R) { return (size_t)((2 * K + 15) & ~15) + (size_t)R * (2 * K + kRowSkew); }

template <int R, bool WEIGHTS>
int launch(const ReorderParams& p, int grid, size_t smem, cudaStream_t st) {
  auto kern = reorder_quantize_kernel<R, WEIGHTS>;
  if (smem > 48 * 1024) MG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, kThreads, smem, st>>>(p);
  MG_CUDA_TRY(cudaGetLastError());
  return MG_OK;
}

int reorder_quantize(bool weights, const void* X, int rows, int K, const int16_t* idx, int KN, int KS,
                     int KO, uint8_t* o4, uint8_t* o6, uint8_t* o8, uint8_t* s4, uint8_t* s6, uint8_t* s8,
                     void* stream) {
  if (rows < 0 || K <= 0 || KN < 0 || KS < 0 || KO < 0 || KN + KS + KO != K) return MG_ERR_SHAPE;
  if ((KN | KS | KO) & 31) return MG_ERR_SHAPE;
  if (K > 32736) return MG_ERR_SHAPE;  // int16 index
  if (rows == 0) return MG_OK;
  if (!X || !idx) return MG_ERR_NULL;
  if ((KN && (!o4 || !s4)) || (KS && (!o6 || !s6)) || (KO && (!o8 || !s8))) return MG_ERR_NULL;
  if (!mg::aligned(X, 16)) return MG_ERR_ALIGN;
  if (!mg::aligned(o4, 16) || !mg::aligned(o6, 8) || !mg::aligned(o8, 16)) return MG_ERR_ALIGN;

  mg::DeviceInfo di;
  int rc = mg::device_info(&di);
  if (rc != MG_OK) return rc;

  ReorderParams p;
  p.X = static_cast<const uint16_t*>(X);
  p.idx = idx;
  p.rows = rows;
  p.K = K;
  p.g4 = KN / 32;
  p.g46 = (KN + KS) / 32;
  p.seg[0] = {o4, s4, (KN + 127) / 128, KN / 2};
  p.seg[1] = {o6, s6, (KS + 127) / 128, weights ? KS / 2 : KS / 4 * 3};
  p.seg[2] = {o8, s8, (KO + 127) / 128, weights ? KO / 2 : KO};

  // Rows per tile: as many as keep three CTAs on an SM, fewer when that would leave SMs idle.
  int R = 8;
  while (R > 1 && (smem_bytes(K, R) > 74 * 1024 || (rows + R - 1) / R < di.sm_count)) R >>= 1;
  const size_t smem = smem_bytes(K, R);
  if (smem > (size_t)di.smem_optin) return MG_ERR_SHAPE;
  p.num_tiles = (rows + R - 1) / R;
  int per_sm = (int)((size_t)228 * 1024 / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  int grid = p.num_tiles < di.sm_count * per_sm ? p.num_tiles : di.sm_count * per_sm;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

#define MG_LAUNCH_R(RR)                                                            \
  case RR:                                                                         \
    return weights ? launch<RR, true>(p, grid, smem, st) : launch<RR, false>(p, grid, smem, st);
  switch (R) {
    MG_LAUNCH_R(8)
    MG_LAUNCH_R(4)
    MG_LAUNCH_R(2)
    MG_LAUNCH_R(1)
  }
#undef MG_LAUNCH_R
  return MG_ERR_SHAPE;
}

}  // namespace

extern "C" int mg_reorder_quantize_x(const void* X, int M, int K, const int16_t* idx, int KN, int KS, int KO,
                                     uint8_t* AN, uint8_t* AS, uint8_t* AO, uint8_t* SFAN, uint8_t* SFAS,
                                     uint8_t* SFAO, void* stream) {
  return reorder_quantize(false, X, M, K, idx, KN, KS, KO, AN, AS, AO, SFAN, SFAS, SFAO, stream);
}

extern "C" int mg_reorder_quantize_w(const void* W, int N, int K, const int16_t* idx, int KN, int KS, int KO,
                                     uint8_t* BN, uint8_t* BS, uint8_t* BO, uint8_t* SFBN, uint8_t* SFBS,
                                     uint8_t* SFBO, void* stream) {
  return reorder_quantize(true, W, N, K, idx, KN, KS, KO, BN, BS, BO, SFBN, SFBS, SFBO, stream);
}
