// Reorder-and-quantise kernels for sm_100a.
//
// One kernel template serves activations (FP4 / FP6 / FP8 by K segment) and weights
// (FP4 in all three segments).  It produces byte-for-byte what MixedGemm's
// reorder_bf16_mixed_kernel / reorder_bf16_fp4_kernel write (src/reorder.cu:94-432 of that
// project), but is organised for an HBM-bound B200:
//   * one persistent CTA per SM; a producer warp streams whole rows into a ring of
//     shared-memory stages with 1-D bulk copies (cp.async.bulk + mbarrier), R rows per stage,
//     while 16 consumer warps quantise the previous stage - loads, math and stores overlap;
//   * the reorder index stays in shared memory for the life of the CTA, pre-multiplied to
//     byte offsets;
//   * a thread owns one (row, 32-element group): lanes of a warp walk the R rows of the same
//     group, and rows are skewed by 16 bytes, so the channel gather hits distinct banks; tasks
//     are dealt round-robin to all threads, so every warp sees the same mix of formats;
//   * the group maximum, the E8M0 scale (exponent arithmetic, no log2) and the codes are
//     computed in registers: round-half-away-from-zero is a fused multiply-add against a magic
//     constant (FMA pipe) and the codes come from cvt.rn.satfinite.{e2m1x2,e3m2x2,e4m3x2}.f32;
//     codes leave as 16/8-byte vector stores.
// Waits on mbarriers are bounded; on expiry a code goes to the device status word and the
// CTA winds down (see wait_parity).
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp6.h>
#include <cuda_fp8.h>

#include "mg_common.h"
#include "ptx_sm100.cuh"

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;  // + one producer warp
constexpr int kRowSkew = 16;               // bytes added to the shared-memory row pitch

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
  int stages;
  long long wait_cycles;
  int* status;
};

// Bounded mbarrier wait; after a timeout every wait of the CTA returns at once.
__device__ __forceinline__ void wait_parity(uint32_t bar, uint32_t parity, volatile int* stop, int* status,
                                            long long limit, int code) {
  if (ptx::mbar_try_wait(bar, parity)) return;
  long long t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (ptx::mbar_try_wait(bar, parity)) return;
    if ((spin & 63u) == 0) {
      if (*stop) return;
      const long long now = clock64();
      if (spin == 0) t0 = now;
      if (now - t0 > limit) {
        *stop = 1;
        atomicOr(status, code);
        return;
      }
    }
  }
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

__device__ __forceinline__ unsigned lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// What a thread keeps for its row across the groups it quantises in one stage.
struct RowCtx {
  uint32_t smem_row;    // shared address of the staged row
  uint32_t sf_row;      // row part of the scale offset: (row%32)*16 + (row/32%4)*4
  uint32_t row_blk;     // row / 128
  uint32_t row;
};

// round(x * 2^e) to the nearest integer, halves away from zero, sign of x kept on a zero result.
// `rs` is 2^e * (1 + 2^-12): the fused multiply-add forms x * rs + 1.5 * 2^23 exactly and rounds it
// once, to nearest even, which leaves the wanted integer in the low mantissa bits.  The factor
// (1 + 2^-12) pushes an exact .5 just past the tie and is too small to move anything else across
// one (x has 8 significant bits, so every other product is at least x * 2^-8 away from a tie).
// Subtracting the constant gives the integer back as a float, and or-ing the sign of x restores
// "-0".  All three run on the FMA / ALU pipes; the conversion unit, which a round-to-integer
// instruction would occupy for sixteen cycles per warp, stays free for the code conversions.
__device__ __forceinline__ float scale_round(float x, float rs) {
  const float kMagic = 12582912.0f;
  const float r = __fadd_rn(__fmaf_rn(x, rs, kMagic), -kMagic);
  return __uint_as_float(__float_as_uint(r) | (__float_as_uint(x) & 0x80000000u));
}

// One (row, group): gather, scale, quantise, pack, store.
template <bool WEIGHTS>
__device__ __forceinline__ void quantise_group(const ReorderParams& p, const RowCtx& rc, uint32_t idx2_addr, int g) {
  float x[32];
  float maxv = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 iv = lds_v4(idx2_addr + g * 64 + q * 16);
    const unsigned o[4] = {iv.x, iv.y, iv.z, iv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const unsigned lo = lds_u16(rc.smem_row + (o[j] & 0xFFFFu));
      const unsigned hi = lds_u16(rc.smem_row + (o[j] >> 16));
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
  so.sf[rc.sf_row + (gs & 3) + (size_t)(gs >> 2) * 512 + (size_t)rc.row_blk * 512 * so.katoms] = (uint8_t)sf;
  const float rs = __uint_as_float(((unsigned)(254 - sf) << 23) | 0x800u);  // 2^(127-sf) * (1 + 2^-12)

#pragma unroll
  for (int i = 0; i < 32; ++i) x[i] = scale_round(x[i], rs);

  uint8_t* out = so.codes + (size_t)rc.row * so.pitch;
  if (fmt == 0) {
    unsigned wds[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      // four cvt.rn.satfinite.e2m1x2.f32 (first source -> high nibble) packed into one word
      asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
          "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
          "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
          "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
          "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
          "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
          : "=r"(wds[q])
          : "f"(x[q * 8]), "f"(x[q * 8 + 1]), "f"(x[q * 8 + 2]), "f"(x[q * 8 + 3]), "f"(x[q * 8 + 4]),
            "f"(x[q * 8 + 5]), "f"(x[q * 8 + 6]), "f"(x[q * 8 + 7]));
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

// One CTA's work: block `blk` of the `nblk` blocks that share the rows of problem p.
template <int R, bool WEIGHTS>
__device__ __forceinline__ void reorder_quantize_cta(const ReorderParams& p, int blk, int nblk) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = p.K;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.stages;
  const int pitch = 2 * K + kRowSkew;
  const int idx_bytes = (2 * K + 15) & ~15;
  uint16_t* idx2 = reinterpret_cast<uint16_t*>(smem);
  uint8_t* tiles = smem + idx_bytes;
  const int stage_bytes = R * pitch;
  uint8_t* tail = tiles + (size_t)S * stage_bytes;  // barriers: full[8], empty[8], then the stop flag
  const uint32_t bar0 = ptx::smem_u32(tail);
  volatile int* stop = reinterpret_cast<volatile int*>(tail + 16 * 8);

  ptx::grid_dep_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(bar0 + 8 * s, 1);                     // full: one expect_tx arrival + bytes
      ptx::mbar_init(bar0 + 8 * (8 + s), kConsumerWarps);  // empty: one arrival per consumer warp
    }
    *stop = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  ptx::grid_dep_wait();  // nothing before this line reads or writes global memory

  // This CTA's contiguous share of the rows, walked in stages of up to R rows.
  const int row_begin = (int)((long long)p.rows * blk / nblk);
  const int row_end = (int)((long long)p.rows * (blk + 1) / nblk);
  const int nstage = (row_end - row_begin + R - 1) / R;

  const int G = K >> 5;
  if (warp == kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < nstage; ++it, s = s + 1 == S ? 0 : s + 1, ph ^= (s == 0)) {
        wait_parity(bar0 + 8 * (8 + s), ph ^ 1u, stop, p.status, p.wait_cycles, 16);
        const int row0 = row_begin + it * R;
        const int nrows = min(R, row_end - row0);
        const uint32_t fb = bar0 + 8 * s;
        ptx::mbar_expect_tx(fb, (uint32_t)nrows * 2u * K);
        const uint32_t dst = ptx::smem_u32(tiles + (size_t)s * stage_bytes);
        for (int r = 0; r < nrows; ++r)
          ptx::bulk_load_1d(dst + r * pitch, p.X + (size_t)(row0 + r) * K, 2u * K, fb);
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers
    // the consumers bring the index in while the producer's first rows are already in flight
    // 16-byte loads, four in flight per thread: element-wise loads through a pointer the compiler must
    // assume may alias shared memory ran one after the other, 8 to 28 L2 round trips (4 to 15 us)
    // before the first row could be touched
    if ((reinterpret_cast<uintptr_t>(p.idx) & 15) == 0) {
      const uint4* src = reinterpret_cast<const uint4*>(p.idx);
      uint4* dst = reinterpret_cast<uint4*>(idx2);
      const int nv = K >> 3;
      const unsigned kmax = (unsigned)(K - 1);
      for (int base = 0; base < nv; base += 4 * kConsumers) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = base + u * kConsumers + tid;
          if (j < nv) v[u] = __ldg(src + j);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = base + u * kConsumers + tid;
          if (j < nv) {
            unsigned w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
              w[k] = (min(w[k] & 0xFFFFu, kmax) * 2u) | ((min(w[k] >> 16, kmax) * 2u) << 16);
            dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    } else {
      for (int i = tid; i < K; i += kConsumers) {
        unsigned v = (uint16_t)p.idx[i];
        v = min(v, (unsigned)(K - 1));
        idx2[i] = (uint16_t)(v * 2);
      }
    }
    ptx::named_barrier_sync(1, kConsumers);
    // a thread keeps its row
    constexpr int kGStep = kConsumers / R;
    const bool worker = tid < R * kGStep;
    const int r = tid % R;
    const int g0 = tid / R;
    const uint32_t idx2_addr = ptx::smem_u32(idx2);
    int s = 0;
    uint32_t ph = 0;
    for (int it = 0; it < nstage; ++it, s = s + 1 == S ? 0 : s + 1, ph ^= (s == 0)) {
      wait_parity(bar0 + 8 * s, ph, stop, p.status, p.wait_cycles, 32);
      const int row = row_begin + it * R + r;
      if (worker && row < row_end && !*stop) {
        RowCtx rc;
        rc.smem_row = ptx::smem_u32(tiles + (size_t)s * stage_bytes) + r * pitch;
        rc.sf_row = (uint32_t)(row & 31) * 16 + (uint32_t)((row >> 5) & 3) * 4;
        rc.row_blk = (uint32_t)row >> 7;
        rc.row = (uint32_t)row;
        for (int g = g0; g < G; g += kGStep) quantise_group<WEIGHTS>(p, rc, idx2_addr, g);
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar0 + 8 * (8 + s));
    }
  }
  __syncthreads();
  if (*stop) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let copies in flight land
  }
}

template <int R, bool WEIGHTS>
__global__ void __launch_bounds__(kThreads, 1) reorder_quantize_kernel(const __grid_constant__ ReorderParams p) {
  reorder_quantize_cta<R, WEIGHTS>(p, (int)blockIdx.x, (int)gridDim.x);
}

// Several independent problems (own input, index, K split and outputs) in one launch: the CTAs are
// dealt out to the problems in proportion to their bytes, so that a step's activations are quantised
// in one wave instead of one launch - and one partly filled wave - each.
constexpr int kMaxQuant = 8;
struct ReorderMulti {
  int nprob;
  int cta_end[kMaxQuant];  // problem j owns CTAs [cta_end[j-1], cta_end[j])
  int rows_per_stage[kMaxQuant];
  ReorderParams prob[kMaxQuant];
};

template <bool WEIGHTS>
__global__ void __launch_bounds__(kThreads, 1) reorder_quantize_multi_kernel(const __grid_constant__ ReorderMulti mp) {
  int j = 0, first = 0;
  while (j + 1 < mp.nprob && (int)blockIdx.x >= mp.cta_end[j]) first = mp.cta_end[j++];
  const ReorderParams& p = mp.prob[j];
  const int blk = (int)blockIdx.x - first, nblk = mp.cta_end[j] - first;
  switch (mp.rows_per_stage[j]) {
    case 8: reorder_quantize_cta<8, WEIGHTS>(p, blk, nblk); break;
    case 4: reorder_quantize_cta<4, WEIGHTS>(p, blk, nblk); break;
    case 2: reorder_quantize_cta<2, WEIGHTS>(p, blk, nblk); break;
    default: reorder_quantize_cta<1, WEIGHTS>(p, blk, nblk); break;
  }
}

size_t smem_bytes(int K, int R, int S) {
  return (size_t)((2 * K + 15) & ~15) + (size_t)S * R * (2 * K + kRowSkew) + 16 * 8 + 16;
}

template <int R, bool WEIGHTS>
int launch(const ReorderParams& p, int grid, size_t smem, cudaStream_t st) {
  auto kern = reorder_quantize_kernel<R, WEIGHTS>;
  if (smem > 48 * 1024) MG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MG_CUDA_TRY(mg::launch_kernel(kern, dim3(grid), dim3(kThreads), smem, st, p));
  return MG_OK;
}

// Checks one problem and fills its kernel parameters (everything but the stage shape, which depends
// on how many CTAs the problem gets).  MG_OK with p->rows == 0 means "nothing to do".
int fill_params(bool weights, const void* X, int rows, int K, const int16_t* idx, int KN, int KS, int KO, uint8_t* o4,
                uint8_t* o6, uint8_t* o8, const size_t* pitches, uint8_t* s4, uint8_t* s6, uint8_t* s8,
                ReorderParams* out) {
  out->rows = 0;
  if (rows < 0 || K <= 0 || KN < 0 || KS < 0 || KO < 0 || KN + KS + KO != K) return MG_ERR_SHAPE;
  if ((KN | KS | KO) & 31) return MG_ERR_SHAPE;
  if (K > 32736) return MG_ERR_SHAPE;  // int16 index
  if (rows == 0) return MG_OK;
  if (!X || !idx) return MG_ERR_NULL;
  if ((KN && (!o4 || !s4)) || (KS && (!o6 || !s6)) || (KO && (!o8 || !s8))) return MG_ERR_NULL;
  if (!mg::aligned(X, 16)) return MG_ERR_ALIGN;
  if (!mg::aligned(o4, 16) || !mg::aligned(o6, 8) || !mg::aligned(o8, 16)) return MG_ERR_ALIGN;

  ReorderParams& p = *out;
  p.X = static_cast<const uint16_t*>(X);
  p.idx = idx;
  p.rows = rows;
  p.K = K;
  p.g4 = KN / 32;
  p.g46 = (KN + KS) / 32;
  const size_t dense[3] = {(size_t)KN / 2, (size_t)(weights ? KS / 2 : KS / 4 * 3), (size_t)(weights ? KO / 2 : KO)};
  const size_t align[3] = {16, (size_t)(weights ? 16 : 8), 16};
  size_t pitch[3];
  for (int i = 0; i < 3; ++i) {
    pitch[i] = pitches && pitches[i] ? pitches[i] : dense[i];
    if (pitch[i] < dense[i] || pitch[i] > 0x7fffffffu) return MG_ERR_SHAPE;
    if (pitch[i] % align[i]) return MG_ERR_ALIGN;
  }
  p.seg[0] = {o4, s4, (KN + 127) / 128, (int)pitch[0]};
  p.seg[1] = {o6, s6, (KS + 127) / 128, (int)pitch[1]};
  p.seg[2] = {o8, s8, (KO + 127) / 128, (int)pitch[2]};
  p.wait_cycles = mg::wait_limit_cycles();
  return mg::device_status_word(&p.status);
}

// Rows per stage and stage count of a problem whose rows are shared by `grid` CTAs; returns the
// shared memory a CTA needs, or 0 when the problem does not fit.
size_t stage_shape(ReorderParams* p, int grid, size_t smem_optin, int* rows_per_stage) {
  const int K = p->K, rows = p->rows;
  const size_t budget = smem_optin - 1024;
  const int rows_per_cta = rows / grid;
  static const int kRs[] = {8, 4, 2, 1};
  int R = 1;
  for (int cand : kRs)
    if (smem_bytes(K, cand, 2) <= budget && (2 * cand <= rows_per_cta || cand == 1)) { R = cand; break; }
  int S = 2;
  while (S < 4 && smem_bytes(K, R, S + 1) <= budget) ++S;
  if (smem_bytes(K, R, 2) > budget) S = 1;
  const size_t smem = smem_bytes(K, R, S);
  if (smem > smem_optin) return 0;
  p->num_tiles = (rows + R - 1) / R;
  p->stages = S;
  *rows_per_stage = R;
  return smem;
}

int reorder_quantize(bool weights, const void* X, int rows, int K, const int16_t* idx, int KN, int KS,
                     int KO, uint8_t* o4, uint8_t* o6, uint8_t* o8, const size_t* pitches, uint8_t* s4, uint8_t* s6,
                     uint8_t* s8, void* stream) {
  ReorderParams p;
  int rc = fill_params(weights, X, rows, K, idx, KN, KS, KO, o4, o6, o8, pitches, s4, s6, s8, &p);
  if (rc != MG_OK || p.rows == 0) return rc;
  mg::DeviceInfo di;
  if ((rc = mg::device_info(&di)) != MG_OK) return rc;

  // Rows per stage (8, 4, 2 or 1): as many as fit twice (double buffering) beside the index, but no more than
  // half of a CTA's share so that its last stage is not mostly empty.  Then as many stages as
  // fit, up to 4.
  int grid = rows < di.sm_count ? rows : di.sm_count;  // rows are dealt out evenly, at least one per CTA
  const int cap = mg::options().reorder_ctas;  // a caller that runs another kernel beside this one may cap the grid
  if (cap > 0 && grid > cap) grid = cap;
  int R = 1;
  const size_t smem = stage_shape(&p, grid, (size_t)di.smem_optin, &R);
  if (smem == 0) return MG_ERR_SHAPE;
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

template <bool WEIGHTS>
int launch_multi(const ReorderMulti& mp, int grid, size_t smem, cudaStream_t st) {
  auto kern = reorder_quantize_multi_kernel<WEIGHTS>;
  if (smem > 48 * 1024) MG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MG_CUDA_TRY(mg::launch_kernel(kern, dim3(grid), dim3(kThreads), smem, st, mp));
  return MG_OK;
}

}  // namespace

extern "C" int mg_reorder_quantize_multi(int weights, int nprob, const mg_quant_problem_t* probs, void* stream) {
  if (nprob < 0 || nprob > kMaxQuant) return MG_ERR_SHAPE;
  if (nprob == 0) return MG_OK;
  if (!probs) return MG_ERR_NULL;
  mg::DeviceInfo di;
  int rc = mg::device_info(&di);
  if (rc != MG_OK) return rc;
  ReorderMulti mp;
  int n = 0;
  double bytes[kMaxQuant], total = 0;
  for (int j = 0; j < nprob; ++j) {
    const mg_quant_problem_t& q = probs[j];
    ReorderParams& p = mp.prob[n];
    rc = fill_params(weights != 0, q.X, q.rows, q.K, q.idx, q.KN, q.KS, q.KO, q.C4, q.C6, q.C8, q.pitch, q.SF4, q.SF6,
                     q.SF8, &p);
    if (rc != MG_OK) return rc;
    if (p.rows == 0) continue;
    // Cost of a problem = its elements, weighted by how well its rows pipeline: a row must be whole
    // in shared memory (the index may gather from anywhere in it), so a large K leaves room for only
    // one or two rows per stage and two or three stages, and a CTA then moves 1.5x / 1.3x fewer bytes
    // per second than with four or more rows per stage (measured per CTA with all SMs busy).
    int r_fit = 1;
    for (int cand : {8, 4, 2})
      if (smem_bytes(p.K, cand, 2) <= (size_t)di.smem_optin - 1024) { r_fit = cand; break; }
    bytes[n] = (double)p.rows * p.K * (r_fit == 1 ? 1.48 : r_fit == 2 ? 1.3 : 1.0);
    total += bytes[n];
    ++n;
  }
  if (n == 0) return MG_OK;
  // CTAs in proportion to the cost, at least one and at most one per row; one CTA per SM in all
  int sms = di.sm_count;
  const int cap = mg::options().reorder_ctas;
  if (cap > 0 && sms > cap) sms = cap;
  if (sms < n) sms = n;
  int share[kMaxQuant], used = 0;
  for (int j = 0; j < n; ++j) {
    int g = (int)(sms * bytes[j] / total);
    if (g < 1) g = 1;
    if (g > mp.prob[j].rows) g = mp.prob[j].rows;
    share[j] = g;
    used += g;
  }
  // what rounding down left over goes, one CTA at a time, to the problem whose CTAs carry the most
  while (used < sms) {
    int best = -1;
    for (int j = 0; j < n; ++j)
      if (share[j] < mp.prob[j].rows && (best < 0 || bytes[j] / share[j] > bytes[best] / share[best])) best = j;
    if (best < 0) break;
    ++share[best];
    ++used;
  }
  int grid = 0;
  size_t smem = 0;
  for (int j = 0; j < n; ++j) {
    const int g = share[j];
    const size_t sm = stage_shape(&mp.prob[j], g, (size_t)di.smem_optin, &mp.rows_per_stage[j]);
    if (sm == 0) return MG_ERR_SHAPE;
    if (sm > smem) smem = sm;
    grid += g;
    mp.cta_end[j] = grid;
  }
  for (int j = n; j < kMaxQuant; ++j) { mp.cta_end[j] = grid; mp.rows_per_stage[j] = 1; }
  mp.nprob = n;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return weights ? launch_multi<true>(mp, grid, smem, st) : launch_multi<false>(mp, grid, smem, st);
}

extern "C" int mg_reorder_quantize_x(const void* X, int M, int K, const int16_t* idx, int KN, int KS, int KO,
                                     uint8_t* AN, uint8_t* AS, uint8_t* AO, uint8_t* SFAN, uint8_t* SFAS,
                                     uint8_t* SFAO, void* stream) {
  return reorder_quantize(false, X, M, K, idx, KN, KS, KO, AN, AS, AO, nullptr, SFAN, SFAS, SFAO, stream);
}

extern "C" int mg_reorder_quantize_w(const void* W, int N, int K, const int16_t* idx, int KN, int KS, int KO,
                                     uint8_t* BN, uint8_t* BS, uint8_t* BO, uint8_t* SFBN, uint8_t* SFBS,
                                     uint8_t* SFBO, void* stream) {
  return reorder_quantize(true, W, N, K, idx, KN, KS, KO, BN, BS, BO, nullptr, SFBN, SFBS, SFBO, stream);
}

extern "C" int mg_reorder_quantize_pitched(int weights, const void* X, int rows, int K, const int16_t* idx, int KN,
                                           int KS, int KO, uint8_t* C4, uint8_t* C6, uint8_t* C8,
                                           const size_t* pitches, uint8_t* SF4, uint8_t* SF6, uint8_t* SF8,
                                           void* stream) {
  return reorder_quantize(weights != 0, X, rows, K, idx, KN, KS, KO, C4, C6, C8, pitches, SF4, SF6, SF8, stream);
}

extern "C" size_t mg_code_pitch(int weights, int segment, int kseg) {
  const int kp = (kseg + 127) / 128 * 128;
  if (segment == 0 || weights) return (size_t)kp / 2;
  return segment == 1 ? (size_t)kp / 4 * 3 : (size_t)kp;
}
