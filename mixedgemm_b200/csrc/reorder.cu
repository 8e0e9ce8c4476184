// Reorder-and-quantise kernels for sm_100a.
//
// One kernel template serves activations (FP4 / FP6 / FP8 by K segment) and weights
// (FP4 in all three segments).  It produces byte-for-byte what MixedGemm's
// reorder_bf16_mixed_kernel / reorder_bf16_fp4_kernel write (src/reorder.cu:94-432 of that
// project), but is organised for an HBM-bound B200.  The channel gather is a random 2-byte
// access per element, so the cost that matters is shared-memory wavefronts and instructions
// per element, not DRAM traffic:
//   * one persistent CTA per SM (16 warps, so that a thread may keep 128 registers) works on PAIRS
//     of rows.  Whole rows stream into a ring of shared-memory stages with 1-D bulk copies
//     (cp.async.bulk + mbarrier), issued by one thread two stages ahead;
//   * when a stage has landed the warps interleave the two rows of every pair in place with
//     ldmatrix.trans / stmatrix (two instructions per 512 bytes, no bank conflicts): afterwards
//     one 32-bit shared-memory word holds a channel for both rows.  One CTA barrier per stage
//     separates this from the gather and tells the copying thread that the previous stage's
//     buffer is free;
//   * then every thread quantises.  A thread owns one (pair slot of the stage, 32-element group)
//     task (two for K > 16384) for the life of the CTA and keeps the 32 shared-memory offsets of
//     its channels in registers, so a gather is one ld.shared.b32 per channel and row pair with
//     no index fetch and no address arithmetic.  Tasks are dealt to threads sorted by format, so
//     that a warp converts to one format (at most two warps straddle a boundary) and the FP6 /
//     FP8 warps are spread evenly over the four schedulers;
//   * group maxima come from max.xorsign.abs.bf16x2 on the packed pair, the E8M0 scale from
//     exponent arithmetic (no log2), round-half-away-from-zero from a 1-ulp nudge and a
//     magic-number add on the FMA pipe (the conversion unit is the scarce pipe), the codes from
//     cvt.rn.satfinite.{e2m1x2,e3m2x2,e4m3x2}.f32; codes leave as 16/8-byte vector stores.
// Waits on mbarriers are bounded; on expiry a code goes to the device status word and the
// CTA winds down (see wait_parity).
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp6.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "mg_common.h"
#include "ptx_sm100.cuh"

namespace {

constexpr int kWarps = 16;
constexpr int kConsumers = kWarps * 32;
constexpr int kThreads = kConsumers;
constexpr int kMaxStages = 4;

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
  int pairs;        // row pairs in all: ceil(rows / 2)
  int P;            // row pairs per stage
  int stages;       // ring depth
  int pitch;        // bytes between the two rows of a pair (and between rows of a stage)
  long long wait_cycles;
  int* status;
  uint8_t chunk_of_warp[kWarps];  // which 32 consecutive tasks warp w takes (balances the schedulers)
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

// E8M0 byte of the smallest power of two 2^e with maxv <= fmt_max * 2^e, from the 15-bit
// magnitude of the bf16 maximum (fmt_max = 1.5 * 2^2, 1.75 * 2^4, 1.75 * 2^8).
__device__ __forceinline__ int scale_byte(unsigned a, int fmt) {
  int E = (int)(a >> 7), m = (int)(a & 0x7F);
  int sh = fmt == 0 ? 2 : fmt == 1 ? 4 : 8;
  int thr = fmt == 0 ? 64 : 96;
  int sf = E - sh + (m > thr ? 1 : 0);
  sf = max(0, min(254, sf));
  return a == 0 ? 126 : sf;
}

// max(|a|, |b|) per bf16 half; the sign bit of a result is the xor of the operands' signs
__device__ __forceinline__ uint32_t max_abs_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Four 8x8 b16 matrices: lane l names row l%8 of matrix l/8; .trans hands thread T, for matrix k,
// the elements [2(T%4)][T/4] (low half) and [2(T%4)+1][T/4] (high half).
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, const uint32_t (&r)[4]) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3])
               : "memory");
}

// Where channel c of a row pair sits after the transposer has been over it, in bytes from the
// first row of the pair.  A warp step takes 256 bytes (16 chunks of 8 channels) of both rows as
// four 8x8 matrices (matrix k: chunks 4k..4k+3, matrix row 2*chunk + row of the pair) and writes
// the transposed matrices back over them: matrix k goes to row k/2 of the pair, 16-byte unit
// (k%2)*8 + j for channel j of a chunk, word chunk%4 inside the unit.
__device__ __forceinline__ uint32_t pair_offset(uint32_t c, uint32_t pitch) {
  const uint32_t chunk = c >> 3, j = c & 7u;
  const uint32_t w = chunk >> 4, k = (chunk >> 2) & 3u, cl = chunk & 3u;
  return (k >> 1) * pitch + w * 256u + (((k & 1u) << 3) + j) * 16u + cl * 4u;
}

// the bf16 in half H of a packed pair as fp32
template <int H>
__device__ __forceinline__ float unpack(uint32_t w) {
  return __uint_as_float(H ? (w & 0xFFFF0000u) : (w << 16));
}

// round(x * 2^e) to the nearest integer, halves away from zero, sign of x kept on a zero result.
// `rs` is 2^e * (1 + 2^-12): the fused multiply-add forms x * rs + 1.5 * 2^23 exactly and rounds it
// once, to nearest even, which leaves the wanted integer in the low mantissa bits.  The factor
// (1 + 2^-12) pushes an exact .5 just past the tie and is too small to move anything else across
// one (x has 8 significant bits, so every other product is at least x * 2^-8 away from a tie).
// Subtracting the constant gives the integer back as a float (both operations on the FMA pipe,
// the conversion unit is the scarce one), and or-ing the sign of x restores "-0".
__device__ __forceinline__ float scale_round(float x, float rs) {
  const float kMagic = 12582912.0f;
  const float r = __fadd_rn(__fmaf_rn(x, rs, kMagic), -kMagic);
  return __uint_as_float(__float_as_uint(r) | (__float_as_uint(x) & 0x80000000u));
}

__device__ __forceinline__ unsigned pack_e2m1x8(const float* x) {
  unsigned w;
  // four cvt.rn.satfinite.e2m1x2.f32 (first source -> high nibble) packed into one word
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(w)
      : "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7]));
  return w;
}

// Quantise the 32 values of row H of the pair and store codes; `out` points at this group's
// bytes in that row.  Scaling and rounding are the same for every format and sit outside the
// format branches, so a warp that holds two formats repeats only the conversion.
template <int H>
__device__ __forceinline__ void quantise_row(const uint32_t (&v)[32], int fmt, float rs, uint8_t* out) {
  unsigned o[8];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    float x[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) x[j] = scale_round(unpack<H>(v[c * 16 + j]), rs);
    if (fmt == 0) {
      o[c * 2] = pack_e2m1x8(x);
      o[c * 2 + 1] = pack_e2m1x8(x + 8);
    } else if (fmt == 1) {
      unsigned w24[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        unsigned p01 = __nv_cvt_float2_to_fp6x2(make_float2(x[q * 4], x[q * 4 + 1]), __NV_E3M2, cudaRoundNearest);
        unsigned p23 = __nv_cvt_float2_to_fp6x2(make_float2(x[q * 4 + 2], x[q * 4 + 3]), __NV_E3M2, cudaRoundNearest);
        w24[q] = (p01 & 0x3Fu) | ((p01 >> 2) & 0xFC0u) | ((p23 & 0x3Fu) << 12) | ((p23 & 0x3F00u) << 10);
      }
      o[c * 3] = w24[0] | (w24[1] << 24);
      o[c * 3 + 1] = (w24[1] >> 8) | (w24[2] << 16);
      o[c * 3 + 2] = (w24[2] >> 16) | (w24[3] << 8);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        unsigned wd = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          // the reference rounds the integer to bf16 before the E4M3 conversion
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(x[q * 4 + j * 2], x[q * 4 + j * 2 + 1]);
          const unsigned hb = *reinterpret_cast<const unsigned*>(&h2);
          unsigned h = __nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(hb << 16), __uint_as_float(hb & 0xFFFF0000u)),
                                               __NV_SATFINITE, __NV_E4M3);
          wd |= (h & 0xFFFFu) << (16 * j);
        }
        o[c * 4 + q] = wd;
      }
    }
  }
  if (fmt == 0) {
    *reinterpret_cast<uint4*>(out) = make_uint4(o[0], o[1], o[2], o[3]);
  } else if (fmt == 1) {
    uint2* o8 = reinterpret_cast<uint2*>(out);
    o8[0] = make_uint2(o[0], o[1]);
    o8[1] = make_uint2(o[2], o[3]);
    o8[2] = make_uint2(o[4], o[5]);
  } else {
    uint4* o16 = reinterpret_cast<uint4*>(out);
    o16[0] = make_uint4(o[0], o[1], o[2], o[3]);
    o16[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// What a consumer thread knows about one group it owns.
struct GroupCtx {
  uint8_t* codes;    // segment's code buffer + this group's byte offset in a row
  uint8_t* sf;       // segment's scale buffer + (gs % 4) + (gs / 4) * 512
  uint32_t pitch;    // bytes per row of the code buffer
  uint32_t sf_blk;   // bytes per 128-row block of the scale buffer
  int fmt;           // 0 E2M1, 1 E3M2, 2 E4M3
};

template <bool WEIGHTS>
__device__ __forceinline__ GroupCtx group_ctx(const ReorderParams& p, int g) {
  const int seg = g < p.g4 ? 0 : (g < p.g46 ? 1 : 2);
  const int gs = g - (seg == 0 ? 0 : (seg == 1 ? p.g4 : p.g46));
  const SegOut so = seg == 0 ? p.seg[0] : (seg == 1 ? p.seg[1] : p.seg[2]);
  GroupCtx c;
  c.fmt = WEIGHTS ? 0 : seg;
  const int bytes = c.fmt == 0 ? 16 : (c.fmt == 1 ? 24 : 32);
  c.codes = so.codes + (size_t)gs * bytes;
  c.sf = so.sf + (gs & 3) + (size_t)(gs >> 2) * 512;
  c.pitch = (uint32_t)so.pitch;
  c.sf_blk = 512u * (uint32_t)so.katoms;
  return c;
}

// Rows 2*pr and 2*pr+1 of one group: scales, codes, stores.
__device__ __forceinline__ void quantise_pair(const uint32_t (&v)[32], const GroupCtx& gc, int pr, int rows) {
  uint32_t m4[4] = {0, 0, 0, 0};  // four short chains instead of one of 32
#pragma unroll
  for (int i = 0; i < 32; ++i) m4[i & 3] = max_abs_bf16x2(m4[i & 3], v[i]);
  const uint32_t m = max_abs_bf16x2(max_abs_bf16x2(m4[0], m4[1]), max_abs_bf16x2(m4[2], m4[3]));
  const int row0 = 2 * pr;
  {
    const int sf = scale_byte(m & 0x7FFFu, gc.fmt);
    gc.sf[(size_t)(row0 >> 7) * gc.sf_blk + (uint32_t)(row0 & 31) * 16 + (uint32_t)((row0 >> 5) & 3) * 4] = (uint8_t)sf;
    quantise_row<0>(v, gc.fmt, __uint_as_float(((unsigned)(254 - sf) << 23) | 0x800u), gc.codes + (size_t)row0 * gc.pitch);
  }
  if (row0 + 1 < rows) {
    const int row1 = row0 + 1;
    const int sf = scale_byte((m >> 16) & 0x7FFFu, gc.fmt);
    gc.sf[(size_t)(row1 >> 7) * gc.sf_blk + (uint32_t)(row1 & 31) * 16 + (uint32_t)((row1 >> 5) & 3) * 4] = (uint8_t)sf;
    quantise_row<1>(v, gc.fmt, __uint_as_float(((unsigned)(254 - sf) << 23) | 0x800u), gc.codes + (size_t)row1 * gc.pitch);
  }
}

// GPT = groups per consumer thread: 1 keeps the 32 channel offsets of the group as 32-bit byte
// offsets, 2 (K > 16384) keeps both groups' offsets as packed 16-bit word offsets.
template <int GPT, bool WEIGHTS>
__global__ void __launch_bounds__(kThreads, 1) reorder_quantize_kernel(const ReorderParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t tiles = (raw + 127u) & ~127u;  // bank analysis of the interleave assumes 128-byte alignment
  const int K = p.K;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.stages;
  const uint32_t pitch = (uint32_t)p.pitch;
  const uint32_t stage_bytes = (uint32_t)p.P * 2u * pitch;
  // barriers: full[4] (copies landed), then the stop flag
  const uint32_t bar0 = tiles + (uint32_t)S * stage_bytes;
  volatile int* stop = reinterpret_cast<volatile int*>(smem_raw + (bar0 - raw) + kMaxStages * 8);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };

  ptx::grid_dep_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < S; ++s) ptx::mbar_init(full_bar(s), 1);  // one expect_tx arrival + bytes
    *stop = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  ptx::grid_dep_wait();  // nothing before this line reads or writes global memory

  // This CTA's contiguous share of the row pairs, walked in stages of up to P pairs.
  const int pair_begin = (int)((long long)p.pairs * blockIdx.x / gridDim.x);
  const int pair_end = (int)((long long)p.pairs * (blockIdx.x + 1) / gridDim.x);
  const int nstage = (pair_end - pair_begin + p.P - 1) / p.P;

  // thread 0 issues the copies of stage `it` (ring slot it % S)
  auto issue_stage = [&](int it, int s) {
    const int pr0 = pair_begin + it * p.P;
    const int row0 = 2 * pr0;
    const int nrows = min(2 * min(p.P, pair_end - pr0), p.rows - row0);
    const uint32_t fb = full_bar(s);
    ptx::mbar_expect_tx(fb, (uint32_t)nrows * 2u * K);
    const uint32_t dst = tiles + (uint32_t)s * stage_bytes;
    for (int r = 0; r < nrows; ++r)
      ptx::bulk_load_1d(dst + r * pitch, p.X + (size_t)(row0 + r) * K, 2u * K, fb);
  };
  if (tid == 0)
    for (int it = 0; it < min(S - 1, nstage); ++it) issue_stage(it, it);

  // interleave: lane l reads row l%8 of matrix l/8, i.e. chunk 4(l/8) + (l%8)/2 of row l%2 of the pair ...
  const uint32_t ld_off = (uint32_t)(lane & 1) * pitch + (uint32_t)((lane >> 3) * 4 + ((lane & 7) >> 1)) * 16u;
  // ... and writes row l%8 of transposed matrix l/8 (see pair_offset)
  const uint32_t st_off = (uint32_t)(lane >> 4) * pitch + (uint32_t)(((lane >> 3) & 1) * 8 + (lane & 7)) * 16u;
  const int steps = (2 * K + 255) >> 8;  // 256-byte steps per pair
  const uint32_t pair_skip = 2u * pitch - (uint32_t)steps * 256u;  // from the end of a pair's steps to the next pair
  int w_first = warp;  // this warp's first step of a stage: step inside its pair, and its offset in the stage
  uint32_t at_first = (uint32_t)warp * 256u;
  while (w_first >= steps) { w_first -= steps; at_first += pair_skip; }

  {
    // ---------------------------------------------------------------- consumers
    // Tasks of a stage = (pair slot, group), numbered with all FP4 groups first (pair slot major),
    // then the FP6 groups, then the FP8 groups; thread j takes task j (and j + 512 when GPT == 2).
    const int G = K >> 5;
    const int n4 = p.g4, n6 = p.g46 - p.g4, n8 = G - p.g46;
    const int tasks = p.P * G;
    const unsigned kmax = (unsigned)(K - 1);

    // the thread's tasks: shared-memory offsets of their 32 channels inside a stage, the pair slot
    // and where the output goes
    constexpr int kOffRegs = GPT == 1 ? 32 : 16;
    uint32_t off[GPT][kOffRegs];
    GroupCtx gc[GPT];
    int slot[GPT];
    bool have[GPT];
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      const int t = (int)p.chunk_of_warp[warp] * 32 + lane + q * kConsumers;
      have[q] = t < tasks;
      slot[q] = 0;
      if (have[q]) {
        int g;
        if (t < p.P * n4) {
          slot[q] = t / n4;
          g = t - slot[q] * n4;
        } else if (t < p.P * (n4 + n6)) {
          const int u = t - p.P * n4;
          slot[q] = u / n6;
          g = n4 + (u - slot[q] * n6);
        } else {
          const int u = t - p.P * (n4 + n6);
          slot[q] = u / n8;
          g = n4 + n6 + (u - slot[q] * n8);
        }
        gc[q] = group_ctx<WEIGHTS>(p, g);
        const uint32_t pair_base = (uint32_t)slot[q] * 2u * pitch;
        const int16_t* src = p.idx + (size_t)g * 32;
        unsigned short c[32];
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(src) + u);
            const unsigned w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              c[u * 8 + k * 2] = (unsigned short)(w[k] & 0xFFFFu);
              c[u * 8 + k * 2 + 1] = (unsigned short)(w[k] >> 16);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) c[i] = (unsigned short)src[i];
        }
        if constexpr (GPT == 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) off[q][i] = pair_base + pair_offset(min((unsigned)c[i], kmax), pitch);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            off[q][i] = ((pair_base + pair_offset(min((unsigned)c[2 * i], kmax), pitch)) >> 2) |
                        (((pair_base + pair_offset(min((unsigned)c[2 * i + 1], kmax), pitch)) >> 2) << 16);
        }
      } else {
        gc[q] = GroupCtx{};
#pragma unroll
        for (int i = 0; i < kOffRegs; ++i) off[q][i] = 0;
      }
    }

    int s = 0;               // ring slot of stage `it`
    int s_next = S > 1 ? S - 1 : 0;  // ring slot of stage it + S - 1, the one issued in this round
    uint32_t ph = 0;
    for (int it = 0; it < nstage; ++it) {
      wait_parity(full_bar(s), ph, stop, p.status, p.wait_cycles, 32);
      const uint32_t sb = tiles + (uint32_t)s * stage_bytes;
      {
        // this warp's share of the stage's 256-byte interleave steps: step i of the stage is step
        // i % steps of pair i / steps, the warp takes steps warp, warp + 16, ..., four per round so
        // that four loads are in flight.  (pair, step) advance without a division.
        const int npairs = min(p.P, pair_end - (pair_begin + it * p.P));
        const int total = npairs * steps;
        int w = w_first;
        uint32_t at = sb + at_first;
        auto advance = [&]() {
          w += kWarps;
          at += kWarps * 256u;
          while (w >= steps) { w -= steps; at += pair_skip; }
        };
        int i = warp;
        for (; i + 3 * kWarps < total; i += 4 * kWarps) {
          uint32_t r[4][4], a4[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            a4[u] = at;
            ldmatrix_x4_trans(at + ld_off, r[u]);
            advance();
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) stmatrix_x4(a4[u] + st_off, r[u]);
        }
        for (; i < total; i += kWarps) {
          uint32_t r[4];
          ldmatrix_x4_trans(at + ld_off, r);
          stmatrix_x4(at + st_off, r);
          advance();
        }
      }
      // every warp has interleaved its share and has finished gathering from the previous stage
      __syncthreads();
      if (tid == 0 && it + S - 1 < nstage) {
        // that stage's buffer was last written with ordinary stores: order them before the copies
        ptx::fence_proxy_async_smem();
        issue_stage(it + S - 1, s_next);
      }
      const bool go = !*stop;
      const uint8_t* sptr = smem_raw + (sb - raw);  // the stage, as a pointer the compiler can fold offsets into
#pragma unroll
      for (int q = 0; q < GPT; ++q) {
        const int pr = pair_begin + it * p.P + slot[q];
        const bool live = go && have[q] && pr < pair_end;
        if (live) {
          uint32_t v[32];
          if constexpr (GPT == 1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = *reinterpret_cast<const uint32_t*>(sptr + off[q][i]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              v[2 * i] = *reinterpret_cast<const uint32_t*>(sptr + ((off[q][i] & 0xFFFFu) << 2));
              v[2 * i + 1] = *reinterpret_cast<const uint32_t*>(sptr + ((off[q][i] >> 16) << 2));
            }
          }
          quantise_pair(v, gc[q], pr, p.rows);
        }
      }
      if (++s == S) { s = 0; ph ^= 1u; }
      if (++s_next == S) s_next = 0;
    }
  }
  __syncthreads();
  if (*stop) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let copies in flight land
  }
}

struct Shape {
  int gpt, P, S, pitch;
  size_t smem;
};

size_t smem_bytes(int pitch, int P, int S) { return 128 + (size_t)S * P * 2 * pitch + kMaxStages * 8 + 16; }

// Pairs per stage and ring depth: as many pairs as give every consumer thread a task, fewer when
// the CTA has fewer pairs or shared memory cannot hold two such stages; then up to four stages
// (three are enough to keep copies in flight, the gather frees a stage early).
Shape plan_shape(int K, int pairs_per_cta, size_t budget) {
  Shape sh{};
  const int G = K / 32;
  sh.gpt = G <= kConsumers ? 1 : 2;
  sh.pitch = (2 * K + 255) / 256 * 256 + 64;  // = 64 mod 128: the two rows of a pair sit in different bank halves
  int P = sh.gpt == 1 ? kConsumers / G : 1;
  if (P > pairs_per_cta) P = pairs_per_cta;
  if (P < 1) P = 1;
  while (P > 1 && smem_bytes(sh.pitch, P, 2) > budget) --P;
  // even out the stages of a CTA: 7 pairs as 4 + 3, not 6 + 1
  const int nst = (pairs_per_cta + P - 1) / P;
  P = (pairs_per_cta + nst - 1) / nst;
  int S = 1;
  while (S < kMaxStages && S < 3 + (nst > 3 ? 1 : 0) && smem_bytes(sh.pitch, P, S + 1) <= budget) ++S;
  sh.P = P;
  sh.S = S;
  sh.smem = smem_bytes(sh.pitch, P, S);
  return sh;
}

template <int GPT, bool WEIGHTS>
int launch(const ReorderParams& p, int grid, size_t smem, cudaStream_t st) {
  auto kern = reorder_quantize_kernel<GPT, WEIGHTS>;
  if (smem > 48 * 1024) MG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MG_CUDA_TRY(mg::launch_kernel(kern, dim3(grid), dim3(kThreads), smem, st, p));
  return MG_OK;
}

int reorder_quantize(bool weights, const void* X, int rows, int K, const int16_t* idx, int KN, int KS,
                     int KO, uint8_t* o4, uint8_t* o6, uint8_t* o8, const size_t* pitches, uint8_t* s4, uint8_t* s6,
                     uint8_t* s8, void* stream) {
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
  const size_t dense[3] = {(size_t)KN / 2, (size_t)(weights ? KS / 2 : KS / 4 * 3), (size_t)(weights ? KO / 2 : KO)};
  const size_t align[3] = {16, (size_t)(weights ? 16 : 8), 16};
  size_t pitch[3];
  for (int i = 0; i < 3; ++i) {
    pitch[i] = pitches ? pitches[i] : dense[i];
    if (pitch[i] < dense[i] || pitch[i] > 0x7fffffffu) return MG_ERR_SHAPE;
    if (pitch[i] % align[i]) return MG_ERR_ALIGN;
  }
  p.seg[0] = {o4, s4, (KN + 127) / 128, (int)pitch[0]};
  p.seg[1] = {o6, s6, (KS + 127) / 128, (int)pitch[1]};
  p.seg[2] = {o8, s8, (KO + 127) / 128, (int)pitch[2]};

  p.pairs = (rows + 1) / 2;
  int grid = p.pairs < di.sm_count ? p.pairs : di.sm_count;  // pairs are dealt out evenly, at least one per CTA
  const int cap = mg::options().reorder_ctas;  // a caller that runs another kernel beside this one may cap the grid
  if (cap > 0 && grid > cap) grid = cap;
  const Shape sh = plan_shape(K, (p.pairs + grid - 1) / grid, (size_t)di.smem_optin);
  if (sh.smem > (size_t)di.smem_optin) return MG_ERR_SHAPE;
  p.P = sh.P;
  p.stages = sh.S;
  p.pitch = sh.pitch;
  p.wait_cycles = mg::wait_limit_cycles();
  {
    // Warp w sits on scheduler w % 4.  Deal the 16 chunks of 32 tasks (sorted by format) to warps so
    // that the four schedulers get about the same work: heaviest chunk first, each to the
    // scheduler with the least work so far that still has a free warp.
    const int G = K / 32, n4 = weights ? G : p.g4, n46 = weights ? G : p.g46;
    const int tasks = sh.P * G;
    auto fmt_of = [&](int t) { return t < sh.P * n4 ? 0 : (t < sh.P * n46 ? 1 : 2); };
    double cost[kWarps];
    for (int c = 0; c < kWarps; ++c) {
      bool has[3] = {false, false, false};
      cost[c] = 0;
      for (int q = 0; q < sh.gpt; ++q) {
        bool any = false;
        for (int l = 0; l < 32; ++l) {
          const int t = c * 32 + l + q * kConsumers;
          if (t < tasks) { has[fmt_of(t)] = true; any = true; }
        }
        if (any) cost[c] += 1.0;  // gather, maxima, scaling and rounding: the same for every format
      }
      cost[c] += (has[0] ? 0.15 : 0) + (has[1] ? 0.6 : 0) + (has[2] ? 0.9 : 0);  // conversion and packing
    }
    int order[kWarps];
    for (int c = 0; c < kWarps; ++c) order[c] = c;
    std::stable_sort(order, order + kWarps, [&](int a, int b) { return cost[a] > cost[b]; });
    double load[4] = {0, 0, 0, 0};
    int used[4] = {0, 0, 0, 0};
    for (int k = 0; k < kWarps; ++k) {
      int best = -1;
      for (int q = 0; q < 4; ++q)
        if (used[q] < kWarps / 4 && (best < 0 || load[q] < load[best])) best = q;
      p.chunk_of_warp[best + 4 * used[best]] = (uint8_t)order[k];
      load[best] += cost[order[k]];
      ++used[best];
    }
  }
  rc = mg::device_status_word(&p.status);
  if (rc != MG_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (sh.gpt == 1) return weights ? launch<1, true>(p, grid, sh.smem, st) : launch<1, false>(p, grid, sh.smem, st);
  return weights ? launch<2, true>(p, grid, sh.smem, st) : launch<2, false>(p, grid, sh.smem, st);
}

}  // namespace

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
