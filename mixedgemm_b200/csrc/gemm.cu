// Mixed MXFP4 / MXFP6 / MXFP8 x MXFP4 block-scaled GEMM for sm_100a.
//
// One persistent, warp-specialised kernel carries all three K segments of MixedGemm's
// matmul_host (src/gemm.cu:22-47 of that project, three chained CUTLASS GEMMs there) in a
// single fp32 accumulator in tensor memory:
//   warp 0      TMA producer: A / B tiles (tiled tensor maps, 128-byte swizzle) and the
//               512-byte scale atoms (1-D bulk copies) into a ring of shared-memory stages
//   warp 1      MMA issuer: copies the scale atoms to TMEM (tcgen05.cp) and issues
//               tcgen05.mma kind::mxf4 (FP4 segment, K=64 per instruction) or
//               kind::mxf8f6f4 (FP6 / FP8 segments, K=32 per instruction)
//   warps 2-5   epilogue: tcgen05.ld the accumulator, round once to bf16, store
// Every stage is 128 bytes of K per row for both operands: 256 FP4 elements in the FP4
// segment (dense nibbles), 128 elements in the FP6 / FP8 segments, where the tensor-map
// types 16U6_ALIGN16B / 16U4_ALIGN16B expand the packed FP6 / FP4 rows to the
// one-byte-per-element slots kind::mxf8f6f4 reads.
// All waits are bounded; on expiry a kernel records a code in the device status word,
// tells the other roles of its CTA to stop, frees its tensor memory and returns.
//
// What runs for a given problem (matmul_impl decides; every choice has an option, see mg_set_option):
//   mixed_gemm_pair_kernel            >= 56 tiles of 256 x 256, bf16 output: two CTAs per tile
//                                     (cta_group::2), TMA-store epilogue, one launch for a list of problems
//   mixed_gemm_kernel<128, -, CS>     <= 33 tiles of 128 x 128: clusters of four CTAs split K and add
//                                     their accumulators through distributed shared memory
//   mixed_gemm_kernel<16..128, SWAP>  M <= 32 with many weight tiles or a long K: weights as the
//                                     128-row operand, tile stored transposed
//   mixed_gemm_kernel<128 | 256>      everything else; with 34..74 tiles and a long K several CTAs
//                                     per tile, partial sums through the caller's workspace
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <random>

#include "mg_common.h"
#include "ptx_sm100.cuh"

namespace {

constexpr int BM = 128;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;

struct SegParams {
  int kseg;     // valid elements of the segment
  int nstages;  // pipeline stages it takes
  int katoms;   // scale atoms along K: ceil(kseg / 128)
  const uint8_t* sfa;
  const uint8_t* sfb;
};

struct GemmParams {
  int M, N, ldd;
  int tiles_m, tiles_n;
  SegParams seg[3];
  const __nv_bfloat16* C;
  __nv_bfloat16* D;
  float* Df32;  // when set, the fp32 accumulator is stored here instead of D
  int* status;
  long long wait_cycles;      // limit of every bounded wait, in SM clock cycles
  uint32_t tx_a[3], tx_b[3];  // bytes one A / B tile load of the segment signals
  int skip_load;  // fault injection for the bounded-wait test: CTA 0 withholds its n-th stage load (0 = off)
  // Split-K (few tiles): `splits` CTAs share a tile, each over a contiguous range of its K stages.
  // Each leaves its fp32 partial in sp_partials and bumps the tile's counter; the CTA that arrives
  // last adds the partials in split order (so the result does not depend on who was last), stores
  // the tile and clears the counter.
  int splits;
  int sp_rows;         // rows per tile in sp_partials (128, or M rounded up to 32 when M <= 96)
  unsigned long long* sp_counters;  // [tile]: (launch token << 8) | arrivals; the last CTA writes 0
  unsigned long long sp_token;      // 56 bits, unique per launch: a word with another token counts as 0
  float* sp_partials;  // [split][tile][column group of 4][sp_rows][4]
};

// Bounded mbarrier wait: true once the phase has completed.  When the limit expires the lane
// records `code`, raises the CTA's stop flag and returns false; from then on every wait of the CTA
// that does not find its phase complete at the first probe returns false at once.  A role whose
// wait failed issues nothing more (no copies, no MMAs, no arrivals) and leaves its loops; the
// kernel then ends normally, with nothing stored.
__device__ __forceinline__ bool wait_parity(uint32_t bar, uint32_t parity, volatile int* stop, int* status,
                                            long long limit, int code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 0) {
      if (*stop) return false;
      const long long now = clock64();
      if (spin == 0) t0 = now;
      if (now - t0 > limit) {
        *stop = 1;
        atomicOr(status, code);
        return false;
      }
    }
  }
}

// The same for a barrier whose phase is completed by other CTAs of the cluster.
__device__ __forceinline__ bool wait_parity_cluster(uint32_t bar, uint32_t parity, volatile int* stop, int* status,
                                                    long long limit, int code) {
  if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
  long long t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
    if ((spin & 63u) == 0) {
      if (*stop) return false;
      const long long now = clock64();
      if (spin == 0) t0 = now;
      if (now - t0 > limit) {
        *stop = 1;
        atomicOr(status, code);
        return false;
      }
    }
  }
}

// Tile order: row blocks in groups of eight, all column blocks of a group before the next group.
// The CTAs (or clusters) running at one time then share about eight A tiles and nine B tiles instead
// of 74 A tiles and one B tile, which keeps operands of problems with many row blocks (M = 16384:
// 150 MB of packed A) in L2.  Up to eight row blocks this is the plain row-fastest order.
__device__ __forceinline__ void raster(int lt, int tiles_m, int tiles_n, int& m_tile, int& n_tile) {
  constexpr int kGroup = 8;
  const int full = tiles_m / kGroup * kGroup;
  const int g = lt / (kGroup * tiles_n);
  if (g * kGroup < full) {
    const int r = lt - g * kGroup * tiles_n;
    m_tile = g * kGroup + r % kGroup;
    n_tile = r / kGroup;
  } else {
    const int rem = tiles_m - full, r = lt - full * tiles_n;
    m_tile = full + r % rem;
    n_tile = r / rem;
  }
}

// CS = cluster split-K: four CTAs of a cluster share a tile, each over a quarter of the K stages,
// and add their accumulators through distributed shared memory (RECV_BYTES: three senders x 128
// rows x 32 columns of fp32 in every CTA).
template <int BN, bool CS = false>
struct Cfg {
  static constexpr int STAGES = CS ? 5 : (BN == 256 ? 4 : (BN == 128 ? 6 : (BN == 64 ? 8 : 10)));
  static constexpr uint32_t RECV_BYTES = CS ? 3u * 128u * 32u * 4u : 0u;
  static constexpr int ACC = BN == 256 ? 1 : 2;
  static constexpr int NB = BN >= 128 ? BN / 128 : 1;
  static constexpr int CHUNKS = (BN + 31) / 32;  // 32-column reads of the accumulator
  static constexpr uint32_t A_BYTES = BM * 128;
  static constexpr uint32_t B_BYTES = BN * 128;
  static constexpr uint32_t SFA_BYTES = 1024;      // up to two atoms
  static constexpr uint32_t SFB_BYTES = NB * 1024;  // up to two atoms per 128 columns
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr uint32_t SF_SLOT_COLS = 8 + NB * 8;  // TMEM columns of one scale slot
  static constexpr uint32_t SF_COL0 = ACC * BN;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + RECV_BYTES;
  static_assert(!CS || BN == 128, "the cluster exchange hands one 32-column chunk to each of four CTAs");
  static_assert(SF_COL0 + 2 * SF_SLOT_COLS <= kTmemCols, "tensor memory budget");
};

// SWAP = true is the decode form (M <= 128): the weights are the MMA's 128-row operand and the
// activations its BN-column operand (BN = M rounded up to 16 / 32 / 64 / 128), so the tensor core
// spends N x BN instead of N x 128 work on M real rows and a stage carries BN instead of 128
// activation rows.  p.tiles_m then counts 128-row weight tiles, p.tiles_n is 1, the host swaps the
// tensor maps, scale pointers and byte counts, and the epilogue stores the tile transposed.
template <int BN, bool SWAP, bool CS = false>
__global__ void __launch_bounds__(kThreads, 1)
mixed_gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmA0,
                  const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmA1,
                  const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmA2,
                  const __grid_constant__ CUtensorMap tmB2) {
  using C = Cfg<BN, CS>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + C::STAGES * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + C::ACC + a); };
  // cluster split-K: "every partial for this tile has arrived here" / "what this CTA sent has been read"
  const uint32_t xfull_bar = bar0 + 8u * (2 * C::STAGES + 2 * C::ACC);
  const uint32_t xfree_bar = xfull_bar + 8u;
  const uint32_t recv = bar0 + 256u;  // [sender slot 0..2][4-column group 0..7][row 0..127] 16-byte units
  volatile uint32_t* tmem_holder =
      reinterpret_cast<volatile uint32_t*>(gbase + C::STAGES * C::STAGE_BYTES + 8 * (2 * C::STAGES + 2 * C::ACC + 2));
  volatile int* stop = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < C::ACC; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 4);
    }
    if (CS) {
      ptx::mbar_init(xfull_bar, 12);  // four epilogue warps of each of the three other CTAs
      ptx::mbar_init(xfree_bar, 12);
    }
    *stop = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmA0);
    ptx::prefetch_tmap(&tmB0);
    ptx::prefetch_tmap(&tmA1);
    ptx::prefetch_tmap(&tmB1);
    ptx::prefetch_tmap(&tmA2);
    ptx::prefetch_tmap(&tmB2);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::grid_dep_launch_dependents();
  ptx::tc_fence_before();
  __syncthreads();
  if (CS) ptx::cluster_sync();  // the other CTAs' exchange barriers exist before anyone arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  ptx::grid_dep_wait();  // the prologue above touched no global memory

  const int total_tiles = p.tiles_m * p.tiles_n;
  // work item w = (tile w / splits, split w % splits); split j covers K stages [S j / splits, S (j+1) / splits)
  const int splits = p.splits;
  const int total_items = total_tiles * splits;
  const int S_units = p.seg[0].nstages + p.seg[1].nstages + p.seg[2].nstages;
  const int seg_off1 = p.seg[0].nstages, seg_off2 = seg_off1 + p.seg[1].nstages;

  // Producer and MMA warps run their loops with all 32 lanes, so that addresses and
  // descriptors are warp-uniform values; one elected lane issues the asynchronous operations.
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    const bool leader = ptx::elect_one();
    int stage = 0;
    uint32_t phase = 0;
    int skip_countdown = p.skip_load;
    bool live = true;  // false once a wait of this role has failed: nothing more is issued
    for (int w = blockIdx.x; w < total_items && live; w += gridDim.x) {
      const int t = w / splits, split = w - t * splits;
      const int u0 = S_units * split / splits, u1 = S_units * (split + 1) / splits;
      int m_tile, n_tile;
      raster(t, p.tiles_m, p.tiles_n, m_tile, n_tile);
#pragma unroll 1
      for (int seg = 0; seg < 3 && live; ++seg) {
        const SegParams sp = seg == 0 ? p.seg[0] : (seg == 1 ? p.seg[1] : p.seg[2]);
        const CUtensorMap* ta = seg == 0 ? &tmA0 : (seg == 1 ? &tmA1 : &tmA2);
        const CUtensorMap* tb = seg == 0 ? &tmB0 : (seg == 1 ? &tmB1 : &tmB2);
        const uint32_t tx_ab = seg == 0 ? p.tx_a[0] + p.tx_b[0]
                                        : (seg == 1 ? p.tx_a[1] + p.tx_b[1] : p.tx_a[2] + p.tx_b[2]);
        const uint8_t* sfa_row = sp.sfa + (size_t)m_tile * sp.katoms * 512;
        const uint8_t* sfb_row = sp.sfb + (size_t)n_tile * C::NB * sp.katoms * 512;
        const int so = seg == 0 ? 0 : (seg == 1 ? seg_off1 : seg_off2);
        const int s_lo = max(u0 - so, 0), s_hi = min(u1 - so, sp.nstages);
#pragma unroll 1
        for (int s = s_lo; s < s_hi; ++s) {
          if (!wait_parity(empty_bar(stage), phase ^ 1u, stop, p.status, p.wait_cycles, 1)) { live = false; break; }
          const int atom0 = seg == 0 ? 2 * s : s;
          const int natoms = seg == 0 ? min(2, sp.katoms - atom0) : 1;
          const uint32_t sbase = base + stage * C::STAGE_BYTES;
          const uint32_t fb = full_bar(stage);
          if (leader) {
            if (p.skip_load != 0 && blockIdx.x == 0 && --skip_countdown == 0) {
              // fault injection: this stage is never loaded, so the MMA warp's wait for it runs out
            } else {
              ptx::mbar_expect_tx(fb, tx_ab + (uint32_t)natoms * 512u * (1 + C::NB));
              ptx::tma_load_2d(sbase, ta, s * 128, m_tile * BM, fb);
              ptx::tma_load_2d(sbase + C::A_BYTES, tb, s * 128, n_tile * BN, fb);
              ptx::bulk_load_1d(sbase + C::A_BYTES + C::B_BYTES, sfa_row + (size_t)atom0 * 512, natoms * 512, fb);
#pragma unroll
              for (int nb = 0; nb < C::NB; ++nb)
                ptx::bulk_load_1d(sbase + C::A_BYTES + C::B_BYTES + C::SFA_BYTES + nb * 1024,
                                  sfb_row + ((size_t)nb * sp.katoms + atom0) * 512, natoms * 512, fb);
            }
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const bool leader = ptx::elect_one();
    // instruction descriptors: scale type UE8M0, M = 128, N = BN, both operands K-major
    constexpr uint32_t kCommon = ((uint32_t)(BN >> 3) << 17) | (1u << 23) | ((uint32_t)(BM >> 4) << 24);
    constexpr uint32_t kIdesc[3] = {kCommon | (1u << 7) | (1u << 10),   // mxf4: E2M1 x E2M1
                                    SWAP ? kCommon | (5u << 7) | (4u << 10) : kCommon | (4u << 7) | (5u << 10),   // E3M2, E2M1
                                    SWAP ? kCommon | (5u << 7) | (0u << 10) : kCommon | (0u << 7) | (5u << 10)};  // E4M3, E2M1
    int stage = 0;
    uint32_t phase = 0, slot = 0;
    int it = 0;
    bool live = true;
    for (int w = blockIdx.x; w < total_items && live; w += gridDim.x, ++it) {
      const int split = w % splits;
      const int u0 = S_units * split / splits, u1 = S_units * (split + 1) / splits;
      const int acc = it % C::ACC;
      const uint32_t acc_phase = (uint32_t)(it / C::ACC) & 1u;
      if (!wait_parity(tempty_bar(acc), acc_phase ^ 1u, stop, p.status, p.wait_cycles, 4)) break;
      ptx::tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
      uint32_t accumulate = 0;
#pragma unroll 1
      for (int seg = 0; seg < 3 && live; ++seg) {
        const SegParams sp = seg == 0 ? p.seg[0] : (seg == 1 ? p.seg[1] : p.seg[2]);
        const uint32_t id0 = seg == 0 ? kIdesc[0] : (seg == 1 ? kIdesc[1] : kIdesc[2]);
        const int so = seg == 0 ? 0 : (seg == 1 ? seg_off1 : seg_off2);
        const int s_lo = max(u0 - so, 0), s_hi = min(u1 - so, sp.nstages);
#pragma unroll 1
        for (int s = s_lo; s < s_hi; ++s) {
          if (!wait_parity(full_bar(stage), phase, stop, p.status, p.wait_cycles, 2)) { live = false; break; }
          ptx::tc_fence_after();
          const uint32_t sbase = base + stage * C::STAGE_BYTES;
          const uint32_t sfa_lo = ptx::desc_lo(sbase + C::A_BYTES + C::B_BYTES);
          const uint32_t sfb_lo = sfa_lo + (C::SFA_BYTES >> 4);
          const uint32_t sfa_t = tmem_base + C::SF_COL0 + slot * C::SF_SLOT_COLS;
          const uint32_t sfb_t = sfa_t + 8;
          const uint32_t a_lo = ptx::desc_lo(sbase), b_lo = ptx::desc_lo(sbase + C::A_BYTES);
          // K elements left in this segment, in MMA steps (64 for FP4, 32 for FP6 / FP8)
          const int nm = seg == 0 ? min(4, (sp.kseg - s * 256) >> 6) : min(4, (sp.kseg - s * 128) >> 5);
          if (leader) {
            // scale atoms -> TMEM: atom a of A to columns a*4.., of B (per 128 columns) to a*NB*4 + nb*4..
            ptx::tc_cp_sf(sfa_t, sfa_lo, ptx::kDescHiSf);
#pragma unroll
            for (int nb = 0; nb < C::NB; ++nb) ptx::tc_cp_sf(sfb_t + nb * 4, sfb_lo + nb * 64, ptx::kDescHiSf);
            if (seg == 0 && nm > 2) {
              ptx::tc_cp_sf(sfa_t + 4, sfa_lo + 32, ptx::kDescHiSf);
#pragma unroll
              for (int nb = 0; nb < C::NB; ++nb)
                ptx::tc_cp_sf(sfb_t + C::NB * 4 + nb * 4, sfb_lo + nb * 64 + 32, ptx::kDescHiSf);
            }
            if (seg == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (j < nm) {
                  constexpr uint32_t kNB4 = C::NB * 4;
                  const uint32_t a = j >> 1, sfid = (j & 1) * 2;
                  ptx::mma_mxf4(d_tmem, a_lo + j * 2, b_lo + j * 2, ptx::kDescHiSw128,
                                id0 | (sfid << 4) | (sfid << 29), sfa_t + a * 4, sfb_t + a * kNB4, accumulate);
                  accumulate = 1;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (j < nm) {
                  ptx::mma_mxf8f6f4(d_tmem, a_lo + j * 2, b_lo + j * 2, ptx::kDescHiSw128,
                                    id0 | ((uint32_t)j << 4) | ((uint32_t)j << 29), sfa_t, sfb_t, accumulate);
                  accumulate = 1;
                }
              }
            }
          }
          accumulate = 1;
          if (leader) ptx::tc_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          slot ^= 1u;
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (leader && live) ptx::tc_commit(tfull_bar(acc));
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int trow = q * 32 + lane;
    volatile int* arrivals = reinterpret_cast<volatile int*>(tmem_holder + 2);  // split-K: counter value seen
    const bool issuer = warp == 2 && lane == 0;
    int it = 0;
    for (int w = blockIdx.x; w < total_items; w += gridDim.x, ++it) {
      const int t = w / splits, split = w - t * splits;
      int m_tile, n_tile;
      raster(t, p.tiles_m, p.tiles_n, m_tile, n_tile);
      const int acc = it % C::ACC;
      const uint32_t acc_phase = (uint32_t)(it / C::ACC) & 1u;
      wait_parity(tfull_bar(acc), acc_phase, stop, p.status, p.wait_cycles, 8);
      __syncwarp();
      ptx::tc_fence_after();
      const int row = m_tile * BM + trow;  // output row, or (SWAP) output column
      const bool store = (SWAP || row < p.M) && !*stop;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * BN;
      const size_t goff = (size_t)row * p.ldd + (size_t)n_tile * BN;
      // 32 accumulator columns of this thread's row -> (+C) -> fp32 or bf16 output
      auto emit = [&](uint32_t (&r)[32], int c) {
        if constexpr (SWAP) {
          // r[j] belongs to output row m = c * 32 + j, column `row`: a warp writes 64 contiguous bytes per m
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = c * 32 + j;
            if (m < p.M) {
              const size_t o = (size_t)m * p.ldd + row;
              float v = __uint_as_float(r[j]);
              if (p.C != nullptr) v += __bfloat162float(p.C[o]);
              if (p.Df32 != nullptr) p.Df32[o] = v;
              else p.D[o] = __float2bfloat16_rn(v);
            }
          }
          return;
        }
        if (p.C != nullptr) {
          const uint4* cp = reinterpret_cast<const uint4*>(p.C + goff + c * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 cv = cp[v];
            const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              r[v * 8 + k * 2] = __float_as_uint(__uint_as_float(r[v * 8 + k * 2]) + __uint_as_float(cw[k] << 16));
              r[v * 8 + k * 2 + 1] =
                  __float_as_uint(__uint_as_float(r[v * 8 + k * 2 + 1]) + __uint_as_float(cw[k] & 0xFFFF0000u));
            }
          }
        }
        if (p.Df32 != nullptr) {
          uint4* fp = reinterpret_cast<uint4*>(p.Df32 + goff + c * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v) fp[v] = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
        } else {
          uint4* dp = reinterpret_cast<uint4*>(p.D + goff + c * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t ow[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + k * 2]),
                                                       __uint_as_float(r[v * 8 + k * 2 + 1]));
              ow[k] = *reinterpret_cast<uint32_t*>(&h);
            }
            dp[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
      };
      if constexpr (CS) {
        // ---- cluster split-K: the four CTAs of the cluster hold partial sums of the same tile.  CTA c
        // finishes columns [32 c, 32 c + 32): the others store that chunk of their accumulator into
        // its shared memory, it adds the four in CTA order and stores the result.
        const uint32_t crank = ptx::cluster_ctarank();
        if (it > 0) wait_parity_cluster(xfree_bar, (uint32_t)(it - 1) & 1u, stop, p.status, p.wait_cycles, 512);
        uint32_t mine[32];
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          if (c == (int)crank) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mine[i] = r[i];
          } else if (store) {
            const uint32_t slot = crank - (crank > (uint32_t)c ? 1u : 0u);
            const uint32_t dst = ptx::map_to_cta(recv + ((slot * 8u) * 128u + (uint32_t)trow) * 16u, (uint32_t)c);
#pragma unroll
            for (int v = 0; v < 8; ++v)
              ptx::st_cluster_v4(dst + (uint32_t)v * 128u * 16u, r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
          }
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        ptx::fence_acq_rel_cluster();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (uint32_t o = 0; o < 4; ++o)
            if (o != crank) ptx::mbar_arrive_release_cluster(ptx::map_to_cta(xfull_bar, o));
        }
        wait_parity_cluster(xfull_bar, (uint32_t)it & 1u, stop, p.status, p.wait_cycles, 512);
        if (store && !*stop) {
          uint32_t r[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0;  // +0.0f
#pragma unroll 1
          for (uint32_t sr = 0; sr < 4; ++sr) {
            if (sr == crank) {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(mine[i]));
            } else {
              const uint32_t slot = sr - (sr > crank ? 1u : 0u);
              const uint32_t src = recv + ((slot * 8u) * 128u + (uint32_t)trow) * 16u;
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                uint4 a;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w)
                             : "r"(src + (uint32_t)v * 128u * 16u));
                r[v * 4] = __float_as_uint(__uint_as_float(r[v * 4]) + __uint_as_float(a.x));
                r[v * 4 + 1] = __float_as_uint(__uint_as_float(r[v * 4 + 1]) + __uint_as_float(a.y));
                r[v * 4 + 2] = __float_as_uint(__uint_as_float(r[v * 4 + 2]) + __uint_as_float(a.z));
                r[v * 4 + 3] = __float_as_uint(__uint_as_float(r[v * 4 + 3]) + __uint_as_float(a.w));
              }
            }
          }
          emit(r, (int)crank);
        }
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (uint32_t o = 0; o < 4; ++o)
            if (o != crank) ptx::mbar_arrive_cluster(ptx::map_to_cta(xfree_bar, o));
        }
        continue;
      }
      if (splits == 1) {
#pragma unroll 1
        for (int c = 0; c < C::CHUNKS; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          if (store) emit(r, c);
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        continue;
      }
      // ---- split-K: leave this CTA's partial (16-byte units, [column group][row]: a warp stores 512
      // contiguous bytes), count the arrival, and let the last CTA of the tile add and store
      const size_t tile_units = (size_t)(BN / 4) * p.sp_rows;
      uint4* part = reinterpret_cast<uint4*>(p.sp_partials) + ((size_t)split * total_tiles + t) * tile_units + trow;
#pragma unroll 1
      for (int c = 0; c < C::CHUNKS; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
        if (store) {
#pragma unroll
          for (int v = 0; v < 8; ++v)
            if (c * 8 + v < BN / 4)
              __stcg(part + (size_t)(c * 8 + v) * p.sp_rows, make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]));
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
      __threadfence();  // the partial is visible device-wide before the arrival is counted
      ptx::named_barrier_sync(1, 128);
      if (issuer) {
        // count this arrival.  The workspace is the caller's and may hold anything: a word that does
        // not carry this launch's token is taken as "nobody has arrived yet".
        unsigned long long* cw = p.sp_counters + t;
        unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(cw);
        int idx = -1;
        for (int tries = 0; tries < 4096; ++tries) {
          const bool mine = (cur >> 8) == p.sp_token;
          const unsigned long long want = mine ? cur + 1 : ((p.sp_token << 8) | 1ull);
          const unsigned long long prev = atomicCAS(cw, cur, want);
          if (prev == cur) {
            idx = mine ? (int)(cur & 0xFF) : 0;
            break;
          }
          cur = prev;
        }
        if (idx < 0) atomicOr(p.status, 256);
        *arrivals = idx;
      }
      ptx::named_barrier_sync(1, 128);
      if (*arrivals == splits - 1) {
        __threadfence();
        if (store) {
          const uint4* src0 = reinterpret_cast<const uint4*>(p.sp_partials) + (size_t)t * tile_units + trow;
#pragma unroll 1
          for (int c = 0; c < C::CHUNKS; ++c) {
            uint32_t r[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0;  // +0.0f
            for (int sp = 0; sp < splits; ++sp) {
              const uint4* src = src0 + (size_t)sp * total_tiles * tile_units + (size_t)(c * 8) * p.sp_rows;
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                if (c * 8 + v >= BN / 4) continue;
                const uint4 a = __ldcg(src + (size_t)v * p.sp_rows);
                r[v * 4] = __float_as_uint(__uint_as_float(r[v * 4]) + __uint_as_float(a.x));
                r[v * 4 + 1] = __float_as_uint(__uint_as_float(r[v * 4 + 1]) + __uint_as_float(a.y));
                r[v * 4 + 2] = __float_as_uint(__uint_as_float(r[v * 4 + 2]) + __uint_as_float(a.z));
                r[v * 4 + 3] = __float_as_uint(__uint_as_float(r[v * 4 + 3]) + __uint_as_float(a.w));
              }
            }
            emit(r, c);
          }
        }
        if (issuer) p.sp_counters[t] = 0;  // every split has arrived: ready for the next launch
      }
    }
  }

  // ------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (CS) ptx::cluster_sync();  // no CTA leaves while another may still store into it or arrive on it
  ptx::tc_fence_after();
  if (*stop) {
    // give copies and MMAs that are still in flight time to land before the CTA goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) ptx::tmem_dealloc(tmem_base, kTmemCols);
}

// ---------------------------------------------------------------- CTA-pair variant
//
// Two CTAs of a cluster (the two SMs of a TPC) compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and only its half (128
// rows) of the B tile, so a stage is 35 KB instead of 51 KB for the same MMA time, and one
// instruction issued by the leader CTA drives both tensor cores.  Per CTA:
//   warp 0      TMA producer for this CTA's operands
//   warp 1      MMA issuer (leader CTA only); owns the pair's TMEM allocation in both CTAs
//   warp 2      relay: when this CTA's stage has landed, arrives on the leader's `ready` barrier
//   warps 3-6   epilogue: TMEM -> registers -> bf16 -> swizzled shared staging -> TMA store;
//               the accumulator is handed back as soon as it is in registers, so the next
//               tile's MMAs overlap the stores
// One launch takes a LIST of problems (up to kMaxProb): each has its own activation, weights,
// output and K split.  The tile list is the concatenation of the problems' tiles, dealt
// round-robin to the clusters, so that small problems fill the slots a large one leaves idle in
// its last wave (q/k/v and gate/up of a layer share the activation; a whole layer's seven
// projections can share a launch).  A problem may carry a ready flag: the producer then waits
// (bounded) until the word at that address is >= the given value before it reads the problem's
// activation - the hook for an exchange that fills the activation buffer while the launch is
// already running.
constexpr int kMaxProb = 8;

struct PairProb {
  SegParams seg[3];
  int M;          // rows of the activation / output
  int tiles_m2;   // 256-row blocks
  int tile_end;   // tiles of problems 0..this one
  int s_units;    // K stages per tile
  // optional: the activation is complete when flag[0 .. flag_count) have all reached the target
  // value, which is *flag_epoch when that pointer is set (a device word the host bumps once per
  // step, so that a captured launch can be replayed) and flag_value otherwise
  const int* flag;
  int flag_count;
  const int* flag_epoch;
  int flag_value;
  // The activation may be stored in row shards (what a multi-GPU exchange fills shard by shard with
  // one copy each): rows [i * shard_rows, (i+1) * shard_rows) of every code buffer are contiguous
  // at the row pitch, consecutive shards lie `shard stride` bytes apart (part of the tensor map),
  // and the scale blocks of shard i start sf_shard_stride[seg] bytes after those of shard i - 1.
  // Unsharded: shard_rows >= M.
  int shard_rows;
  uint32_t sf_shard_stride[3];
  int flag_rows;  // > 0: flag i covers rows [i * flag_rows, (i + 1) * flag_rows) and a tile waits only for its own rows' flag
  int m_rot;      // 256-row block the problem's tile order starts with (the blocks whose rows are there first)
};

struct PairParams {
  int nprob;
  PairProb prob[kMaxProb];
  uint32_t tx_a[3], tx_b[3];  // bytes one A / B tile load of the segment signals
  int* status;
  long long wait_cycles;
};

// Which tiles a cluster computes, in order.  Tiles of different problems differ in cost (K), and
// dealing them out round-robin leaves the clusters that drew more of the expensive ones working
// while the others are done (6.7 % of the launch on the 8B projection set).  The host deals the
// tile list out in order, each tile to the cluster that is free first under a cost model (K stages
// + a constant), and passes the result; without a table (equal costs, or more tiles than fit)
// cluster c takes tiles c, c + clusters, ...
constexpr int kMaxClusters = 96;
constexpr int kMaxSched = 8192;
struct PairSchedule {
  int use;
  uint16_t off[kMaxClusters + 1];  // cluster c owns tile[off[c] .. off[c + 1])
  uint16_t tile[kMaxSched];
};

struct PairMaps {
  CUtensorMap a[kMaxProb][3];  // activation codes per problem and K segment
  CUtensorMap b[kMaxProb][3];  // weight codes
  CUtensorMap d[kMaxProb];     // outputs
};

template <int STAGES_, int NSLOT_>
struct PairCfgT {
  static constexpr int STAGES = STAGES_;
  static constexpr int NSLOT = NSLOT_;  // 64-column output panels that can be staged at once
  static constexpr int THREADS = 224;
  static constexpr uint32_t A_BYTES = 128 * 128;
  static constexpr uint32_t B_BYTES = 128 * 128;
  static constexpr uint32_t SFA_BYTES = 1024;
  static constexpr uint32_t SFB_BYTES = 2048;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;  // 35 KB
  static constexpr uint32_t PANEL_BYTES = 128 * 128;         // 128 rows x 64 bf16 columns
  static constexpr uint32_t STAGING_BYTES = NSLOT * PANEL_BYTES;
  static constexpr uint32_t SF_COL0 = 256;
  static constexpr uint32_t SF_SLOT_COLS = 8 + 16;
  static constexpr size_t SMEM = 1024 + STAGING_BYTES + (size_t)STAGES * STAGE_BYTES + 256;
};
using PairCfg = PairCfgT<5, 2>;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg::THREADS, 1)
mixed_gemm_pair_kernel(const __grid_constant__ PairParams p, const __grid_constant__ PairMaps gm,
                       const __grid_constant__ PairSchedule sched) {
  using C = PairCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // staging first, then the stage ring, then barriers
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t ring = base + C::STAGING_BYTES;
  const uint32_t bar0 = ring + C::STAGES * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto ready_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  auto empty_bar = [&](int s) { return bar0 + 8u * (2 * C::STAGES + s); };
  const uint32_t tfull_bar = bar0 + 8u * (3 * C::STAGES);
  const uint32_t tempty_bar = bar0 + 8u * (3 * C::STAGES + 1);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(
      gbase + C::STAGING_BYTES + C::STAGES * C::STAGE_BYTES + 8 * (3 * C::STAGES + 2));
  volatile int* stop = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const long long wait_limit = p.wait_cycles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(ready_bar(s), 2);  // one relay arrival per CTA (used in the leader only)
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(tfull_bar, 1);
    ptx::mbar_init(tempty_bar, 8);  // four epilogue warps in each CTA (used in the leader only)
    *stop = 0;
    ptx::fence_mbar_init();
    for (int j = 0; j < p.nprob; ++j) {
      for (int s = 0; s < 3; ++s) {
        ptx::prefetch_tmap(&gm.a[j][s]);
        ptx::prefetch_tmap(&gm.b[j][s]);
      }
      ptx::prefetch_tmap(&gm.d[j]);
    }
  }
  ptx::cluster_sync();  // both CTAs' barriers exist before anything arrives on them
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::grid_dep_launch_dependents();
  ptx::tc_fence_before();
  ptx::cluster_sync();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  ptx::grid_dep_wait();  // the prologue above touched no global memory

  const int total_tiles = p.prob[p.nprob - 1].tile_end;
  const int first_tile = (int)ptx::cluster_id_x(), tile_step = (int)ptx::nclusters_x();
  // this cluster's tiles: a range of the host's table, or every tile_step-th tile
  const int my_begin = sched.use ? (int)sched.off[first_tile] : 0;
  const int my_count = sched.use ? (int)sched.off[first_tile + 1] - my_begin
                                 : (total_tiles - first_tile + tile_step - 1) / tile_step;
  auto tile_of = [&](int i) -> int { return sched.use ? (int)sched.tile[my_begin + i] : first_tile + i * tile_step; };
  // pair tile t -> (problem, 256-row block, 256-column block of that problem); rows vary fastest
  auto locate = [&](int t, int& prob, int& m_pt, int& n_tile) {
    prob = 0;
    int start = 0;
    while (prob + 1 < p.nprob && t >= p.prob[prob].tile_end) start = p.prob[prob++].tile_end;
    const int tm2 = p.prob[prob].tiles_m2;
    raster(t - start, tm2, (p.prob[prob].tile_end - start) / tm2, m_pt, n_tile);
    m_pt += p.prob[prob].m_rot;
    if (m_pt >= tm2) m_pt -= tm2;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    const bool leader = ptx::elect_one();
    int stage = 0;
    uint32_t phase = 0;
    int flag_prob = -1;      // problem the mask below belongs to
    uint32_t flag_mask = 0;  // its flags that have been seen up
    bool live = true;        // false once a wait of this role has failed: nothing more is issued
    for (int i = 0; i < my_count && live; ++i) {
      const int t = tile_of(i);
      int prob, m_pt, n_tile;
      locate(t, prob, m_pt, n_tile);
      const PairProb& pp = p.prob[prob];
      if (pp.flag != nullptr) {
        // The activation of this problem is being filled by somebody else (copy engines, other
        // GPUs over NVLink): wait until the flag of this tile's rows - or, without per-row flags,
        // every flag - has reached the target, then order the tensor-map reads after it.
        if (flag_prob != prob) { flag_prob = prob; flag_mask = 0; }
        const int f0 = pp.flag_rows > 0 ? min((m_pt * 256) / pp.flag_rows, pp.flag_count - 1) : 0;
        const int f1 = pp.flag_rows > 0 ? f0 + 1 : pp.flag_count;
        bool waited = false;
        for (int f = f0; f < f1; ++f) {
          if (flag_mask & (1u << (f & 31))) continue;
          const long long t0 = clock64();
          int target = pp.flag_value;
          if (pp.flag_epoch != nullptr)
            asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(target) : "l"(pp.flag_epoch) : "memory");
          for (;;) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(pp.flag + f) : "memory");
            if (v - target >= 0) break;
            if (*stop) { live = false; break; }
            __nanosleep(200);
            if (clock64() - t0 > wait_limit) {
              *stop = 1;
              atomicOr(p.status, 1024);
            }
          }
          if (!live) break;
          flag_mask |= 1u << (f & 31);
          waited = true;
        }
        if (!live) break;
        if (waited) asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      const int m_row0 = m_pt * 256 + (int)rank * 128, n_row0 = n_tile * 256 + (int)rank * 128;
      // this CTA's 128 rows inside their shard (the map is 3-D: byte, row of the shard, shard), and
      // their scale blocks; a CTA whose 128 rows lie wholly beyond M reads the last real row
      // block's scales (its accumulator rows are never stored), so that no copy leaves the buffer
      const int a_shard = m_row0 / pp.shard_rows, a_row = m_row0 - a_shard * pp.shard_rows;
      const int row_blk = min(m_pt * 2 + (int)rank, (pp.M + 127) / 128 - 1);
      const int sf_shard = (row_blk * 128) / pp.shard_rows, sf_blk = row_blk - sf_shard * (pp.shard_rows >> 7);
#pragma unroll 1
      for (int seg = 0; seg < 3 && live; ++seg) {
        const SegParams sp = seg == 0 ? pp.seg[0] : (seg == 1 ? pp.seg[1] : pp.seg[2]);
        const CUtensorMap* ta = &gm.a[prob][seg];
        const CUtensorMap* tb = &gm.b[prob][seg];
        const uint32_t tx_ab = seg == 0 ? p.tx_a[0] + p.tx_b[0]
                                        : (seg == 1 ? p.tx_a[1] + p.tx_b[1] : p.tx_a[2] + p.tx_b[2]);
        const uint32_t sf_stride = seg == 0 ? pp.sf_shard_stride[0] : (seg == 1 ? pp.sf_shard_stride[1] : pp.sf_shard_stride[2]);
        const uint8_t* sfa_row = sp.sfa + (size_t)sf_shard * sf_stride + (size_t)sf_blk * sp.katoms * 512;
        const uint8_t* sfb_row = sp.sfb + (size_t)(n_tile * 2) * sp.katoms * 512;
#pragma unroll 1
        for (int s = 0; s < sp.nstages; ++s) {
          if (!wait_parity(empty_bar(stage), phase ^ 1u, stop, p.status, wait_limit, 1)) { live = false; break; }
          const int atom0 = seg == 0 ? 2 * s : s;
          const int natoms = seg == 0 ? min(2, sp.katoms - atom0) : 1;
          const uint32_t sbase = ring + stage * C::STAGE_BYTES;
          const uint32_t fb = full_bar(stage);
          if (leader) {
            ptx::mbar_expect_tx(fb, tx_ab + (uint32_t)natoms * 512u * 3u);
            ptx::tma_load_3d(sbase, ta, s * 128, a_row, a_shard, fb);
            ptx::tma_load_2d(sbase + C::A_BYTES, tb, s * 128, n_row0, fb);
            ptx::bulk_load_1d(sbase + C::A_BYTES + C::B_BYTES, sfa_row + (size_t)atom0 * 512, natoms * 512, fb);
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
              ptx::bulk_load_1d(sbase + C::A_BYTES + C::B_BYTES + C::SFA_BYTES + nb * 1024,
                                sfb_row + ((size_t)nb * sp.katoms + atom0) * 512, natoms * 512, fb);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ relay: stage landed -> leader's ready barrier
    int stage = 0;
    uint32_t phase = 0;
    bool live = true;
    for (int i = 0; i < my_count && live; ++i) {
      const int t = tile_of(i);
      int prob, m_pt, n_tile;
      locate(t, prob, m_pt, n_tile);
      const int s_units = p.prob[prob].s_units;
#pragma unroll 1
      for (int s = 0; s < s_units; ++s) {
        if (!wait_parity(full_bar(stage), phase, stop, p.status, wait_limit, 64)) { live = false; break; }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ready_bar(stage), 0));
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA)
    if (rank == 0) {
      const bool leader = ptx::elect_one();
      // instruction descriptors: scale type UE8M0, M = 256 (pair), N = 256, both operands K-major
      constexpr uint32_t kCommon = ((uint32_t)(256 >> 3) << 17) | (1u << 23) | ((uint32_t)(256 >> 4) << 24);
      constexpr uint32_t kIdesc[3] = {kCommon | (1u << 7) | (1u << 10), kCommon | (4u << 7) | (5u << 10),
                                      kCommon | (0u << 7) | (5u << 10)};
      int stage = 0;
      uint32_t phase = 0, slot = 0;
      int it = 0;
      bool live = true;
      for (; it < my_count && live; ++it) {
        const int t = tile_of(it);
        int prob, m_pt, n_tile;
        locate(t, prob, m_pt, n_tile);
        const PairProb& pp = p.prob[prob];
        if (!wait_parity(tempty_bar, ((uint32_t)it & 1u) ^ 1u, stop, p.status, wait_limit, 4)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base;
        uint32_t accumulate = 0;
#pragma unroll 1
        for (int seg = 0; seg < 3 && live; ++seg) {
          const SegParams sp = seg == 0 ? pp.seg[0] : (seg == 1 ? pp.seg[1] : pp.seg[2]);
          const uint32_t id0 = seg == 0 ? kIdesc[0] : (seg == 1 ? kIdesc[1] : kIdesc[2]);
#pragma unroll 1
          for (int s = 0; s < sp.nstages; ++s) {
            if (!wait_parity(ready_bar(stage), phase, stop, p.status, wait_limit, 2)) { live = false; break; }
            ptx::tc_fence_after();
            const uint32_t sbase = ring + stage * C::STAGE_BYTES;
            const uint32_t sfa_lo = ptx::desc_lo(sbase + C::A_BYTES + C::B_BYTES);
            const uint32_t sfb_lo = sfa_lo + (C::SFA_BYTES >> 4);
            const uint32_t sfa_t = tmem_base + C::SF_COL0 + slot * C::SF_SLOT_COLS;
            const uint32_t sfb_t = sfa_t + 8;
            const uint32_t a_lo = ptx::desc_lo(sbase), b_lo = ptx::desc_lo(sbase + C::A_BYTES);
            // K elements left in this segment, in MMA steps (64 for FP4, 32 for FP6 / FP8)
            const int nm = seg == 0 ? min(4, (sp.kseg - s * 256) >> 6) : min(4, (sp.kseg - s * 128) >> 5);
            if (leader) {
              ptx::tc_cp_sf_pair(sfa_t, sfa_lo, ptx::kDescHiSf);
              ptx::tc_cp_sf_pair(sfb_t, sfb_lo, ptx::kDescHiSf);
              ptx::tc_cp_sf_pair(sfb_t + 4, sfb_lo + 64, ptx::kDescHiSf);
              if (seg == 0 && nm > 2) {
                ptx::tc_cp_sf_pair(sfa_t + 4, sfa_lo + 32, ptx::kDescHiSf);
                ptx::tc_cp_sf_pair(sfb_t + 8, sfb_lo + 32, ptx::kDescHiSf);
                ptx::tc_cp_sf_pair(sfb_t + 12, sfb_lo + 64 + 32, ptx::kDescHiSf);
              }
              if (seg == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (j < nm) {
                    const uint32_t a = j >> 1, sfid = (j & 1) * 2;
                    ptx::mma_mxf4_pair(d_tmem, a_lo + j * 2, b_lo + j * 2, ptx::kDescHiSw128,
                                       id0 | (sfid << 4) | (sfid << 29), sfa_t + a * 4, sfb_t + a * 8, accumulate);
                    accumulate = 1;
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (j < nm) {
                    ptx::mma_mxf8f6f4_pair(d_tmem, a_lo + j * 2, b_lo + j * 2, ptx::kDescHiSw128,
                                           id0 | ((uint32_t)j << 4) | ((uint32_t)j << 29), sfa_t, sfb_t, accumulate);
                    accumulate = 1;
                  }
                }
              }
              ptx::tc_commit_pair(empty_bar(stage), 3);  // frees the stage in both CTAs
            }
            accumulate = 1;
            slot ^= 1u;
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          }
        }
        if (leader && live) ptx::tc_commit_pair(tfull_bar, 3);  // accumulators of both CTAs are complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 3-6)
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int trow = q * 32 + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t tempty_leader = ptx::map_to_cta(tempty_bar, 0);
    const bool issuer = warp == 3 && lane == 0;
    int it = 0;
    for (; it < my_count; ++it) {
      const int t = tile_of(it);
      int prob, m_pt, n_tile;
      locate(t, prob, m_pt, n_tile);
      wait_parity(tfull_bar, (uint32_t)it & 1u, stop, p.status, wait_limit, 8);
      __syncwarp();
      ptx::tc_fence_after();
      // Drain the accumulator in one go: every 32-column chunk is rounded to bf16 as it arrives, so
      // the whole 256-column row fits in 128 registers and TMEM goes back to the MMA warp before the
      // first byte is staged; the staging and the stores then overlap the next tile's MMAs instead
      // of holding them up.
      uint32_t pk[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r0[32], r1[32];
        ptx::tmem_ld_32x32(taddr + c * 64, r0);
        ptx::tmem_ld_32x32(taddr + c * 64 + 32, r1);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r0[k * 2]), __uint_as_float(r0[k * 2 + 1]));
          __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r1[k * 2]), __uint_as_float(r1[k * 2 + 1]));
          pk[c * 32 + k] = *reinterpret_cast<uint32_t*>(&h0);
          pk[c * 32 + 16 + k] = *reinterpret_cast<uint32_t*>(&h1);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader);
      const int m0 = m_pt * 256 + (int)rank * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (issuer) ptx::bulk_wait_group_read<C::NSLOT - 1>();  // the slot's last store has read it
        ptx::named_barrier_sync(1, 128);
        const uint32_t slot_addr = base + (uint32_t)(j % C::NSLOT) * C::PANEL_BYTES;
        const uint32_t prow = slot_addr + trow * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          ptx::sts_v4(prow + ((uint32_t)(c ^ (trow & 7)) << 4), pk[j * 32 + c * 4], pk[j * 32 + c * 4 + 1],
                      pk[j * 32 + c * 4 + 2], pk[j * 32 + c * 4 + 3]);
        ptx::fence_proxy_async_smem();
        ptx::named_barrier_sync(1, 128);
        if (issuer) {
          if (m0 < p.prob[prob].M && !*stop) ptx::tma_store_2d(&gm.d[prob], n_tile * 256 + j * 64, m0, slot_addr);
          ptx::bulk_commit_group();  // one group per panel, also when nothing was stored
        }
      }
    }
    if (issuer) ptx::bulk_wait_group0();
  }

  // ------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  // A CTA that gave up tells its peer (which is still here: it cannot pass the barrier below before
  // this CTA arrives), so that both take the same path through the second barrier.
  __syncthreads();
  if (threadIdx.x == 0 && *stop) ptx::st_cluster_u32(ptx::map_to_cta(ptx::smem_u32(const_cast<int*>(stop)), rank ^ 1u), 1u);
  ptx::cluster_sync();
  ptx::tc_fence_after();
  if (*stop) {
    // give copies and MMAs that are still in flight time to land before either CTA goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    ptx::cluster_sync();
  }
  if (warp == 1) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
}

// Copies `rows` rows of `src_pitch` bytes to a wider pitch, zero-filling the tail; up to
// four such jobs per launch (blockIdx.y).  Used for segments that are not a multiple of 128.
struct RepackJob {
  const uint8_t* src;
  uint8_t* dst;
  int rows, src_pitch, dst_pitch, copy_bytes;  // copy_bytes of every source row are real data
};
struct RepackJobs {
  RepackJob j[4];
};

__global__ void repack_rows_kernel(const RepackJobs jobs) {
  const RepackJob jb = blockIdx.y == 0 ? jobs.j[0] : blockIdx.y == 1 ? jobs.j[1] : blockIdx.y == 2 ? jobs.j[2] : jobs.j[3];
  const int words = jb.dst_pitch >> 2, src_words = jb.copy_bytes >> 2;
  const size_t total = (size_t)jb.rows * words;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / words), w = (int)(i - (size_t)r * words);
    uint32_t v = 0;
    if (w < src_words) v = reinterpret_cast<const uint32_t*>(jb.src + (size_t)r * jb.src_pitch)[w];
    reinterpret_cast<uint32_t*>(jb.dst + (size_t)r * jb.dst_pitch)[w] = v;
  }
}

// ---------------------------------------------------------------- host side
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_encode_once;

int get_encoder(PFN_cuTensorMapEncodeTiled_v12000* out) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  *out = g_encode;
  return g_encode ? MG_OK : MG_ERR_CUDA;
}

// 2-D K-major operand: `kdim` elements of type `dt` per row, `rows` rows, `pitch` bytes.
int make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, uint64_t kdim, uint64_t rows,
             uint64_t pitch, uint32_t box_k, uint32_t box_rows) {
  PFN_cuTensorMapEncodeTiled_v12000 enc;
  if (get_encoder(&enc) != MG_OK) return MG_ERR_CUDA;
  cuuint64_t dims[2] = {kdim, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {box_k, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    mg::note_cuda_error(cudaErrorInvalidValue);
    return MG_ERR_CUDA;
  }
  return MG_OK;
}

// 3-D K-major operand stored in row shards: `kdim` elements per row, `shard_rows` rows `pitch` bytes
// apart per shard, `nshards` shards `shard_stride` bytes apart.  One shard describes a plain 2-D operand.
int make_map3(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, uint64_t kdim, uint64_t shard_rows,
              uint64_t nshards, uint64_t pitch, uint64_t shard_stride, uint32_t box_k, uint32_t box_rows) {
  PFN_cuTensorMapEncodeTiled_v12000 enc;
  if (get_encoder(&enc) != MG_OK) return MG_ERR_CUDA;
  cuuint64_t dims[3] = {kdim, shard_rows, nshards};
  cuuint64_t strides[2] = {pitch, shard_stride};
  cuuint32_t box[3] = {box_k, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    mg::note_cuda_error(cudaErrorInvalidValue);
    return MG_ERR_CUDA;
  }
  return MG_OK;
}

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Where each of the six code buffers (AN, BN, AS, BS, AO, BO) is read from and with which row
// pitch.  The tensor-map types that unpack FP6 / FP4 for kind::mxf8f6f4 need a pitch that is a
// multiple of 32 bytes and covers the segment rounded up to 128 elements; a buffer that does
// not offer that (the dense layout of a segment that is only a multiple of 64) is first copied
// to such a pitch in the workspace.
struct Plan {
  size_t pitch[6];   // pitch the GEMM reads with
  bool repack[6];
  size_t off[6];     // workspace offset of the padded copy
  size_t dense[6];   // bytes of real data per row
  size_t total;      // workspace bytes
  int ksp, kop;      // segment sizes rounded up to 128
  int status;
};

Plan make_plan(int M, int N, int KN, int KS, int KO, const size_t* pitches) {
  Plan pl{};
  pl.ksp = round_up(KS, 128);
  pl.kop = round_up(KO, 128);
  const size_t dense[6] = {(size_t)KN / 2, (size_t)KN / 2, (size_t)KS / 4 * 3, (size_t)KS / 2, (size_t)KO, (size_t)KO / 2};
  const size_t need[6] = {(size_t)KN / 2, (size_t)KN / 2, (size_t)pl.ksp / 4 * 3, (size_t)pl.ksp / 2, (size_t)pl.kop,
                          (size_t)pl.kop / 2};
  const size_t align[6] = {16, 16, 32, 32, 16, 32};
  const int rows[6] = {M, N, M, N, M, N};
  const int kseg[6] = {KN, KN, KS, KS, KO, KO};
  size_t off = 0;
  pl.status = MG_OK;
  for (int i = 0; i < 6; ++i) {
    pl.dense[i] = dense[i];
    const size_t given = pitches ? pitches[i] : dense[i];
    if (kseg[i] == 0) { pl.pitch[i] = 0; continue; }
    if (given < dense[i]) { pl.status = MG_ERR_SHAPE; return pl; }
    if (given % align[i] == 0 && given >= need[i]) {
      pl.pitch[i] = given;
    } else if (i < 2) {
      pl.status = MG_ERR_ALIGN;  // the FP4 segment is a multiple of 128: only a bad pitch gets here
      return pl;
    } else {
      pl.repack[i] = true;
      pl.pitch[i] = need[i];
      pl.off[i] = off;
      off = align_up(off + (size_t)rows[i] * need[i], 1024);
    }
  }
  pl.total = off;
  return pl;
}

int choose_bn(int M, int N, int sms, const mg::Options& opt) {
  if (opt.gemm_bn == 128 || (opt.gemm_bn == 256 && N % 256 == 0)) return opt.gemm_bn;
  if (N % 256 != 0) return 128;
  const int tm = (M + BM - 1) / BM;
  auto eff = [&](int bn, double w) {
    const int tiles = tm * (N / bn);
    const int waves = (tiles + sms - 1) / sms;
    return w * (double)tiles / ((double)waves * sms);
  };
  return eff(256, 1.0) >= eff(128, 0.92) ? 256 : 128;
}

template <int BN, bool SWAP = false>
int launch_gemm(const GemmParams& p, const CUtensorMap* maps, int sms, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kern = mixed_gemm_kernel<BN, SWAP>;
  MG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
  const int items = p.tiles_m * p.tiles_n * p.splits;
  const int grid = items < sms ? items : sms;
  MG_CUDA_TRY(mg::launch_kernel(kern, dim3(grid), dim3(kThreads), C::SMEM, st, p, maps[0], maps[1], maps[2], maps[3],
                                maps[4], maps[5]));
  return MG_OK;
}

// Cluster split-K launch: clusters of four CTAs, one tile per cluster at a time.
int launch_gemm_cs(const GemmParams& p, const CUtensorMap* maps, int sms, cudaStream_t st) {
  using C = Cfg<128, true>;
  auto kern = mixed_gemm_kernel<128, false, true>;
  MG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
  const int tiles = p.tiles_m * p.tiles_n;
  const int clusters = tiles < sms / 4 ? tiles : sms / 4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * 4);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 4;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = mg::pdl_enabled() ? 2 : 1;
  MG_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5]));
  return MG_OK;
}

// How many clusters of four of these CTAs the device holds at one time (asked once per device; 33
// on a B200, 0 where no GPC has four free SMs, e.g. on a partitioned GPU).
int cluster_split_capacity() {
  static std::atomic<int> known[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int k = known[dev].load();
  if (k == 0) {
    using C = Cfg<128, true>;
    auto kern = mixed_gemm_kernel<128, false, true>;
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(4);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 4;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool ok = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM) == cudaSuccess &&
                    cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n >= 1;
    if (!ok) (void)cudaGetLastError();  // the question is allowed to fail; the answer is then "no"
    k = ok ? n : -1;
    known[dev].store(k);
  }
  return k > 0 ? k : 0;
}

// Cluster split-K is taken when the 128 x 128 tiles of the problem fit the clusters the device
// holds at one time (at most a quarter of the SMs) and every quarter of K has at least two stages.
// At these sizes a launch is bound by the fixed cost of a K stage on the tensor pipe (about 255 ns,
// whatever the stage holds), so a quarter of the stages per CTA is what shortens it; the
// accumulators meet in distributed shared memory, not in L2.  Option GEMM_CSPLIT = 0 turns it off.
bool csplit_wanted(int M, int N, int s_units, int sms, const mg::Options& opt) {
  if (N % 128 != 0 || opt.gemm_csplit == 0) return false;
  const int tiles = (M + BM - 1) / BM * (N / 128);
  return tiles <= sms / 4 && s_units >= 8 && tiles <= cluster_split_capacity();
}

// Scratch behind the padded copies, for split-K: 32 KB of tile counters (each carries a per-launch
// token, so the bytes may hold anything when a call starts), then fp32 partials
// [split][tile][column group][row].
constexpr size_t kSpCounterBytes = 32 * 1024;
constexpr int kSpMaxTiles = (int)(kSpCounterBytes / sizeof(unsigned long long));

// Split-K plan of the single-CTA kernel: only when the tiles occupy at most half of the SMs, each
// split keeps at least 16 K stages (below that the partial round trip through L2 costs more than
// the shorter K loop saves: 12.6 against 8.9 us at 16 x 4096 x 4096), at most eight splits.
// Option GEMM_SPLITK = 0 turns it off, n > 0 forces n splits.
struct SplitPlan {
  int splits, rows;
  size_t bytes;  // fp32 partials
};
// True when the decode form of the single-CTA kernel takes the problem.  Measured on B200 it wins
// for M <= 32 when there are many weight tiles or a long K (16 x 14336 x 4096: 11.2 against 13.8 us,
// 16 x 8192 x 28672: 28.1 against 37.5 us) and loses when M > 32, where its element-wise transposed
// stores dominate (128 x 4096 x 4096: 16.3 against 9.8 us), or when the problem is a handful of
// short tiles (16 x 4096 x 4096: 9.9 against 8.9 us).  Option GEMM_SWAP = 0 / 1 turns it off / on
// for every M <= 128.
bool swap_wanted(int M, int N, int s_units, const mg::Options& opt) {
  if (M > 128 || N % 128 != 0) return false;
  if (opt.gemm_swap >= 0) return opt.gemm_swap != 0;
  return M <= 32 && (N / 128 >= 64 || s_units >= 32);
}
int swap_bn(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }

SplitPlan plan_splitk(int M, int N, int s_units, int bn, int sms, bool swap, const mg::Options& opt) {
  SplitPlan sp{1, 128, 0};
  const int tiles_m = (M + BM - 1) / BM, tiles = swap ? N / 128 : tiles_m * (N / bn);
  const int want = opt.gemm_splitk;
  if (want == 0 || tiles > kSpMaxTiles) return sp;
  int splits = std::min(std::min(sms / tiles, s_units / 16), 8);  // the arrival count has 8 bits
  if (tiles * 2 > sms) splits = 1;
  if (want > 0) splits = std::min(std::min(want, s_units), 64);
  if (splits < 2) return sp;
  sp.splits = splits;
  sp.rows = (!swap && tiles_m == 1 && M <= 96) ? (M + 31) / 32 * 32 : 128;
  sp.bytes = (size_t)splits * tiles * sp.rows * bn * sizeof(float);
  return sp;
}

// One problem of a CTA-pair launch as the host sees it (device pointers).
struct PairProblem {
  const uint8_t* a[3];    // AN, AS, AO
  const uint8_t* sfa[3];
  size_t pitch_a[3];
  const uint8_t* b[3];    // BN, BS, BO
  const uint8_t* sfb[3];
  size_t pitch_b[3];
  int M, N, KN, KS, KO;
  void* D;
  int ldd;
  const int* flag;
  int flag_count;
  const int* flag_epoch;
  int flag_value;
  int flag_rows;
  int first_row;
  int shard_rows;              // 0: the activation is one block of M rows
  size_t a_shard_stride[3];    // bytes between consecutive shards of AN / AS / AO
  size_t sfa_shard_stride[3];  // and of their scale buffers
};

// The schedule of a problem list: tiles in list order, each to the cluster that is free first when a
// tile of problem j costs cost[j].  Lists whose tiles all cost the same keep the round-robin order
// (use = 0).  The last few distinct lists are remembered: a caller repeats the same shapes step after
// step and the dealing is a few thousand heap operations.
struct ScheduleKey {
  int nprob, clusters;
  int tiles[kMaxProb], cost[kMaxProb];
  bool operator==(const ScheduleKey& o) const { return memcmp(this, &o, sizeof(*this)) == 0; }
};

const PairSchedule& schedule_for(const ScheduleKey& key) {
  static std::mutex mu;
  static ScheduleKey keys[4];
  static PairSchedule tables[4];
  static int used = 0, next = 0;
  static thread_local PairSchedule mine;  // the caller's copy: another thread may evict the cached one
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (keys[i] == key) { mine = tables[i]; return mine; }
  const int slot = used < 4 ? used++ : (next++ & 3);
  PairSchedule& t = tables[slot];
  keys[slot] = key;
  int total = 0;
  bool same = true;
  for (int j = 0; j < key.nprob; ++j) {
    total += key.tiles[j];
    same = same && key.cost[j] == key.cost[0];
  }
  t.use = 0;
  if (!same && total <= kMaxSched && key.clusters <= kMaxClusters && total > key.clusters) {
    // (time free, cluster) min-heap; per-cluster lists are built in two passes: counts, then entries
    // fixed-size scratch (guarded by the mutex): nothing here allocates
    static std::pair<long long, int> heap[kMaxClusters];
    static uint16_t owner[kMaxSched];
    static int count[kMaxClusters], fill[kMaxClusters];
    for (int c = 0; c < key.clusters; ++c) { heap[c] = {0, -c}; count[c] = fill[c] = 0; }
    auto cmp = [](const std::pair<long long, int>& a, const std::pair<long long, int>& b) {
      return a.first != b.first ? a.first > b.first : a.second < b.second;  // earliest first, then lowest cluster
    };
    std::make_heap(heap, heap + key.clusters, cmp);
    int tix = 0;
    for (int j = 0; j < key.nprob; ++j)
      for (int i = 0; i < key.tiles[j]; ++i, ++tix) {
        std::pop_heap(heap, heap + key.clusters, cmp);
        std::pair<long long, int>& top = heap[key.clusters - 1];
        const int c = -top.second;
        owner[tix] = (uint16_t)c;
        ++count[c];
        top.first += key.cost[j];
        std::push_heap(heap, heap + key.clusters, cmp);
      }
    int off = 0;
    for (int c = 0; c < key.clusters; ++c) { t.off[c] = (uint16_t)off; off += count[c]; }
    for (int c = key.clusters; c <= kMaxClusters; ++c) t.off[c] = (uint16_t)off;
    for (int i = 0; i < total; ++i) {
      const int c = owner[i];
      t.tile[t.off[c] + fill[c]++] = (uint16_t)i;
    }
    t.use = 1;
  }
  mine = t;
  return mine;
}

// Validates the problems, builds their tensor maps and launches the CTA-pair kernel once.
// Every code buffer must be readable in place (a pitch the unpacking tensor maps take).
int launch_pair(int nprob, const PairProblem* pr, int sms, cudaStream_t st) {
  if (nprob < 1 || nprob > kMaxProb) return MG_ERR_SHAPE;
  PairParams p{};
  PairMaps gm;
  int rc;
  int tiles = 0;
  for (int j = 0; j < nprob; ++j) {
    const PairProblem& q = pr[j];
    if (q.M <= 0 || q.N <= 0 || q.N % 256 || q.KN < 0 || q.KS < 0 || q.KO < 0 || q.KN + q.KS + q.KO <= 0) return MG_ERR_SHAPE;
    if (q.KN % 128 || q.KS % 64 || q.KO % 64 || q.ldd < q.N || q.ldd % 8) return MG_ERR_SHAPE;
    if (!q.D) return MG_ERR_NULL;
    if (!mg::aligned(q.D, 16)) return MG_ERR_ALIGN;
    const size_t pitches[6] = {q.pitch_a[0], q.pitch_b[0], q.pitch_a[1], q.pitch_b[1], q.pitch_a[2], q.pitch_b[2]};
    const Plan pl = make_plan(q.M, q.N, q.KN, q.KS, q.KO, pitches);
    if (pl.status != MG_OK) return pl.status;
    if (pl.total) return MG_ERR_ALIGN;  // a buffer would need the padded copy: not in this launch
    const int kseg[3] = {q.KN, q.KS, q.KO};
    const int first = q.KN ? 0 : (q.KS ? 1 : 2);
    for (int seg = 0; seg < 3; ++seg) {
      // a zero-sized segment still needs valid maps as kernel arguments: alias the first real one
      const int sg = kseg[seg] ? seg : first;
      if (!q.a[sg] || !q.sfa[sg] || !q.b[sg] || !q.sfb[sg]) return MG_ERR_NULL;
      if (!mg::aligned(q.a[sg], 32) || !mg::aligned(q.b[sg], 32) || !mg::aligned(q.sfa[sg], 16) || !mg::aligned(q.sfb[sg], 16))
        return MG_ERR_ALIGN;
      const uint64_t kd = sg == 0 ? q.KN / 2 : (sg == 1 ? pl.ksp : pl.kop);
      const CUtensorMapDataType da = sg == 1 ? CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8;
      const CUtensorMapDataType db = sg == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B;
      const int srows = q.shard_rows > 0 ? q.shard_rows : q.M;
      const int nshards = (q.M + srows - 1) / srows;
      if (nshards > 1) {
        if (srows % 128 || q.M % srows || q.a_shard_stride[sg] % 32 || q.sfa_shard_stride[sg] % 16 || q.sfa_shard_stride[sg] > 0xffffffffull ||
            q.a_shard_stride[sg] < (size_t)srows * pl.pitch[sg * 2])
          return MG_ERR_SHAPE;
      }
      const uint64_t sstride = nshards > 1 ? q.a_shard_stride[sg] : (uint64_t)align_up((size_t)srows * pl.pitch[sg * 2], 32);
      if ((rc = make_map3(&gm.a[j][seg], da, q.a[sg], kd, srows, nshards, pl.pitch[sg * 2], sstride, 128, BM))) return rc;
      if ((rc = make_map(&gm.b[j][seg], db, q.b[sg], kd, q.N, pl.pitch[sg * 2 + 1], 128, 128))) return rc;
    }
    if ((rc = make_map(&gm.d[j], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, q.D, q.N, q.M, (uint64_t)q.ldd * 2, 64, 128))) return rc;
    PairProb& d = p.prob[j];
    d.seg[0] = {q.KN, (q.KN + 255) / 256, (q.KN + 127) / 128, q.sfa[0], q.sfb[0]};
    d.seg[1] = {q.KS, (q.KS + 127) / 128, (q.KS + 127) / 128, q.sfa[1], q.sfb[1]};
    d.seg[2] = {q.KO, (q.KO + 127) / 128, (q.KO + 127) / 128, q.sfa[2], q.sfb[2]};
    d.M = q.M;
    d.shard_rows = q.shard_rows > 0 && q.shard_rows < q.M ? q.shard_rows : ((q.M + 127) / 128) * 128;
    for (int seg = 0; seg < 3; ++seg) d.sf_shard_stride[seg] = (uint32_t)q.sfa_shard_stride[seg];
    d.tiles_m2 = (q.M + 255) / 256;
    tiles += d.tiles_m2 * (q.N / 256);
    d.tile_end = tiles;
    d.s_units = d.seg[0].nstages + d.seg[1].nstages + d.seg[2].nstages;
    d.flag = q.flag;
    d.flag_count = q.flag ? (q.flag_count > 0 ? q.flag_count : 1) : 0;
    d.flag_epoch = q.flag_epoch;
    d.flag_value = q.flag_value;
    if (q.flag && q.flag_count > 32) return MG_ERR_SHAPE;
    if (q.flag_rows < 0 || q.flag_rows % 256 || q.first_row < 0 || q.first_row % 256) return MG_ERR_SHAPE;
    d.flag_rows = q.flag ? q.flag_rows : 0;
    d.m_rot = (q.first_row / 256) % d.tiles_m2;
  }
  for (int j = nprob; j < kMaxProb; ++j) {  // unused slots: valid maps, never dereferenced
    for (int seg = 0; seg < 3; ++seg) {
      gm.a[j][seg] = gm.a[0][seg];
      gm.b[j][seg] = gm.b[0][seg];
    }
    gm.d[j] = gm.d[0];
  }
  p.nprob = nprob;
  // A tensor-map load signals the packed byte count of its box on the mbarrier.
  p.tx_a[0] = BM * 128; p.tx_b[0] = 128 * 128;
  p.tx_a[1] = BM * 96;  p.tx_b[1] = 128 * 64;
  p.tx_a[2] = BM * 128; p.tx_b[2] = 128 * 64;
  p.wait_cycles = mg::wait_limit_cycles();
  rc = mg::device_status_word(&p.status);
  if (rc != MG_OK) return rc;
  int max_clusters = sms / 2;
  const int cap = mg::options().gemm_max_clusters;
  if (cap > 0 && cap < max_clusters) max_clusters = cap;
  const int clusters = tiles < max_clusters ? tiles : max_clusters;
  ScheduleKey key;
  memset(&key, 0, sizeof(key));
  key.nprob = nprob;
  key.clusters = clusters;
  for (int j = 0; j < nprob; ++j) {
    key.tiles[j] = p.prob[j].tile_end - (j ? p.prob[j - 1].tile_end : 0);
    key.cost[j] = p.prob[j].s_units + 1;  // K stages, plus the accumulator drain between two tiles
  }
  if (mg::options().gemm_sched == 0) key.nprob = 1, key.tiles[0] = tiles;  // one cost: round-robin
  const PairSchedule& sched = schedule_for(key);
  MG_CUDA_TRY(cudaFuncSetAttribute(mixed_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairCfg::SMEM));
  MG_CUDA_TRY(mg::launch_kernel(mixed_gemm_pair_kernel, dim3(2 * clusters), dim3(PairCfg::THREADS), PairCfg::SMEM, st, p, gm, sched));
  return MG_OK;
}

}  // namespace

extern "C" int mg_pair_schedule(int nprob, const int* tiles, const int* cost, int clusters, int* use,
                                uint16_t* off, uint16_t* tile) {
  if (!tiles || !cost || !use || !off || !tile) return MG_ERR_NULL;
  if (nprob < 1 || nprob > kMaxProb || clusters < 1 || clusters > kMaxClusters) return MG_ERR_SHAPE;
  ScheduleKey key;
  memset(&key, 0, sizeof(key));
  key.nprob = nprob;
  key.clusters = clusters;
  long long total = 0;
  for (int j = 0; j < nprob; ++j) {
    if (tiles[j] < 0 || cost[j] < 1) return MG_ERR_SHAPE;
    key.tiles[j] = tiles[j];
    key.cost[j] = cost[j];
    total += tiles[j];
  }
  const PairSchedule& sc = schedule_for(key);
  *use = sc.use;
  if (sc.use) {
    memcpy(off, sc.off, sizeof(uint16_t) * (size_t)(clusters + 1));
    memcpy(tile, sc.tile, sizeof(uint16_t) * (size_t)total);
  }
  return MG_OK;
}

extern "C" size_t mg_matmul_workspace_bytes(int M, int N, int KN, int KS, int KO) {
  if (M <= 0 || N <= 0 || KN < 0 || KS < 0 || KO < 0) return 0;
  return make_plan(M, N, KN, KS, KO, nullptr).total;
}

// `allow_split`: whether split-K through the workspace may be chosen (mg_matmul_static_ws turns it
// off so that its result does not depend on how large the built-in scratch happens to be).
static int matmul_impl(bool f32_out, bool allow_split, const uint8_t* AN, const uint8_t* BN_, const uint8_t* AS, const uint8_t* BS,
                       const uint8_t* AO, const uint8_t* BO, const size_t* pitches, int M, int N, int KN, int KS, int KO,
                       const void* C_bf16, void* D_bf16, int ldd, const uint8_t* SFAN, const uint8_t* SFBN,
                       const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO, const uint8_t* SFBO,
                       void* workspace, size_t workspace_bytes, void* stream) {
  if (M < 0 || N <= 0 || KN < 0 || KS < 0 || KO < 0 || KN + KS + KO <= 0) return MG_ERR_SHAPE;
  if (KN % 128 || KS % 64 || KO % 64 || N % 128 || ldd < N || ldd % 8) return MG_ERR_SHAPE;
  if (M == 0) return MG_OK;
  if (!D_bf16) return MG_ERR_NULL;
  if ((KN && (!AN || !BN_ || !SFAN || !SFBN)) || (KS && (!AS || !BS || !SFAS || !SFBS)) ||
      (KO && (!AO || !BO || !SFAO || !SFBO)))
    return MG_ERR_NULL;
  if (!mg::aligned(D_bf16, 16) || !mg::aligned(C_bf16, 16)) return MG_ERR_ALIGN;
  const void* ptrs[] = {AN, BN_, AS, BS, AO, BO};
  for (const void* q : ptrs)
    if (!mg::aligned(q, 32)) return MG_ERR_ALIGN;
  const void* sfs[] = {SFAN, SFBN, SFAS, SFBS, SFAO, SFBO};
  for (const void* q : sfs)
    if (!mg::aligned(q, 16)) return MG_ERR_ALIGN;

  mg::DeviceInfo di;
  int rc = mg::device_info(&di);
  if (rc != MG_OK) return rc;
  const mg::Options opt = mg::options();
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // Buffers whose pitch the unpacking tensor maps cannot take go through a padded copy.
  const Plan pl = make_plan(M, N, KN, KS, KO, pitches);
  if (pl.status != MG_OK) return pl.status;
  const uint8_t* src[6] = {AN, BN_, AS, BS, AO, BO};
  if (pl.total) {
    if (!workspace || workspace_bytes < pl.total) return MG_ERR_WORKSPACE;
    if (!mg::aligned(workspace, 1024)) return MG_ERR_ALIGN;
    uint8_t* w = static_cast<uint8_t*>(workspace);
    RepackJobs jobs{};
    int nj = 0;
    for (int i = 2; i < 6; ++i) {
      if (!pl.repack[i]) continue;
      jobs.j[nj++] = {src[i], w + pl.off[i], (i & 1) ? N : M, (int)(pitches ? pitches[i] : pl.dense[i]),
                      (int)pl.pitch[i], (int)pl.dense[i]};
      src[i] = w + pl.off[i];
    }
    repack_rows_kernel<<<dim3(di.sm_count * 2, nj), 256, 0, st>>>(jobs);
    MG_CUDA_TRY(cudaGetLastError());
  }
  AS = src[2]; BS = src[3]; AO = src[4]; BO = src[5];

  // The CTA-pair kernel wants enough 256 x 256 tiles to occupy most SM pairs; smaller problems
  // spread better as 128-row tiles over single SMs.
  bool use_pair = !f32_out && C_bf16 == nullptr && N % 256 == 0 && M > 128;
  const int pair_tiles = ((M + 255) / 256) * (N / 256);
  if (opt.gemm_2cta >= 0) use_pair = use_pair && opt.gemm_2cta != 0;
  else use_pair = use_pair && pair_tiles * 4 >= (di.sm_count / 2) * 3;
  if (use_pair) {
    PairProblem q{};
    const uint8_t* a[3] = {AN, AS, AO};
    const uint8_t* b[3] = {BN_, BS, BO};
    const uint8_t* sa[3] = {SFAN, SFAS, SFAO};
    const uint8_t* sb[3] = {SFBN, SFBS, SFBO};
    for (int i = 0; i < 3; ++i) {
      q.a[i] = a[i]; q.b[i] = b[i]; q.sfa[i] = sa[i]; q.sfb[i] = sb[i];
      q.pitch_a[i] = pl.pitch[2 * i]; q.pitch_b[i] = pl.pitch[2 * i + 1];
    }
    q.M = M; q.N = N; q.KN = KN; q.KS = KS; q.KO = KO; q.D = D_bf16; q.ldd = ldd;
    return launch_pair(1, &q, di.sm_count, st);
  }

  // Split-K scratch sits behind the padded copies, when the caller's workspace has room for it.
  const size_t sk_off = align_up(pl.total, 1024);
  uint8_t* sk_ws = nullptr;
  size_t sk_bytes = 0;
  if (allow_split && workspace && mg::aligned(workspace, 1024) && workspace_bytes >= sk_off + kSpCounterBytes) {
    sk_ws = static_cast<uint8_t*>(workspace) + sk_off;
    sk_bytes = workspace_bytes - sk_off;
  }
  const int s_units = (KN + 255) / 256 + (KS + 127) / 128 + (KO + 127) / 128;
  const bool csplit = csplit_wanted(M, N, s_units, di.sm_count, opt);
  const bool swap = !csplit && swap_wanted(M, N, s_units, opt);
  // rows of one load of the MMA's column operand: weights, or (decode form) activations
  const int bn = csplit ? 128 : (swap ? swap_bn(M) : choose_bn(M, N, di.sm_count, opt));

  GemmParams p{};
  p.M = M;
  p.N = N;
  p.ldd = ldd;
  p.tiles_m = swap ? N / BM : (M + BM - 1) / BM;
  p.tiles_n = swap ? 1 : N / bn;
  p.seg[0] = {KN, (KN + 255) / 256, (KN + 127) / 128, swap ? SFBN : SFAN, swap ? SFAN : SFBN};
  p.seg[1] = {KS, (KS + 127) / 128, (KS + 127) / 128, swap ? SFBS : SFAS, swap ? SFAS : SFBS};
  p.seg[2] = {KO, (KO + 127) / 128, (KO + 127) / 128, swap ? SFBO : SFAO, swap ? SFAO : SFBO};
  p.C = static_cast<const __nv_bfloat16*>(C_bf16);
  p.D = f32_out ? nullptr : static_cast<__nv_bfloat16*>(D_bf16);
  p.Df32 = f32_out ? static_cast<float*>(D_bf16) : nullptr;
  p.wait_cycles = mg::wait_limit_cycles();
  p.skip_load = opt.fault_skip_load > 0 ? opt.fault_skip_load : 0;
  rc = mg::device_status_word(&p.status);
  if (rc != MG_OK) return rc;
  // A tensor-map load signals the packed byte count of its box on the mbarrier.
  p.tx_a[0] = BM * 128;       p.tx_b[0] = (uint32_t)bn * 128;
  p.tx_a[1] = BM * 96;        p.tx_b[1] = (uint32_t)bn * 64;
  p.tx_a[2] = BM * 128;       p.tx_b[2] = (uint32_t)bn * 64;
  if (swap) {  // 128 weight rows (E2M1 in every segment) against bn activation rows
    p.tx_a[1] = BM * 64;      p.tx_b[1] = (uint32_t)bn * 96;
    p.tx_a[2] = BM * 64;      p.tx_b[2] = (uint32_t)bn * 128;
  }

  CUtensorMap maps[6];
  // a zero-sized segment still needs valid maps as kernel arguments: alias the first real one
  const int first = KN ? 0 : (KS ? 1 : 2);
  for (int seg = 0; seg < 3; ++seg) {
    const int s = (seg == 0 ? KN : seg == 1 ? KS : KO) ? seg : first;
    // activations go to map 2 seg, weights to 2 seg + 1; the decode form hands them over swapped
    CUtensorMap* ma = &maps[seg * 2 + (swap ? 1 : 0)];
    CUtensorMap* mb = &maps[seg * 2 + (swap ? 0 : 1)];
    const int box_a = swap ? bn : BM, box_b = swap ? BM : bn;
    if (s == 0) {
      if ((rc = make_map(ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, AN, KN / 2, M, pl.pitch[0], 128, box_a))) return rc;
      if ((rc = make_map(mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, BN_, KN / 2, N, pl.pitch[1], 128, box_b))) return rc;
    } else if (s == 1) {
      if ((rc = make_map(ma, CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, AS, pl.ksp, M, pl.pitch[2], 128, box_a))) return rc;
      if ((rc = make_map(mb, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, BS, pl.ksp, N, pl.pitch[3], 128, box_b))) return rc;
    } else {
      if ((rc = make_map(ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, AO, pl.kop, M, pl.pitch[4], 128, box_a))) return rc;
      if ((rc = make_map(mb, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, BO, pl.kop, N, pl.pitch[5], 128, box_b))) return rc;
    }
  }
  p.splits = 1;
  if (csplit) {
    p.splits = 4;
    return launch_gemm_cs(p, maps, di.sm_count, st);
  }
  if (sk_ws) {
    const SplitPlan sp = plan_splitk(M, N, s_units, bn, di.sm_count, swap, opt);
    if (sp.splits > 1 && sk_bytes >= kSpCounterBytes + sp.bytes) {
      p.splits = sp.splits;
      p.sp_rows = sp.rows;
      p.sp_counters = reinterpret_cast<unsigned long long*>(sk_ws);
      p.sp_partials = reinterpret_cast<float*>(sk_ws + kSpCounterBytes);
      static std::atomic<unsigned long long> token{std::random_device{}() | 1ull};
      p.sp_token = (token.fetch_add(0x9E3779B97F4A7C15ull) >> 8) | 1ull;  // 56 bits, never 0
    }
  }
  if (swap) {
    switch (bn) {
      case 16: return launch_gemm<16, true>(p, maps, di.sm_count, st);
      case 32: return launch_gemm<32, true>(p, maps, di.sm_count, st);
      case 64: return launch_gemm<64, true>(p, maps, di.sm_count, st);
      default: return launch_gemm<128, true>(p, maps, di.sm_count, st);
    }
  }
  return bn == 256 ? launch_gemm<256>(p, maps, di.sm_count, st) : launch_gemm<128>(p, maps, di.sm_count, st);
}

extern "C" int mg_matmul(const uint8_t* AN, const uint8_t* BN_, const uint8_t* AS, const uint8_t* BS,
                         const uint8_t* AO, const uint8_t* BO, int M, int N, int KN, int KS, int KO,
                         const void* C_bf16, void* D_bf16, int ldd, const uint8_t* SFAN, const uint8_t* SFBN,
                         const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO, const uint8_t* SFBO,
                         void* workspace, size_t workspace_bytes, void* stream) {
  return matmul_impl(false, true, AN, BN_, AS, BS, AO, BO, nullptr, M, N, KN, KS, KO, C_bf16, D_bf16, ldd, SFAN, SFBN,
                     SFAS, SFBS, SFAO, SFBO, workspace, workspace_bytes, stream);
}

extern "C" int mg_matmul_pitched(const uint8_t* AN, const uint8_t* BN_, const uint8_t* AS, const uint8_t* BS,
                                 const uint8_t* AO, const uint8_t* BO, const size_t* pitches, int out_f32, int M, int N,
                                 int KN, int KS, int KO, const void* C_bf16, void* D, int ldd, const uint8_t* SFAN,
                                 const uint8_t* SFBN, const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO,
                                 const uint8_t* SFBO, void* workspace, size_t workspace_bytes, void* stream) {
  return matmul_impl(out_f32 != 0, true, AN, BN_, AS, BS, AO, BO, pitches, M, N, KN, KS, KO, C_bf16, D, ldd, SFAN, SFBN, SFAS,
                     SFBS, SFAO, SFBO, workspace, workspace_bytes, stream);
}

extern "C" size_t mg_matmul_pitched_workspace_bytes(int M, int N, int KN, int KS, int KO, const size_t* pitches) {
  if (M <= 0 || N <= 0 || KN < 0 || KS < 0 || KO < 0) return 0;
  const size_t need = make_plan(M, N, KN, KS, KO, pitches).total;
  // On top: what split-K of the single-CTA kernel (few tiles, long K) would use, if it may be chosen
  // for this problem.  A smaller workspace still works, without it.
  mg::DeviceInfo di;
  const int sms = mg::device_info(&di) == MG_OK ? di.sm_count : 148;
  const mg::Options opt = mg::options();
  const int s_units = (KN + 255) / 256 + (KS + 127) / 128 + (KO + 127) / 128;
  size_t extra = 0;
  for (int bn : {128, 256})
    if (N % bn == 0) extra = std::max(extra, plan_splitk(M, N, s_units, bn, sms, false, opt).bytes);
  if (M <= 128 && N % 128 == 0) extra = std::max(extra, plan_splitk(M, N, s_units, swap_bn(M), sms, true, opt).bytes);
  if (extra == 0) return need;
  return align_up(need, 1024) + kSpCounterBytes + extra;
}

extern "C" int mg_matmul_f32(const uint8_t* AN, const uint8_t* BN_, const uint8_t* AS, const uint8_t* BS,
                             const uint8_t* AO, const uint8_t* BO, int M, int N, int KN, int KS, int KO,
                             const void* C_bf16, float* D_f32, int ldd, const uint8_t* SFAN, const uint8_t* SFBN,
                             const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO, const uint8_t* SFBO,
                             void* workspace, size_t workspace_bytes, void* stream) {
  return matmul_impl(true, true, AN, BN_, AS, BS, AO, BO, nullptr, M, N, KN, KS, KO, C_bf16, D_f32, ldd, SFAN, SFBN, SFAS,
                     SFBS, SFAO, SFBO, workspace, workspace_bytes, stream);
}

extern "C" int mg_matmul_fp4(const uint8_t* A, const uint8_t* B, int M, int N, int K, const void* C_bf16,
                             void* D_bf16, const uint8_t* SFA, const uint8_t* SFB, void* stream) {
  return mg_matmul(A, B, nullptr, nullptr, nullptr, nullptr, M, N, K, 0, 0, C_bf16, D_bf16, N, SFA, SFB, nullptr,
                   nullptr, nullptr, nullptr, nullptr, 0, stream);
}
extern "C" int mg_matmul_fp6(const uint8_t* A, const uint8_t* B, int M, int N, int K, const void* C_bf16,
                             void* D_bf16, const uint8_t* SFA, const uint8_t* SFB, void* stream) {
  if (K % 128) return MG_ERR_SHAPE;
  return mg_matmul(nullptr, nullptr, A, B, nullptr, nullptr, M, N, 0, K, 0, C_bf16, D_bf16, N, nullptr, nullptr, SFA,
                   SFB, nullptr, nullptr, nullptr, 0, stream);
}
extern "C" int mg_matmul_fp8(const uint8_t* A, const uint8_t* B, int M, int N, int K, const void* C_bf16,
                             void* D_bf16, const uint8_t* SFA, const uint8_t* SFB, void* stream) {
  if (K % 128) return MG_ERR_SHAPE;
  return mg_matmul(nullptr, nullptr, nullptr, nullptr, A, B, M, N, 0, 0, K, C_bf16, D_bf16, N, nullptr, nullptr,
                   nullptr, nullptr, SFA, SFB, nullptr, 0, stream);
}

// ---------------------------------------------------------------- several weights, one activation
extern "C" int mg_matmul_group_pitched(int nprob, const uint8_t* AN, const uint8_t* AS, const uint8_t* AO,
                                       const size_t* pitches_a, const uint8_t* const* BN_, const uint8_t* const* BS,
                                       const uint8_t* const* BO, const size_t* pitches_b, int M, const int* N, int KN,
                                       int KS, int KO, void* const* D_bf16, const int* ldd, const uint8_t* SFAN,
                                       const uint8_t* SFAS, const uint8_t* SFAO, const uint8_t* const* SFBN,
                                       const uint8_t* const* SFBS, const uint8_t* const* SFBO, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  if (nprob < 1 || nprob > kMaxProb || M <= 128) return MG_ERR_SHAPE;
  if (!pitches_a || !pitches_b || !N || !D_bf16 || !ldd) return MG_ERR_NULL;
  mg::DeviceInfo di;
  int rc = mg::device_info(&di);
  if (rc != MG_OK) return rc;
  PairProblem pr[kMaxProb] = {};
  for (int j = 0; j < nprob; ++j) {
    PairProblem& q = pr[j];
    q.a[0] = AN; q.a[1] = AS; q.a[2] = AO;
    q.sfa[0] = SFAN; q.sfa[1] = SFAS; q.sfa[2] = SFAO;
    q.b[0] = BN_ ? BN_[j] : nullptr; q.b[1] = BS ? BS[j] : nullptr; q.b[2] = BO ? BO[j] : nullptr;
    q.sfb[0] = SFBN ? SFBN[j] : nullptr; q.sfb[1] = SFBS ? SFBS[j] : nullptr; q.sfb[2] = SFBO ? SFBO[j] : nullptr;
    for (int i = 0; i < 3; ++i) {
      q.pitch_a[i] = pitches_a[i];
      q.pitch_b[i] = pitches_b[j * 3 + i];
    }
    q.M = M; q.N = N[j]; q.KN = KN; q.KS = KS; q.KO = KO;
    q.D = D_bf16[j]; q.ldd = ldd[j];
  }
  return launch_pair(nprob, pr, di.sm_count, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- a list of independent problems
extern "C" int mg_matmul_multi(int nprob, const mg_problem_t* probs, void* stream) {
  if (!probs) return MG_ERR_NULL;
  if (nprob < 1 || nprob > kMaxProb) return MG_ERR_SHAPE;
  mg::DeviceInfo di;
  int rc = mg::device_info(&di);
  if (rc != MG_OK) return rc;
  PairProblem pr[kMaxProb] = {};
  for (int j = 0; j < nprob; ++j) {
    const mg_problem_t& s = probs[j];
    PairProblem& q = pr[j];
    if (s.M <= 128) return MG_ERR_SHAPE;
    q.a[0] = s.AN; q.a[1] = s.AS; q.a[2] = s.AO;
    q.sfa[0] = s.SFAN; q.sfa[1] = s.SFAS; q.sfa[2] = s.SFAO;
    q.b[0] = s.BN; q.b[1] = s.BS; q.b[2] = s.BO;
    q.sfb[0] = s.SFBN; q.sfb[1] = s.SFBS; q.sfb[2] = s.SFBO;
    for (int i = 0; i < 3; ++i) {
      q.pitch_a[i] = s.pitch_a[i];
      q.pitch_b[i] = s.pitch_b[i];
    }
    q.M = s.M; q.N = s.N; q.KN = s.KN; q.KS = s.KS; q.KO = s.KO;
    q.D = s.D_bf16; q.ldd = s.ldd;
    q.flag = s.ready_flags; q.flag_count = s.ready_count; q.flag_epoch = s.ready_epoch; q.flag_value = s.ready_value;
    q.flag_rows = s.ready_rows; q.first_row = s.first_row;
    q.shard_rows = s.a_shard_rows;
    for (int i = 0; i < 3; ++i) { q.a_shard_stride[i] = s.a_shard_stride[i]; q.sfa_shard_stride[i] = s.sfa_shard_stride[i]; }
  }
  return launch_pair(nprob, pr, di.sm_count, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- entry point that allocates nothing
//
// Some hosts of this library cannot obtain device memory at the moment they need a product:
// a serving runtime that handed all free HBM to its own pool at start-up (a later cudaMalloc
// simply fails there), or a plugin whose execute callback is forbidden to allocate because an
// allocation may synchronise the whole device.  mg_matmul needs scratch only for K segments
// that are not a multiple of 128, and only as much as the padded copies take; for those
// callers the scratch below is part of the library image instead.  Every device that loads
// the library carries it until the process exits.
namespace {
static __device__ __align__(256) uint8_t g_static_ws[MG_STATIC_WS_BYTES + 1024];
uint8_t* g_static_ws_ptr[64];  // resolved address per device, 1024-aligned inside the array
std::mutex g_static_ws_mu;
}  // namespace

extern "C" int mg_matmul_static_ws(const uint8_t* AN, const uint8_t* BN_, const uint8_t* AS, const uint8_t* BS,
                                   const uint8_t* AO, const uint8_t* BO, int M, int N, int KN, int KS, int KO,
                                   const void* C_bf16, void* D_bf16, int ldd, const uint8_t* SFAN,
                                   const uint8_t* SFBN, const uint8_t* SFAS, const uint8_t* SFBS,
                                   const uint8_t* SFAO, const uint8_t* SFBO, void* stream) {
  if (M < 0 || N <= 0 || KN < 0 || KS < 0 || KO < 0) return MG_ERR_SHAPE;
  const size_t need = make_plan(M, N, KN, KS, KO, nullptr).total;
  if (need > (size_t)MG_STATIC_WS_BYTES) return MG_ERR_WORKSPACE;  // beyond the built-in scratch
  int dev = 0;
  MG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return MG_ERR_DEVICE;
  uint8_t* ws = nullptr;
  {
    // The array's name is only a host-side handle; the device address has to be asked for,
    // once per device, with that device current.
    std::lock_guard<std::mutex> lk(g_static_ws_mu);
    if (!g_static_ws_ptr[dev]) {
      void* p = nullptr;
      MG_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_ws));
      g_static_ws_ptr[dev] = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~(uintptr_t)1023);
    }
    ws = g_static_ws_ptr[dev];
  }
  // Only the padded copies live in the array: split-K through scratch is not taken, so the kernel
  // chosen (and with it the result) is that of mg_matmul given a workspace of exactly
  // mg_matmul_workspace_bytes() bytes.
  return matmul_impl(false, false, AN, BN_, AS, BS, AO, BO, nullptr, M, N, KN, KS, KO, C_bf16, D_bf16, ldd, SFAN, SFBN,
                     SFAS, SFBS, SFAO, SFBO, ws, (size_t)MG_STATIC_WS_BYTES, stream);
}
