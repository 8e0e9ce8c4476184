/*
 * mixedgemm_c.h - C ABI of the B200 (sm_100a) implementation of MixedGemm's hot path:
 * activation / weight reorder-and-quantise followed by the mixed MXFP4/6/8 x MXFP4
 * block-scaled GEMM.
 *
 * Conventions for every entry point:
 *   - plain pointers and sizes only; all data pointers are DEVICE pointers on the
 *     current CUDA device unless a comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream); calls are
 *     asynchronous, never synchronise the device and never print;
 *   - the return value is an MG_* status; nothing throws or exits;
 *   - output buffers are caller-owned; the library allocates no device memory (the one
 *     exception, mg_xbuf_alloc, says so).
 *
 * Paths below (src/..., include/...) are relative to the MixedGemm project and name
 * the reference interface each entry point replaces.
 */
#ifndef MIXEDGEMM_C_H
#define MIXEDGEMM_C_H

#include <stddef.h>
#include <stdint.h>

#include "fp4.h"
#include "fp6.h"
#include "fp8.h"
#include "mxdtype.h"

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MG_OK = 0,
  MG_ERR_SHAPE = 1,      /* a size is not supported (segments must be multiples of 32, ...) */
  MG_ERR_NULL = 2,       /* a required pointer is NULL */
  MG_ERR_ALIGN = 3,      /* a pointer or pitch breaks an alignment rule */
  MG_ERR_WORKSPACE = 4,  /* workspace missing or too small */
  MG_ERR_CUDA = 5,       /* a CUDA runtime / driver call failed (see mg_last_cuda_error) */
  MG_ERR_DEVICE = 6,     /* the device is not an sm_100 part */
  MG_ERR_TIMEOUT = 7,    /* a kernel gave up on a bounded wait (see mg_device_status) */
  MG_ERR_NCCL = 8        /* NCCL is not available in this process, or one of its calls failed */
};

/* Human-readable text of a status. */
const char* mg_strerror(int status);

/* cudaError_t value of the last failing CUDA call seen by this library on this thread. */
int mg_last_cuda_error(void);

/* Library version, major*100 + minor. */
int mg_version(void);

/*
 * Reads and clears the device-side error word that kernels set when a bounded wait
 * expires.  Synchronises `stream`.  *status_host receives 0 or the kernel-specific code
 * (1 / 2 / 4 / 8: the GEMM's producer / MMA / accumulator-free / accumulator-full waits;
 * 16 / 32: the quantiser's; 64: the CTA pair's relay; 256: split-K arrival counter;
 * 512: cluster split-K exchange; 1024: a problem's ready flag).  Returns MG_ERR_TIMEOUT when the
 * word was non-zero: results of the launches since the last call are then not valid, and the
 * context is still usable (the kernels gave up and returned, nothing trapped).
 */
int mg_device_status(int* status_host, void* stream);

/*
 * Limit of every bounded wait inside the kernels, in microseconds of SM clock at 2 GHz
 * (0 restores the default of about one second).  Applies to launches made after the call.
 */
int mg_set_wait_limit_us(long long us);

/*
 * Switches that choose between kernels or turn a mode off.  Each is read from the environment
 * once (MG_<NAME>), when the library is first used, and can be changed at run time here;
 * -1 means "let the library decide".  Names (with or without the MG_ prefix):
 *   GEMM_BN          128 / 256: tile width of the single-CTA kernel
 *   GEMM_2CTA        0 / 1: CTA-pair kernel off / on where it applies
 *   GEMM_CSPLIT      0: cluster split-K off
 *   GEMM_SPLITK      0: split-K through the workspace off;  n > 0: n splits
 *   GEMM_SWAP        0 / 1: decode form off / on for every M <= 128
 *   GEMM_SCHED       0: tiles of a multi-problem launch dealt out round-robin, not by cost
 *   GEMM_MAX_CLUSTERS n > 0: the CTA-pair kernel uses at most n SM pairs (to leave SMs to a kernel that
 *                    runs beside it, e.g. mg_push_block)
 *   PDL              0: no programmatic dependent launch
 *   REORDER_CTAS     n > 0: at most n CTAs for the quantiser (to share the GPU with another kernel)
 *   FAULT_SKIP_LOAD  n > 0: host-side fault injection for tests - the first CTA of the single-CTA
 *                    GEMM never issues its n-th stage load, so the wait for it runs out
 * mg_set_option returns MG_ERR_SHAPE for an unknown name; mg_reset_options re-reads the environment.
 */
int mg_set_option(const char* name, int value);
int mg_get_option(const char* name, int* value);
void mg_reset_options(void);

/* Bytes of a scale buffer for `rows` rows of a `kseg`-element segment: whole atoms,
 * ceil(rows/128) * ceil(kseg/128) * 512. */
size_t mg_sf_bytes(int rows, int kseg);

/*
 * Activation reorder-and-quantise.
 * Replaces run_reorder_bf16_mixed<32,K> (include/reorder.cuh:295-308, src/reorder.cu:434-469)
 * and its kernel reorder_bf16_mixed_kernel (src/reorder.cu:94-269), for any K = KN+KS+KO with
 * all three multiples of 32 and K <= 32736.
 *   X      [M,K] bf16 row-major, 16-byte aligned
 *   idx    [K]   int16: reordered position j takes input channel idx[j]
 *   AN     [M,KN/2]    AS [M,3*KS/4]    AO [M,KO]          packed codes (mxdtype.h)
 *   SFAN / SFAS / SFAO  at least mg_sf_bytes(M, KN / KS / KO) bytes each; only the
 *          positions of real (row, 32-block) pairs are written.
 * A segment of size 0 may pass NULL buffers.
 */
int mg_reorder_quantize_x(const void* X, int M, int K, const int16_t* idx, int KN, int KS, int KO,
                          uint8_t* AN, uint8_t* AS, uint8_t* AO, uint8_t* SFAN, uint8_t* SFAS,
                          uint8_t* SFAO, void* stream);

/*
 * Weight reorder-and-quantise: all three segments become MXFP4.
 * Replaces run_reorder_bf16_fp4<32,K> (include/reorder.cuh:310-323, src/reorder.cu:471-506)
 * and reorder_bf16_fp4_kernel (src/reorder.cu:271-432).
 *   W [N,K] bf16;  BN [N,KN/2]  BS [N,KS/2]  BO [N,KO/2];  SFB* as above with rows = N.
 */
int mg_reorder_quantize_w(const void* W, int N, int K, const int16_t* idx, int KN, int KS, int KO,
                          uint8_t* BN, uint8_t* BS, uint8_t* BO, uint8_t* SFBN, uint8_t* SFBS,
                          uint8_t* SFBO, void* stream);

/*
 * Bytes of scratch mg_matmul needs for this problem (0 when every segment is a multiple
 * of 128 elements).  Segments that are only multiples of 64 are first copied to a
 * 128-padded pitch there, because the tensor-map types that unpack FP4/FP6 need it.
 */
size_t mg_matmul_workspace_bytes(int M, int N, int KN, int KS, int KO);

/*
 * Mixed block-scaled GEMM:  D[M,N] = bf16( sum over the three segments of A_seg * B_seg^T
 * (+ C when C != NULL) ), fp32 accumulation in one accumulator, one rounding at the end.
 * Replaces matmul_host (include/gemm.h:21-41, src/gemm.cu:22-47) and the three CUTLASS
 * GEMMs it chains (src/fp4.cu, src/fp6.cu, src/fp8.cu).
 *   AN/AS/AO, SFAN/SFAS/SFAO   as written by mg_reorder_quantize_x (M rows)
 *   BN/BS/BO, SFBN/SFBS/SFBO   as written by mg_reorder_quantize_w (N rows, N % 128 == 0)
 *   D      [M,N] bf16, row pitch `ldd` elements (ldd % 8 == 0, 16-byte aligned base)
 *   C      optional [M,N] bf16 with the same pitch, added before the final rounding
 *   workspace / workspace_bytes   scratch of mg_matmul_workspace_bytes() bytes, 1024-aligned
 * Segments must be multiples of 64 (KN of 128); code buffers 32-byte aligned.
 */
int mg_matmul(const uint8_t* AN, const uint8_t* BN, const uint8_t* AS, const uint8_t* BS,
              const uint8_t* AO, const uint8_t* BO, int M, int N, int KN, int KS, int KO,
              const void* C_bf16, void* D_bf16, int ldd, const uint8_t* SFAN, const uint8_t* SFBN,
              const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO, const uint8_t* SFBO,
              void* workspace, size_t workspace_bytes, void* stream);

/*
 * Row-pitched variants.  The reference keeps every code buffer dense ([rows, K/2] and so on,
 * src/bindings.cpp:88-90, :207-209); a segment that is only a multiple of 64 elements (K = 14336
 * gives 4928 and 448) then has a row pitch that the unpacking tensor maps cannot take, and
 * mg_matmul has to copy it.  Buffers allocated with the pitch mg_code_pitch() returns are read in
 * place instead.  Logical contents are unchanged: row r of a buffer starts at r * pitch and its
 * first K/2 (3K/4, K) bytes are the reference's row; the bytes after them are never interpreted.
 *   pitches of mg_reorder_quantize_pitched: {FP4 buffer, FP6 (or second FP4) buffer, FP8 (or third FP4) buffer}
 *   pitches of mg_matmul_pitched:           {AN, BN, AS, BS, AO, BO}
 * mg_matmul_pitched needs workspace only for operands whose pitch does not qualify.  What
 * mg_matmul_pitched_workspace_bytes reports on top (32 KB + fp32 partials, only for problems that
 * could use it) lets split-K run; with a smaller workspace the call still works, without it:
 * a problem whose 128-row tiles occupy at most half of the SMs and whose K has at least 32 stages
 * of 128 bytes (decode shapes and narrow weight shards at large K) runs up to eight CTAs per tile,
 * each over a range of K; the CTA that arrives last adds the fp32 partials in a fixed order and
 * stores the tile.  The result is deterministic and differs from the unsplit kernel by fp32
 * re-association only.  The arrival counters carry a per-launch token, so the workspace may hold
 * anything when the call starts.  Option GEMM_SPLITK = 0 turns it off.
 * A workspace must not be shared by calls that may run at the same time.
 * out_f32 != 0 selects the fp32 output of mg_matmul_f32.
 */
size_t mg_code_pitch(int weights, int segment, int kseg);
int mg_reorder_quantize_pitched(int weights, const void* X, int rows, int K, const int16_t* idx, int KN, int KS,
                                int KO, uint8_t* C4, uint8_t* C6, uint8_t* C8, const size_t* pitches,
                                uint8_t* SF4, uint8_t* SF6, uint8_t* SF8, void* stream);
/*
 * Up to eight independent quantisations (own input, reorder index, K split and output buffers) in one
 * launch: the CTAs are dealt out to the problems in proportion to their sizes, so that the
 * activations of a step are quantised in one wave.  Every problem is what one
 * mg_reorder_quantize_pitched call takes (pitch = {0, 0, 0} means dense rows) and gives the same bytes.
 */
typedef struct mg_quant_problem {
  const void* X; /* [rows, K] bf16 */
  int rows, K;
  const int16_t* idx;
  int KN, KS, KO;
  uint8_t *C4, *C6, *C8;
  size_t pitch[3];
  uint8_t *SF4, *SF6, *SF8;
} mg_quant_problem_t;
int mg_reorder_quantize_multi(int weights, int nprob, const mg_quant_problem_t* probs, void* stream);
size_t mg_matmul_pitched_workspace_bytes(int M, int N, int KN, int KS, int KO, const size_t* pitches);
int mg_matmul_pitched(const uint8_t* AN, const uint8_t* BN, const uint8_t* AS, const uint8_t* BS,
                      const uint8_t* AO, const uint8_t* BO, const size_t* pitches, int out_f32, int M, int N,
                      int KN, int KS, int KO, const void* C_bf16, void* D, int ldd, const uint8_t* SFAN,
                      const uint8_t* SFBN, const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO,
                      const uint8_t* SFBO, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Reorder-index calibration: idx = stable ascending argsort of the per-channel absmax of X.
 * The reference leaves this to the caller (main.py:29 uses arange; the absmax/argsort variant at
 * main.py:31-33 is commented out and uses an unstable torch.sort).  Ties are ubiquitous in bf16
 * maxima, so the order is pinned: equal maxima keep channel order.
 *   X [M,K] bf16 (K % 8 == 0, K <= 32736);  idx [K] int16 out;
 *   absmax_bits [K] uint16 out: bf16 bit pattern of each channel's largest magnitude.
 */
int mg_reorder_index(const void* X, int M, int K, int16_t* idx, uint16_t* absmax_bits, void* stream);

/*
 * Several weight matrices that consume the same quantised activation (q/k/v; gate/up) in ONE
 * launch: D[j] = bf16(A * B[j]^T), j < nprob <= 8.  The reference calls matmul_host once per weight
 * (main.py:59 per layer); sharing the launch lets small projections fill SMs that a large one
 * leaves idle in its last wave.  Restrictions: M > 128, every N[j] a multiple of 256, bf16 output,
 * and every code buffer row-pitched so that it is read in place (mg_code_pitch) - otherwise
 * MG_ERR_SHAPE / MG_ERR_ALIGN is returned and the caller issues mg_matmul per weight instead.
 *   pitches_a[3] = {AN, AS, AO};  pitches_b[3*j + s] = pitch of weight j, segment s
 *   BN/BS/BO/SFBN/SFBS/SFBO/D/N/ldd are arrays of nprob entries.  workspace / workspace_bytes are
 *   not used (kept for callers of earlier versions); pass NULL / 0.
 */
int mg_matmul_group_pitched(int nprob, const uint8_t* AN, const uint8_t* AS, const uint8_t* AO,
                            const size_t* pitches_a, const uint8_t* const* BN, const uint8_t* const* BS,
                            const uint8_t* const* BO, const size_t* pitches_b, int M, const int* N, int KN, int KS,
                            int KO, void* const* D_bf16, const int* ldd, const uint8_t* SFAN, const uint8_t* SFAS,
                            const uint8_t* SFAO, const uint8_t* const* SFBN, const uint8_t* const* SFBS,
                            const uint8_t* const* SFBO, void* workspace, size_t workspace_bytes, void* stream);

/*
 * A list of INDEPENDENT problems in one launch of the CTA-pair kernel: each has its own quantised
 * activation, weights, K split and output.  The reference calls matmul_host once per layer
 * (main.py:59); a layer's projections each leave SM pairs idle in their last wave, and one launch
 * over the concatenated tile lists (dealt round-robin in the order given) closes those gaps.
 * Restrictions per problem: M > 128, N a multiple of 256, bf16 output, every code buffer row-pitched
 * so that it is read in place (mg_code_pitch); nprob <= 8.  Otherwise MG_ERR_SHAPE / MG_ERR_ALIGN is
 * returned, nothing is launched, and the caller issues mg_matmul per problem instead.
 *
 * ready_flags (optional): device address of ready_count ints (0 counts as 1).  The kernel does not
 * read the problem's activation before every one of them has reached the target value
 * (flag - target >= 0; acquire loads at system scope, bounded wait, status code 1024 on expiry).
 * The target is *ready_epoch when that device pointer is set - a word the host bumps once per step
 * (mg_epoch_bump), so that a captured launch can be replayed - and ready_value otherwise.  It lets
 * an exchange that is still filling the activation buffer - copy engines, other GPUs writing over
 * NVLink (mg_push_shard) - overlap the problems listed before it.
 * ready_rows > 0 (a multiple of 256) makes flag i stand for rows [i ready_rows, (i+1) ready_rows)
 * only: a tile then waits for the flag of its own rows, not for all of them.  first_row (a
 * multiple of 256) is the row the problem's tile order starts with, wrapping around - the rows
 * that are there first, e.g. the ones this GPU quantised itself.
 *
 * a_shard_rows > 0 (a multiple of 128): the activation is stored in row shards - rows
 * [i a_shard_rows, (i+1) a_shard_rows) of AN / AS / AO are contiguous at the row pitch, shard i + 1
 * starts a_shard_stride[seg] bytes after shard i, and likewise the scale blocks with
 * sfa_shard_stride[seg].  It is the layout in which a rank's rows of all six buffers can be one
 * contiguous block, so that an exchange moves them with one copy per peer.
 */
typedef struct mg_problem {
  const uint8_t *AN, *AS, *AO, *SFAN, *SFAS, *SFAO; /* activation, as written by mg_reorder_quantize_pitched */
  size_t pitch_a[3];
  const uint8_t *BN, *BS, *BO, *SFBN, *SFBS, *SFBO; /* weights */
  size_t pitch_b[3];
  int M, N, KN, KS, KO;
  void* D_bf16; /* [M,N] bf16, row pitch ldd elements */
  int ldd;
  const int* ready_flags;
  int ready_count;
  const int* ready_epoch;
  int ready_value;
  int ready_rows;
  int first_row;
  int a_shard_rows;
  size_t a_shard_stride[3];
  size_t sfa_shard_stride[3];
} mg_problem_t;
int mg_matmul_multi(int nprob, const mg_problem_t* probs, void* stream);
/*
 * The tile order a multi-problem launch uses, for inspection and tests (host only, no CUDA call):
 * problem j has tiles[j] tile pairs of cost[j] (the library uses K stages + 1); the concatenated
 * tile list is dealt out in order, each tile to the SM pair that is free first.  *use = 0 means
 * "round-robin" (equal costs, no more tiles than pairs, or more than 8192 tiles); otherwise pair c
 * computes tile[off[c]] .. tile[off[c + 1] - 1] in that order.  off holds clusters + 1 entries, tile
 * the total number of tiles.  clusters <= 96.
 */
int mg_pair_schedule(int nprob, const int* tiles, const int* cost, int clusters, int* use, uint16_t* off,
                     uint16_t* tile);

/*
 * Same product with the fp32 accumulator written unrounded: D_f32 [M,N] float, pitch `ldd`
 * elements (ldd % 4 == 0).  The reference has no such output (its GEMMs write bf16,
 * src/fp4.cu:175-179); it exists so that the accumulation can be checked against a
 * float64 product without the bf16 rounding step in between.
 */
int mg_matmul_f32(const uint8_t* AN, const uint8_t* BN, const uint8_t* AS, const uint8_t* BS,
                  const uint8_t* AO, const uint8_t* BO, int M, int N, int KN, int KS, int KO,
                  const void* C_bf16, float* D_f32, int ldd, const uint8_t* SFAN, const uint8_t* SFBN,
                  const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO, const uint8_t* SFBO,
                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * Multi-GPU use, one process per GPU.  The GEMM shards along N (rank r owns rows
 * [r N/P, (r+1) N/P) of the quantised weight, whole 128-row scale blocks); K is never split, so
 * every output element is the same K-ordered sum as on one GPU.  The reference has no multi-GPU
 * mode; these entry points have no counterpart there.
 *
 * Plain collectives (NCCL, taken from the process or loaded by name; MG_ERR_NCCL when absent):
 *   mg_dist_unique_id    rank 0 makes the 128-byte id, the host hands it to the other ranks
 *   mg_dist_init         communicator of `world` ranks for the current device
 *   mg_bcast_activations one grouped broadcast of up to six buffers from `root` into every rank's
 *                        own memory ("quantise once, broadcast")
 *   mg_allgather_inplace every rank has written its shard (bytes [rank * shard, (rank+1) * shard)
 *                        of each buffer); the others' shards are gathered in place
 *   mg_allgather_output  [M, N/P] shards -> P consecutive [M, N/P] blocks, for callers that need
 *                        the whole output
 */
int mg_dist_unique_id(void* id128);
int mg_dist_init(void** comm, const void* id128, int world, int rank);
int mg_dist_destroy(void* comm);
int mg_bcast_activations(void* comm, int root, void* const* bufs, const size_t* bytes, int nbuf, void* stream);
int mg_allgather_inplace(void* comm, void* const* bufs, const size_t* shard_bytes, int nbuf, void* stream);
int mg_allgather_output(void* comm, const void* Y_local, void* Y_shards, size_t bytes_per_rank, void* stream);

/*
 * The overlapped exchange: every rank quantises M / P rows of an activation in place in its own
 * full-size buffer and pushes them into every peer's buffer with copy-engine copies over NVLink,
 * followed by a 4-byte flag; the GEMM that consumes the activation is launched at once and waits,
 * problem by problem, for the flags (mg_problem_t.ready_flags).  No SM takes part in the transfer.
 *   mg_xbuf_alloc / mg_xbuf_free   an exchange buffer (plain device allocation, zero-filled): the
 *                        one place where this library allocates, because the buffer must be
 *                        exportable as a whole
 *   mg_ipc_export / mg_ipc_import / mg_ipc_close   64-byte handle of such a buffer for the other
 *                        processes of the node; importing enables peer access
 *   mg_epoch_bump        *epoch_word += 1 on `stream` (one thread); call once per step before the
 *                        quantisers
 *   mg_push_shard        bases[r] = rank r's buffer as seen from this process (bases[rank] the own
 *                        one); byte ranges seg_off / seg_bytes (the same in every buffer) go to
 *                        each peer on streams[0 .. world-2], then the int at flag_off + rank * 4
 *                        receives *epoch_word.  The streams must already wait for the quantiser.
 * Buffers are used in turn by consecutive steps; keep two sets and alternate, because a rank may
 * start pushing the next step while a slower peer still multiplies the current one.
 */
int mg_xbuf_alloc(void** ptr, size_t bytes);
int mg_xbuf_free(void* ptr);
int mg_ipc_export(const void* ptr, void* handle64);
int mg_ipc_import(const void* handle64, void** ptr);
int mg_ipc_close(void* ptr);
int mg_epoch_bump(int* epoch_word, void* stream);
int mg_push_shard(int world, int rank, void* const* bases, const size_t* seg_off, const size_t* seg_bytes, int nseg,
                  size_t flag_off, const int* epoch_word, void* const* streams);
/*
 * The same push made by a kernel instead of the copy engines: the block [block_off, block_off +
 * block_bytes) of bases[rank] is stored into the same place of every other rank's buffer with plain
 * peer stores, and the CTA that finishes last writes *epoch_word into this rank's flag word
 * (flag_off + 4 rank) on every rank, its own included.  One launch, no per-copy latency.
 * ctas > 0: that many CTAs, each of which claims 32 KB of shared memory it does not use, so that it
 * does not share its SM with a GEMM or quantiser CTA (sharing slows the GEMM CTA by a third, and a
 * GEMM ends with its slowest SM pair): launch the GEMM that runs beside it on correspondingly fewer
 * SM pairs (option GEMM_MAX_CLUSTERS).  ctas == 0: one CTA per SM, no shared memory (for a push that
 * has the GPU to itself).  `counter` is a zeroed device word that the kernel leaves at zero.
 * world <= 16.
 */
int mg_push_block(int world, int rank, void* const* bases, size_t block_off, size_t block_bytes, size_t flag_off,
                  const int* epoch_word, int* counter, int ctas, void* stream);
/*
 * Both pushes for a subset of the peers, so that the copy engines and a kernel can share a push
 * (they reach different parts of the link rate): bit s - 1 of ring_mask names the peer s places down
 * the ring, (rank - s + world) % world; 0 means all of them, as in the calls above.  With a mask,
 * mg_push_block_to still writes this rank's own flag and mg_push_shard_to does not.
 */
int mg_push_shard_to(int world, int rank, unsigned ring_mask, void* const* bases, const size_t* seg_off,
                     const size_t* seg_bytes, int nseg, size_t flag_off, const int* epoch_word, void* const* streams);
int mg_push_block_to(int world, int rank, unsigned ring_mask, void* const* bases, size_t block_off, size_t block_bytes,
                     size_t flag_off, const int* epoch_word, int* counter, int ctas, void* stream);

/*
 * mg_matmul for callers that cannot allocate.  No counterpart in the reference (its binding
 * allocates with torch on every call, src/bindings.cpp:36).
 *
 * Meant for hosts that have no way to get device memory when they need the product - a serving
 * process whose own pool already owns all free HBM, so that cudaMalloc fails; a plugin whose
 * execute callback must not allocate.  The scratch that mg_matmul takes from the caller lives in
 * a fixed array inside the library instead (MG_STATIC_WS_BYTES, held by every device that loads
 * the library until the process ends).  Same arguments and result as mg_matmul without the two
 * workspace arguments.
 *
 *  - Problems whose padded copies need more than MG_STATIC_WS_BYTES (see
 *    mg_matmul_workspace_bytes) are refused with MG_ERR_WORKSPACE; nothing is launched.
 *  - The call itself makes no cudaMalloc / cudaFree and uses no allocating library routine.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress);
 *    make that first call outside any stream capture.
 *  - Only the padded copies live in the array (split-K through scratch is not taken), so the
 *    kernel that runs, and with it the result, is that of mg_matmul given a workspace of exactly
 *    mg_matmul_workspace_bytes() bytes.
 *  - All calls share the one array and it keeps whatever the previous call left there.  Nothing
 *    has to be cleared: each call rewrites every byte it later reads, zero padding included.
 *    Two calls that overlap on the GPU (different streams, no dependency) race on it - order
 *    them.
 */
#define MG_STATIC_WS_BYTES (24u << 20)
int mg_matmul_static_ws(const uint8_t* AN, const uint8_t* BN, const uint8_t* AS, const uint8_t* BS,
                        const uint8_t* AO, const uint8_t* BO, int M, int N, int KN, int KS, int KO,
                        const void* C_bf16, void* D_bf16, int ldd, const uint8_t* SFAN, const uint8_t* SFBN,
                        const uint8_t* SFAS, const uint8_t* SFBS, const uint8_t* SFAO, const uint8_t* SFBO,
                        void* stream);

#ifdef __cplusplus
}
#endif
#endif
