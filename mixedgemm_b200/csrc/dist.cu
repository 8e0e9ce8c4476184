// Multi-GPU exchange behind the C ABI (one process per GPU).
//
// The GEMM shards along N, so every rank needs the whole quantised activation.  Two ways to get
// it there:
//   * plain NCCL collectives on the caller's stream (mg_bcast_activations, mg_allgather_inplace,
//     mg_allgather_output).  NCCL is taken from the process (the libnccl that the host framework
//     already loaded) or loaded by name; nothing links against it, so the library loads without it.
//   * the overlapped exchange: every rank quantises its M / P rows and PUSHES them into every
//     peer's buffer over NVLink - with copy-engine copies (mg_push_shard: cudaMemcpyAsync on
//     per-peer streams, no SM involved, followed by a 4-byte flag copy), with a kernel that stores
//     into the peers' buffers from SMs of its own (mg_push_block), or with both sharing the peers
//     (the _to forms).  The GEMM that consumes the activation may already be running: its producer
//     waits for the flags (mg_problem_t.ready_flags).  Peer buffers are opened through CUDA IPC.
// The GEMM and the quantiser never have another GPU's memory as an operand and no tensor map covers
// it; what crosses NVLink are NCCL's transfers, those copies and the push kernel's plain stores.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "mg_common.h"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  bool ok = false;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

const NcclApi& nccl() {
  std::call_once(g_nccl_once, [] {
    // the copy the process already holds (one NCCL per process), else by name
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    g_nccl.handle = h;
#define MG_SYM(field, name) g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name))
    MG_SYM(GetUniqueId, "ncclGetUniqueId");
    MG_SYM(CommInitRank, "ncclCommInitRank");
    MG_SYM(CommDestroy, "ncclCommDestroy");
    MG_SYM(Broadcast, "ncclBroadcast");
    MG_SYM(AllGather, "ncclAllGather");
    MG_SYM(GroupStart, "ncclGroupStart");
    MG_SYM(GroupEnd, "ncclGroupEnd");
#undef MG_SYM
    g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.Broadcast &&
                g_nccl.AllGather && g_nccl.GroupStart && g_nccl.GroupEnd;
  });
  return g_nccl;
}

struct Comm {
  ncclComm_t nccl;
  int world, rank;
};

#define MG_NCCL_TRY(expr)                      \
  do {                                         \
    if ((expr) != ncclSuccess) return MG_ERR_NCCL; \
  } while (0)

__global__ void epoch_bump_kernel(int* word) { *word += 1; }

// The same push made by SMs: every CTA copies a share of this rank's block into every peer's buffer
// with 16-byte loads (four in flight per thread) and plain peer stores; the CTA that finishes last
// raises this rank's flag on every rank.  One launch, no per-copy latency, and all-to-all traffic at
// the link rate where concurrent copy-engine copies fall to half of it.  Sharing an SM with a GEMM
// CTA slows that CTA by a third (measured), and the GEMM ends with its slowest SM pair, so the few
// CTAs of the default form ask for shared memory they do not use: an SM that holds one has no room
// for a GEMM or quantiser CTA, and the GEMM is launched on correspondingly fewer SM pairs.
constexpr int kMaxPeers = 15;
struct PushParams {
  const uint4* src;
  uint4* dst[kMaxPeers];   // the block's place in each peer's buffer, nearest peer first
  int* flag[kMaxPeers + 1];  // this rank's flag word on each peer, then on this rank itself
  int npeers;
  size_t n16;
  const int* epoch_word;
  int* counter;  // CTAs that have finished (returns to zero)
};

constexpr int kPushThreads = 1024;
constexpr int kPushUnroll = 8;

__global__ void __launch_bounds__(kPushThreads) push_block_kernel(const __grid_constant__ PushParams p) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < p.n16; i0 += stride * kPushUnroll) {
    uint4 v[kPushUnroll];
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      const size_t i = i0 + (size_t)u * stride;
      if (i < p.n16)
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                     : "l"(p.src + i));
    }
#pragma unroll 1
    for (int q = 0; q < p.npeers; ++q) {
      uint4* dst = p.dst[q];
#pragma unroll
      for (int u = 0; u < kPushUnroll; ++u) {
        const size_t i = i0 + (size_t)u * stride;
        if (i < p.n16) dst[i] = v[u];
      }
    }
  }
  // release: every thread's stores, then the CTA's arrival; the last CTA's flag stores come after
  // every other CTA's arrival, hence after their stores
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(p.counter, 1);
    if (done == (int)gridDim.x - 1) {
      *p.counter = 0;
      __threadfence_system();
      const int e = *reinterpret_cast<const volatile int*>(p.epoch_word);
      for (int q = 0; q <= p.npeers; ++q)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.flag[q]), "r"(e) : "memory");
    }
  }
}

}  // namespace

extern "C" int mg_dist_unique_id(void* id128) {
  if (!id128) return MG_ERR_NULL;
  const NcclApi& n = nccl();
  if (!n.ok) return MG_ERR_NCCL;
  static_assert(sizeof(ncclUniqueId) == 128, "the C ABI hands the id around as 128 bytes");
  MG_NCCL_TRY(n.GetUniqueId(static_cast<ncclUniqueId*>(id128)));
  return MG_OK;
}

extern "C" int mg_dist_init(void** comm, const void* id128, int world, int rank) {
  if (!comm || !id128) return MG_ERR_NULL;
  if (world < 1 || rank < 0 || rank >= world) return MG_ERR_SHAPE;
  const NcclApi& n = nccl();
  if (!n.ok) return MG_ERR_NCCL;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  Comm* c = new Comm{nullptr, world, rank};
  if (n.CommInitRank(&c->nccl, world, id, rank) != ncclSuccess) {
    delete c;
    return MG_ERR_NCCL;
  }
  *comm = c;
  return MG_OK;
}

extern "C" int mg_dist_destroy(void* comm) {
  if (!comm) return MG_OK;
  Comm* c = static_cast<Comm*>(comm);
  const NcclApi& n = nccl();
  const bool ok = n.ok && n.CommDestroy(c->nccl) == ncclSuccess;
  delete c;
  return ok ? MG_OK : MG_ERR_NCCL;
}

extern "C" int mg_bcast_activations(void* comm, int root, void* const* bufs, const size_t* bytes, int nbuf,
                                    void* stream) {
  if (!comm || !bufs || !bytes) return MG_ERR_NULL;
  Comm* c = static_cast<Comm*>(comm);
  if (root < 0 || root >= c->world || nbuf < 0) return MG_ERR_SHAPE;
  const NcclApi& n = nccl();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MG_NCCL_TRY(n.GroupStart());
  for (int i = 0; i < nbuf; ++i) {
    if (bytes[i] == 0) continue;
    if (!bufs[i]) {
      n.GroupEnd();
      return MG_ERR_NULL;
    }
    if (n.Broadcast(bufs[i], bufs[i], bytes[i], ncclUint8, root, c->nccl, st) != ncclSuccess) {
      n.GroupEnd();
      return MG_ERR_NCCL;
    }
  }
  MG_NCCL_TRY(n.GroupEnd());
  return MG_OK;
}

extern "C" int mg_allgather_inplace(void* comm, void* const* bufs, const size_t* shard_bytes, int nbuf, void* stream) {
  if (!comm || !bufs || !shard_bytes) return MG_ERR_NULL;
  Comm* c = static_cast<Comm*>(comm);
  const NcclApi& n = nccl();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MG_NCCL_TRY(n.GroupStart());
  for (int i = 0; i < nbuf; ++i) {
    if (shard_bytes[i] == 0) continue;
    if (!bufs[i]) {
      n.GroupEnd();
      return MG_ERR_NULL;
    }
    uint8_t* base = static_cast<uint8_t*>(bufs[i]);
    if (n.AllGather(base + (size_t)c->rank * shard_bytes[i], base, shard_bytes[i], ncclUint8, c->nccl, st) != ncclSuccess) {
      n.GroupEnd();
      return MG_ERR_NCCL;
    }
  }
  MG_NCCL_TRY(n.GroupEnd());
  return MG_OK;
}

extern "C" int mg_allgather_output(void* comm, const void* Y_local, void* Y_shards, size_t bytes_per_rank,
                                   void* stream) {
  if (!comm || !Y_local || !Y_shards) return MG_ERR_NULL;
  Comm* c = static_cast<Comm*>(comm);
  const NcclApi& n = nccl();
  MG_NCCL_TRY(n.AllGather(Y_local, Y_shards, bytes_per_rank, ncclUint8, c->nccl, static_cast<cudaStream_t>(stream)));
  return MG_OK;
}

// ---------------------------------------------------------------- peer buffers
extern "C" int mg_xbuf_alloc(void** ptr, size_t bytes) {
  if (!ptr) return MG_ERR_NULL;
  if (bytes == 0) return MG_ERR_SHAPE;
  MG_CUDA_TRY(cudaMalloc(ptr, bytes));
  MG_CUDA_TRY(cudaMemset(*ptr, 0, bytes));
  return MG_OK;
}

extern "C" int mg_xbuf_free(void* ptr) {
  if (ptr) MG_CUDA_TRY(cudaFree(ptr));
  return MG_OK;
}

extern "C" int mg_ipc_export(const void* ptr, void* handle64) {
  if (!ptr || !handle64) return MG_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI hands the handle around as 64 bytes");
  MG_CUDA_TRY(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), const_cast<void*>(ptr)));
  return MG_OK;
}

extern "C" int mg_ipc_import(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return MG_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  MG_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return MG_OK;
}

extern "C" int mg_ipc_close(void* ptr) {
  if (ptr) MG_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return MG_OK;
}

extern "C" int mg_epoch_bump(int* epoch_word, void* stream) {
  if (!epoch_word) return MG_ERR_NULL;
  epoch_bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(epoch_word);
  MG_CUDA_TRY(cudaGetLastError());
  return MG_OK;
}

extern "C" int mg_push_shard(int world, int rank, void* const* bases, const size_t* seg_off, const size_t* seg_bytes,
                             int nseg, size_t flag_off, const int* epoch_word, void* const* streams) {
  return mg_push_shard_to(world, rank, 0u, bases, seg_off, seg_bytes, nseg, flag_off, epoch_word, streams);
}

extern "C" int mg_push_shard_to(int world, int rank, unsigned ring_mask, void* const* bases, const size_t* seg_off,
                                const size_t* seg_bytes, int nseg, size_t flag_off, const int* epoch_word,
                                void* const* streams) {
  if (!bases || !seg_off || !seg_bytes || !epoch_word || !streams) return MG_ERR_NULL;
  if (world < 1 || world > 32 || rank < 0 || rank >= world || nseg < 0) return MG_ERR_SHAPE;
  const uint8_t* mine = static_cast<const uint8_t*>(bases[rank]);
  if (!mine) return MG_ERR_NULL;
  for (int step = 0; step < world; ++step) {
    // peers in ring order downwards from this rank, so that at any moment the ranks write to
    // different targets and rank r hears from r + 1 first, then r + 2, ...; step 0 is this rank
    // itself: its rows are already in place, only its own flag goes up
    const int peer = (rank - step + world) % world;
    // a mask names the peers this call serves by their distance down the ring (bit step - 1); the
    // own flag then belongs to the call that serves the others (mg_push_block_to)
    if (ring_mask != 0 && (step == 0 || !(ring_mask >> (step - 1) & 1u))) continue;
    uint8_t* dst = static_cast<uint8_t*>(bases[peer]);
    if (!dst) return MG_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(streams[step == 0 ? 0 : step - 1]);
    for (int i = 0; i < nseg && step > 0; ++i)
      if (seg_bytes[i])
        MG_CUDA_TRY(cudaMemcpyAsync(dst + seg_off[i], mine + seg_off[i], seg_bytes[i], cudaMemcpyDefault, st));
    // stream order: the flag leaves after the data has arrived
    MG_CUDA_TRY(cudaMemcpyAsync(dst + flag_off + (size_t)rank * sizeof(int), epoch_word, sizeof(int), cudaMemcpyDefault, st));
  }
  return MG_OK;
}

extern "C" int mg_push_block(int world, int rank, void* const* bases, size_t block_off, size_t block_bytes,
                             size_t flag_off, const int* epoch_word, int* counter, int ctas, void* stream) {
  return mg_push_block_to(world, rank, 0u, bases, block_off, block_bytes, flag_off, epoch_word, counter, ctas, stream);
}

extern "C" int mg_push_block_to(int world, int rank, unsigned ring_mask, void* const* bases, size_t block_off,
                                size_t block_bytes, size_t flag_off, const int* epoch_word, int* counter, int ctas,
                                void* stream) {
  if (!bases || !epoch_word || !counter) return MG_ERR_NULL;
  if (world < 1 || world > kMaxPeers + 1 || rank < 0 || rank >= world || ctas < 0) return MG_ERR_SHAPE;
  if (block_bytes % 16 || block_off % 16 || flag_off % 4) return MG_ERR_ALIGN;
  PushParams p{};
  uint8_t* mine = static_cast<uint8_t*>(bases[rank]);
  if (!mine) return MG_ERR_NULL;
  p.src = reinterpret_cast<const uint4*>(mine + block_off);
  int np = 0;
  for (int step = 1; step < world; ++step) {
    // ring order downwards from this rank, as in mg_push_shard; a mask keeps only the named distances
    if (ring_mask != 0 && !(ring_mask >> (step - 1) & 1u)) continue;
    uint8_t* peer = static_cast<uint8_t*>(bases[(rank - step + world) % world]);
    if (!peer) return MG_ERR_NULL;
    if (!mg::aligned(peer, 16)) return MG_ERR_ALIGN;
    p.dst[np] = reinterpret_cast<uint4*>(peer + block_off);
    p.flag[np] = reinterpret_cast<int*>(peer + flag_off) + rank;
    ++np;
  }
  p.npeers = np;
  if (!mg::aligned(mine, 16)) return MG_ERR_ALIGN;
  p.flag[np] = reinterpret_cast<int*>(mine + flag_off) + rank;
  p.n16 = block_bytes / 16;
  p.epoch_word = epoch_word;
  p.counter = counter;
  mg::DeviceInfo di;
  int rc = mg::device_info(&di);
  if (rc != MG_OK) return rc;
  int grid = ctas > 0 ? ctas : di.sm_count;
  const size_t need = (p.n16 + kPushThreads - 1) / kPushThreads;
  if ((size_t)grid > need) grid = need ? (int)need : 1;
  // ctas > 0: each CTA claims 32 KB of shared memory, so that it has its SM to itself beside kernels
  // that fill shared memory (see above); ctas == 0: one CTA per SM, sharing it with whatever runs
  // and they are launched as clusters of two, which land on the two SMs of one pair: n CTAs then
  // cost the CTA-pair GEMM n / 2 of its SM pairs, not n
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  cfg.blockDim = dim3(kPushThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  if (ctas > 0) {
    grid = (grid + 1) & ~1;
    cfg.dynamicSmemBytes = 32 * 1024;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cfg.gridDim = dim3(grid);
  MG_CUDA_TRY(cudaLaunchKernelEx(&cfg, push_block_kernel, p));
  return MG_OK;
}
