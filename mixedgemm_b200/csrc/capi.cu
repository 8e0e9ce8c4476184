// Status, device queries and small helpers of the C ABI.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "mg_common.h"

namespace {
thread_local int tl_last_cuda_error = 0;

// Set by kernels whose bounded waits expire; read and cleared by mg_device_status().
__device__ int g_device_status = 0;

constexpr int kMaxDevices = 64;
mg::DeviceInfo g_info[kMaxDevices];
bool g_info_ok[kMaxDevices];
int* g_status_ptr[kMaxDevices];
std::mutex g_mu;

constexpr long long kDefaultWaitCycles = 2000000000LL;  // about one second of SM clock
std::atomic<long long> g_wait_cycles{kDefaultWaitCycles};
}  // namespace

namespace {
struct OptionSlot {
  const char* name;
  int mg::Options::*field;
  int fallback;
};
const OptionSlot kOptionSlots[] = {
    {"GEMM_BN", &mg::Options::gemm_bn, -1},         {"GEMM_2CTA", &mg::Options::gemm_2cta, -1},
    {"GEMM_CSPLIT", &mg::Options::gemm_csplit, -1}, {"GEMM_SPLITK", &mg::Options::gemm_splitk, -1},
    {"GEMM_SWAP", &mg::Options::gemm_swap, -1},     {"PDL", &mg::Options::pdl, 1},
    {"REORDER_CTAS", &mg::Options::reorder_ctas, 0}, {"FAULT_SKIP_LOAD", &mg::Options::fault_skip_load, 0},
    {"GEMM_SCHED", &mg::Options::gemm_sched, 1},    {"GEMM_MAX_CLUSTERS", &mg::Options::gemm_max_clusters, 0},
};
mg::Options g_options;
bool g_options_ready = false;
std::mutex g_options_mu;

void load_options_locked() {
  for (const OptionSlot& s : kOptionSlots) {
    g_options.*(s.field) = s.fallback;
    const std::string env = std::string("MG_") + s.name;
    if (const char* e = std::getenv(env.c_str()))
      if (e[0] != 0) g_options.*(s.field) = std::atoi(e);
  }
  g_options_ready = true;
}
}  // namespace

namespace mg {

Options options() {
  std::lock_guard<std::mutex> lk(g_options_mu);
  if (!g_options_ready) load_options_locked();
  return g_options;
}

bool pdl_enabled() { return options().pdl != 0; }

long long wait_limit_cycles() { return g_wait_cycles.load(std::memory_order_relaxed); }

int note_cuda_error(cudaError_t e) {
  tl_last_cuda_error = (int)e;
  return MG_ERR_CUDA;
}

int device_info(DeviceInfo* out) {
  int dev = 0;
  MG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return MG_ERR_DEVICE;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_info_ok[dev]) {
    DeviceInfo di;
    MG_CUDA_TRY(cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev));
    MG_CUDA_TRY(cudaDeviceGetAttribute(&di.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    MG_CUDA_TRY(cudaDeviceGetAttribute(&di.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    g_info[dev] = di;
    g_info_ok[dev] = true;
  }
  *out = g_info[dev];
  return out->cc_major == 10 ? MG_OK : MG_ERR_DEVICE;
}

int device_status_word(int** dev_ptr) {
  int dev = 0;
  MG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return MG_ERR_DEVICE;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    MG_CUDA_TRY(cudaGetSymbolAddress(&p, g_device_status));
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  *dev_ptr = g_status_ptr[dev];
  return MG_OK;
}

}  // namespace mg

extern "C" const char* mg_strerror(int status) {
  switch (status) {
    case MG_OK: return "ok";
    case MG_ERR_SHAPE: return "unsupported shape";
    case MG_ERR_NULL: return "null pointer";
    case MG_ERR_ALIGN: return "misaligned pointer or pitch";
    case MG_ERR_WORKSPACE: return "workspace missing or too small";
    case MG_ERR_CUDA: return "CUDA call failed";
    case MG_ERR_DEVICE: return "device is not sm_100";
    case MG_ERR_TIMEOUT: return "kernel gave up on a bounded wait";
    case MG_ERR_NCCL: return "NCCL unavailable or an NCCL call failed";
    default: return "unknown status";
  }
}

extern "C" int mg_set_wait_limit_us(long long us) {
  if (us < 0) return MG_ERR_SHAPE;
  // clock64 ticks at the SM clock, at most 2 GHz on this part: 2000 cycles per microsecond
  g_wait_cycles.store(us == 0 ? kDefaultWaitCycles : us * 2000LL, std::memory_order_relaxed);
  return MG_OK;
}

extern "C" int mg_set_option(const char* name, int value) {
  if (!name) return MG_ERR_NULL;
  if (std::strncmp(name, "MG_", 3) == 0) name += 3;
  std::lock_guard<std::mutex> lk(g_options_mu);
  if (!g_options_ready) load_options_locked();
  for (const OptionSlot& s : kOptionSlots)
    if (std::strcmp(name, s.name) == 0) {
      g_options.*(s.field) = value;
      return MG_OK;
    }
  return MG_ERR_SHAPE;
}

extern "C" int mg_get_option(const char* name, int* value) {
  if (!name || !value) return MG_ERR_NULL;
  if (std::strncmp(name, "MG_", 3) == 0) name += 3;
  const mg::Options o = mg::options();
  for (const OptionSlot& s : kOptionSlots)
    if (std::strcmp(name, s.name) == 0) {
      *value = o.*(s.field);
      return MG_OK;
    }
  return MG_ERR_SHAPE;
}

extern "C" void mg_reset_options(void) {
  std::lock_guard<std::mutex> lk(g_options_mu);
  load_options_locked();
}

extern "C" int mg_last_cuda_error(void) { return tl_last_cuda_error; }

extern "C" int mg_version(void) { return 1; }

extern "C" size_t mg_sf_bytes(int rows, int kseg) {
  if (rows <= 0 || kseg <= 0) return 0;
  return (size_t)((rows + 127) / 128) * (size_t)((kseg + 127) / 128) * 512;
}

extern "C" int mg_device_status(int* status_host, void* stream) {
  if (!status_host) return MG_ERR_NULL;
  int* dptr = nullptr;
  int rc = mg::device_status_word(&dptr);
  if (rc != MG_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MG_CUDA_TRY(cudaStreamSynchronize(st));
  MG_CUDA_TRY(cudaMemcpy(status_host, dptr, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_host != 0) {
    MG_CUDA_TRY(cudaMemset(dptr, 0, sizeof(int)));
    return MG_ERR_TIMEOUT;
  }
  return MG_OK;
}
