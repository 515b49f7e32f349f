// Library-wide pieces of the C ABI: version, per-thread error text, device report.
#include "common.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>

namespace b200ops {

namespace {
const char* const kKnobNames[kKnobCount] = {
    "B200OPS_GMM_PAIR",    "B200OPS_GMM_KSPLIT",        "B200OPS_GMM_SHORT", "B200OPS_PA_MODE",
    "B200OPS_PA_STAGES",   "B200OPS_PA_CHUNK_TOKENS",
    "B200OPS_RMSNORM_VPT", "B200OPS_RMSNORM_CTA_WARPS", "B200OPS_RAC_DEDUP", "B200OPS_PDL"};
std::atomic<int> g_knob_state[kKnobCount];  // 0 not read yet, 1 unset, 2 set
std::atomic<int> g_knob_value[kKnobCount];
}  // namespace

int knob(Knob k, int fallback) {
  int st = g_knob_state[k].load(std::memory_order_acquire);
  if (st == 0) {  // two threads may both get here; they store the same thing
    const char* s = std::getenv(kKnobNames[k]);
    st = (s && *s) ? 2 : 1;
    g_knob_value[k].store(st == 2 ? std::atoi(s) : 0, std::memory_order_relaxed);
    g_knob_state[k].store(st, std::memory_order_release);
  }
  return st == 2 ? g_knob_value[k].load(std::memory_order_relaxed) : fallback;
}

char* last_error_buffer() {
  static thread_local char buf[kLastErrorLen] = {0};
  return buf;
}

int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace b200ops

extern "C" int b200ops_version(void) { return 200; }

extern "C" void b200ops_reload_options(void) {
  for (int k = 0; k < b200ops::kKnobCount; ++k) b200ops::g_knob_state[k].store(0, std::memory_order_release);
}

extern "C" const char* b200ops_last_error(void) { return b200ops::last_error_buffer(); }

// Replaces native::print_info (csrc/ffi/bind.cpp:26-51), which prints the Ascend core counts
// and the sizes / bandwidths of its on-chip memories; the CUDA counterpart of those figures
// is what cudaDeviceProp and the device attributes report.
extern "C" int b200ops_print_info(int device_id, char* buf, size_t buf_len) {
  using namespace b200ops;
  cudaDeviceProp prop;
  B200OPS_CUDA(cudaGetDeviceProperties(&prop, device_id));
  int mem_clock_khz = 0, bus_bits = 0, smem_optin = 0;
  B200OPS_CUDA(cudaDeviceGetAttribute(&mem_clock_khz, cudaDevAttrMemoryClockRate, device_id));
  B200OPS_CUDA(cudaDeviceGetAttribute(&bus_bits, cudaDevAttrGlobalMemoryBusWidth, device_id));
  B200OPS_CUDA(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device_id));
  char text[1024];
  snprintf(text, sizeof(text),
           "device %d: %s (sm_%d%d)\n"
           "SMs: %d, max threads/SM: %d, registers/SM: %d\n"
           "shared memory/SM: %zu, shared memory/block (opt-in): %d, L2: %d, HBM: %zu\n"
           "memory clock kHz: %d, memory bus bits: %d, nominal HBM GB/s: %.0f\n",
           device_id, prop.name, prop.major, prop.minor, prop.multiProcessorCount,
           prop.maxThreadsPerMultiProcessor, prop.regsPerMultiprocessor,
           prop.sharedMemPerMultiprocessor, smem_optin, prop.l2CacheSize, prop.totalGlobalMem,
           mem_clock_khz, bus_bits, 2.0 * mem_clock_khz * 1e3 * (bus_bits / 8.0) / 1e9);
  fputs(text, stdout);
  fflush(stdout);
  if (buf != nullptr && buf_len > 0) {
    strncpy(buf, text, buf_len - 1);
    buf[buf_len - 1] = '\0';
  }
  return B200OPS_OK;
}

namespace b200ops {
namespace gmm { int status_take(); }
namespace pa { int fast_path_status_take(); }
}  // namespace b200ops

// Codes 1-9 come from grouped_matmul's pipeline, 11-19 from paged_attention's TMA path.
extern "C" int b200ops_pipeline_status(int* status) {
  using namespace b200ops;
  B200OPS_REQUIRE(status != nullptr, "pipeline_status: null pointer");
  B200OPS_CUDA(cudaDeviceSynchronize());
  const int g = gmm::status_take();
  const int p = pa::fast_path_status_take();
  if (g < 0 || p < 0) return fail(B200OPS_ECUDA, "pipeline_status: could not read the status words");
  *status = g != 0 ? g : p;
  return B200OPS_OK;
}
