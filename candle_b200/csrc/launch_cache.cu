// Per-device launch configuration that is computed once instead of on every call: the SM count,
// and for each kernel its dynamic shared-memory limit, shared-memory carve-out preference and the
// number of CTAs of a given shape that fit on an SM.
//
// Function attributes are global to a (kernel, device) pair, so setting the dynamic shared-memory
// limit to "what this call needs" races between threads that launch the same kernel with different
// shapes.  Here the limit is raised once to the architectural maximum and never lowered; the
// carve-out preference is only a hint (a stale value costs speed, never correctness) and is
// re-applied only when the wanted value changes.
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "launch.h"

namespace cb200 {

namespace {

constexpr int kMaxDevices = 64;
constexpr int kMaxDynamicSmem = 227 * 1024;

struct OccupancyEntry {
  int threads;
  size_t smem;
  int ctas_per_sm;
};

struct KernelState {
  bool limit_raised = false;
  int carveout = -1;
  std::vector<OccupancyEntry> occupancy;
};

struct Key {
  int device;
  const void* func;
  bool operator==(const Key& o) const { return device == o.device && func == o.func; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    return std::hash<const void*>()(k.func) ^ (static_cast<size_t>(k.device) * 0x9E3779B97F4A7C15ull);
  }
};

std::mutex g_mutex;
std::unordered_map<Key, KernelState, KeyHash> g_kernels;
int g_sm_count[kMaxDevices] = {};

std::atomic<uint64_t> g_wait_tuning{(static_cast<uint64_t>(kWaitSpins) << 32) | 0u};

}  // namespace

WaitTuning wait_tuning() {
  const uint64_t v = g_wait_tuning.load(std::memory_order_relaxed);
  return WaitTuning{static_cast<uint32_t>(v >> 32), static_cast<uint32_t>(v & 0xFFFFFFFFu)};
}

void set_wait_tuning(WaitTuning t) {
  g_wait_tuning.store((static_cast<uint64_t>(t.spins) << 32) | t.extra_tx, std::memory_order_relaxed);
}

cudaError_t device_sm_count(int* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_sm_count[dev] == 0) {
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    g_sm_count[dev] = n > 0 ? n : 1;
  }
  *out = g_sm_count[dev];
  return cudaSuccess;
}

cudaError_t kernel_launch_config(const void* func, int threads, size_t smem, int carveout_percent,
                                 int* ctas_per_sm) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(g_mutex);
  KernelState& st = g_kernels[Key{dev, func}];
  if (!st.limit_raised) {
    e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
    if (e != cudaSuccess) return e;
    st.limit_raised = true;
  }
  if (carveout_percent >= 0 && carveout_percent != st.carveout) {
    if (carveout_percent > 100) carveout_percent = 100;
    e = cudaFuncSetAttribute(func, cudaFuncAttributePreferredSharedMemoryCarveout, carveout_percent);
    if (e != cudaSuccess) return e;
    st.carveout = carveout_percent;
  }
  if (ctas_per_sm != nullptr) {
    for (const OccupancyEntry& o : st.occupancy) {
      if (o.threads == threads && o.smem == smem) {
        *ctas_per_sm = o.ctas_per_sm;
        return cudaSuccess;
      }
    }
    int n = 1;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, func, threads, smem);
    if (e != cudaSuccess) return e;
    if (n < 1) n = 1;
    st.occupancy.push_back(OccupancyEntry{threads, smem, n});
    *ctas_per_sm = n;
  }
  return cudaSuccess;
}

}  // namespace cb200
