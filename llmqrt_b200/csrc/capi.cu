// Process-wide pieces of the C ABI: error buffer, version, workspace size, device properties.
#include "common.cuh"

#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

namespace llmqrt {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return 148;
    cached = p.multiProcessorCount;
    cached_dev = dev;
  }
  return cached;
}

static std::atomic<long long> g_launches{0};

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(LLMQRT_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return LLMQRT_OK;
}

long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("LLMQRT_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

int ensure_dynamic_smem(const void* func, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> configured;
  // The 48 KiB a kernel gets without opting in covers static + dynamic shared memory together, so
  // opt in from 32 KiB of dynamic memory on.
  if (bytes <= 32 * 1024) return LLMQRT_OK;
  int dev = 0;
  LLMQRT_CUDA_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  int& have = configured[{dev, func}];
  if (bytes > have) {
    LLMQRT_CUDA_OK(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    have = bytes;
  }
  return LLMQRT_OK;
}

}  // namespace llmqrt

extern "C" {

const char* llmqrt_last_error(void) { return llmqrt::last_error_buffer(); }

int llmqrt_abi_version(void) { return 5; }

long long llmqrt_launch_count(void) { return llmqrt::launch_count(); }

// 64 KiB of arrival counters followed by 160 MiB of partial sums.  Every kernel that splits its
// reduction clamps the number of slices so that its partials fit (8 slices of a 64 x 18944 fp32
// tile are 39 MiB).
size_t llmqrt_workspace_bytes(void) { return llmqrt::LLMQRT_WS_COUNTER_BYTES + llmqrt::LLMQRT_WS_PARTIAL_BYTES; }

}  // extern "C"
