// abi.cu -- error plumbing and process-wide bookkeeping of the C ABI.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace ieb {

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char *what) {
  snprintf(g_err, sizeof g_err, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return IE_B200_E_CUDA;
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool pdl_enabled() {
  static const bool on = [] {
    const char *v = getenv("IE_B200_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

int ensure_dynamic_smem(const void *func, size_t bytes) {
  if (bytes <= 48u * 1024u) return IE_B200_OK;
  static std::mutex mu;
  static std::map<std::pair<const void *, int>, size_t> set_to;
  int dev = 0;
  IEB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  size_t &cur = set_to[{func, dev}];
  if (bytes > cur) {
    IEB_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    cur = bytes;
  }
  return IE_B200_OK;
}

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n, cached_dev = dev;
  }
  return cached;
}

}  // namespace ieb

extern "C" const char *ie_b200_last_error(void) { return ieb::g_err; }

extern "C" int ie_b200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

extern "C" uint64_t ie_b200_launch_count(void) { return ieb::g_launches.load(std::memory_order_relaxed); }
