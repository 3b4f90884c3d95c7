// Version and thread-local error text of the C ABI; per-device kernel attribute bookkeeping.
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace hb200 {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int ensure_dynamic_smem(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, size_t> done;
  int dev = 0;
  HB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  size_t& have = done[std::make_pair(kernel, dev)];
  if (bytes > have) {
    HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    have = bytes;
  }
  return 0;
}
}  // namespace hb200

extern "C" int hb200_version(void) { return 100; }
extern "C" const char* hb200_last_error(void) { return hb200::g_err; }
