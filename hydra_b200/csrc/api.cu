// Version and thread-local error text of the C ABI.
#include "common.cuh"

namespace hb200 {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
}  // namespace hb200

extern "C" int hb200_version(void) { return 100; }
extern "C" const char* hb200_last_error(void) { return hb200::g_err; }
