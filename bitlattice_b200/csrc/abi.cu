// Error reporting and device queries of the C ABI.
#include "common.cuh"

#include <cstring>
#include <mutex>

namespace blb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count(int device) {
  static std::mutex mu;
  static int cached[64];
  std::lock_guard<std::mutex> lock(mu);
  if (device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cached[device] = n;
  }
  return cached[device];
}

}  // namespace blb

extern "C" int bl_version(void) { return 1; }

extern "C" const char* bl_last_error(void) { return blb::g_error; }
