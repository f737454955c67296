// ABI version, per-thread error string and the device-capability check shared by all entry points.
#include <cstring>

#include "common.cuh"

namespace moddit {

static thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_error[0] = '\0'; }

int require_sm100() {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail(MODDIT_E_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(err));
  int major = 0;
  err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (err != cudaSuccess)
    return fail(MODDIT_E_CUDA, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(err));
  if (major != 10)
    return fail(MODDIT_E_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only",
                dev, major);
  return MODDIT_OK;
}

}  // namespace moddit

extern "C" int moddit_abi_version(void) { return 2; }

extern "C" const char* moddit_last_error_string(void) { return moddit::g_error; }
