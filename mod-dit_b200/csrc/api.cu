// ABI version, per-thread error string and the device-capability check shared by all entry points.
#include <cstring>
#include <mutex>

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

namespace {
struct SmemOptIn {
  const void* kernel;
  int device;
  size_t bytes;
};
constexpr int kMaxOptIns = 256;
SmemOptIn g_optins[kMaxOptIns];
int g_optin_count = 0;
std::mutex g_optin_mutex;
}  // namespace

int ensure_dynamic_smem(const void* kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return MODDIT_OK;          // available without opting in
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail(MODDIT_E_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(err));
  std::lock_guard<std::mutex> lock(g_optin_mutex);
  SmemOptIn* slot = nullptr;
  for (int i = 0; i < g_optin_count; ++i)
    if (g_optins[i].kernel == kernel && g_optins[i].device == dev) slot = &g_optins[i];
  if (slot != nullptr && slot->bytes >= bytes) return MODDIT_OK;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (err != cudaSuccess)
    return fail(MODDIT_E_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize, %zu) failed: %s", bytes,
                cudaGetErrorString(err));
  if (slot == nullptr && g_optin_count < kMaxOptIns) slot = &g_optins[g_optin_count++];
  if (slot != nullptr) *slot = SmemOptIn{kernel, dev, bytes};
  return MODDIT_OK;
}

}  // namespace moddit

extern "C" int moddit_abi_version(void) { return 2; }

extern "C" const char* moddit_last_error_string(void) { return moddit::g_error; }
