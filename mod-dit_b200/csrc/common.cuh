// Shared host-side helpers for the C-ABI entry points: argument checks and error reporting.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "moddit.h"

namespace moddit {

// Stores a printf-style message for moddit_last_error_string() on this thread and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Returns 0 when the current device is compute capability 10.x, else a failure code.
int require_sm100();

#define MODDIT_CHECK_ARG(cond, ...)                                  \
  do {                                                               \
    if (!(cond)) return ::moddit::fail(MODDIT_E_ARG, __VA_ARGS__);   \
  } while (0)

#define MODDIT_CHECK_CUDA(expr)                                                              \
  do {                                                                                       \
    cudaError_t err__ = (expr);                                                              \
    if (err__ != cudaSuccess)                                                                \
      return ::moddit::fail(MODDIT_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
  } while (0)

#define MODDIT_CHECK_LAUNCH(name)                                                            \
  do {                                                                                       \
    cudaError_t err__ = cudaGetLastError();                                                  \
    if (err__ != cudaSuccess)                                                                \
      return ::moddit::fail(MODDIT_E_CUDA, "launch of %s failed: %s", name,                  \
                            cudaGetErrorString(err__));                                      \
  } while (0)

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Opt-in to `bytes` of dynamic shared memory for `kernel` on the current device.  The attribute is a per-device
// property of the kernel: the driver call is made only when a launch needs more than any earlier one did, not
// once per call.  Returns MODDIT_OK or a failure code (message set).
int ensure_dynamic_smem(const void* kernel, size_t bytes);

}  // namespace moddit
