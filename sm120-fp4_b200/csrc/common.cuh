// Shared declarations of the CUDA translation units: error codes and launch-check helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Error codes returned by every C entry point (0 = success). Mirrored in include/b200moe.h.
enum {
  B200MOE_OK = 0,
  B200MOE_ERR_ARG = -1,        // null pointer, negative size, misaligned buffer
  B200MOE_ERR_SHAPE = -2,      // a dimension the kernels do not take
  B200MOE_ERR_CUDA = -3,       // a CUDA runtime / driver call failed (see b200moe_last_cuda_error)
  B200MOE_ERR_DEVICE = -4,     // no sm_100 device, or the driver entry point for tensor maps is missing
  B200MOE_ERR_TIMEOUT = -5,    // a bounded device-side wait ran out (status word set by the kernel)
  B200MOE_ERR_WORKSPACE = -6,  // workspace too small
  B200MOE_ERR_LIMIT = -7,      // size beyond a stated maximum
  B200MOE_ERR_RANGE = -8,      // an intermediate activation exceeded the range of the fixed activation scale (results clipped)
  B200MOE_ERR_ORDER = -9,      // the routing inputs changed while the call was running (they were not complete when it started)
};

namespace b200 {
extern thread_local cudaError_t g_last_cuda_error;
inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = e;
  return B200MOE_ERR_CUDA;
}
}  // namespace b200

#define B200_CUDA_TRY(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::b200::cuda_fail(_e);      \
  } while (0)

#define B200_LAUNCH_CHECK()                                   \
  do {                                                        \
    cudaError_t _e = cudaGetLastError();                      \
    if (_e != cudaSuccess) return ::b200::cuda_fail(_e);      \
  } while (0)
