// Host-side helpers shared by the translation units of libmegamoe_sm100.so.
#pragma once

#include <cuda_runtime.h>

#include <mutex>

#include "../../include/mega_moe_b200.h"

namespace mm {

// printf-style; stores the message for mm_last_error() of the calling thread.
void set_error(const char* fmt, ...);

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

// A kernel's function attributes (e.g. the opt-in dynamic shared-memory size) belong to the
// device the call was made on, so a process that drives several GPUs must set them once per
// device.  `run` is called with the device current, under the guard's lock, the first time
// each device comes by; it returns MM_OK or an error (then it is retried on the next call).
struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  std::mutex mutex;
  bool done[kMaxDevices] = {};

  template <class F>
  int operator()(F&& run) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
      set_error("cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
      return MM_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(mutex);
    if (done[dev]) return MM_OK;
    const int rc = run();
    if (rc == MM_OK) done[dev] = true;
    return rc;
  }
};

}  // namespace mm
