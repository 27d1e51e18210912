// Host-side helpers shared by the translation units of libmegamoe_sm100.so.
#pragma once

#include <cuda_runtime.h>

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

}  // namespace mm
