// Library-level entry points: error text, status record, device query and the CUDA-IPC
// symmetric buffers.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace mm {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

}  // namespace mm

using namespace mm;

extern "C" {

int mm_abi_version(void) { return 3; }

const char* mm_last_error(void) { return g_error; }

int mm_num_sms(int* out_host) {
  if (!out_host) {
    set_error("mm_num_sms: null argument");
    return MM_ERR_ARG;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(out_host, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) {
    set_error("mm_num_sms: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

int mm_status_reset(void* status, cudaStream_t stream) {
  if (!status) {
    set_error("mm_status_reset: null argument");
    return MM_ERR_ARG;
  }
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(mm_status_record), stream);
  if (e != cudaSuccess) {
    set_error("mm_status_reset: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

int mm_status_read(const void* status, mm_status_record* out_host, cudaStream_t stream) {
  if (!status || !out_host) {
    set_error("mm_status_read: null argument");
    return MM_ERR_ARG;
  }
  cudaError_t e = cudaMemcpyAsync(out_host, status, sizeof(mm_status_record),
                                  cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    set_error("mm_status_read: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

int mm_symm_alloc(size_t bytes, void** dptr_host, unsigned char handle_host[64]) {
  if (!dptr_host || !handle_host || bytes == 0) {
    set_error("mm_symm_alloc: bad arguments");
    return MM_ERR_ARG;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    set_error("mm_symm_alloc: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  e = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    set_error("mm_symm_alloc: %s", cudaGetErrorString(e));
    cudaFree(p);
    return MM_ERR_CUDA;
  }
  memcpy(handle_host, &h, 64);
  *dptr_host = p;
  return MM_OK;
}

int mm_symm_open(const unsigned char handle_host[64], void** peer_ptr_host) {
  if (!handle_host || !peer_ptr_host) {
    set_error("mm_symm_open: null argument");
    return MM_ERR_ARG;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_host, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_error("mm_symm_open: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  *peer_ptr_host = p;
  return MM_OK;
}

int mm_symm_close(void* peer_ptr) {
  if (!peer_ptr) {
    set_error("mm_symm_close: null argument");
    return MM_ERR_ARG;
  }
  cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  if (e != cudaSuccess) {
    set_error("mm_symm_close: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

int mm_symm_free(void* dptr) {
  if (!dptr) {
    set_error("mm_symm_free: null argument");
    return MM_ERR_ARG;
  }
  cudaError_t e = cudaFree(dptr);
  if (e != cudaSuccess) {
    set_error("mm_symm_free: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

}  // extern "C"
