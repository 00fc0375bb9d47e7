// Symmetric buffers for one-process-per-GPU ranks on one node: a plain
// cudaMalloc allocation exported through a CUDA IPC handle and opened by every
// peer, which yields ordinary device pointers that kernels can load from and
// store to over NVLink.  No TMA is ever pointed at a peer mapping.
#include "comm.h"

#include <cstring>

namespace nfb {

const char* symm_alloc(size_t bytes, void** ptr, unsigned char handle_out[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) { cudaFree(p); return cudaGetErrorString(e); }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return cudaGetErrorString(e); }
  std::memcpy(handle_out, &h, 64);
  *ptr = p;
  return nullptr;
}

const char* symm_open(const unsigned char handle[64], void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* symm_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* symm_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
