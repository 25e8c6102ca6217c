// Peer-visible device buffers for the tensor-parallel all-reduce that is fused into the
// linear kernel's epilogue: allocation, export and import of inter-process memory handles.
// One process per GPU; a rank allocates its workspace and arrival counters here, sends the
// 64-byte handles to its peers (any host channel), and opens theirs.  The kernels only
// ever use plain loads and stores (and system-scope atomics) on these buffers.
#include <string.h>

#include "nz_common.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");

extern "C" int nz_peer_alloc(uint64_t bytes, void **ptr, void *handle64) {
  if (!ptr || !handle64 || bytes == 0) {
    nz::set_error("nz_peer_alloc: null pointer or zero size");
    return NZ_E_ARG;
  }
  void *p = nullptr;
  NZ_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaError_t err = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, p);
  if (err != cudaSuccess) {
    cudaFree(p);
    return nz::cuda_fail(err, "nz_peer_alloc");
  }
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return NZ_OK;
}

extern "C" int nz_peer_open(const void *handle64, void **ptr) {
  if (!ptr || !handle64) {
    nz::set_error("nz_peer_open: null pointer");
    return NZ_E_ARG;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  NZ_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return NZ_OK;
}

extern "C" int nz_peer_close(void *ptr) {
  if (ptr) NZ_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return NZ_OK;
}

extern "C" int nz_peer_free(void *ptr) {
  if (ptr) NZ_CUDA_TRY(cudaFree(ptr));
  return NZ_OK;
}
