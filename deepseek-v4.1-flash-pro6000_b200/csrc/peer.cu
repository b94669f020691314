// Peer-visible device buffers for the vocabulary-sharded path: one process per GPU, each exports one buffer (the full
// logits rows it will sample) and maps the other ranks' buffers, so that the head kernel's epilogue can store its
// vocabulary slice of every row directly into the row's owner (ds41_b200_head_fp8_scatter).  Plain CUDA IPC mappings,
// written with ordinary peer stores: no NVSwitch group object is created for them.
#include <cuda_runtime.h>

#include <cstring>

#include "ds41_b200.h"
#include "host_error.h"

using namespace ds41;

static_assert(sizeof(cudaIpcMemHandle_t) == DS41_B200_PEER_HANDLE_BYTES, "handle size is part of the ABI");

extern "C" int ds41_b200_peer_alloc(size_t bytes, void **ptr, void *handle) {
  if (!bytes || !ptr || !handle) return invalid("peer_alloc arguments");
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return int(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return int(e);
  }
  std::memcpy(handle, &h, sizeof h);
  *ptr = p;
  return 0;
}

extern "C" int ds41_b200_peer_open(const void *handle, void **ptr) {
  if (!handle || !ptr) return invalid("peer_open arguments");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof h);
  return int(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

extern "C" int ds41_b200_peer_close(void *ptr) { return ptr ? int(cudaIpcCloseMemHandle(ptr)) : 0; }

extern "C" int ds41_b200_peer_free(void *ptr) { return ptr ? int(cudaFree(ptr)) : 0; }
