// Symmetric heap: one device buffer per rank, exported through CUDA IPC so that every rank of the
// node can map every peer's buffer and address it with plain loads and stores over NVLink/NVSwitch.
// The handle exchange itself is done by the host control plane (torch.distributed object
// all-gather, see parallel/symm.py).  Replaces the per-tensor CUDA-IPC handles that the reference
// ships through the Ray object store (python/ray/tensor_transfer.py:35-96).
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "runtime.h"

extern "C" {

int mmt_symm_alloc(size_t bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}

int mmt_symm_free(void* p) { return (int)cudaFree(p); }

// handle: 64 bytes
int mmt_symm_export(void* p, unsigned char* handle) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  memcpy(handle, &h, sizeof(h));
  return 0;
}

int mmt_symm_import(const unsigned char* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}

int mmt_symm_unimport(void* p) { return (int)cudaIpcCloseMemHandle(p); }

int mmt_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}

}  // extern "C"
