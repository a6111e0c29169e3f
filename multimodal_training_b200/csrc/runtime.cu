// Host-side runtime of the kernel library: device properties and the error word
// that kernels use to report a bounded wait that ran out.
#include "runtime.h"

#include "common.cuh"

namespace {
int g_sms = 0;
MmtErrorWord* g_err = nullptr;
}  // namespace

int mmt_sm_count() {
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  return g_sms;
}

MmtErrorWord* mmt_error_word() {
  if (!g_err) {
    if (cudaMalloc(&g_err, sizeof(MmtErrorWord)) != cudaSuccess) return nullptr;
    cudaMemset(g_err, 0, sizeof(MmtErrorWord));
  }
  return g_err;
}

// Driver-API calls (tensor-map encoding) need a current context on the calling thread.  Threads that
// PyTorch creates for backward may not have one yet when our first call arrives, so the first call on
// each thread binds the primary context of the device that owns `ptr`.
int mmt_ensure_context(const void* ptr) {
  thread_local int bound_device = -1;
  if (bound_device >= 0) return 0;
  cudaPointerAttributes attr;
  int dev = -1;
  if (ptr && cudaPointerGetAttributes(&attr, ptr) == cudaSuccess && attr.type == cudaMemoryTypeDevice)
    dev = attr.device;
  else
    cudaGetLastError();
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) return -1;
  cudaError_t e = cudaSetDevice(dev);
  if (e == cudaSuccess) e = cudaFree(0);
  if (e != cudaSuccess) return (int)e;
  bound_device = dev;
  return 0;
}

extern "C" int mmt_get_error(int* out) {
  MmtErrorWord* w = mmt_error_word();
  if (!w) return -1;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpy(out, w, sizeof(MmtErrorWord), cudaMemcpyDeviceToHost);
}

// Device address of the error word (for an asynchronous copy to pinned host memory behind a step).
extern "C" void* mmt_error_word_address() { return mmt_error_word(); }

extern "C" int mmt_clear_error() {
  MmtErrorWord* w = mmt_error_word();
  if (!w) return -1;
  return (int)cudaMemset(w, 0, sizeof(MmtErrorWord));
}

extern "C" const char* mmt_version() { return "mmt_b200 sm_100a"; }
