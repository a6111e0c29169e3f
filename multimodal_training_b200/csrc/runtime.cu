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

extern "C" int mmt_get_error(int* out) {
  MmtErrorWord* w = mmt_error_word();
  if (!w) return -1;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpy(out, w, sizeof(MmtErrorWord), cudaMemcpyDeviceToHost);
}

extern "C" int mmt_clear_error() {
  MmtErrorWord* w = mmt_error_word();
  if (!w) return -1;
  return (int)cudaMemset(w, 0, sizeof(MmtErrorWord));
}

extern "C" const char* mmt_version() { return "mmt_b200 sm_100a"; }
