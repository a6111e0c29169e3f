// Host-side runtime shared by every translation unit of the kernel library.
#pragma once
#include <cuda_runtime.h>

struct MmtErrorWord;

// Number of SMs of the current device (cached).
int mmt_sm_count();
// Device address of the library's error word for the current device
// (allocated on first use; kernels record bounded-wait failures there).
MmtErrorWord* mmt_error_word();

// Makes sure the calling thread has the CUDA context of the device that owns `ptr` (first call per thread).
int mmt_ensure_context(const void* ptr);

extern "C" {
// Copies the error word to out[4] = {code, where, block, aux}; synchronises the device.
int mmt_get_error(int* out);
// Device address of the error word ([4] int32), or nullptr if it could not be allocated.
void* mmt_error_word_address();
// Resets the error word to zero.
int mmt_clear_error();
// Library build tag, for tests that check the native path is loaded.
const char* mmt_version();
}
