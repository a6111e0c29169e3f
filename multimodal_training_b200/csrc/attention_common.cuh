// Shared pieces of the forward and backward flash-attention kernels.
#pragma once
#include <cudaTypedefs.h>

#include "common.cuh"
#include "runtime.h"

extern "C" int mmt_make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                                uint32_t box_inner, uint32_t box_outer);

namespace attn {

constexpr int BQ = 128;   // query rows per tile
constexpr int BKV = 128;  // kv rows per tile
constexpr int kThreads = 192;
constexpr uint32_t CHUNK = 128 * 64 * 2;  // one [128 x 64] bf16 swizzled box = 16 KB
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* qkv;
  __nv_bfloat16* out;          // [T, n_q*dim]
  float* lse;                  // [n_q, T]
  const int* seq_lo;
  const int* seq_hi;
  int T, n_q, n_kv, dim;
  long ld;
  int causal;
  float scale;
  MmtErrorWord* ew;
  // backward only
  const __nv_bfloat16* dout;   // [T, n_q*dim]
  const float* delta;          // [n_q, T]  rowsum(out * dout)
  __nv_bfloat16* dqkv;         // [T, ld]
  float* ws_dk;                // optional [n_q, T, dim] fp32 per-q-head partial dK (GQA: one CTA per q head)
  float* ws_dv;
};

// byte offset of element (row, col) inside a [128 x 64] SW128 box with 128-byte rows
MMT_DEVICE uint32_t sw128_offset(int row, int col) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 3) ^ (row & 7)) & 7) << 4) + (col & 7) * 2);
}

// descriptor address of K-step k (16 columns) of a K-major operand whose columns sit in two
// 64-column boxes at `base` and `base + CHUNK`
MMT_DEVICE uint32_t kmajor_kstep_addr(uint32_t base, int k) {
  return base + (k >> 2) * CHUNK + (k & 3) * 32;
}

// K-major operand tile (rows x up-to-128 columns in two boxes): descriptor of K-step k
MMT_DEVICE uint64_t desc_kmajor(uint32_t base, int k) { return make_smem_desc(kmajor_kstep_addr(base, k), 16, 1024); }
// MN-major operand tile: rows are the K dimension (16 rows per step), columns the M/N dimension
MMT_DEVICE uint64_t desc_mnmajor(uint32_t base, int k) { return make_smem_desc(base + k * 2048, CHUNK, 1024); }

}  // namespace attn
