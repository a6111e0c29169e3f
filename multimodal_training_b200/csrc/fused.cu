// Producer and consumer halves of the fused compute+collective paths that are not GEMMs.
//
// All of them address peer GPUs' memory directly (symmetric heap, plain loads/stores over
// NVLink/NVSwitch) and synchronise with epoch flags: a producer finishes its stores, fences
// system-wide and release-stores the epoch into a flag word on the consumer's GPU; a consumer
// spins on its LOCAL flag words with acquire loads, bounded by a deadline (error word on expiry).
// Flags only ever grow, so nothing is reset between uses.
//
//   rmsnorm_push     RMSNorm (optional) of a token shard, each output row stored into the gather
//                    buffer of EVERY tensor-parallel peer: the all-gather of "all-gather -> GEMM" happens
//                    in the epilogue of the norm; the GEMM's TMA producer waits on the flags (gemm.cu)
//   rs_reduce        owner side of "GEMM -> reduce-scatter": sum the partial tiles that the peers' GEMM
//                    epilogues pushed into this rank's staging slots (+ residual)
//   route_rows       vision->text handoff and its gradient: rows stored to (peer, row) destinations
//   wait_flags       stand-alone bounded wait (consumer side of route_rows)
//   zero1_adamw      ZeRO-1 step in one pass: pull the peers' gradient shards, sum, AdamW on the fp32 master
//                    shard, push the bf16 parameters into every peer's parameter buffer
//
// Replaces NCCL call sites C1-C12/C18 of the reference (all-to-all in modeling_qwen2_5_vl.py:628-746, DTensor
// all-reduces from python/ray/text.py:1165-1177, DeepSpeed ZeRO-1 configured at python/ray/trainer.py:764-785,
// IPC handoff python/ray/tensor_transfer.py:35-96).
#include "common.cuh"
#include "runtime.h"

namespace {

typedef __nv_bfloat16 bf16;

MMT_DEVICE void load8(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(w[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
MMT_DEVICE uint4 pack8(const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  return o;
}

struct PeerSet {
  unsigned long long base[8];   // destination base address on each peer (region offset included)
  int* flag[8];                 // flag word to set on each peer
  int n;
};

// Last CTA of the grid publishes the epoch to every peer's flag word.
MMT_DEVICE void publish_when_last(int* counter, const PeerSet& ps, int epoch) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y;
    if (atomicAdd(counter, 1) == (int)total - 1) {
      *counter = 0;
      __threadfence_system();
      for (int r = 0; r < ps.n; ++r) flag_store_release_sys(ps.flag[r], epoch);
    }
  }
}

// A CTA that gives up (its bounded wait ran out) still counts itself out, so that the counter is back at zero for
// the next launch; it publishes nothing: the peers' own waits run out and the host reads the error word.
MMT_DEVICE void retire_without_publishing(int* counter) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y;
    if (atomicAdd(counter, 1) == (int)total - 1) *counter = 0;
  }
}

// One CTA waits for n local flag words (skipping `self`); all threads learn the outcome.
MMT_DEVICE bool wait_all_flags(const int* flags, int n, int self, int epoch, MmtErrorWord* ew, int where) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int s = 0; s < n && ok; ++s)
      if (s != self) ok = flag_wait_ge(&flags[s], epoch, MMT_WAIT_NS, ew, where);
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  return ok_s != 0;
}

// ----------------------------------------------------------------------------
// RMSNorm (or plain copy when w == nullptr) of x[rows, cols], every row stored to all peers at
// row_offset + row of their gather buffers.  One CTA per row.
// ----------------------------------------------------------------------------
constexpr int kNT = 256, kNV = 4;

__global__ void __launch_bounds__(kNT) rmsnorm_push_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          float* __restrict__ rstd_out, PeerSet ps, int* counter,
                                                          int epoch, long row_offset, int cols, float eps) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  const int nvec = cols >> 3;
  float v[kNV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNV; ++i) {
    const int c = threadIdx.x + i * kNT;
    if (c < nvec) {
      load8(x + row * cols + c * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  float rstd = 1.f;
  if (w) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = threadIdx.x < kNT / 32 ? red[threadIdx.x] : 0.f;
    if (threadIdx.x < 32) {
      t = warp_sum(t);
      if (threadIdx.x == 0) red[0] = t;
    }
    __syncthreads();
    rstd = rsqrtf(red[0] / (float)cols + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < kNV; ++i) {
    const int c = threadIdx.x + i * kNT;
    if (c < nvec) {
      float o[8];
      if (w) {
        float wv[8];
        load8(w + c * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j];
      }
      const uint4 packed = pack8(o);
      const long off = (row_offset + row) * cols + c * 8;
      for (int r = 0; r < ps.n; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(ps.base[r]) + off) = packed;
    }
  }
  publish_when_last(counter, ps, epoch);
}

// ----------------------------------------------------------------------------
// out[r, c] = residual[r, c] + sum_s staging[s][r][c]   (fp32 sum in rank order, so all ranks agree bit for bit)
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rs_reduce_kernel(const bf16* __restrict__ staging, const int* __restrict__ flags,
                                                       int epoch, int n_src, int self, const bf16* __restrict__ residual,
                                                       bf16* __restrict__ out, long rows, int cols, MmtErrorWord* ew) {
  if (!wait_all_flags(flags, n_src, self, epoch, ew, 900)) return;
  const long n8 = rows * cols / 8;
  const long slot = rows * cols;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float acc[8];
    if (residual) {
      load8(residual + i * 8, acc);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int s = 0; s < n_src; ++s) {
      float v[8];
      load8(staging + s * slot + i * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    *reinterpret_cast<uint4*>(out + i * 8) = pack8(acc);
  }
}

// ----------------------------------------------------------------------------
// Row routing: src row i goes to peer dest_rank[i], row dest_row[i] of the region at ps.base[peer].
// One warp per row.  Used for the vision->text handoff (forward) and its gradient (backward).
// ----------------------------------------------------------------------------
__global__ void route_rows_kernel(const bf16* __restrict__ src, const int* __restrict__ dest_rank,
                                  const long* __restrict__ dest_row, PeerSet ps, int* counter, int epoch, long rows,
                                  int cols, long src_ld, long dst_ld, long dst_rows, MmtErrorWord* ew) {
  const long r = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r < rows) {
    const int lane = threadIdx.x & 31;
    const int dr = dest_rank[r];
    const long drow = dest_row[r];
    if (dr < 0 || dr >= ps.n || drow < 0 || drow >= dst_rows) {
      // a destination outside the region would be a wild store into a peer's memory: skip it and say so
      if (lane == 0) mmt_report(ew, MMT_ERR_BOUNDS, 920, (int)r);
    } else {
      bf16* dst = reinterpret_cast<bf16*>(ps.base[dr]) + drow * dst_ld;
      for (int c = lane * 8; c < cols; c += 256)
        *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + r * src_ld + c);
    }
  }
  publish_when_last(counter, ps, epoch);
}

__global__ void wait_flags_kernel(const int* __restrict__ flags, int n, int self, int epoch, MmtErrorWord* ew) {
  wait_all_flags(flags, n, self, epoch, ew, 910);
}

// ----------------------------------------------------------------------------
// ZeRO-1 in one pass over the owned shard [lo, lo + n):
//   g = sum over ranks of their gradient at [lo, lo+n)  (peer loads; fp32 sum in rank order)
//   AdamW on master / m / v (fp32), p = bf16(master) stored into EVERY rank's parameter buffer (peer stores)
// Before: every rank's backward must be complete (grad_flags, set by publish at the end of backward).
// After: param flags tell every rank that this shard of the parameters is up to date.
// ----------------------------------------------------------------------------
struct ZeroPeers {
  unsigned long long grad[8];    // each rank's flat gradient base
  unsigned long long param[8];   // each rank's flat parameter base
  int* param_flag[8];            // flag word on each rank: "shard of rank `self` is updated"
  int n;
};

__global__ void __launch_bounds__(256) zero1_adamw_kernel(ZeroPeers zp, const int* __restrict__ grad_flags,
                                                         int grad_epoch, int self, int* counter, int param_epoch,
                                                         float* __restrict__ master, float* __restrict__ m,
                                                         float* __restrict__ v, long lo, long n, long n_decay,
                                                         float lr, float b1, float b2, float eps, float wd, float bc1,
                                                         float bc2, const float* __restrict__ gscale_ptr,
                                                         float* __restrict__ normsq_out, MmtErrorWord* ew) {
  if (!wait_all_flags(grad_flags, zp.n, self, grad_epoch, ew, 920)) {
    retire_without_publishing(counter);
    return;
  }
  const float gs = gscale_ptr ? *gscale_ptr : 1.f;
  const long n8 = n >> 3;
  float nsq = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long e = i * 8;
    float g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = 0.f;
    for (int r = 0; r < zp.n; ++r) {
      float t[8];
      load8(reinterpret_cast<const bf16*>(zp.grad[r]) + lo + e, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] += t[j];
    }
    float4 w0 = *reinterpret_cast<float4*>(master + e), w1 = *reinterpret_cast<float4*>(master + e + 4);
    float4 m0 = *reinterpret_cast<float4*>(m + e), m1 = *reinterpret_cast<float4*>(m + e + 4);
    float4 v0 = *reinterpret_cast<float4*>(v + e), v1 = *reinterpret_cast<float4*>(v + e + 4);
    float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gs;
      nsq += gj * gj;
      mv[j] = b1 * mv[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      const float upd = (mv[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
      const float decay = (e + j < n_decay) ? wd : 0.f;
      wv[j] = wv[j] - lr * (upd + decay * wv[j]);
    }
    *reinterpret_cast<float4*>(master + e) = make_float4(wv[0], wv[1], wv[2], wv[3]);
    *reinterpret_cast<float4*>(master + e + 4) = make_float4(wv[4], wv[5], wv[6], wv[7]);
    *reinterpret_cast<float4*>(m + e) = make_float4(mv[0], mv[1], mv[2], mv[3]);
    *reinterpret_cast<float4*>(m + e + 4) = make_float4(mv[4], mv[5], mv[6], mv[7]);
    *reinterpret_cast<float4*>(v + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(v + e + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    const uint4 packed = pack8(wv);
    for (int r = 0; r < zp.n; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(zp.param[r]) + lo + e) = packed;
  }
  if (normsq_out) {
    nsq = warp_sum(nsq);
    if ((threadIdx.x & 31) == 0) atomicAdd(normsq_out, nsq);
  }
  PeerSet ps;
  ps.n = zp.n;
  for (int r = 0; r < zp.n; ++r) ps.flag[r] = zp.param_flag[r];
  publish_when_last(counter, ps, param_epoch);
}

// ----------------------------------------------------------------------------
// Ulysses exchange (sequence <-> heads) as direct peer stores.
//   to_heads:  src [rows, parts, groups, W] (token-major rows of this rank, all heads) ->
//              peer g's buffer [T_all, parts, W] at row dst_row[r]: group g's heads of every part
//   to_tokens: src [T_all, parts, W] (all rows, this rank's heads) ->
//              owner's buffer [rows_owner, parts, groups, W] at (row_local[r], part, my group)
// One warp per (row, part, group) segment of W elements (W % 8 == 0).
// ----------------------------------------------------------------------------
__global__ void ulysses_to_heads_kernel(const bf16* __restrict__ src, const int* __restrict__ dst_row, PeerSet ps,
                                        int* counter, int epoch, long rows, int parts, int groups, int W) {
  const long seg = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const long nseg = rows * parts * groups;
  if (seg < nseg) {
    const int lane = threadIdx.x & 31;
    const int g = (int)(seg % groups);
    const int pt = (int)((seg / groups) % parts);
    const long r = seg / ((long)groups * parts);
    const bf16* s = src + ((r * parts + pt) * groups + g) * (long)W;
    bf16* d = reinterpret_cast<bf16*>(ps.base[g]) + ((long)dst_row[r] * parts + pt) * W;
    for (int c = lane * 8; c < W; c += 256) *reinterpret_cast<uint4*>(d + c) = *reinterpret_cast<const uint4*>(s + c);
  }
  publish_when_last(counter, ps, epoch);
}

__global__ void ulysses_to_tokens_kernel(const bf16* __restrict__ src, const int* __restrict__ owner,
                                         const int* __restrict__ row_local, PeerSet ps, int* counter, int epoch,
                                         long rows, int parts, int groups, int my_group, int W) {
  const long seg = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const long nseg = rows * parts;
  if (seg < nseg) {
    const int lane = threadIdx.x & 31;
    const int pt = (int)(seg % parts);
    const long r = seg / parts;
    const bf16* s = src + (r * parts + pt) * (long)W;
    bf16* d = reinterpret_cast<bf16*>(ps.base[owner[r]]) + (((long)row_local[r] * parts + pt) * groups + my_group) * W;
    for (int c = lane * 8; c < W; c += 256) *reinterpret_cast<uint4*>(d + c) = *reinterpret_cast<const uint4*>(s + c);
  }
  publish_when_last(counter, ps, epoch);
}

// Publishes an epoch to all peers (e.g. "my backward pass is complete") without moving data.
__global__ void publish_kernel(PeerSet ps, int epoch) {
  __threadfence_system();
  if (threadIdx.x == 0)
    for (int r = 0; r < ps.n; ++r) flag_store_release_sys(ps.flag[r], epoch);
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" {

// Plain-data mirror of PeerSet for the ctypes boundary.
struct MmtPeerSet {
  unsigned long long base[8];
  unsigned long long flag[8];
  int n;
};

static PeerSet to_ps(const MmtPeerSet* in) {
  PeerSet ps;
  ps.n = in->n;
  for (int i = 0; i < 8; ++i) {
    ps.base[i] = in->base[i];
    ps.flag[i] = reinterpret_cast<int*>(in->flag[i]);
  }
  return ps;
}

int mmt_rmsnorm_push(const void* x, const void* w, float* rstd, const MmtPeerSet* peers, int* counter, int epoch,
                     long row_offset, long rows, int cols, float eps, void* stream) {
  if (cols % 8 || cols > 8 * kNT * kNV || peers->n < 1 || peers->n > 8) return -2;
  if (rows == 0) return -3;  // a rank with no rows could never publish its flag
  rmsnorm_push_kernel<<<(unsigned)rows, kNT, 0, ST(stream)>>>(reinterpret_cast<const bf16*>(x),
                                                             reinterpret_cast<const bf16*>(w), rstd, to_ps(peers),
                                                             counter, epoch, row_offset, cols, eps);
  return (int)cudaGetLastError();
}

int mmt_rs_reduce(const void* staging, const int* flags, int epoch, int n_src, int self, const void* residual,
                  void* out, long rows, int cols, void* stream) {
  if ((rows * cols) % 8) return -2;
  long blocks = (rows * cols / 8 + 255) / 256;
  const long cap = (long)mmt_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  rs_reduce_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(reinterpret_cast<const bf16*>(staging), flags, epoch,
                                                            n_src, self, reinterpret_cast<const bf16*>(residual),
                                                            reinterpret_cast<bf16*>(out), rows, cols,
                                                            mmt_error_word());
  return (int)cudaGetLastError();
}

// dest_rank: int32 index into `peers`; dest_row: int64 row of the destination region, which has dst_rows rows.
int mmt_route_rows(const void* src, const int* dest_rank, const long* dest_row, const MmtPeerSet* peers, int* counter,
                   int epoch, long rows, int cols, long src_ld, long dst_ld, long dst_rows, void* stream) {
  if (cols % 8 || src_ld % 8 || dst_ld % 8) return -2;
  const long blocks = rows > 0 ? (rows + 7) / 8 : 1;
  route_rows_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(reinterpret_cast<const bf16*>(src), dest_rank, dest_row,
                                                             to_ps(peers), counter, epoch, rows, cols, src_ld, dst_ld, dst_rows,
                                                             mmt_error_word());
  return (int)cudaGetLastError();
}

int mmt_wait_flags(const int* flags, int n, int self, int epoch, void* stream) {
  wait_flags_kernel<<<1, 32, 0, ST(stream)>>>(flags, n, self, epoch, mmt_error_word());
  return (int)cudaGetLastError();
}

int mmt_publish(const MmtPeerSet* peers, int epoch, void* stream) {
  publish_kernel<<<1, 32, 0, ST(stream)>>>(to_ps(peers), epoch);
  return (int)cudaGetLastError();
}

int mmt_ulysses_to_heads(const void* src, const int* dst_row, const MmtPeerSet* peers, int* counter, int epoch,
                         long rows, int parts, int groups, int W, void* stream) {
  if (W % 8 || peers->n != groups) return -2;
  const long nseg = rows * parts * groups;
  const long blocks = nseg > 0 ? (nseg + 7) / 8 : 1;
  ulysses_to_heads_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(reinterpret_cast<const bf16*>(src), dst_row,
                                                                   to_ps(peers), counter, epoch, rows, parts, groups, W);
  return (int)cudaGetLastError();
}

int mmt_ulysses_to_tokens(const void* src, const int* owner, const int* row_local, const MmtPeerSet* peers,
                          int* counter, int epoch, long rows, int parts, int groups, int my_group, int W,
                          void* stream) {
  if (W % 8 || peers->n != groups) return -2;
  const long nseg = rows * parts;
  const long blocks = nseg > 0 ? (nseg + 7) / 8 : 1;
  ulysses_to_tokens_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(reinterpret_cast<const bf16*>(src), owner,
                                                                    row_local, to_ps(peers), counter, epoch, rows,
                                                                    parts, groups, my_group, W);
  return (int)cudaGetLastError();
}

struct MmtZeroPeers {
  unsigned long long grad[8];
  unsigned long long param[8];
  unsigned long long param_flag[8];
  int n;
};

int mmt_zero1_adamw(const MmtZeroPeers* peers, const int* grad_flags, int grad_epoch, int self, int* counter,
                    int param_epoch, float* master, float* m, float* v, long lo, long n, long n_decay, float lr,
                    float b1, float b2, float eps, float wd, int step, const float* gscale_ptr, float* normsq_out,
                    void* stream) {
  if (n % 8 || lo % 8 || peers->n < 1 || peers->n > 8) return -2;
  ZeroPeers zp;
  zp.n = peers->n;
  for (int i = 0; i < 8; ++i) {
    zp.grad[i] = peers->grad[i];
    zp.param[i] = peers->param[i];
    zp.param_flag[i] = reinterpret_cast<int*>(peers->param_flag[i]);
  }
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  long blocks = (n / 8 + 255) / 256;
  const long cap = (long)mmt_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  zero1_adamw_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(zp, grad_flags, grad_epoch, self, counter, param_epoch,
                                                              master, m, v, lo, n, n_decay, lr, b1, b2, eps, wd, bc1,
                                                              bc2, gscale_ptr, normsq_out, mmt_error_word());
  return (int)cudaGetLastError();
}

}  // extern "C"
