// Memory-bound kernels of the training step, written for HBM3e streaming:
// 16-byte vector accesses, one pass over each tensor, fp32 math, bf16 storage.
//
//   RMSNorm fwd/bwd            (reference: HF Qwen2RMSNorm used at modeling_qwen2_5_vl.py:253,771,1302)
//   rotate-half RoPE, in place (reference: modeling_qwen2_5_vl.py:272-283 vision, 1153-1191 M-RoPE)
//   SwiGLU / GELU fwd/bwd      (reference: modeling_qwen2_5_vl.py:204,256,1149)
//   row gather / scatter(-add) (embedding lookup, window permutation, vision->text splice)
//   column sums                (bias gradients)
//   vocab-parallel cross-entropy statistics and in-place gradient
//                              (reference: python/tensor_parallel/cross_entropy.py:41-236)
//   fused AdamW over a flat parameter shard, sum of squares (grad norm)
//                              (reference: torch.optim.Adam at python/ray/trainer.py:503-572)
#include <stdio.h>

#include "common.cuh"
#include "noalloc.h"
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
MMT_DEVICE void store8(bf16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

template <int kThreads>
MMT_DEVICE float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < kThreads / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  const float r = red[0];
  __syncthreads();
  return r;
}
template <int kThreads>
MMT_DEVICE float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < kThreads / 32) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) {
    t = warp_max(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  const float r = red[0];
  __syncthreads();
  return r;
}

// ----------------------------------------------------------------------------
// RMSNorm.  One CTA per row; the row stays in registers between the two passes.
// cols % 8 == 0, cols <= 8 * kThreads * kVec.
// ----------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormVec = 4;  // up to 8192 columns

__global__ void __launch_bounds__(kNormThreads) rmsnorm_fwd_kernel(const bf16* __restrict__ x,
                                                                  const bf16* __restrict__ w, bf16* __restrict__ y,
                                                                  float* __restrict__ rstd_out, int cols, float eps) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  const bf16* xr = x + row * cols;
  float v[kNormVec][8];
  float ss = 0.f;
  const int nvec = cols >> 3;
#pragma unroll
  for (int i = 0; i < kNormVec; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) {
      load8(xr + c * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float rstd = rsqrtf(ss / (float)cols + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < kNormVec; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) {
      float wv[8], o[8];
      load8(w + c * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
      store8(y + row * cols + c * 8, o);
    }
  }
}

MMT_DEVICE void unpack8(const uint4& u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(w[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}

// Forward for rows of up to 4096 columns: one warp per row (the row stays in registers as raw bf16, the sum of
// squares needs shuffles only), eight rows per CTA, no block-wide barrier.
template <int VPL>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_fwd_warp_kernel(const bf16* __restrict__ x,
                                                                       const bf16* __restrict__ w,
                                                                       bf16* __restrict__ y,
                                                                       float* __restrict__ rstd_out, long rows,
                                                                       int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (kNormThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols >> 3;
  const bf16* xr = x + row * cols;
  uint4 raw[VPL];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + i * 32;
    raw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (c < nvec) raw[i] = *reinterpret_cast<const uint4*>(xr + c * 8);
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    float v[8];
    unpack8(raw[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)cols + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      float v[8], wv[8], o[8];
      unpack8(raw[i], v);
      load8(w + c * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[j] * rstd * wv[j];
      store8(y + row * cols + c * 8, o);
    }
  }
}

// dx = rstd * (g - x * rstd^2 * mean(g * x)) (+ extra),  g = dy * w.
// A thread owns VEC fixed 8-column vectors, so its share of dw = sum_rows(dy * x * rstd) stays in registers; the
// per-CTA partial sums go to `dw_partial` [gridDim.x, cols] (fp32 scratch) for the second-stage reduction.
// A CTA takes R rows per iteration: all their loads are issued before the one block reduction of the R row
// dots (one __syncthreads per iteration, the exchange buffer alternates), which keeps enough bytes in flight per SM
// to run at memory speed; the rows are held as raw bf16 so that R x VEC vectors fit in registers.
template <int VEC, int R>
__global__ void __launch_bounds__(kNormThreads, VEC <= 2 ? 2 : 1) rmsnorm_bwd_kernel(const bf16* __restrict__ dy,
                                                                     const bf16* __restrict__ x,
                                                                     const bf16* __restrict__ w,
                                                                     const float* __restrict__ rstd_in,
                                                                     bf16* __restrict__ dx,
                                                                     float* __restrict__ dw_partial, int rows, int cols,
                                                                     const bf16* __restrict__ extra) {
  constexpr int kWarps = kNormThreads / 32;
  __shared__ float red[2][R][kWarps];
  const int nvec = cols >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float dwacc[VEC][8];
  float wv[VEC][8];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f, wv[i][j] = 0.f;
    if (c < nvec) load8(w + c * 8, wv[i]);
  }
  int buf = 0;
  for (long row0 = (long)blockIdx.x * R; row0 < rows; row0 += (long)gridDim.x * R, buf ^= 1) {
    uint4 xr[R][VEC], dr[R][VEC], er[R][VEC];
    float rs[R], dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long row = row0 + r;
      const bool ok = row < rows;
      rs[r] = ok ? rstd_in[row] : 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        xr[r][i] = dr[r][i] = er[r][i] = make_uint4(0u, 0u, 0u, 0u);
        if (ok && c < nvec) {
          xr[r][i] = *reinterpret_cast<const uint4*>(x + row * cols + c * 8);
          dr[r][i] = *reinterpret_cast<const uint4*>(dy + row * cols + c * 8);
          if (extra) er[r][i] = *reinterpret_cast<const uint4*>(extra + row * cols + c * 8);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float xv[8], d[8];
        unpack8(xr[r][i], xv);
        unpack8(dr[r][i], d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc += d[j] * wv[i][j] * xv[j];
          dwacc[i][j] += d[j] * xv[j] * rs[r];
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) red[buf][r][warp] = acc;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < kWarps; ++k) t += red[buf][r][k];
      dot[r] = t;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long row = row0 + r;
      if (row >= rows) continue;
      const float coef = dot[r] * rs[r] * rs[r] / (float)cols;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        if (c < nvec) {
          float xv[8], d[8], e[8], o[8];
          unpack8(xr[r][i], xv);
          unpack8(dr[r][i], d);
          unpack8(er[r][i], e);      // zeros without `extra`
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = rs[r] * (d[j] * wv[i][j] - xv[j] * coef) + e[j];
          store8(dx + row * cols + c * 8, o);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) {
      float* dst = dw_partial + (long)blockIdx.x * cols + c * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// out[c] (+)= sum_p partial[p, c]; out is bf16.  Block (32 columns, 8 part lanes): the parts are summed by eight
// lanes with independent loads and combined in a fixed order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partial, bf16* __restrict__ out,
                                                              int parts, int cols, int accumulate) {
  __shared__ float red[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < cols) {
#pragma unroll 4
    for (int p = threadIdx.y; p < parts; p += 8) s += partial[(long)p * cols + c];
  }
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x];
    if (accumulate) t += __bfloat162float(out[c]);
    out[c] = __float2bfloat16(t);
  }
}

// ----------------------------------------------------------------------------
// Rotate-half rotary embedding, in place, over the first `heads` heads of each row.
// x: [tokens, row_stride] with head h at column h*dim; cs: cos [tokens, dim], sin [tokens, dim] (fp32).
// sign = +1 forward, -1 backward (the transpose of the rotation).
// ----------------------------------------------------------------------------
__global__ void rope_kernel(bf16* __restrict__ x, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            long tokens, int heads, int dim, long row_stride, float sign) {
  const int half = dim >> 1;
  const int pairs_per_head = half >> 1;  // two adjacent columns per thread
  const long total = tokens * heads * pairs_per_head;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int pp = (int)(i % pairs_per_head);
    const long th = i / pairs_per_head;
    const int h = (int)(th % heads);
    const long t = th / heads;
    const int c = pp * 2;
    bf16* base = x + t * row_stride + (long)h * dim;
    const float2 lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + c));
    const float2 hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + c + half));
    const float2 c_lo = *reinterpret_cast<const float2*>(cos_t + t * dim + c);
    const float2 c_hi = *reinterpret_cast<const float2*>(cos_t + t * dim + c + half);
    const float2 s_lo = *reinterpret_cast<const float2*>(sin_t + t * dim + c);
    const float2 s_hi = *reinterpret_cast<const float2*>(sin_t + t * dim + c + half);
    float o_lo0, o_lo1, o_hi0, o_hi1;
    if (sign > 0.f) {
      // y_lo = x_lo*cos_lo - x_hi*sin_lo ; y_hi = x_hi*cos_hi + x_lo*sin_hi
      o_lo0 = lo.x * c_lo.x - hi.x * s_lo.x;
      o_lo1 = lo.y * c_lo.y - hi.y * s_lo.y;
      o_hi0 = hi.x * c_hi.x + lo.x * s_hi.x;
      o_hi1 = hi.y * c_hi.y + lo.y * s_hi.y;
    } else {
      // transpose: dx_lo = dy_lo*cos_lo + dy_hi*sin_hi ; dx_hi = dy_hi*cos_hi - dy_lo*sin_lo
      o_lo0 = lo.x * c_lo.x + hi.x * s_hi.x;
      o_lo1 = lo.y * c_lo.y + hi.y * s_hi.y;
      o_hi0 = hi.x * c_hi.x - lo.x * s_lo.x;
      o_hi1 = hi.y * c_hi.y - lo.y * s_lo.y;
    }
    *reinterpret_cast<uint32_t*>(base + c) = pack_bf16x2(o_lo0, o_lo1);
    *reinterpret_cast<uint32_t*>(base + c + half) = pack_bf16x2(o_hi0, o_hi1);
  }
}

// Same rotation with 16-byte accesses: a thread takes eight adjacent columns of the low half of a head and the
// matching eight of the high half (needs dim / 2 to be a multiple of 8).
__global__ void __launch_bounds__(256, 4) rope_vec8_kernel(bf16* __restrict__ x, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 long tokens, int heads, int dim, long row_stride, float sign) {
  const int half = dim >> 1;
  const int vecs = half >> 3;
  const long total = tokens * heads * vecs;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int vv = (int)(i % vecs);
    const long th = i / vecs;
    const int h = (int)(th % heads);
    const long t = th / heads;
    const int c = vv * 8;
    bf16* base = x + t * row_stride + (long)h * dim;
    float lo[8], hi[8], o_lo[8], o_hi[8];
    load8(base + c, lo);
    load8(base + c + half, hi);
    const float* cr = cos_t + t * dim;
    const float* sr = sin_t + t * dim;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const float4 c_lo = *reinterpret_cast<const float4*>(cr + c + 4 * q);
      const float4 c_hi = *reinterpret_cast<const float4*>(cr + c + half + 4 * q);
      const float4 s_lo = *reinterpret_cast<const float4*>(sr + c + 4 * q);
      const float4 s_hi = *reinterpret_cast<const float4*>(sr + c + half + 4 * q);
      const float cl[4] = {c_lo.x, c_lo.y, c_lo.z, c_lo.w}, ch[4] = {c_hi.x, c_hi.y, c_hi.z, c_hi.w};
      const float sl[4] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w}, sh[4] = {s_hi.x, s_hi.y, s_hi.z, s_hi.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k = 4 * q + j;
        if (sign > 0.f) {
          o_lo[k] = lo[k] * cl[j] - hi[k] * sl[j];
          o_hi[k] = hi[k] * ch[j] + lo[k] * sh[j];
        } else {
          o_lo[k] = lo[k] * cl[j] + hi[k] * sh[j];
          o_hi[k] = hi[k] * ch[j] - lo[k] * sl[j];
        }
      }
    }
    store8(base + c, o_lo);
    store8(base + c + half, o_hi);
  }
}

// ----------------------------------------------------------------------------
// SwiGLU on a fused [rows, 2*inter] gate|up buffer.
// ----------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long rows, int inter) {
  const int nvec = inter >> 3;
  const long total = rows * nvec;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / nvec;
    const int c = (int)(i % nvec) * 8;
    float g[8], u[8], o[8];
    load8(gu + r * 2 * inter + c, g);
    load8(gu + r * 2 * inter + inter + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = silu(g[j]) * u[j];
    store8(out + r * inter + c, o);
  }
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu, bf16* __restrict__ dgu,
                                  long rows, int inter) {
  const int nvec = inter >> 3;
  const long total = rows * nvec;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / nvec;
    const int c = (int)(i % nvec) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + r * 2 * inter + c, g);
    load8(gu + r * 2 * inter + inter + c, u);
    load8(dout + r * inter + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float sl = g[j] * sg;
      dg[j] = d[j] * u[j] * (sg + sl * (1.f - sg));
      du[j] = d[j] * sl;
    }
    store8(dgu + r * 2 * inter + c, dg);
    store8(dgu + r * 2 * inter + inter + c, du);
  }
}

__global__ void gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long n8) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_erf(v[j]);
    store8(y + i * 8, v);
  }
}
__global__ void gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx,
                                long n8) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float v[8], d[8];
    load8(x + i * 8, v);
    load8(dy + i * 8, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] *= gelu_erf_grad(v[j]);
    store8(dx + i * 8, d);
  }
}

// y = a + b (bf16), used for residual adds outside GEMM epilogues.
__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ y, long n8) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float u[8], v[8];
    load8(a + i * 8, u);
    load8(b + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] += v[j];
    store8(y + i * 8, u);
  }
}

// ----------------------------------------------------------------------------
// Row gather / scatter.  idx[r] < 0 (or outside [lo, hi)) gives a zero row on
// gather and is skipped on scatter.  One warp per row.
// ----------------------------------------------------------------------------
__global__ void gather_rows_kernel(const bf16* __restrict__ src, const long* __restrict__ idx, bf16* __restrict__ dst,
                                   long rows, int cols, long lo, long hi, long src_ld, long dst_ld) {
  const long r = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const long s = idx[r];
  const bool valid = s >= lo && s < hi;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int c = lane * 8; c < cols; c += 256) {
    uint4 v = valid ? *reinterpret_cast<const uint4*>(src + (s - lo) * src_ld + c) : zero;
    *reinterpret_cast<uint4*>(dst + r * dst_ld + c) = v;
  }
}

// dst[idx[r]] = src[r]   (add == 0)   or   dst[idx[r]] += src[r]  (add == 1, bf16x2 atomics)
__global__ void scatter_rows_kernel(const bf16* __restrict__ src, const long* __restrict__ idx, bf16* __restrict__ dst,
                                    long rows, int cols, long lo, long hi, long src_ld, long dst_ld, int add) {
  const long r = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const long d = idx[r];
  if (d < lo || d >= hi) return;
  if (!add) {
    for (int c = lane * 8; c < cols; c += 256)
      *reinterpret_cast<uint4*>(dst + (d - lo) * dst_ld + c) = *reinterpret_cast<const uint4*>(src + r * src_ld + c);
  } else {
    for (int c = lane * 2; c < cols; c += 64) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(src + r * src_ld + c);
      atomicAdd(reinterpret_cast<__nv_bfloat162*>(dst + (d - lo) * dst_ld + c), v);
    }
  }
}

// ----------------------------------------------------------------------------
// Column sums: out[c] (+)= sum_r x[r, c].  Stage 1 writes per-CTA partials.
// ----------------------------------------------------------------------------
__global__ void colsum_partial_kernel(const bf16* __restrict__ x, float* __restrict__ partial, long rows, int cols,
                                      long ld) {
  // blockDim = (32 column-vectors, 8 row lanes); grid = (ceil(cols/256), row splits)
  __shared__ float red[8][32][8];
  const int cv = blockIdx.x * 32 + threadIdx.x;
  const int c = cv * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < cols) {
    for (long r = blockIdx.y * 8 + threadIdx.y; r < rows; r += (long)gridDim.y * 8) {
      float v[8];
      load8(x + r * ld + c, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x][j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
      for (int k = 0; k < 8; ++k) s += red[k][threadIdx.x][j];
      partial[(long)blockIdx.y * cols + c + j] = s;
    }
  }
}

// ----------------------------------------------------------------------------
// Vocab-parallel cross-entropy.
// stats: per row, max over the local vocab shard, sum exp(l - max), and the target logit if the
// label falls into [vocab_lo, vocab_lo + V) (else 0).
// grad (in place): l <- (exp(l - gmax) / gsum - [label == col]) * scale for valid rows, 0 otherwise.
// ----------------------------------------------------------------------------
constexpr int kCeThreads = 512;

__global__ void __launch_bounds__(kCeThreads) ce_stats_kernel(const bf16* __restrict__ logits,
                                                             const long* __restrict__ labels, float* __restrict__ omax,
                                                             float* __restrict__ osum, float* __restrict__ otgt, int V,
                                                             long ld, long vocab_lo) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  const bf16* l = logits + row * ld;
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < nvec; c += kCeThreads) {
    float v[8];
    load8(l + c * 8, v);
    float lm = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, v[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(v[j] - m);
  }
  const float gm = block_max<kCeThreads>(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum<kCeThreads>(s, red);
  if (threadIdx.x == 0) {
    omax[row] = gm;
    osum[row] = s;
    const long lab = labels[row] - vocab_lo;
    otgt[row] = (lab >= 0 && lab < V) ? __bfloat162float(l[lab]) : 0.f;
  }
}

__global__ void __launch_bounds__(kCeThreads) ce_grad_kernel(bf16* __restrict__ logits, const long* __restrict__ labels,
                                                            const float* __restrict__ gmax,
                                                            const float* __restrict__ gsum,
                                                            const float* __restrict__ scale_ptr, int V, long ld,
                                                            long vocab_lo) {
  const long row = blockIdx.x;
  bf16* l = logits + row * ld;
  const int nvec = V >> 3;
  const long lab_g = labels[row];
  const bool valid = lab_g >= 0;
  const long lab = lab_g - vocab_lo;
  const float scale = valid ? *scale_ptr : 0.f;
  const float m = gmax[row];
  const float inv = valid ? 1.f / gsum[row] : 0.f;
  for (int c = threadIdx.x; c < nvec; c += kCeThreads) {
    float v[8];
    load8(l + c * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(v[j] - m) * inv;
      if ((long)(c * 8 + j) == lab) p -= 1.f;
      v[j] = p * scale;
    }
    store8(l + c * 8, v);
  }
}

// ----------------------------------------------------------------------------
// Fused AdamW (decoupled weight decay) over a flat shard.
//   g <- g * gscale;  m,v update;  master -= lr * (mhat / (sqrt(vhat) + eps) + wd * master);  p = bf16(master)
// Elements [0, n_decay) use `wd`, the rest 0.  gscale_ptr may be null (1.0).
// ----------------------------------------------------------------------------
__global__ void adamw_kernel(bf16* __restrict__ p, const bf16* __restrict__ g, float* __restrict__ master,
                             float* __restrict__ m, float* __restrict__ v, long n, long n_decay, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ gscale_ptr) {
  const float gs = gscale_ptr ? *gscale_ptr : 1.f;
  const long n8 = n >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long e = i * 8;
    float gv[8], out[8];
    load8(g + e, gv);
    float4 w0 = *reinterpret_cast<float4*>(master + e), w1 = *reinterpret_cast<float4*>(master + e + 4);
    float4 m0 = *reinterpret_cast<float4*>(m + e), m1 = *reinterpret_cast<float4*>(m + e + 4);
    float4 v0 = *reinterpret_cast<float4*>(v + e), v1 = *reinterpret_cast<float4*>(v + e + 4);
    float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = gv[j] * gs;
      mv[j] = b1 * mv[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      const float upd = (mv[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
      const float decay = (e + j < n_decay) ? wd : 0.f;
      wv[j] = wv[j] - lr * (upd + decay * wv[j]);
      out[j] = wv[j];
    }
    *reinterpret_cast<float4*>(master + e) = make_float4(wv[0], wv[1], wv[2], wv[3]);
    *reinterpret_cast<float4*>(master + e + 4) = make_float4(wv[4], wv[5], wv[6], wv[7]);
    *reinterpret_cast<float4*>(m + e) = make_float4(mv[0], mv[1], mv[2], mv[3]);
    *reinterpret_cast<float4*>(m + e + 4) = make_float4(mv[4], mv[5], mv[6], mv[7]);
    *reinterpret_cast<float4*>(v + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(v + e + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    store8(p + e, out);
  }
}

// AdamW with the states of an optimizer that runs directly on bf16 parameters (what torch.optim.AdamW does on a
// bf16 model, the reference's setting: python/ray/trainer.py:503-572): no fp32 master copy, moments in bf16.  The
// arithmetic of an element is fp32; weight, m and v are rounded to bf16 when stored.  14 bytes of traffic per
// parameter instead of 28.
__global__ void adamw_bf16_kernel(bf16* __restrict__ p, const bf16* __restrict__ g, bf16* __restrict__ m,
                                  bf16* __restrict__ v, long n, long n_decay, float lr, float b1, float b2, float eps,
                                  float wd, float bc1, float bc2, const float* __restrict__ gscale_ptr) {
  const float gs = gscale_ptr ? *gscale_ptr : 1.f;
  const long n8 = n >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long e = i * 8;
    float gv[8], wv[8], mv[8], vv[8];
    load8(g + e, gv);
    load8(p + e, wv);
    load8(m + e, mv);
    load8(v + e, vv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = gv[j] * gs;
      mv[j] = b1 * mv[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      const float upd = (mv[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
      const float decay = (e + j < n_decay) ? wd : 0.f;
      wv[j] = wv[j] - lr * (upd + decay * wv[j]);
    }
    store8(m + e, mv);
    store8(v + e, vv);
    store8(p + e, wv);
  }
}

// out[0] += sum(x^2)   (fp32 atomic; caller zeroes out)
__global__ void sumsq_kernel(const bf16* __restrict__ x, long n8, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j] * v[j];
  }
  s = block_sum<256>(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// coef = min(1, max_norm / (sqrt(normsq) + 1e-6)) * extra
__global__ void clip_coef_kernel(const float* __restrict__ normsq, float max_norm, float extra,
                                 float* __restrict__ coef) {
  const float n = sqrtf(*normsq);
  float c = max_norm > 0.f ? fminf(1.f, max_norm / (n + 1e-6f)) : 1.f;
  *coef = c * extra;
}

inline int grid_for(long work, int threads, int max_blocks) {
  long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<bf16*>(p)
#define CBF(p) reinterpret_cast<const bf16*>(p)

extern "C" {

int mmt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long rows, int cols, float eps, void* stream) {
  if (cols % 8 || cols > 8 * kNormThreads * kNormVec) return -2;
  if (rows == 0) return 0;
  const int vpl = (cols / 8 + 31) / 32;
  const unsigned grid8 = (unsigned)((rows + kNormThreads / 32 - 1) / (kNormThreads / 32));
  if (vpl <= 8) {
    rmsnorm_fwd_warp_kernel<8><<<grid8, kNormThreads, 0, ST(stream)>>>(CBF(x), CBF(w), BF(y), rstd, rows, cols, eps);
  } else if (vpl <= 16) {
    rmsnorm_fwd_warp_kernel<16><<<grid8, kNormThreads, 0, ST(stream)>>>(CBF(x), CBF(w), BF(y), rstd, rows, cols, eps);
  } else {
    rmsnorm_fwd_kernel<<<(unsigned)rows, kNormThreads, 0, ST(stream)>>>(CBF(x), CBF(w), BF(y), rstd, cols, eps);
  }
  return (int)cudaGetLastError();
}

// Number of per-CTA partial rows that mmt_rmsnorm_bwd writes; scratch must hold parts*cols floats.
int mmt_rmsnorm_bwd_parts(long rows) {
  const int cap = mmt_sm_count() * 2;
  return (int)(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

static void launch_reduce_partials(const float* scratch, void* out, int parts, int cols, int accumulate,
                                   void* stream) {
  reduce_partials_kernel<<<(cols + 31) / 32, dim3(32, 8), 0, ST(stream)>>>(scratch, BF(out), parts, cols, accumulate);
}

// Launches the backward kernel on at most `max_parts` CTAs; returns the number of partial rows it wrote.
static int launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* extra,
                              void* dx, float* scratch, long rows, int cols, int max_parts, void* stream) {
  const int vec = (cols / 8 + kNormThreads - 1) / kNormThreads;
  const int r = vec == 1 ? 4 : 2;
  long grid = (rows + r - 1) / r;
  if (grid > max_parts) grid = max_parts;
  if (grid < 1) grid = 1;
#define MMT_NORM_BWD(V, RR)                                                                                        \
  rmsnorm_bwd_kernel<V, RR><<<(unsigned)grid, kNormThreads, 0, ST(stream)>>>(CBF(dy), CBF(x), CBF(w), rstd, BF(dx), \
                                                                             scratch, (int)rows, cols, CBF(extra))
  switch (vec) {
    case 1: MMT_NORM_BWD(1, 4); break;
    case 2: MMT_NORM_BWD(2, 2); break;
    case 3: MMT_NORM_BWD(3, 2); break;
    default: MMT_NORM_BWD(4, 2); break;
  }
#undef MMT_NORM_BWD
  return (int)grid;
}

// dx and dw (bf16; accumulate_dw adds to the existing dw).  scratch: fp32 [parts, cols].
int mmt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                    float* scratch, long rows, int cols, int accumulate_dw, void* stream) {
  if (cols % 8 || cols > 8 * kNormThreads * kNormVec) return -2;
  if (rows < 0 || rows > 0x7fffffffL) return -5;      // the kernel indexes rows with 32-bit integers
  if (rows == 0) return 0;
  const int parts = launch_rmsnorm_bwd(dy, x, w, rstd, nullptr, dx, scratch, rows, cols, mmt_rmsnorm_bwd_parts(rows),
                                       stream);
  launch_reduce_partials(scratch, dw, parts, cols, accumulate_dw, stream);
  return (int)cudaGetLastError();
}

// As mmt_rmsnorm_bwd, with dx = (gradient through the norm) + extra: the pre-norm residual block's
// "gradient of the norm input plus gradient of the skip path" in one pass instead of a separate add.
int mmt_rmsnorm_bwd_add(const void* dy, const void* x, const void* w, const float* rstd, const void* extra, void* dx,
                        void* dw, float* scratch, long rows, int cols, int accumulate_dw, void* stream) {
  if (cols % 8 || cols > 8 * kNormThreads * kNormVec) return -2;
  if (rows < 0 || rows > 0x7fffffffL) return -5;      // the kernel indexes rows with 32-bit integers
  if (rows == 0) return 0;
  const int parts = launch_rmsnorm_bwd(dy, x, w, rstd, extra, dx, scratch, rows, cols, mmt_rmsnorm_bwd_parts(rows),
                                       stream);
  launch_reduce_partials(scratch, dw, parts, cols, accumulate_dw, stream);
  return (int)cudaGetLastError();
}

int mmt_rope(void* x, const float* cos_t, const float* sin_t, long tokens, int heads, int dim, long row_stride,
             int backward, void* stream) {
  if (dim % 4) return -2;
  const long work = tokens * heads * (dim / 4);
  if (work == 0) return 0;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(cos_t) |
                         reinterpret_cast<uintptr_t>(sin_t)) & 15) == 0;
  if (dim % 16 == 0 && row_stride % 8 == 0 && aligned) {
    const long work8 = tokens * heads * (dim / 16);
    rope_vec8_kernel<<<grid_for(work8, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(
        BF(x), cos_t, sin_t, tokens, heads, dim, row_stride, backward ? -1.f : 1.f);
    return (int)cudaGetLastError();
  }
  rope_kernel<<<grid_for(work, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(BF(x), cos_t, sin_t, tokens, heads, dim,
                                                                              row_stride, backward ? -1.f : 1.f);
  return (int)cudaGetLastError();
}

int mmt_swiglu_fwd(const void* gu, void* out, long rows, int inter, void* stream) {
  if (inter % 8) return -2;
  const long work = rows * (inter / 8);
  if (work == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(work, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(CBF(gu), BF(out), rows, inter);
  return (int)cudaGetLastError();
}
int mmt_swiglu_bwd(const void* dout, const void* gu, void* dgu, long rows, int inter, void* stream) {
  if (inter % 8) return -2;
  const long work = rows * (inter / 8);
  if (work == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(work, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(CBF(dout), CBF(gu), BF(dgu), rows,
                                                                                    inter);
  return (int)cudaGetLastError();
}
int mmt_gelu_fwd(const void* x, void* y, long n, void* stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  gelu_fwd_kernel<<<grid_for(n / 8, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(CBF(x), BF(y), n / 8);
  return (int)cudaGetLastError();
}
int mmt_gelu_bwd(const void* dy, const void* x, void* dx, long n, void* stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  gelu_bwd_kernel<<<grid_for(n / 8, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(CBF(dy), CBF(x), BF(dx), n / 8);
  return (int)cudaGetLastError();
}
int mmt_add(const void* a, const void* b, void* y, long n, void* stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  add_kernel<<<grid_for(n / 8, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(CBF(a), CBF(b), BF(y), n / 8);
  return (int)cudaGetLastError();
}

int mmt_gather_rows(const void* src, const long* idx, void* dst, long rows, int cols, long lo, long hi, long src_ld,
                    long dst_ld, void* stream) {
  if (cols % 8 || src_ld % 8 || dst_ld % 8) return -2;
  if (rows == 0) return 0;
  gather_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ST(stream)>>>(CBF(src), idx, BF(dst), rows, cols, lo, hi,
                                                                        src_ld, dst_ld);
  return (int)cudaGetLastError();
}
int mmt_scatter_rows(const void* src, const long* idx, void* dst, long rows, int cols, long lo, long hi, long src_ld,
                     long dst_ld, int add, void* stream) {
  if (cols % 8 || src_ld % 8 || dst_ld % 8) return -2;
  if (rows == 0) return 0;
  scatter_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ST(stream)>>>(CBF(src), idx, BF(dst), rows, cols, lo, hi,
                                                                         src_ld, dst_ld, add);
  return (int)cudaGetLastError();
}

int mmt_colsum_parts(long rows) {
  long p = (rows + 63) / 64;
  const int cap = 64;
  return (int)(p < 1 ? 1 : (p > cap ? cap : p));
}
// out[c] (+)= sum_r x[r,c]; scratch fp32 [parts, cols].
int mmt_colsum(const void* x, void* out, float* scratch, long rows, int cols, long ld, int accumulate, void* stream) {
  if (cols % 8 || ld % 8) return -2;
  const int parts = mmt_colsum_parts(rows);
  dim3 grid((cols + 255) / 256, parts), block(32, 8);
  colsum_partial_kernel<<<grid, block, 0, ST(stream)>>>(CBF(x), scratch, rows, cols, ld);
  launch_reduce_partials(scratch, out, parts, cols, accumulate, stream);
  return (int)cudaGetLastError();
}

int mmt_ce_stats(const void* logits, const long* labels, float* omax, float* osum, float* otgt, long rows, int V,
                 long ld, long vocab_lo, void* stream) {
  if (V % 8 || ld % 8) return -2;
  if (rows == 0) return 0;
  ce_stats_kernel<<<(unsigned)rows, kCeThreads, 0, ST(stream)>>>(CBF(logits), labels, omax, osum, otgt, V, ld,
                                                                vocab_lo);
  return (int)cudaGetLastError();
}
int mmt_ce_grad(void* logits, const long* labels, const float* gmax, const float* gsum, const float* scale_ptr,
                long rows, int V, long ld, long vocab_lo, void* stream) {
  if (V % 8 || ld % 8) return -2;
  if (rows == 0) return 0;
  ce_grad_kernel<<<(unsigned)rows, kCeThreads, 0, ST(stream)>>>(BF(logits), labels, gmax, gsum, scale_ptr, V, ld,
                                                               vocab_lo);
  return (int)cudaGetLastError();
}

int mmt_adamw(void* p, const void* g, float* master, float* m, float* v, long n, long n_decay, float lr, float b1,
              float b2, float eps, float wd, int step, const float* gscale_ptr, void* stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamw_kernel<<<grid_for(n / 8, 256, mmt_sm_count() * 16), 256, 0, ST(stream)>>>(
      BF(p), CBF(g), master, m, v, n, n_decay, lr, b1, b2, eps, wd, bc1, bc2, gscale_ptr);
  return (int)cudaGetLastError();
}

// AdamW on bf16 parameters with bf16 moments and no master copy (see adamw_bf16_kernel).
int mmt_adamw_bf16(void* p, const void* g, void* m, void* v, long n, long n_decay, float lr, float b1, float b2,
                   float eps, float wd, int step, const float* gscale_ptr, void* stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamw_bf16_kernel<<<grid_for(n / 8, 256, mmt_sm_count() * 16), 256, 0, ST(stream)>>>(
      BF(p), CBF(g), BF(m), BF(v), n, n_decay, lr, b1, b2, eps, wd, bc1, bc2, gscale_ptr);
  return (int)cudaGetLastError();
}

int mmt_sumsq(const void* x, long n, float* out, void* stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  sumsq_kernel<<<grid_for(n / 8, 256, mmt_sm_count() * 8), 256, 0, ST(stream)>>>(CBF(x), n / 8, out);
  return (int)cudaGetLastError();
}
int mmt_clip_coef(const float* normsq, float max_norm, float extra, float* coef, void* stream) {
  clip_coef_kernel<<<1, 1, 0, ST(stream)>>>(normsq, max_norm, extra, coef);
  return (int)cudaGetLastError();
}

}  // extern "C"

// ----------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared and documented in noalloc.h).
// ----------------------------------------------------------------------------
namespace {
// Scratch for the per-CTA partial sums of dw.  In host code this name is only a stand-in for the
// symbol: kernels must be given the device address obtained with cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[MMT_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (resolved once per device).
float* noalloc_scratch_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_noalloc_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "mmt_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return nullptr;
    }
    g_noalloc_ptr[dev] = ptr;
  }
  return g_noalloc_ptr[dev];
}
}  // namespace

extern "C" int mmt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                       void* dw, long rows, int cols, int accumulate_dw, void* stream) {
  if (cols % 8) return -2;
  if (cols <= 0 || cols > MMT_NOALLOC_MAX_COLS || rows < 0 || rows > 0x7fffffffL) {
    fprintf(stderr,
            "mmt_rmsnorm_bwd_noalloc: size [%ld, %d] is outside the built-in scratch's limits (cols <= %d, "
            "rows < 2^31)\n", rows, cols, MMT_NOALLOC_MAX_COLS);
    return -5;
  }
  if (rows == 0) return 0;
  float* scratch = noalloc_scratch_ptr();
  if (scratch == nullptr) return -6;
  // as many per-CTA partial rows as the regular entry point would use, capped by the scratch size
  int parts = mmt_rmsnorm_bwd_parts(rows);
  const int cap = MMT_NOALLOC_SCRATCH_FLOATS / cols;
  if (parts > cap) parts = cap;
  parts = launch_rmsnorm_bwd(dy, x, w, rstd, nullptr, dx, scratch, rows, cols, parts, stream);
  launch_reduce_partials(scratch, dw, parts, cols, accumulate_dw, stream);
  return (int)cudaGetLastError();
}
