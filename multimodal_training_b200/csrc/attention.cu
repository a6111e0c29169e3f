// Packed variable-length flash attention on tcgen05 (sm_100a), forward and backward.
//
// Layout.  One fused activation buffer qkv[T, ld] (bf16): q heads, then k heads, then v heads,
// `dim` columns each (dim = 80 for the vision encoder, 128 for the text decoder).  Sequences are
// packed along T; per-token arrays seq_lo[t], seq_hi[t] give the row range of the token's own
// sequence, which expresses window attention, whole-image attention and packed causal text with
// one mechanism: a query tile of 128 consecutive rows may span several (short) sequences and the
// mask keeps every row inside its own.  GQA: q head h reads kv head h / (n_q / n_kv).
//
// Forward, one CTA per (128-row query tile, q head), 6 warps:
//   warps 0-3  softmax: thread i owns query row i (tensor-memory lane i); two passes over the
//              128 scores of a KV tile held in tensor memory (row max, then exp2 / sum / bf16 P
//              written to swizzled shared memory); output accumulator in registers
//   warp 4     TMA producer: Q once, K and V tiles through 2-stage rings
//   warp 5     MMA issuer: S = Q K^T (both operands K-major in shared memory) into a
//              double-buffered tensor-memory tile, then PV = P V (V is the MN-major operand)
// head_dim 80 is not a multiple of the 64-column swizzle atom: every operand tile is fetched as two
// 64-column boxes (columns 0-63 and 64-127 of the head; the tail of the second box belongs to the
// next head or is zero fill and is never read).  As a K-major operand the fifth K=16 step reads the
// first 16 columns of the second box; as an MN-major operand N=80 covers box 0 and a quarter of
// box 1.  So there are no padded FLOPs and a single swizzle mode.
//
// Backward is two kernels without atomics: dK/dV (one CTA per KV tile, looping over the query
// tiles and the q heads of the group, accumulating in tensor memory) and dQ (one CTA per query
// tile, looping over KV tiles).  Both recompute P from the saved log-sum-exp.
//
// Replaces flash-attn's flash_attn_varlen_func reached through HF in the reference
// (python/models/qwen2_5_vl/modeling_qwen2_5_vl.py:431-448,540-557,694-711,1266-1281).
#include "attention_common.cuh"

namespace {
using namespace attn;

template <int DIM>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                         // 2 boxes
  uint8_t* sK = sQ + 2 * CHUNK;               // 2 stages x 2 boxes
  uint8_t* sV = sK + 4 * CHUNK;               // 2 stages x 2 boxes
  uint8_t* sP = sV + 4 * CHUNK;               // 2 boxes
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * CHUNK);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* s_empty = bars + 11;    // 2
  uint64_t* p_full = bars + 13;     // 1
  uint64_t* pv_full = bars + 14;    // 1
  uint64_t* o_empty = bars + 15;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ;
  const int head = blockIdx.y;
  const int kv_head = head / (p.n_q / p.n_kv);
  const int q_last = min(q0 + BQ, p.T) - 1;
  const int kv_lo = p.seq_lo[q0];
  const int kv_hi = p.causal ? min(p.seq_hi[q_last], q_last + 1) : p.seq_hi[q_last];
  const int n_tiles = (kv_hi - kv_lo + BKV - 1) / BKV;
  const int xq = head * DIM, xk = (p.n_q + kv_head) * DIM, xv = (p.n_q + p.n_kv + kv_head) * DIM;
  constexpr int X2 = 64;  // column offset of the second box of a tile

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_full, 1);
    mbar_init(o_empty, 4);
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_pv = tmem_base + 256;

  if (warp == 4) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * CHUNK);
      tma_load_2d(sQ, &tm, q_full, xq, q0);
      tma_load_2d(sQ + CHUNK, &tm, q_full, xq + X2, q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int r0 = kv_lo + j * BKV;
        if (!mbar_wait(&k_empty[s], ph ^ 1, p.ew, 400)) break;
        mbar_expect_tx(&k_full[s], 2 * CHUNK);
        tma_load_2d(sK + s * 2 * CHUNK, &tm, &k_full[s], xk, r0);
        tma_load_2d(sK + s * 2 * CHUNK + CHUNK, &tm, &k_full[s], xk + X2, r0);
        if (!mbar_wait(&v_empty[s], ph ^ 1, p.ew, 401)) break;
        mbar_expect_tx(&v_full[s], 2 * CHUNK);
        tma_load_2d(sV + s * 2 * CHUNK, &tm, &v_full[s], xv, r0);
        tma_load_2d(sV + s * 2 * CHUNK + CHUNK, &tm, &v_full[s], xv + 64, r0);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BQ, DIM, 0, 1);
      const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, p.ew, 500);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph, p.ew, 501)) return false;
        if (!mbar_wait(&s_empty[s], ph ^ 1, p.ew, 502)) return false;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sK + s * 2 * CHUNK);
#pragma unroll
        for (int k = 0; k < DIM / 16; ++k) {
          tc_mma_ss(tmem_base + s * 128, make_smem_desc(kmajor_kstep_addr(q_base, k), 16, 1024),
                    make_smem_desc(kmajor_kstep_addr(k_base, k), 16, 1024), idesc_s, k != 0);
        }
        tc_commit(&s_full[s]);
        tc_commit(&k_empty[s]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_tiles) {
          if (!issue_s(j + 1)) break;
        }
        if (!mbar_wait(&v_full[s], ph, p.ew, 503)) break;
        if (!mbar_wait(p_full, j & 1, p.ew, 504)) break;
        if (!mbar_wait(o_empty, (j & 1) ^ 1, p.ew, 505)) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(sV + s * 2 * CHUNK);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          tc_mma_ss(tmem_pv, make_smem_desc(p_base + (k >> 2) * CHUNK + (k & 3) * 32, 16, 1024),
                    make_smem_desc(v_base + k * 2048, CHUNK, 1024), idesc_pv, k != 0);
        }
        tc_commit(pv_full);
        tc_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------------
    const int row = warp * 32 + lane;
    const int qrow = q0 + row;
    const bool row_ok = qrow < p.T;
    const int lo = row_ok ? p.seq_lo[qrow] : 0;
    int hi = row_ok ? p.seq_hi[qrow] : 0;
    if (p.causal) hi = min(hi, qrow + 1);
    const float sl2 = p.scale * LOG2E;
    const uint32_t lane_addr = ((uint32_t)(warp * 32) << 16);
    float m = -INFINITY, l = 0.f;
    float o[DIM];
#pragma unroll
    for (int i = 0; i < DIM; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int kv0 = kv_lo + j * BKV;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], ph, p.ew, 600));
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_addr + s * 128;
      // pass 1: row maximum over the valid columns
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + c * 32 + i;
          if (kv >= lo && kv < hi) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f((m - m_use) * sl2);
      // P of the previous tile must have been consumed before it is overwritten: pv_full(j-1) was
      // awaited at the end of the previous iteration.
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int kv = kv0 + c * 32 + i;
          float p0 = (kv >= lo && kv < hi) ? exp2f((__uint_as_float(r[i]) - m_use) * sl2) : 0.f;
          float p1 = (kv + 1 >= lo && kv + 1 < hi) ? exp2f((__uint_as_float(r[i + 1]) - m_use) * sl2) : 0.f;
          // sum what the tensor core will see (bf16-rounded), so that O / l is consistent
          const uint32_t u = pack_bf16x2(p0, p1);
          const float2 f = unpack_bf16x2(u);
          sum += f.x + f.y;
          pk[i >> 1] = u;
        }
        uint8_t* dst = sP + (c >> 1) * CHUNK;
        const int col0 = (c & 1) * 32;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          *reinterpret_cast<uint4*>(dst + sw128_offset(row, col0 + g * 8)) =
              make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
        }
      }
      l = l * alpha + sum;
      m = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[s]);
        mbar_arrive(p_full);
      }
      ok = __all_sync(0xffffffffu, mbar_wait(pv_full, j & 1, p.ew, 601));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DIM / 16; ++c) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(tmem_pv + lane_addr + c * 16, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) o[c * 16 + i] = o[c * 16 + i] * alpha + __uint_as_float(r[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_empty);
    }
    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (long)qrow * (p.n_q * DIM) + head * DIM;
#pragma unroll
      for (int c = 0; c < DIM; c += 8) {
        uint4 v;
        v.x = pack_bf16x2(o[c] * inv, o[c + 1] * inv);
        v.y = pack_bf16x2(o[c + 2] * inv, o[c + 3] * inv);
        v.z = pack_bf16x2(o[c + 4] * inv, o[c + 5] * inv);
        v.w = pack_bf16x2(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = v;
      }
      p.lse[(long)head * p.T + qrow] = l > 0.f ? m * p.scale + logf(l) : INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, 512);
}

constexpr size_t kFwdSmem = 1024 + 12 * CHUNK + 17 * 8 + 16;

template <int DIM>
int launch_fwd(const CUtensorMap& tm, const AttnParams& p, cudaStream_t st) {
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kFwdSmem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  dim3 grid((p.T + BQ - 1) / BQ, p.n_q);
  attn_fwd_kernel<DIM><<<grid, kThreads, kFwdSmem, st>>>(tm, p);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" int mmt_attn_fwd(const void* qkv, void* out, float* lse, const int* seq_lo, const int* seq_hi, long T,
                            int n_q, int n_kv, int dim, long ld, int causal, float scale, void* stream) {
  if (T <= 0) return 0;
  if (mmt_ensure_context(qkv)) return -7;
  if ((dim != 80 && dim != 128) || n_q % n_kv || (ld & 7)) return -2;
  CUtensorMap tm;
  const uint64_t width = (uint64_t)(n_q + 2 * n_kv) * dim;
  int r = mmt_make_tmap_2d(&tm, qkv, width, (uint64_t)T, (uint64_t)ld, 64, 128);
  if (r) return 1000 + r;
  AttnParams p;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.seq_lo = seq_lo;
  p.seq_hi = seq_hi;
  p.T = (int)T; p.n_q = n_q; p.n_kv = n_kv; p.dim = dim; p.ld = ld;
  p.causal = causal; p.scale = scale;
  p.ew = mmt_error_word();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dim == 80 ? launch_fwd<80>(tm, p, st) : launch_fwd<128>(tm, p, st);
}
