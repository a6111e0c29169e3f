// Packed variable-length flash attention on tcgen05 (sm_100a), forward and backward.
//
// Layout.  One fused activation buffer qkv[T, ld] (bf16): q heads, then k heads, then v heads,
// `dim` columns each (dim = 80 for the vision encoder, 128 for the text decoder).  Sequences are
// packed along T; per-token arrays seq_lo[t], seq_hi[t] give the row range of the token's own
// sequence, which expresses window attention, whole-image attention and packed causal text with
// one mechanism: a query tile of 128 consecutive rows may span several (short) sequences and the
// mask keeps every row inside its own.  GQA: q head h reads kv head h / (n_q / n_kv).
//
// Forward: one CTA per pair of (128-row query tile, q head) items, 10 warps (two softmax warp groups, a TMA
// producer, an MMA issuer); see the comment at attn_fwd2_kernel.
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

// ------------------------------------------------------------------------------------------------
// Forward: two (query tile, head) items per CTA worked in ping-pong.
//
// With one item per CTA the four softmax warps are the limit: while they convert S of tile j the tensor core
// idles.  Here a CTA owns two items, each with its own
// softmax warp group (4 warps, one query row per thread), its own K and V buffers and its own tensor-memory
// columns, while ONE TMA warp and ONE MMA warp serve both, so the tensor core computes S or PV of one item
// while the other item's rows are in the exponentials.
//   * P never touches shared memory: the softmax threads write it as packed bf16 pairs over the first 64
//     columns of the S tile they have just read (tcgen05.st), and PV takes it as the tensor-memory A operand.
//   * O stays in tensor memory for the whole KV loop (PV accumulates).  The running maximum is lazy: O and l
//     are rescaled only when a row's maximum grew by more than 2^8 since the value in use, which after the
//     first tiles is rare; the rescale is a tensor-memory read-modify-write by the row's own thread, safe
//     because S of tile j is only published after PV of tile j-1 has completed.
//   * KV tiles that are entirely visible to every row of a warp skip the per-element mask.
// Tensor memory: S/P of item w at columns [128w, 128w+128), O of item w at [256+128w, 256+128w+DIM).
// Shared memory: Q, K, V of each item, 32 KB each (two 64-column boxes).
// ------------------------------------------------------------------------------------------------
constexpr int kFwd2Threads = 320;

template <int DIM>
__global__ void __launch_bounds__(kFwd2Threads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p, const int n_items) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                         // [item][2 boxes]
  uint8_t* sK = sQ + 4 * CHUNK;
  uint8_t* sV = sK + 4 * CHUNK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 4 * CHUNK);
  uint64_t* q_full = bars;          // [2]
  uint64_t* k_full = bars + 2;      // [2]
  uint64_t* k_empty = bars + 4;     // [2]
  uint64_t* v_full = bars + 6;      // [2]
  uint64_t* v_empty = bars + 8;     // [2]
  uint64_t* s_full = bars + 10;     // [2]
  uint64_t* p_full = bars + 12;     // [2]
  uint64_t* pv_done = bars + 14;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int X2 = 64;
  // the two items of this CTA: heads fastest, so both usually share the query rows (and, with GQA, K and V)
  int q0[2], head[2], kv_lo[2], n_tiles[2], xq[2], xk[2], xv[2];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    // causal: the last query tiles see the most KV tiles, so they are started first (longest work first)
    const int cta = p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    const int item = cta * 2 + w;
    n_tiles[w] = 0;
    q0[w] = head[w] = kv_lo[w] = xq[w] = xk[w] = xv[w] = 0;
    if (item < n_items) {
      head[w] = item % p.n_q;
      q0[w] = (item / p.n_q) * BQ;
      const int kv_head = head[w] / (p.n_q / p.n_kv);
      const int q_last = min(q0[w] + BQ, p.T) - 1;
      kv_lo[w] = p.seq_lo[q0[w]];
      const int kv_hi = p.causal ? min(p.seq_hi[q_last], q_last + 1) : p.seq_hi[q_last];
      n_tiles[w] = (kv_hi - kv_lo[w] + BKV - 1) / BKV;
      xq[w] = head[w] * DIM;
      xk[w] = (p.n_q + kv_head) * DIM;
      xv[w] = (p.n_q + p.n_kv + kv_head) * DIM;
    }
  }
  const int max_tiles = max(n_tiles[0], n_tiles[1]);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      bool ok = true;
      for (int w = 0; w < 2; ++w) {
        if (n_tiles[w] == 0) continue;
        mbar_expect_tx(&q_full[w], 2 * CHUNK);
        tma_load_2d(sQ + w * 2 * CHUNK, &tm, &q_full[w], xq[w], q0[w]);
        tma_load_2d(sQ + w * 2 * CHUNK + CHUNK, &tm, &q_full[w], xq[w] + X2, q0[w]);
      }
      for (int j = 0; j < max_tiles && ok; ++j) {
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= n_tiles[w]) continue;
          if (j > 0 && !mbar_wait(&k_empty[w], (j - 1) & 1, p.ew, 410)) { ok = false; break; }
          const int r0 = kv_lo[w] + j * BKV;
          mbar_expect_tx(&k_full[w], 2 * CHUNK);
          tma_load_2d(sK + w * 2 * CHUNK, &tm, &k_full[w], xk[w], r0);
          tma_load_2d(sK + w * 2 * CHUNK + CHUNK, &tm, &k_full[w], xk[w] + X2, r0);
        }
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= n_tiles[w]) continue;
          if (j > 0 && !mbar_wait(&v_empty[w], (j - 1) & 1, p.ew, 411)) { ok = false; break; }
          const int r0 = kv_lo[w] + j * BKV;
          mbar_expect_tx(&v_full[w], 2 * CHUNK);
          tma_load_2d(sV + w * 2 * CHUNK, &tm, &v_full[w], xv[w], r0);
          tma_load_2d(sV + w * 2 * CHUNK + CHUNK, &tm, &v_full[w], xv[w] + X2, r0);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BQ, DIM, 0, 1);
      const uint32_t hi_k = smem_desc_hi(1024), hi_v = smem_desc_hi(1024);
      uint32_t q_lo[2], k_lo[2], v_lo[2];
      for (int w = 0; w < 2; ++w) {
        q_lo[w] = smem_desc_lo(smem_u32(sQ + w * 2 * CHUNK), 16);
        k_lo[w] = smem_desc_lo(smem_u32(sK + w * 2 * CHUNK), 16);
        v_lo[w] = smem_desc_lo(smem_u32(sV + w * 2 * CHUNK), CHUNK);
      }
      auto issue_s = [&](int w) {
        const uint32_t d = tmem_base + (uint32_t)(w * 128);
#pragma unroll
        for (int k = 0; k < DIM / 16; ++k) {
          const uint32_t off = (uint32_t)(((k >> 2) * CHUNK + (k & 3) * 32) >> 4);
          tc_mma_ss(d, smem_desc_join(hi_k, q_lo[w] + off), smem_desc_join(hi_k, k_lo[w] + off), idesc_s, k != 0);
        }
        tc_commit(&s_full[w]);
        tc_commit(&k_empty[w]);
      };
      bool ok = true;
      for (int w = 0; w < 2 && ok; ++w) {
        if (n_tiles[w] == 0) continue;
        ok = mbar_wait(&q_full[w], 0, p.ew, 510) && mbar_wait(&k_full[w], 0, p.ew, 511);
        if (ok) issue_s(w);
      }
      for (int j = 0; j < max_tiles && ok; ++j) {
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= n_tiles[w]) continue;
          if (!mbar_wait(&p_full[w], j & 1, p.ew, 512) || !mbar_wait(&v_full[w], j & 1, p.ew, 513)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + 256u + (uint32_t)(w * 128);
          const uint32_t a = tmem_base + (uint32_t)(w * 128);
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            tc_mma_ts(d, a + (uint32_t)(k * 8), smem_desc_join(hi_v, v_lo[w] + (uint32_t)(k * (2048 >> 4))), idesc_pv,
                      (j | k) != 0);
          }
          tc_commit(&v_empty[w]);
          if (j == n_tiles[w] - 1) tc_commit(&pv_done[w]);
          if (j + 1 < n_tiles[w]) {
            if (!mbar_wait(&k_full[w], (j + 1) & 1, p.ew, 514)) { ok = false; break; }
            issue_s(w);
          }
        }
      }
    }
  } else {
    // ------------------------------ softmax + epilogue, one warp group per item ------------------------------
    const int w = warp >> 2;             // item
    const int q = warp & 3;              // tensor-memory lane quadrant of this warp
    if (n_tiles[w] > 0) {
      const int row = q * 32 + lane;
      const int qrow = q0[w] + row;
      const bool row_ok = qrow < p.T;
      const int lo = row_ok ? p.seq_lo[qrow] : 0;
      int hi = row_ok ? p.seq_hi[qrow] : 0;
      if (p.causal) hi = min(hi, qrow + 1);
      const float sl2 = p.scale * LOG2E;
      const uint32_t lane_addr = ((uint32_t)(q * 32) << 16);
      const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)(w * 128);
      const uint32_t o_addr = tmem_base + lane_addr + 256u + (uint32_t)(w * 128);
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j < n_tiles[w]; ++j) {
        const int kv0 = kv_lo[w] + j * BKV;
        ok = __all_sync(0xffffffffu, mbar_wait(&s_full[w], j & 1, p.ew, 610));
        if (!ok) break;
        tc_fence_after();
        const bool full = __all_sync(0xffffffffu, kv0 >= lo && kv0 + BKV <= hi);
        // pass 1: row maximum over the visible columns
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(s_addr + c * 32, r);
          tmem_wait_ld();
          if (full) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kv = kv0 + c * 32 + i;
              if (kv >= lo && kv < hi) mx = fmaxf(mx, __uint_as_float(r[i]));
            }
          }
        }
        // lazy running maximum: adopt a new reference only when it moved by more than 2^8
        const float m_new = fmaxf(m_ref, mx);
        const bool need = (m_new - m_ref) * sl2 > 8.f;        // false when both are -inf (NaN compares false)
        if (j == 0) {
          if (need) m_ref = m_new;                             // O does not exist yet: nothing to rescale
        } else if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? exp2f((m_ref - m_new) * sl2) : 1.f;   // exp2(-inf) = 0 for a row without history
          l *= alpha;
          if (need) m_ref = m_new;
#pragma unroll
          for (int c = 0; c < DIM / 16; ++c) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(o_addr + c * 16, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x16(o_addr + c * 16, r);
          }
          tmem_wait_st();
        }
        const float bias = (m_ref == -INFINITY) ? 0.f : -m_ref * sl2;
        // pass 2: P = exp2(S * sl2 + bias) as bf16 pairs, written over the columns of S already consumed
        float sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(s_addr + c * 32, r);
          tmem_wait_ld();
          uint32_t pk[16];
          if (full) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = exp2f(fmaf(__uint_as_float(r[i]), sl2, bias));
              const float p1 = exp2f(fmaf(__uint_as_float(r[i + 1]), sl2, bias));
              sum += p0 + p1;
              pk[i >> 1] = pack_bf16x2(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int kv = kv0 + c * 32 + i;
              const float p0 = (kv >= lo && kv < hi) ? exp2f(fmaf(__uint_as_float(r[i]), sl2, bias)) : 0.f;
              const float p1 = (kv + 1 >= lo && kv + 1 < hi) ? exp2f(fmaf(__uint_as_float(r[i + 1]), sl2, bias)) : 0.f;
              sum += p0 + p1;
              pk[i >> 1] = pack_bf16x2(p0, p1);
            }
          }
          tmem_st_32x32b_x16(s_addr + c * 16, pk);
        }
        l += sum;
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[w]);
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[w], 0, p.ew, 611));
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + (long)qrow * (p.n_q * DIM) + head[w] * DIM;
#pragma unroll
        for (int c = 0; c < DIM / 16; ++c) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(o_addr + c * 16, r);
          tmem_wait_ld();
          if (row_ok) {
            uint4 v0, v1;
            v0.x = pack_bf16x2(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
            v0.y = pack_bf16x2(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
            v0.z = pack_bf16x2(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
            v0.w = pack_bf16x2(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
            v1.x = pack_bf16x2(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
            v1.y = pack_bf16x2(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
            v1.z = pack_bf16x2(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
            v1.w = pack_bf16x2(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 16) = v0;
            *reinterpret_cast<uint4*>(dst + c * 16 + 8) = v1;
          }
        }
        if (row_ok) p.lse[(long)head[w] * p.T + qrow] = l > 0.f ? m_ref * p.scale + logf(l) : INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

constexpr size_t kFwdSmem = 1024 + 12 * CHUNK + 17 * 8 + 16;

template <int DIM>
int launch_fwd2(const CUtensorMap& tm, const AttnParams& p, cudaStream_t st) {
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kFwdSmem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const int n_items = ((p.T + BQ - 1) / BQ) * p.n_q;
  attn_fwd2_kernel<DIM><<<(n_items + 1) / 2, kFwd2Threads, kFwdSmem, st>>>(tm, p, n_items);
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
  return dim == 80 ? launch_fwd2<80>(tm, p, st) : launch_fwd2<128>(tm, p, st);
}
