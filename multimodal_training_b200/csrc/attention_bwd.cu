// Backward of the packed variable-length flash attention (see attention.cu for the layout).
//
// Three launches, no atomics, deterministic:
//   1. delta[h, t] = sum_d out[t,h,d] * dout[t,h,d]
//   2. dK/dV: one CTA per (128-row KV tile, kv head), looping over the q heads of the GQA group and over blocks
//      of 64 queries that can see the KV tile; transposed scores S^T = K Q^T and dP^T = V dO^T in tensor memory,
//      P^T and dS^T written back over them as packed bf16 and used as tensor-memory A operands of
//      dV += P^T dO and dK += dS^T Q, whose accumulators stay in tensor memory across the whole loop
//   3. dQ: one CTA per (128-row query tile, q head), looping over KV tiles with the same pipeline
//      (dQ += dS K, dS as a tensor-memory operand)
// P = exp(S * scale - lse) and dS = P * (dP - delta) * scale are recomputed from the saved log-sum-exp.
// Every tile is fetched as 64-column TMA boxes that serve as K-major or MN-major operands, so Q, K, V and dO
// need no transposes.  Details at the kernels.
#include "attention_common.cuh"

namespace {
using namespace attn;

// ----------------------------------------------------------------------------------------------
// 1. delta
// ----------------------------------------------------------------------------------------------
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int T, int n_q, int dim) {
  const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long)T * n_q) return;
  const long t = w / n_q;
  const int h = (int)(w % n_q);
  const __nv_bfloat16* o = out + t * (long)(n_q * dim) + h * dim;
  const __nv_bfloat16* d = dout + t * (long)(n_q * dim) + h * dim;
  float s = 0.f;
  for (int c = lane * 2; c < dim; c += 64) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o + c));
    const float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(d + c));
    s += a.x * b.x + a.y * b.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(long)h * T + t] = s;
}

// P and dS of one 32-column chunk for query row `qrow` (lo <= kv < hi is the row's visible range).
// r_s / r_dp hold raw S and dP; on return pk_p / pk_ds hold the bf16 pairs.
MMT_DEVICE void p_ds_chunk(const uint32_t (&r_s)[32], const uint32_t (&r_dp)[32], int kv_base, int lo, int hi,
                           float sl2, float lse_l2, float delta, float scale, uint32_t (&pk_p)[16],
                           uint32_t (&pk_ds)[16]) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const int kv = kv_base + i;
    const float p0 = (kv >= lo && kv < hi) ? exp2f(__uint_as_float(r_s[i]) * sl2 - lse_l2) : 0.f;
    const float p1 = (kv + 1 >= lo && kv + 1 < hi) ? exp2f(__uint_as_float(r_s[i + 1]) * sl2 - lse_l2) : 0.f;
    const float d0 = p0 * (__uint_as_float(r_dp[i]) - delta) * scale;
    const float d1 = p1 * (__uint_as_float(r_dp[i + 1]) - delta) * scale;
    pk_p[i >> 1] = pack_bf16x2(p0, p1);
    pk_ds[i >> 1] = pack_bf16x2(d0, d1);
  }
}

MMT_DEVICE void store_chunk(uint8_t* tile, int row, int c, const uint32_t (&pk)[16]) {
  uint8_t* dst = tile + (c >> 1) * CHUNK;
  const int col0 = (c & 1) * 32;
#pragma unroll
  for (int g = 0; g < 4; ++g)
    *reinterpret_cast<uint4*>(dst + sw128_offset(row, col0 + g * 8)) =
        make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
}

// dK / dV of a GQA group = sum of its q heads' fp32 partials, in head order (deterministic), rounded once.
__global__ void attn_group_reduce_kernel(const float* __restrict__ ws_dk, const float* __restrict__ ws_dv,
                                         __nv_bfloat16* __restrict__ dqkv, int T, int n_q, int n_kv, int dim, long ld) {
  const int group = n_q / n_kv;
  const int per_row = n_kv * dim / 4;                 // float4 items per token and tensor
  const long idx = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (idx >= (long)T * per_row * 2) return;
  const int which = (int)(idx / ((long)T * per_row));  // 0 = dK, 1 = dV
  const long rem = idx - (long)which * T * per_row;
  const int t = (int)(rem / per_row);
  const int e = (int)(rem % per_row) * 4;
  const int kvh = e / dim, c = e % dim;
  const float* ws = which ? ws_dv : ws_dk;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int g = 0; g < group; ++g) {
    const float4 v = *reinterpret_cast<const float4*>(ws + ((long)(kvh * group + g) * T + t) * dim + c);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  __nv_bfloat16* dst = dqkv + (long)t * ld + (long)(n_q + which * n_kv + kvh) * dim + c;
  uint2 o;
  o.x = pack_bf16x2(acc.x, acc.y);
  o.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(dst) = o;
}

// ----------------------------------------------------------------------------------------------
// 2. dK / dV: transposed scores, P^T / dS^T as tensor-memory operands, pipelined.
//
// A kernel that runs its four stages (TMA, S/dP MMAs, softmax, dV/dK MMAs) strictly one after the other and moves
// P and dS through shared memory leaves the tensor core idle most of the time.  Here one CTA owns a 128-row KV
// tile, and
//   * it computes the TRANSPOSED tiles S^T = K Q^T and dP^T = V dO^T for blocks of 64 queries, so the KV rows
//     are the tensor-memory lanes and P^T, dS^T can be written back (packed bf16, tcgen05.st) over the columns
//     they were computed from and fed to dV += P^T dO and dK += dS^T Q as tensor-memory A operands: no P/dS in
//     shared memory, which leaves room for a 3-deep ring of Q/dO blocks;
//   * S^T/dP^T are double buffered in tensor memory (2 x 128 columns) next to dV and dK (128 columns each), so
//     the MMAs of block i+1 run while the eight softmax warps (two per lane quadrant, 32 query columns each)
//     work on block i;
//   * per-query values (visible range, log-sum-exp, delta) are staged in shared memory one block ahead.
// Tensor memory: stage s at columns 128 s: S^T [0,64) (P^T over [0,32)), dP^T [64,128) (dS^T over [64,96));
// dV at 256, dK at 384.
// ----------------------------------------------------------------------------------------------
constexpr int BQ2 = 64;                       // queries per block
constexpr uint32_t QBOX = BQ2 * 64 * 2;       // one [64 x 64] bf16 box = 8 KB
constexpr int kRing = 3;
constexpr int kBwd2Threads = 320;             // 8 softmax warps, TMA warp, MMA warp

MMT_DEVICE void softmax_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int DIM>
__global__ void __launch_bounds__(kBwd2Threads, 1)
attn_bwd_dkdv2_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q64,
                      const __grid_constant__ CUtensorMap tm_do64, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                               // 2 boxes of [128 x 64]
  uint8_t* sV = sK + 2 * CHUNK;
  uint8_t* sRing = sV + 2 * CHUNK;                  // kRing x (Q: 2 boxes of [64 x 64], dO: 2 boxes)
  float* sRow = reinterpret_cast<float*>(sRing + kRing * 4 * QBOX);   // [2 stages][4][64]: lo, hi, lse*log2e, delta
  int* sFull = reinterpret_cast<int*>(sRow + 2 * 4 * BQ2);           // [2 stages][2 warps]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sFull + 4);
  uint64_t* kv_full = bars;               // 1
  uint64_t* slot_full = bars + 1;         // kRing
  uint64_t* slot_free = bars + 1 + kRing; // kRing
  uint64_t* s_full = bars + 1 + 2 * kRing;   // 2
  uint64_t* pds_full = s_full + 2;           // 2
  uint64_t* done = pds_full + 2;             // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv0 = blockIdx.x * BKV;
  const bool split = p.ws_dk != nullptr;
  const int full_group = p.n_q / p.n_kv;
  const int kv_head = split ? (int)blockIdx.y / full_group : (int)blockIdx.y;
  const int head0 = split ? (int)blockIdx.y : kv_head * full_group;
  const int group = split ? 1 : full_group;
  const int kv_last = min(kv0 + BKV, p.T) - 1;
  const int q_lo = p.causal ? kv0 : p.seq_lo[kv0];
  const int q_hi = p.seq_hi[kv_last];
  const int n_qb = (q_hi - q_lo + BQ2 - 1) / BQ2;
  const int n_iter = n_qb * group;
  const int xk = (p.n_q + kv_head) * DIM, xv = (p.n_q + p.n_kv + kv_head) * DIM;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_kv);
    tma_prefetch_desc(&tm_q64);
    tma_prefetch_desc(&tm_do64);
    mbar_init(kv_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&pds_full[i], 8);
    }
    mbar_init(done, 1);
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
  const uint32_t t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(kv_full, 4 * CHUNK);
      tma_load_2d(sK, &tm_kv, kv_full, xk, kv0);
      tma_load_2d(sK + CHUNK, &tm_kv, kv_full, xk + 64, kv0);
      tma_load_2d(sV, &tm_kv, kv_full, xv, kv0);
      tma_load_2d(sV + CHUNK, &tm_kv, kv_full, xv + 64, kv0);
      for (int it = 0; it < n_iter; ++it) {
        const int g = it / n_qb, i = it % n_qb;
        const int head = head0 + g;
        const int r0 = q_lo + i * BQ2;
        const int r = it % kRing;
        if (!mbar_wait(&slot_free[r], ((it / kRing) & 1) ^ 1, p.ew, 730)) break;
        uint8_t* sQ = sRing + (size_t)r * 4 * QBOX;
        uint8_t* sDO = sQ + 2 * QBOX;
        mbar_expect_tx(&slot_full[r], 4 * QBOX);
        tma_load_2d(sQ, &tm_q64, &slot_full[r], head * DIM, r0);
        tma_load_2d(sQ + QBOX, &tm_q64, &slot_full[r], head * DIM + 64, r0);
        tma_load_2d(sDO, &tm_do64, &slot_full[r], head * DIM, r0);
        tma_load_2d(sDO + QBOX, &tm_do64, &slot_full[r], head * DIM + 64, r0);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc_1 = make_idesc_bf16(BKV, BQ2, 0, 0);     // S^T, dP^T: M = 128 kv rows, N = 64 queries
      const uint32_t idesc_2 = make_idesc_bf16(BKV, DIM, 0, 1);     // dV, dK: A from tensor memory, B MN-major
      const uint32_t hi = smem_desc_hi(1024);
      const uint32_t k_lo = smem_desc_lo(smem_u32(sK), 16), v_lo = smem_desc_lo(smem_u32(sV), 16);
      const uint32_t ring_k = smem_desc_lo(smem_u32(sRing), 16);       // Q / dO as K-major B of the first MMAs
      const uint32_t ring_mn = smem_desc_lo(smem_u32(sRing), QBOX);    // dO / Q as MN-major B of the second MMAs
      auto mma2 = [&](int j) {
        const uint32_t st = tmem_base + (uint32_t)((j & 1) * 128);
        const uint32_t slot = (uint32_t)(j % kRing) * ((4 * QBOX) >> 4);
#pragma unroll
        for (int k = 0; k < BQ2 / 16; ++k)        // dV += P^T dO
          tc_mma_ts(t_dv, st + (uint32_t)(k * 8), smem_desc_join(hi, ring_mn + slot + ((2 * QBOX) >> 4) + (uint32_t)(k * 128)),
                    idesc_2, (j | k) != 0);
#pragma unroll
        for (int k = 0; k < BQ2 / 16; ++k)        // dK += dS^T Q
          tc_mma_ts(t_dk, st + 64u + (uint32_t)(k * 8), smem_desc_join(hi, ring_mn + slot + (uint32_t)(k * 128)), idesc_2,
                    (j | k) != 0);
        tc_commit(&slot_free[j % kRing]);
      };
      bool ok = mbar_wait(kv_full, 0, p.ew, 740);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int r = it % kRing;
        if (!mbar_wait(&slot_full[r], (it / kRing) & 1, p.ew, 741)) { ok = false; break; }
        const uint32_t st = tmem_base + (uint32_t)((it & 1) * 128);
        const uint32_t slot = (uint32_t)r * ((4 * QBOX) >> 4);
#pragma unroll
        for (int k = 0; k < DIM / 16; ++k) {
          const uint32_t a_off = (uint32_t)(((k >> 2) * CHUNK + (k & 3) * 32) >> 4);
          const uint32_t b_off = (uint32_t)(((k >> 2) * QBOX + (k & 3) * 32) >> 4);
          tc_mma_ss(st, smem_desc_join(hi, k_lo + a_off), smem_desc_join(hi, ring_k + slot + b_off), idesc_1, k != 0);
        }
#pragma unroll
        for (int k = 0; k < DIM / 16; ++k) {
          const uint32_t a_off = (uint32_t)(((k >> 2) * CHUNK + (k & 3) * 32) >> 4);
          const uint32_t b_off = (uint32_t)(((k >> 2) * QBOX + (k & 3) * 32) >> 4) + ((2 * QBOX) >> 4);
          tc_mma_ss(st + 64u, smem_desc_join(hi, v_lo + a_off), smem_desc_join(hi, ring_k + slot + b_off), idesc_1,
                    k != 0);
        }
        tc_commit(&s_full[it & 1]);
        if (it > 0) {
          const int j = it - 1;
          if (!mbar_wait(&pds_full[j & 1], (j >> 1) & 1, p.ew, 742)) { ok = false; break; }
          tc_fence_after();
          mma2(j);
        }
      }
      if (ok && n_iter > 0) {
        const int j = n_iter - 1;
        if (mbar_wait(&pds_full[j & 1], (j >> 1) & 1, p.ew, 743)) {
          tc_fence_after();
          mma2(j);
        }
      }
      tc_commit(done);
    }
  } else {
    // ------------------------------ softmax warps (8) + epilogue ------------------------------
    const int q4 = warp & 3;               // tensor-memory lane quadrant
    const int half = warp >> 2;            // which 32 of the 64 query columns
    const int row = q4 * 32 + lane;        // kv row of this thread inside the tile
    const int kvrow = kv0 + row;
    const int tid = threadIdx.x;           // 0..255
    const uint32_t lane_addr = ((uint32_t)(q4 * 32) << 16);
    const float sl2 = p.scale * LOG2E;
    // per-query values of block `it`, fetched by threads 0..63 one block ahead
    float pre[4] = {0.f, 0.f, 0.f, 0.f};
    auto fetch = [&](int it) {
      if (tid < BQ2 && it < n_iter) {
        const int g = it / n_qb, i = it % n_qb;
        const int head = head0 + g;
        const int q = q_lo + i * BQ2 + tid;
        int lo = 0, hi2 = 0;
        float l2 = 0.f, dl = 0.f;
        if (q < q_hi) {
          lo = p.seq_lo[q];
          hi2 = p.seq_hi[q];
          if (p.causal) hi2 = min(hi2, q + 1);
          l2 = p.lse[(long)head * p.T + q] * LOG2E;
          dl = p.delta[(long)head * p.T + q];
        }
        pre[0] = __int_as_float(lo);
        pre[1] = __int_as_float(hi2);
        pre[2] = l2;
        pre[3] = dl;
      }
    };
    fetch(0);
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int s = it & 1;
      float* rowv = sRow + s * 4 * BQ2;
      if (tid < BQ2) {
        rowv[tid] = pre[0];
        rowv[BQ2 + tid] = pre[1];
        rowv[2 * BQ2 + tid] = pre[2];
        rowv[3 * BQ2 + tid] = pre[3];
        // does this query see the whole KV tile?
        const int lo = __float_as_int(pre[0]), hi2 = __float_as_int(pre[1]);
        const bool cover = __all_sync(0xffffffffu, lo <= kv0 && hi2 >= kv0 + BKV);
        if (lane == 0) sFull[s * 2 + warp] = cover ? 1 : 0;
      }
      fetch(it + 1);
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (it >> 1) & 1, p.ew, 750));
      if (!ok) break;
      tc_fence_after();
      const uint32_t st = tmem_base + lane_addr + (uint32_t)(s * 128);
      uint32_t r_s[32], r_dp[32];
      tmem_ld_32x32b_x32(st + (uint32_t)(half * 32), r_s);
      tmem_ld_32x32b_x32(st + 64u + (uint32_t)(half * 32), r_dp);
      tmem_wait_ld();
      softmax_bar_sync();      // every warp has read its columns (P^T / dS^T overwrite them) and sRow is complete
      const bool full = (sFull[s * 2] & sFull[s * 2 + 1]) != 0;
      const float* lo_v = rowv + half * 32;
      const float* hi_v = rowv + BQ2 + half * 32;
      const float* l2_v = rowv + 2 * BQ2 + half * 32;
      const float* dl_v = rowv + 3 * BQ2 + half * 32;
      uint32_t pk_p[16], pk_ds[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = exp2f(fmaf(__uint_as_float(r_s[i]), sl2, -l2_v[i]));
        float p1 = exp2f(fmaf(__uint_as_float(r_s[i + 1]), sl2, -l2_v[i + 1]));
        if (!full) {
          if (!(kvrow >= __float_as_int(lo_v[i]) && kvrow < __float_as_int(hi_v[i]))) p0 = 0.f;
          if (!(kvrow >= __float_as_int(lo_v[i + 1]) && kvrow < __float_as_int(hi_v[i + 1]))) p1 = 0.f;
        }
        const float d0 = p0 * (__uint_as_float(r_dp[i]) - dl_v[i]) * p.scale;
        const float d1 = p1 * (__uint_as_float(r_dp[i + 1]) - dl_v[i + 1]) * p.scale;
        pk_p[i >> 1] = pack_bf16x2(p0, p1);
        pk_ds[i >> 1] = pack_bf16x2(d0, d1);
      }
      tmem_st_32x32b_x16(st + (uint32_t)(half * 16), pk_p);
      tmem_st_32x32b_x16(st + 64u + (uint32_t)(half * 16), pk_ds);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[s]);
    }
    // epilogue: thread = kv row; warps 0-3 write dK, warps 4-7 write dV
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(done, 0, p.ew, 751));
    tc_fence_after();
    const uint32_t acc = (half == 0 ? t_dk : t_dv) + lane_addr;
    const int xo = half == 0 ? xk : xv;
#pragma unroll 1
    for (int c = 0; c < DIM / 16; ++c) {
      uint32_t r[16];
      if (n_iter > 0 && ok) {
        tmem_ld_32x32b_x16(acc + c * 16, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = 0u;
      }
      if (kvrow < p.T && split) {
        float* w = (half == 0 ? p.ws_dk : p.ws_dv) + ((long)head0 * p.T + kvrow) * DIM + c * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 4) *reinterpret_cast<uint4*>(w + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
      } else if (kvrow < p.T) {
        __nv_bfloat16* dst = p.dqkv + (long)kvrow * p.ld + xo + c * 16;
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          uint4 a;
          a.x = pack_bf16x2(__uint_as_float(r[h2 * 8 + 0]), __uint_as_float(r[h2 * 8 + 1]));
          a.y = pack_bf16x2(__uint_as_float(r[h2 * 8 + 2]), __uint_as_float(r[h2 * 8 + 3]));
          a.z = pack_bf16x2(__uint_as_float(r[h2 * 8 + 4]), __uint_as_float(r[h2 * 8 + 5]));
          a.w = pack_bf16x2(__uint_as_float(r[h2 * 8 + 6]), __uint_as_float(r[h2 * 8 + 7]));
          *reinterpret_cast<uint4*>(dst + h2 * 8) = a;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

constexpr size_t kBwd2Smem = 1024 + 4 * CHUNK + kRing * 4 * QBOX + 2 * 4 * BQ2 * 4 + 16 + (2 + 2 * kRing + 5) * 8 + 16;

// ----------------------------------------------------------------------------------------------
// 3. dQ: same pipeline as the dK/dV kernel above with the roles of Q and KV exchanged.
// One CTA owns a 128-row query tile of one head and walks the visible KV range in blocks of 64 rows:
//   S = Q K_blk^T, dP = dO V_blk^T   (query rows are the tensor-memory lanes, 64 + 64 columns, double buffered)
//   dS = exp2(S*scale*log2e - lse*log2e) * (dP - delta) * scale   (eight softmax warps; per-row values in registers)
//   dQ += dS K_blk                   (dS written as packed bf16 over the dP columns: tensor-memory A operand;
//                                     the K block is the MN-major B operand)
// Tensor memory: stage s at columns 128 s: S [0,64), dP [64,128) (dS over [64,96)); dQ at 256.
// ----------------------------------------------------------------------------------------------
template <int DIM>
__global__ void __launch_bounds__(kBwd2Threads, 1)
attn_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_kv64, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                               // 2 boxes of [128 x 64]
  uint8_t* sDO = sQ + 2 * CHUNK;
  uint8_t* sRing = sDO + 2 * CHUNK;                 // kRing x (K block: 2 boxes of [64 x 64], V block: 2 boxes)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRing + kRing * 4 * QBOX);
  uint64_t* q_full = bars;                // 1
  uint64_t* slot_full = bars + 1;         // kRing
  uint64_t* slot_free = bars + 1 + kRing; // kRing
  uint64_t* s_full = bars + 1 + 2 * kRing;   // 2
  uint64_t* ds_full = s_full + 2;            // 2
  uint64_t* done = ds_full + 2;              // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal: the last query tiles see the most KV blocks and are started first
  const int q0 = (p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x) * BQ;
  const int head = blockIdx.y;
  const int kv_head = head / (p.n_q / p.n_kv);
  const int q_last = min(q0 + BQ, p.T) - 1;
  const int kv_lo = p.seq_lo[q0];
  const int kv_hi = p.causal ? min(p.seq_hi[q_last], q_last + 1) : p.seq_hi[q_last];
  const int n_iter = (kv_hi - kv_lo + BQ2 - 1) / BQ2;
  const int xq = head * DIM, xk = (p.n_q + kv_head) * DIM, xv = (p.n_q + p.n_kv + kv_head) * DIM;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_kv64);
    mbar_init(q_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&ds_full[i], 8);
    }
    mbar_init(done, 1);
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
  const uint32_t t_dq = tmem_base + 256;

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 4 * CHUNK);
      tma_load_2d(sQ, &tm_q, q_full, xq, q0);
      tma_load_2d(sQ + CHUNK, &tm_q, q_full, xq + 64, q0);
      tma_load_2d(sDO, &tm_do, q_full, xq, q0);
      tma_load_2d(sDO + CHUNK, &tm_do, q_full, xq + 64, q0);
      for (int it = 0; it < n_iter; ++it) {
        const int r0 = kv_lo + it * BQ2;
        const int r = it % kRing;
        if (!mbar_wait(&slot_free[r], ((it / kRing) & 1) ^ 1, p.ew, 760)) break;
        uint8_t* sKb = sRing + (size_t)r * 4 * QBOX;
        uint8_t* sVb = sKb + 2 * QBOX;
        mbar_expect_tx(&slot_full[r], 4 * QBOX);
        tma_load_2d(sKb, &tm_kv64, &slot_full[r], xk, r0);
        tma_load_2d(sKb + QBOX, &tm_kv64, &slot_full[r], xk + 64, r0);
        tma_load_2d(sVb, &tm_kv64, &slot_full[r], xv, r0);
        tma_load_2d(sVb + QBOX, &tm_kv64, &slot_full[r], xv + 64, r0);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_1 = make_idesc_bf16(BQ, BQ2, 0, 0);      // S, dP: M = 128 queries, N = 64 kv rows
      const uint32_t idesc_2 = make_idesc_bf16(BQ, DIM, 0, 1);      // dQ: A from tensor memory, B = K block MN-major
      const uint32_t hi = smem_desc_hi(1024);
      const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16), do_lo = smem_desc_lo(smem_u32(sDO), 16);
      const uint32_t ring_k = smem_desc_lo(smem_u32(sRing), 16);
      const uint32_t ring_mn = smem_desc_lo(smem_u32(sRing), QBOX);
      auto mma2 = [&](int j) {
        const uint32_t st = tmem_base + (uint32_t)((j & 1) * 128);
        const uint32_t slot = (uint32_t)(j % kRing) * ((4 * QBOX) >> 4);
#pragma unroll
        for (int k = 0; k < BQ2 / 16; ++k)
          tc_mma_ts(t_dq, st + 64u + (uint32_t)(k * 8), smem_desc_join(hi, ring_mn + slot + (uint32_t)(k * 128)), idesc_2,
                    (j | k) != 0);
        tc_commit(&slot_free[j % kRing]);
      };
      bool ok = mbar_wait(q_full, 0, p.ew, 770);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int r = it % kRing;
        if (!mbar_wait(&slot_full[r], (it / kRing) & 1, p.ew, 771)) { ok = false; break; }
        const uint32_t st = tmem_base + (uint32_t)((it & 1) * 128);
        const uint32_t slot = (uint32_t)r * ((4 * QBOX) >> 4);
#pragma unroll
        for (int k = 0; k < DIM / 16; ++k) {
          const uint32_t a_off = (uint32_t)(((k >> 2) * CHUNK + (k & 3) * 32) >> 4);
          const uint32_t b_off = (uint32_t)(((k >> 2) * QBOX + (k & 3) * 32) >> 4);
          tc_mma_ss(st, smem_desc_join(hi, q_lo + a_off), smem_desc_join(hi, ring_k + slot + b_off), idesc_1, k != 0);
        }
#pragma unroll
        for (int k = 0; k < DIM / 16; ++k) {
          const uint32_t a_off = (uint32_t)(((k >> 2) * CHUNK + (k & 3) * 32) >> 4);
          const uint32_t b_off = (uint32_t)(((k >> 2) * QBOX + (k & 3) * 32) >> 4) + ((2 * QBOX) >> 4);
          tc_mma_ss(st + 64u, smem_desc_join(hi, do_lo + a_off), smem_desc_join(hi, ring_k + slot + b_off), idesc_1,
                    k != 0);
        }
        tc_commit(&s_full[it & 1]);
        if (it > 0) {
          const int j = it - 1;
          if (!mbar_wait(&ds_full[j & 1], (j >> 1) & 1, p.ew, 772)) { ok = false; break; }
          tc_fence_after();
          mma2(j);
        }
      }
      if (ok && n_iter > 0) {
        const int j = n_iter - 1;
        if (mbar_wait(&ds_full[j & 1], (j >> 1) & 1, p.ew, 773)) {
          tc_fence_after();
          mma2(j);
        }
      }
      tc_commit(done);
    }
  } else {
    const int q4 = warp & 3;
    const int half = warp >> 2;
    const int row = q4 * 32 + lane;
    const int qrow = q0 + row;
    const bool row_ok = qrow < p.T;
    const uint32_t lane_addr = ((uint32_t)(q4 * 32) << 16);
    const float sl2 = p.scale * LOG2E;
    int lo = 0, hi2 = 0;
    float lse_l2 = 0.f, delta = 0.f;
    if (row_ok) {
      lo = p.seq_lo[qrow];
      hi2 = p.seq_hi[qrow];
      if (p.causal) hi2 = min(hi2, qrow + 1);
      lse_l2 = p.lse[(long)head * p.T + qrow] * LOG2E;
      delta = p.delta[(long)head * p.T + qrow];
    }
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int s = it & 1;
      const int kvb = kv_lo + it * BQ2 + half * 32;          // first kv row of this warp's 32 columns
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (it >> 1) & 1, p.ew, 780));
      if (!ok) break;
      tc_fence_after();
      const uint32_t st = tmem_base + lane_addr + (uint32_t)(s * 128);
      uint32_t r_s[32], r_dp[32];
      tmem_ld_32x32b_x32(st + (uint32_t)(half * 32), r_s);
      tmem_ld_32x32b_x32(st + 64u + (uint32_t)(half * 32), r_dp);
      tmem_wait_ld();
      softmax_bar_sync();      // every warp has read its dP columns before dS overwrites them
      const bool full = __all_sync(0xffffffffu, kvb >= lo && kvb + 32 <= hi2);
      uint32_t pk_ds[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = exp2f(fmaf(__uint_as_float(r_s[i]), sl2, -lse_l2));
        float p1 = exp2f(fmaf(__uint_as_float(r_s[i + 1]), sl2, -lse_l2));
        if (!full) {
          const int kv = kvb + i;
          if (!(kv >= lo && kv < hi2)) p0 = 0.f;
          if (!(kv + 1 >= lo && kv + 1 < hi2)) p1 = 0.f;
        }
        const float d0 = p0 * (__uint_as_float(r_dp[i]) - delta) * p.scale;
        const float d1 = p1 * (__uint_as_float(r_dp[i + 1]) - delta) * p.scale;
        pk_ds[i >> 1] = pack_bf16x2(d0, d1);
      }
      tmem_st_32x32b_x16(st + 64u + (uint32_t)(half * 16), pk_ds);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[s]);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(done, 0, p.ew, 781));
    tc_fence_after();
    // epilogue: the two warps of a lane quadrant split the head's columns in 16-column chunks
    __nv_bfloat16* dst = p.dqkv + (long)qrow * p.ld + xq;
#pragma unroll 1
    for (int c = half; c < DIM / 16; c += 2) {
      uint32_t r[16];
      if (n_iter > 0 && ok) {
        tmem_ld_32x32b_x16(t_dq + lane_addr + c * 16, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          uint4 a;
          a.x = pack_bf16x2(__uint_as_float(r[h2 * 8 + 0]), __uint_as_float(r[h2 * 8 + 1]));
          a.y = pack_bf16x2(__uint_as_float(r[h2 * 8 + 2]), __uint_as_float(r[h2 * 8 + 3]));
          a.z = pack_bf16x2(__uint_as_float(r[h2 * 8 + 4]), __uint_as_float(r[h2 * 8 + 5]));
          a.w = pack_bf16x2(__uint_as_float(r[h2 * 8 + 6]), __uint_as_float(r[h2 * 8 + 7]));
          *reinterpret_cast<uint4*>(dst + c * 16 + h2 * 8) = a;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

constexpr size_t kDq2Smem = 1024 + 4 * CHUNK + kRing * 4 * QBOX + (2 + 2 * kRing + 5) * 8 + 16;

template <int DIM>
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tq64, const CUtensorMap& tdo64,
               const AttnParams& p, cudaStream_t st) {
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkdv2_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kBwd2Smem);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_bwd_dq2_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDq2Smem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const int tiles = (p.T + BQ - 1) / BQ;
  attn_bwd_dkdv2_kernel<DIM><<<dim3(tiles, p.ws_dk ? p.n_q : p.n_kv), kBwd2Threads, kBwd2Smem, st>>>(tq, tq64, tdo64, p);
  if (p.ws_dk) {
    const long items = (long)p.T * (p.n_kv * DIM / 4) * 2;
    attn_group_reduce_kernel<<<(unsigned)((items + 255) / 256), 256, 0, st>>>(p.ws_dk, p.ws_dv, p.dqkv, p.T, p.n_q,
                                                                             p.n_kv, DIM, p.ld);
  }
  attn_bwd_dq2_kernel<DIM><<<dim3(tiles, p.n_q), kBwd2Threads, kDq2Smem, st>>>(tq, tdo, tq64, p);
  return (int)cudaGetLastError();
}

}  // namespace

// dqkv [T, ld] receives dq | dk | dv in the layout of qkv.  delta is fp32 scratch [n_q, T].  ws is optional fp32
// scratch of 2 * n_q * T * dim floats: with it (and n_q > n_kv) dK/dV run one CTA per q head and are summed over
// each GQA group afterwards, which fills the GPU when there are few KV tiles.
extern "C" int mmt_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                            void* dqkv, const int* seq_lo, const int* seq_hi, long T, int n_q, int n_kv, int dim,
                            long ld, int causal, float scale, float* ws, void* stream) {
  if (T <= 0) return 0;
  if (mmt_ensure_context(qkv)) return -7;
  if ((dim != 80 && dim != 128) || n_q % n_kv || (ld & 7)) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  {
    const long warps = T * n_q;
    const int threads = 256;
    const long blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                           reinterpret_cast<const __nv_bfloat16*>(dout), delta,
                                                           (int)T, n_q, dim);
  }
  CUtensorMap tq, tdo;
  const uint64_t width = (uint64_t)(n_q + 2 * n_kv) * dim;
  int r = mmt_make_tmap_2d(&tq, qkv, width, (uint64_t)T, (uint64_t)ld, 64, 128);
  if (r) return 1000 + r;
  r = mmt_make_tmap_2d(&tdo, dout, (uint64_t)n_q * dim, (uint64_t)T, (uint64_t)n_q * dim, 64, 128);
  if (r) return 2000 + r;
  AttnParams p;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.out = nullptr;
  p.lse = const_cast<float*>(lse);
  p.seq_lo = seq_lo;
  p.seq_hi = seq_hi;
  p.T = (int)T; p.n_q = n_q; p.n_kv = n_kv; p.dim = dim; p.ld = ld;
  p.causal = causal; p.scale = scale;
  p.ew = mmt_error_word();
  p.dout = reinterpret_cast<const __nv_bfloat16*>(dout);
  p.delta = delta;
  p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  const bool split = ws != nullptr && n_q > n_kv;
  p.ws_dk = split ? ws : nullptr;
  p.ws_dv = split ? ws + (long)n_q * T * dim : nullptr;
  CUtensorMap tq64, tdo64;   // 64-row boxes for the second-generation kernels' query / KV blocks
  r = mmt_make_tmap_2d(&tq64, qkv, width, (uint64_t)T, (uint64_t)ld, 64, 64);
  if (r) return 3000 + r;
  r = mmt_make_tmap_2d(&tdo64, dout, (uint64_t)n_q * dim, (uint64_t)T, (uint64_t)n_q * dim, 64, 64);
  if (r) return 4000 + r;
  return dim == 80 ? launch_bwd<80>(tq, tdo, tq64, tdo64, p, st) : launch_bwd<128>(tq, tdo, tq64, tdo64, p, st);
}
