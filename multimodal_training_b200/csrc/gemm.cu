// bf16 GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   C[M,N] = epilogue( alpha * sum_k A[m,k] * B[n,k] )
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: global -> 128B-swizzled shared-memory ring
//   warp 1      MMA issuer: one thread issues tcgen05.mma (cta_group::1) with both
//               operands in shared memory and the fp32 accumulator in tensor memory;
//               tcgen05.commit frees ring slots and publishes finished accumulators
//   warps 2..9  epilogue: tcgen05.ld accumulator rows -> registers -> fused bias / GELU / residual /
//               accumulate -> bf16 through per-warp shared-memory slabs and TMA stores (or direct stores)
// The accumulator is double buffered in tensor memory (2 x BN columns) so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Operand layouts.  A is logically [M,K], B is logically [N,K].  Each may be
// "K-major" (memory [rows][K]) or "MN-major" (memory [K][rows]); the three
// combinations cover a linear layer's forward (K,K), its input gradient
// (K,MN) and its weight gradient (MN,MN) without any transpose pass.
// Tails in M, N and K are handled by TMA zero fill on loads and bounds checks
// on stores.  Requirements: leading dimensions multiples of 8 elements, N % 8 == 0.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference
// (python/models/qwen2_5_vl/modeling_qwen2_5_vl.py:198-200,334-338,1143-1145,1226-1229).
#include <cudaTypedefs.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cstddef>
#include "common.cuh"
#include "runtime.h"

// Measurement builds only (-DMMT_GEMM_MEASURE, see csrc/build.py): switches that drop parts of the kernel's work
// (results are then wrong), the in-kernel clock probe and the descriptor bring-up knob.  In a regular build none of
// them exists: the tests read MMT_DBG as the constant 0 and the setters are not exported.
#ifdef MMT_GEMM_MEASURE
#define MMT_DBG (p.dbg)
#define MMT_CLK (p.clk)
#else
#define MMT_DBG 0
#define MMT_CLK ((unsigned long long*)nullptr)
#endif

namespace {

constexpr int BM = 128;
constexpr int BK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 8;
constexpr uint32_t kSlabBytes = 32 * 64 * 2;   // one epilogue warp's [32 x 64] bf16 staging slab
constexpr int kThreads = 64 + kEpiWarps * 32 + 32;   // TMA warp, MMA warp, eight epilogue warps, one forwarder warp
constexpr int kAgChunks = 64;                  // chunk flags per source rank of a fused all-gather

struct GemmParams {
  int M, N, K;
  void* C;
  int ldc;
  const __nv_bfloat16* bias;      // [N] or nullptr
  const __nv_bfloat16* residual;  // [M, ldr] or nullptr (added after the activation)
  int ldr;
  int act;                        // 0 none, 1 GELU(erf)
  int accumulate;                 // C += result
  int out_f32;                    // C is float
  float alpha;
  int a_mn, b_mn;                 // operand majors
  int tma_store;                  // bf16 output leaves through the epilogue warps' shared-memory slabs
  int group_m, tiles_n;           // raster: m-tiles per band (0 = all), number of n-tiles
  uint32_t mn_lbo, mn_sbo, mn_kstep;  // descriptor constants of MN-major tiles
  MmtErrorWord* ew;
  // --- stream-K for the last partial wave: the final `sk_tiles` tiles are cut along K into gridDim.x equal runs of
  //     k-blocks, one per CTA; a CTA that does not reach the end of a tile leaves its fp32 partial in `sk_ws`
  //     (slot = CTA index) and raises sk_flags[CTA] to sk_epoch; the CTA that reaches the end adds the partials of
  //     the CTAs before it, in CTA order, and runs the epilogue.  sk_tiles == 0: off.
  int sk_tiles;
  float* sk_ws;
  int* sk_flags;
  int sk_epoch;
  int dbg;                        // measurement only: bit 0 = operands are loaded once (ring filled, then reused), bit 1 = no
                                  // per-stage commit, bit 2 = no TMA stores, bit 3 = no epilogue work at all
  unsigned long long* clk;        // optional: CTA 0 writes {SM cycles, nanoseconds} it spent in the kernel
  // --- all-gather consumer (A rows arrive from peers): rows [s*ag_rows, (s+1)*ag_rows) come from rank s and
  //     are complete once ag_flags[s] >= ag_epoch; this rank's own rows need no wait.  ag_flags == nullptr: off.
  const int* ag_flags;
  int ag_epoch, ag_rows, ag_self;
  // --- all-gather FORWARDER inside the same kernel (fwd_peers > 0).  The CTAs that compute the first fwd_split
  //     column tiles of a block of this rank's own rows also send that block to the peers: of the A stages the TMA
  //     producer loads for the MMA, column tile tn forwards the k-blocks with kb % fwd_split == tn, storing the stage
  //     from shared memory into the same place of every destination's gathered buffer (bulk tensor stores over
  //     NVLink).  The rows cross the link while the tensor core works on them, are read from HBM once, and the work
  //     is spread over fwd_split CTAs per row block.  Each of those CTAs counts itself into fwd_counter[block] once
  //     its stores have landed; the last one writes ag_epoch to flag word [ag_self * kAgChunks + block] on every
  //     peer, and the consumer side waits per (source rank, block) on ag_flags.  ag_chunk = rows per block = rows of
  //     a tile.  fwd_direct: own rows are loaded from the caller's shard (tensor map 9 of the table) instead of the
  //     gathered buffer, and this rank's gathered buffer is one more destination (fwd_dsts = fwd_peers + 1).
  int* fwd_flag[8];                 // flag arrays of the fwd_peers remote peers
  int* fwd_counter;                 // [kAgChunks] ints, zero between launches
  int fwd_peers, fwd_dsts, fwd_split, fwd_direct, ag_chunk;
  // --- reduce-scatter producer: row r of C belongs to rank r / rs_rows and is stored to that rank's staging
  //     slot `rs_self` ([rs_self*rs_rows + r % rs_rows, :] at rs_base[owner]); when the whole GEMM is done,
  //     rs_flag[p] on every peer receives rs_epoch.  rs_rows == 0: off.
  unsigned long long rs_base[8];
  int* rs_flag[8];
  int* rs_counter;
  int rs_rows, rs_self, rs_ranks, rs_epoch;
  // --- column scatter (Ulysses sequence -> heads exchange as the epilogue of the QKV projection): the output is
  //     `parts` blocks of sc_part columns; inside every block, columns [r * sc_w, (r + 1) * sc_w) belong to rank r
  //     and go to row sc_row[row] of that rank's buffer rs_base[r] ([*, sc_ld], sc_ld = parts * sc_w) at column
  //     part * sc_w + (column inside the owner's range).  A [32 x 64] slab with one owner and 32 consecutive
  //     destination rows leaves as one bulk store (tensor map r of the table); anything else as 16-byte stores.
  //     When the whole GEMM is done, rs_flag[r] on every rank receives rs_epoch.  C is not written.  nullptr: off.
  const int* sc_row;
  int sc_part, sc_w, sc_ld;
  // --- K-slice consumer (Ulysses heads -> sequence exchange as the prologue of the output projection): columns
  //     [s * kf_w, (s + 1) * kf_w) of A were written by rank s and are complete once kf_flags[s] >= kf_epoch.  The
  //     k-blocks are walked starting with this rank's own slice (kf_self), which needs no wait.  nullptr: off.
  const int* kf_flags;
  int kf_epoch, kf_w, kf_self, kf_ranks;
};

// tile index -> (tile_m, tile_n); with an all-gather consumer the m tiles are rotated so that the CTA wave
// starts on this rank's own rows while the peers' rows are still in flight; with a reduce-scatter producer they
// are rotated so that the ranks' stores are spread over the owners.
MMT_DEVICE void tile_coords(const GemmParams& p, int tile, int tiles_m, int bmt, int& tm, int& tn) {
  // Grouped raster: tiles are walked in bands of `group_m` m-tiles, n-fastest inside a band... i.e. a wave of
  // CTAs covers a roughly square block of the output, so every A and B tile it needs is shared by many CTAs
  // and stays in L2 instead of being re-streamed from DRAM once per n-tile.
  const int g = p.group_m > 0 ? p.group_m : tiles_m;
  const int band = tile / (g * p.tiles_n);
  const int first = band * g;
  const int rows = min(g, tiles_m - first);
  const int local = tile - band * g * p.tiles_n;
  tm = first + local % rows;
  tn = local / rows;
  if (p.ag_flags) tm = (tm + (int)(((long)p.ag_self * p.ag_rows) / bmt)) % tiles_m;
  // reduce-scatter producer: rank r starts on the rows owned by rank r + 1, so at any moment the ranks store
  // into different owners instead of all converging on rank 0's NVLink ingress
  else if (p.rs_rows) tm = (tm + (int)(((long)((p.rs_self + 1) % p.rs_ranks) * p.rs_rows) / bmt)) % tiles_m;
}

// One unit of work of a CTA: k-blocks [k0, k1) of tile `tile`.
//   kind 0: a whole tile;  kind 1: a run that stops before the tile's last k-block (partial sums go to the
//   workspace);  kind 2: a run that ends the tile after other CTAs did its first k-blocks (their partial sums
//   are added before the epilogue; `first_contrib` .. cta - 1 are those CTAs).
struct WorkItem {
  int tile, k0, k1, kind, first_contrib;
};

// i-th work item of CTA `cta`: the stream-K runs first (partial sums before finishing runs, so that they are ready
// when their tile ends), then this CTA's whole tiles.
MMT_DEVICE bool work_item(const GemmParams& p, int i, int cta, int grid, int KB, int ntiles, WorkItem& w) {
  const int i0 = i;
  const int full = ntiles - p.sk_tiles;
  int n_sk = 0;
  if (p.sk_tiles > 0) {
    const long units = (long)p.sk_tiles * KB;
    const long u0 = units * cta / grid, u1 = units * (cta + 1) / grid;
    if (u1 > u0) {
      const int ta = (int)(u0 / KB);
      const long end_a = min(u1, (long)(ta + 1) * KB);
      n_sk = u1 > end_a ? 2 : 1;
      // a run that crosses into the next tile is worked in two items; the head of the NEXT tile (a partial sum, which
      // depends on nobody) goes first and the tail of the current tile (which may have to wait for the CTAs before
      // this one) second: partial sums are then produced by all CTAs at once instead of one CTA after the other
      if (n_sk == 2) i = 1 - i;
      if (i == 0) {
        w.tile = full + ta;
        w.k0 = (int)(u0 - (long)ta * KB);
        w.k1 = (int)(end_a - (long)ta * KB);
        w.first_contrib = cta;
        if (w.k1 < KB) {
          w.kind = 1;
        } else if (w.k0 == 0) {
          w.kind = 0;
        } else {
          w.kind = 2;
          int c = cta;                       // CTAs before this one whose run ends inside this tile
          while (c > 0 && units * c / grid > (long)ta * KB) --c;
          w.first_contrib = c;
        }
        return true;
      }
      if (i == 1 && n_sk == 2) {
        w.tile = full + ta + 1;
        w.k0 = 0;
        w.k1 = (int)(u1 - (long)(ta + 1) * KB);
        w.kind = 1;
        w.first_contrib = cta;
        return true;
      }
    }
  }
  const int t = cta + (i0 - n_sk) * grid;
  if (t >= full) return false;
  w.tile = t;
  w.k0 = 0;
  w.k1 = KB;
  w.kind = 0;
  w.first_contrib = cta;
  return true;
}

// MT = number of 128-row accumulators per CTA tile.  MT == 1: 128 x BN tile, the accumulator is double
// buffered in tensor memory (epilogue of tile i overlaps the main loop of tile i+1).  MT == 2: 256 x BN tile,
// both halves share every B tile in shared memory (a third less L2 -> shared-memory traffic per flop, which is
// what bounds the MT == 1 kernel); the two halves fill tensor memory, so the epilogue overlaps the next tile
// half by half.
template <int BN, int MT>
struct Cfg {
  static constexpr int BMT = BM * MT;
  static constexpr uint32_t A_BYTES = BMT * BK * 2;
  static constexpr uint32_t B_BYTES = BN * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t STORE_BYTES = kEpiWarps * kSlabBytes;   // one [32 x 64] bf16 slab per epilogue warp
  static constexpr int kStages = (int)((227u * 1024u - 2048u - STORE_BYTES) / STAGE_BYTES) > 8
                                     ? 8 : (int)((227u * 1024u - 2048u - STORE_BYTES) / STAGE_BYTES);
  static constexpr uint32_t TMEM_COLS = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);
  static constexpr size_t SMEM = 1024 + (size_t)kStages * STAGE_BYTES + STORE_BYTES + (4 * kStages + 4) * 8 + 16;
  static_assert(MT == 1 || 2 * BN <= 512, "two accumulators must fit tensor memory");
};


// Tensor maps beside A and B.  Output ([32 x 64] boxes): index 0 for a plain GEMM; one per owner rank for a
// reduce-scatter producer.  All-gather forwarder: 1 .. 8 = the destinations' gathered buffers (boxes of an A stage),
// 9 = this rank's shard as the source of its own rows.
struct OutMaps {
  CUtensorMap m[10];
};

// byte offset of (row, col) in a [rows x 64] bf16 box (1024-byte aligned) with 128-byte rows and the 128B swizzle
MMT_DEVICE uint32_t store_box_offset(int row, int col) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 3) ^ (row & 7)) & 7) << 4) + (col & 7) * 2);
}

MMT_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
MMT_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
MMT_DEVICE uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
MMT_DEVICE void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
MMT_DEVICE void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
MMT_DEVICE void tc_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}
MMT_DEVICE void tc_mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
MMT_DEVICE void tmem_alloc_pair(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
}
MMT_DEVICE void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
MMT_DEVICE void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}


// ------------------------------------------------------------------------------------
// Epilogue of one 128-row accumulator, shared by both kernels.
//
// Eight warps drain an accumulator: warp e owns tensor-memory lanes (rows) 32*(e%4).. and every second group of
// 64 columns.  A warp never synchronises with another warp: it reads 64 columns of its 32 rows with two
// tcgen05.ld, converts them, writes its own 32 x 64 bf16 slab of shared memory (128-byte rows, 128B swizzle) and
// hands that slab to a TMA store of its own (full 128-byte rows per request, also when C is a peer GPU's buffer).
// The next group's tcgen05.ld is issued before the warp waits for its previous store to have read the slab, and
// the accumulator is released to the MMA warp as soon as this warp's last tcgen05.ld has completed, i.e. before
// the conversion and the stores of the last group.
// fp32 outputs, C += and ragged reduce-scatter rows use direct 16-byte global stores instead of the slab.
// ------------------------------------------------------------------------------------

// sk_part / sk_n / sk_stride: stream-K partial sums of this accumulator left by sk_n earlier CTAs (fp32, [128][BN],
// one slot of sk_stride floats per CTA), added in CTA order before the epilogue arithmetic.
#if defined(MMT_GEMM_TRACE) && defined(MMT_GEMM_MEASURE)
// measurement build: warp 2 of CTA 0 appends SM cycle stamps to MMT_CLK[2..] (see the epilogue loop)
#define MMT_TRACE_STAMP(id)                                                                         \
  do {                                                                                              \
    if (MMT_CLK && blockIdx.x == 0 && (threadIdx.x >> 5) == 2 && (threadIdx.x & 31) == 0) {            \
      const unsigned long long n_ = MMT_CLK[2];                                                       \
      if (n_ < 500) { MMT_CLK[3 + 2 * n_] = (id); MMT_CLK[4 + 2 * n_] = (unsigned long long)clock64(); MMT_CLK[2] = n_ + 1; } \
    }                                                                                               \
  } while (0)
#else
#define MMT_TRACE_STAMP(id) do { } while (0)
#endif

template <int BN>
MMT_DEVICE void epilogue_block(const GemmParams& p, uint32_t tmem_acc, int row0, int col_tile0,
                               int q, int half, int lane, uint8_t* slab, uint32_t release_bar,
                               const float* sk_part = nullptr, int sk_n = 0, long sk_stride = 0) {
  constexpr int kGroups = BN / 64;
  const bool tma_out = !p.out_f32 && p.tma_store;
  const int srow0 = row0 + q * 32;                 // first row of this warp's slab
  const long grow = (long)srow0 + lane;
  const bool row_ok = grow < p.M;
  const uint32_t taddr0 = tmem_acc + ((uint32_t)(q * 32) << 16);
  int last_g = -1;
  for (int g = half; g < kGroups; g += 2) last_g = g;
  if (last_g < 0) {                                 // no columns for this warp (BN == 64, second half)
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(release_bar);
    return;
  }
#pragma unroll 1
  for (int g = half; g < kGroups; g += 2) {
    uint32_t r0[32], r1[32];
    tmem_ld_32x32b_x32(taddr0 + (uint32_t)(g * 64), r0);
    tmem_ld_32x32b_x32(taddr0 + (uint32_t)(g * 64 + 32), r1);
    tmem_wait_ld();
    MMT_TRACE_STAMP(10 + g);
    if (g == last_g) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(release_bar);
    }
    MMT_TRACE_STAMP(20 + g);
    for (int c = 0; c < sk_n; ++c) {
      // slot layout: [64-column group][16-byte chunk][row], so that a warp reads 512 contiguous bytes per request
      const float4* src = reinterpret_cast<const float4*>(sk_part + (long)c * sk_stride) + (long)g * 16 * 128 +
                          (q * 32 + lane);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 a = src[i * 128], b = src[(8 + i) * 128];
        r0[4 * i] = __float_as_uint(__uint_as_float(r0[4 * i]) + a.x);
        r0[4 * i + 1] = __float_as_uint(__uint_as_float(r0[4 * i + 1]) + a.y);
        r0[4 * i + 2] = __float_as_uint(__uint_as_float(r0[4 * i + 2]) + a.z);
        r0[4 * i + 3] = __float_as_uint(__uint_as_float(r0[4 * i + 3]) + a.w);
        r1[4 * i] = __float_as_uint(__uint_as_float(r1[4 * i]) + b.x);
        r1[4 * i + 1] = __float_as_uint(__uint_as_float(r1[4 * i + 1]) + b.y);
        r1[4 * i + 2] = __float_as_uint(__uint_as_float(r1[4 * i + 2]) + b.z);
        r1[4 * i + 3] = __float_as_uint(__uint_as_float(r1[4 * i + 3]) + b.w);
      }
    }
    const int colg = col_tile0 + g * 64;
    if (MMT_DBG & 8) continue;                        // measurement only: drain the accumulator, store nothing
    if (colg < p.N && (row_ok || tma_out)) {
#pragma unroll
      for (int j8 = 0; j8 < 8; ++j8) {
        const int col = colg + j8 * 8;
        if (col >= p.N) break;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = __uint_as_float(j8 < 4 ? r0[j8 * 8 + j] : r1[(j8 - 4) * 8 + j]) * p.alpha;
        if (p.bias) {
          const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
          const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(bw[j]);
            v[2 * j] += f.x;
            v[2 * j + 1] += f.y;
          }
        }
        if (p.act == 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = gelu_erf(v[j]);
        }
        if (p.residual && row_ok) {
          const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + grow * p.ldr + col);
          const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(rw[j]);
            v[2 * j] += f.x;
            v[2 * j + 1] += f.y;
          }
        }
        if (p.out_f32) {
          float* dst = reinterpret_cast<float*>(p.C) + grow * p.ldc + col;
          if (p.accumulate) {
            const float4 o0 = *reinterpret_cast<const float4*>(dst);
            const float4 o1 = *reinterpret_cast<const float4*>(dst + 4);
            v[0] += o0.x; v[1] += o0.y; v[2] += o0.z; v[3] += o0.w;
            v[4] += o1.x; v[5] += o1.y; v[6] += o1.z; v[7] += o1.w;
          }
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
          __nv_bfloat16* dst = nullptr;
          if (!tma_out || (p.accumulate && row_ok)) {
            if (p.rs_rows) {
              const int owner = (int)(grow / p.rs_rows);
              dst = reinterpret_cast<__nv_bfloat16*>(p.rs_base[owner]) +
                    ((long)p.rs_self * p.rs_rows + (grow - (long)owner * p.rs_rows)) * p.ldc + col;
            } else {
              dst = reinterpret_cast<__nv_bfloat16*>(p.C) + grow * p.ldc + col;
            }
            if (p.accumulate) {       // C += : the old value is read directly, the sum leaves like any other result
              const uint4 ov = *reinterpret_cast<const uint4*>(dst);
              const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16x2(ow[j]);
                v[2 * j] += f.x;
                v[2 * j + 1] += f.y;
              }
            }
          }
          uint4 o;
          o.x = pack_bf16x2(v[0], v[1]);
          o.y = pack_bf16x2(v[2], v[3]);
          o.z = pack_bf16x2(v[4], v[5]);
          o.w = pack_bf16x2(v[6], v[7]);
          if (tma_out) *reinterpret_cast<uint4*>(slab + store_box_offset(lane, j8 * 8)) = o;
          else *reinterpret_cast<uint4*>(dst) = o;
        }
      }
    }
    MMT_TRACE_STAMP(30 + g);
    if (tma_out) {
      // The warp's 32 x 64 slab leaves as full 128-byte row segments: lane l copies 16 bytes of row (l >> 3) of
      // every group of four rows, so each store instruction of the warp writes four complete lines.  Plain
      // stores on purpose: a bulk (TMA) store would queue behind the operand loads that the producer warp has
      // already issued for the next tile, and the warp would wait for that queue before it may refill its slab.
      __syncwarp();
      if (colg < p.N && !(MMT_DBG & 4)) {
        const int chunk = lane & 7;
        const int col = colg + chunk * 8;
        if (col < p.N) {
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = it * 4 + (lane >> 3);
            const long gr = (long)srow0 + row;
            if (gr < p.M) {
              const uint4 val = *reinterpret_cast<const uint4*>(slab + store_box_offset(row, chunk * 8));
              __nv_bfloat16* dst;
              if (p.rs_rows) {
                const int owner = (int)(gr / p.rs_rows);
                dst = reinterpret_cast<__nv_bfloat16*>(p.rs_base[owner]) +
                      ((long)p.rs_self * p.rs_rows + (gr - (long)owner * p.rs_rows)) * p.ldc + col;
              } else {
                dst = reinterpret_cast<__nv_bfloat16*>(p.C) + gr * p.ldc + col;
              }
              *reinterpret_cast<uint4*>(dst) = val;
            }
          }
        }
      }
      __syncwarp();                                  // the slab may be refilled
    }
    MMT_TRACE_STAMP(40 + g);
  }
}

// The common case of epilogue_block as straight-line code: alpha == 1, no activation, bf16 output that overwrites C,
// no stream-K partial sums; bias and residual are compile-time options.  Every linear layer's forward, input-gradient
// and (first) weight-gradient GEMM ends here; epilogue_block keeps the general arithmetic.
// Releases an accumulator to the MMA warp.  Within one CTA a CTA-scope arrive is enough (tensor-memory accesses are
// ordered by the tcgen05 fences); the cluster-scope release that a barrier in the partner CTA needs would first wait
// until this thread's earlier global stores are visible cluster-wide, i.e. for their round trip to L2.
MMT_DEVICE void release_acc(uint32_t release_bar, bool remote) {
  if (remote) mbar_arrive_cluster(release_bar);
  else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(release_bar) : "memory");
}

template <int BN, bool kBias, bool kResid>
MMT_DEVICE void epilogue_fast(const GemmParams& p, const OutMaps& tmC, uint32_t tmem_acc, int row0, int col_tile0,
                              int q, int half, int lane, uint8_t* slab, uint32_t release_bar, bool remote) {
  constexpr int kGroups = BN / 64;
  const int srow0 = row0 + q * 32;
  const long grow = (long)srow0 + lane;
  const bool row_ok = grow < p.M;
  const uint32_t taddr0 = tmem_acc + ((uint32_t)(q * 32) << 16);
  const int N = p.N;
  const int chunk = lane & 7, sub = lane >> 3;
  constexpr int last_g_of[2] = {((kGroups - 1) & ~1), ((kGroups - 2) | 1)};
  const int last_g = kGroups == 1 ? (half == 0 ? 0 : -1) : last_g_of[half];
  if (last_g < 0 || half >= kGroups) {
    __syncwarp();
    if (lane == 0) release_acc(release_bar, remote);
    return;
  }
  // bulk (TMA) stores: the warp hands its slab to the copy engine and goes on; the burst of all CTAs' results then
  // drains into L2 behind the next tile's main loop instead of stalling the epilogue warps on store back-pressure
  const bool bulk = p.tma_store == 2;
  // column scatter: destination rows of the slab's first and last row, fetched now so that the loads are in flight
  // while the accumulator is read; 32 consecutive rows can leave as one box
  int sc_first = 0;
  bool sc_rows_in_a_run = false;
  if (p.sc_row && srow0 + 32 <= p.M) {
    sc_first = p.sc_row[srow0];
    sc_rows_in_a_run = p.sc_row[srow0 + 31] - sc_first == 31;
  }
#pragma unroll 1
  for (int g = half; g < kGroups; g += 2) {
    uint32_t r0[32], r1[32];
    tmem_ld_32x32b_x32(taddr0 + (uint32_t)(g * 64), r0);
    tmem_ld_32x32b_x32(taddr0 + (uint32_t)(g * 64 + 32), r1);
    tmem_wait_ld();
    MMT_TRACE_STAMP(10 + g);
    if (g == last_g) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release_acc(release_bar, remote);
    }
    MMT_TRACE_STAMP(20 + g);
    const int colg = col_tile0 + g * 64;
    if (colg >= N) continue;
    uint4 o[8];
#pragma unroll
    for (int j8 = 0; j8 < 8; ++j8) {
      const int col = colg + j8 * 8;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(j8 < 4 ? r0[j8 * 8 + j] : r1[(j8 - 4) * 8 + j]);
      if (kBias || kResid) {
        if (col < N) {
          if (kBias) {
            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
            const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16x2(bw[j]);
              v[2 * j] += f.x;
              v[2 * j + 1] += f.y;
            }
          }
          if (kResid && row_ok) {
            const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + grow * p.ldr + col);
            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16x2(rw[j]);
              v[2 * j] += f.x;
              v[2 * j + 1] += f.y;
            }
          }
        }
      }
      o[j8].x = pack_bf16x2(v[0], v[1]);
      o[j8].y = pack_bf16x2(v[2], v[3]);
      o[j8].z = pack_bf16x2(v[4], v[5]);
      o[j8].w = pack_bf16x2(v[6], v[7]);
    }
    if (bulk) {
      if (lane == 0) tma_store_wait_read();          // the previous bulk store has read the slab
      __syncwarp();
    }
#pragma unroll
    for (int j8 = 0; j8 < 8; ++j8) *reinterpret_cast<uint4*>(slab + store_box_offset(lane, j8 * 8)) = o[j8];
    MMT_TRACE_STAMP(30 + g);
    if (bulk) {
      fence_proxy_async_smem();
      __syncwarp();
      bool stored = true;
      if (p.sc_row) {
        // one owner, one column block and 32 consecutive destination rows, or else plain stores below
        const int part = colg / p.sc_part, within = colg - part * p.sc_part, owner = within / p.sc_w;
        const int in_owner = within - owner * p.sc_w;
        stored = sc_rows_in_a_run && colg + 64 <= N && within + 64 <= p.sc_part && in_owner + 64 <= p.sc_w;
        if (stored && lane == 0) {
          tma_store_2d(&tmC.m[owner], slab, part * p.sc_w + in_owner, sc_first);
          tma_store_commit();
        }
      } else if (lane == 0) {
        if (srow0 < p.M) {
          if (p.rs_rows) {
            const int owner = srow0 / p.rs_rows;      // rs_rows is a multiple of 32: a slab has one owner
            tma_store_2d(&tmC.m[owner], slab, colg, srow0 - owner * p.rs_rows);
          } else {
            tma_store_2d(&tmC.m[0], slab, colg, srow0);
          }
        }
        tma_store_commit();
      }
      if (stored) {
        MMT_TRACE_STAMP(40 + g);
        continue;
      }
    }
    __syncwarp();
    const int col = colg + chunk * 8;
    if (p.sc_row) {
      if (col < N) {
        const int part = col / p.sc_part, within = col - part * p.sc_part, owner = within / p.sc_w;
        const long dcol = (long)part * p.sc_w + (within - owner * p.sc_w);
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.rs_base[owner]);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int row = it * 4 + sub;
          const long gr = (long)srow0 + row;
          if (gr < p.M)
            *reinterpret_cast<uint4*>(base + (long)p.sc_row[gr] * p.sc_ld + dcol) =
                *reinterpret_cast<const uint4*>(slab + store_box_offset(row, chunk * 8));
        }
      }
    } else if (col < N) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int row = it * 4 + sub;
        const long gr = (long)srow0 + row;
        if (gr < p.M) {
          const uint4 val = *reinterpret_cast<const uint4*>(slab + store_box_offset(row, chunk * 8));
          __nv_bfloat16* dst;
          if (p.rs_rows) {
            const int owner = (int)(gr / p.rs_rows);
            dst = reinterpret_cast<__nv_bfloat16*>(p.rs_base[owner]) +
                  ((long)p.rs_self * p.rs_rows + (gr - (long)owner * p.rs_rows)) * p.ldc + col;
          } else {
            dst = reinterpret_cast<__nv_bfloat16*>(p.C) + gr * p.ldc + col;
          }
          *reinterpret_cast<uint4*>(dst) = val;
        }
      }
    }
    __syncwarp();
    MMT_TRACE_STAMP(40 + g);
  }
}

// Picks the straight-line epilogue when the GEMM's options allow it.
template <int BN>
MMT_DEVICE void epilogue_any(const GemmParams& p, const OutMaps& tmC, bool remote, uint32_t tmem_acc, int row0,
                             int col_tile0, int q, int half, int lane, uint8_t* slab, uint32_t release_bar,
                             const float* sk_part = nullptr, int sk_n = 0, long sk_stride = 0) {
  const bool fast = p.alpha == 1.0f && p.act == 0 && !p.accumulate && !p.out_f32 && sk_n == 0 && !(MMT_DBG & 12);
  if (!fast) {
    epilogue_block<BN>(p, tmem_acc, row0, col_tile0, q, half, lane, slab, release_bar, sk_part, sk_n, sk_stride);
  } else if (p.bias) {
    if (p.residual) epilogue_fast<BN, true, true>(p, tmC, tmem_acc, row0, col_tile0, q, half, lane, slab, release_bar, remote);
    else epilogue_fast<BN, true, false>(p, tmC, tmem_acc, row0, col_tile0, q, half, lane, slab, release_bar, remote);
  } else {
    if (p.residual) epilogue_fast<BN, false, true>(p, tmC, tmem_acc, row0, col_tile0, q, half, lane, slab, release_bar, remote);
    else epilogue_fast<BN, false, false>(p, tmC, tmem_acc, row0, col_tile0, q, half, lane, slab, release_bar, remote);
  }
}

// Stream-K run that stops before the end of its tile: the accumulator goes to this CTA's workspace slot as fp32.
template <int BN>
MMT_DEVICE void epilogue_partial(uint32_t tmem_acc, float* dst, int q, int half, int lane, uint32_t release_bar) {
  constexpr int kGroups = BN / 64;
  const uint32_t taddr0 = tmem_acc + ((uint32_t)(q * 32) << 16);
  int last_g = -1;
  for (int g = half; g < kGroups; g += 2) last_g = g;
  if (last_g < 0) {
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(release_bar);
    return;
  }
#pragma unroll 1
  for (int g = half; g < kGroups; g += 2) {
    uint32_t r0[32], r1[32];
    tmem_ld_32x32b_x32(taddr0 + (uint32_t)(g * 64), r0);
    tmem_ld_32x32b_x32(taddr0 + (uint32_t)(g * 64 + 32), r1);
    tmem_wait_ld();
    if (g == last_g) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(release_bar);
    }
    // [64-column group][16-byte chunk][row]: every store request of a warp covers 512 contiguous bytes
    uint4* out = reinterpret_cast<uint4*>(dst) + (long)g * 16 * 128 + (q * 32 + lane);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      out[i * 128] = make_uint4(r0[4 * i], r0[4 * i + 1], r0[4 * i + 2], r0[4 * i + 3]);
      out[(8 + i) * 128] = make_uint4(r1[4 * i], r1[4 * i + 1], r1[4 * i + 2], r1[4 * i + 3]);
    }
  }
}

MMT_DEVICE void epi_bar_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }

// Does the CTA that computes tile (tm, tn) also forward the tile's rows of A to the peers?  (GemmParams::fwd_peers)
MMT_DEVICE bool forwards_tile(const GemmParams& p, int tm, int tn, int bmt) {
  if (p.fwd_peers <= 0 || tn >= p.fwd_split) return false;
  const int r0 = tm * bmt, own0 = p.ag_self * p.ag_rows;
  return r0 >= own0 && r0 < own0 + p.ag_rows;
}

// Consumer half: rows [r0, r1] of the gathered A are complete once the chunk flags of their (source rank, chunk)
// pairs carry this launch's epoch.  `seen` remembers the pairs this thread has already waited for.
MMT_DEVICE bool ag_wait_chunks(const GemmParams& p, int r0, int r1, uint32_t (&seen)[16]) {
  for (int row = r0; row <= r1;) {
    const int src = row / p.ag_rows;
    if (src == p.ag_self) {                            // own rows were written by this stream before the launch
      row = (src + 1) * p.ag_rows;
      continue;
    }
    const int c = (row - src * p.ag_rows) / p.ag_chunk;
    const int idx = src * kAgChunks + c;
    if (!((seen[idx >> 5] >> (idx & 31)) & 1u)) {
      if (!flag_wait_ge(&p.ag_flags[idx], p.ag_epoch, MMT_WAIT_NS, p.ew, 111)) return false;
      seen[idx >> 5] |= 1u << (idx & 31);
    }
    row = src * p.ag_rows + (c + 1) * p.ag_chunk;      // first row of the next chunk (or of the next rank)
    if (row > (src + 1) * p.ag_rows) row = (src + 1) * p.ag_rows;
  }
  return true;
}

template <int BN, int MT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ OutMaps tmC, const GemmParams p) {
  using C_ = Cfg<BN, MT>;
  constexpr int kStages = C_::kStages;
  constexpr int BMT = C_::BMT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sStore = smem + (size_t)kStages * C_::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStore + C_::STORE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;   // [2]: accumulator slot filled
  uint64_t* tempty = tfull + 2;           // [2]: accumulator slot drained
  // all-gather forwarding only: the MMA thread tells the forwarder that a stage of a forwarded tile has landed
  // (fwd_go), the forwarder tells the TMA producer that its stores have read the stage (fwd_done).  Both rings see
  // one phase per FORWARDED use of a stage, and each has a single waiter that follows every phase.
  uint64_t* fwd_go = tempty + 2;          // [kStages]
  uint64_t* fwd_done = fwd_go + kStages;  // [kStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fwd_done + kStages);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  long long clk_c0 = 0;
  unsigned long long clk_t0 = 0;
  if (MMT_CLK && blockIdx.x == 0 && threadIdx.x == 0) {
    clk_c0 = clock64();
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(clk_t0));
  }
  const int tiles_m = (p.M + BMT - 1) / BMT;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int ntiles = tiles_m * tiles_n;
  const int KB = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&fwd_go[s], 1);
      mbar_init(&fwd_done[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], kEpiWarps);
    mbar_init(&tempty[1], kEpiWarps);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C_::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      uint32_t ag_seen = p.ag_flags ? (1u << p.ag_self) : 0u;
      uint32_t ag_chunk_seen[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
      uint32_t fwd_pending = 0, fwd_parity = 0;   // per stage: last use is being forwarded / parity of that hand-back
      // K-slice consumer: source ranks already waited for (own slice needs no wait), all of them, first k-block
      uint32_t kf_seen = p.kf_flags ? (1u << p.kf_self) : 0u;
      const uint32_t kf_all = p.kf_flags ? ((1u << p.kf_ranks) - 1u) : 0u;
      const int kf_kb0 = p.kf_flags ? (p.kf_self * p.kf_w) / BK : 0;
      int kcount = 0;
      WorkItem w;
      for (int wi = 0; ok && work_item(p, wi, blockIdx.x, gridDim.x, KB, ntiles, w); ++wi) {
        int tm, tn;
        tile_coords(p, w.tile, tiles_m, BMT, tm, tn);
        const bool fwd_tile = forwards_tile(p, tm, tn, BMT);
        const bool own_direct = p.fwd_direct && tm * BMT >= p.ag_self * p.ag_rows && tm * BMT < (p.ag_self + 1) * p.ag_rows;
        if (p.ag_flags) {
          const int r0 = tm * BMT, r1 = min(r0 + BMT, p.M) - 1;
          if (p.ag_chunk > 0) {
            ok = ag_wait_chunks(p, r0, r1, ag_chunk_seen);
          } else {
            for (int src = r0 / p.ag_rows; src <= r1 / p.ag_rows && ok; ++src) {
              if (ag_seen & (1u << src)) continue;
              ok = flag_wait_ge(&p.ag_flags[src], p.ag_epoch, MMT_WAIT_NS, p.ew, 110);
              ag_seen |= 1u << src;
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        // K-slice consumer: only until every source has been seen once (normally the CTA's first tile); after that
        // the k-blocks are walked in plain order with no per-block work in this thread
        const bool kf_tile = p.kf_flags && kf_seen != kf_all;
        for (int kb0 = w.k0; kb0 < w.k1; ++kb0) {
          int kb = kb0;
          if (kf_tile) {
            // start with this rank's own columns of A, wait for a peer's slice when it is reached
            kb = kb0 + kf_kb0;
            if (kb >= KB) kb -= KB;
            const int s0 = (kb * BK) / p.kf_w, s1 = min((kb * BK + BK - 1) / p.kf_w, p.kf_ranks - 1);
            bool waited = false;
            for (int src = s0; src <= s1 && ok; ++src) {
              if (kf_seen & (1u << src)) continue;
              ok = flag_wait_ge(&p.kf_flags[src], p.kf_epoch, MMT_WAIT_NS, p.ew, 112);
              kf_seen |= 1u << src;
              waited = true;
            }
            if (!ok) break;
            if (waited) asm volatile("fence.proxy.async;" ::: "memory");
          }
          if ((MMT_DBG & 1) && kcount++ >= kStages) continue;
          if (!mbar_wait(&empty[s], ph ^ 1, p.ew, 100)) { ok = false; break; }
          if (fwd_pending & (1u << s)) {
            // the stage's previous contents also went to the peers: the forwarder's stores must have read them
            if (!mbar_wait(&fwd_done[s], (fwd_parity >> s) & 1u, p.ew, 101)) { ok = false; break; }
            fwd_parity ^= 1u << s;
            fwd_pending &= ~(1u << s);
          }
          if (fwd_tile && kb % p.fwd_split == tn) fwd_pending |= 1u << s;
          uint8_t* sA = smem + (size_t)s * C_::STAGE_BYTES;
          uint8_t* sB = sA + C_::A_BYTES;
          mbar_expect_tx(&full[s], C_::STAGE_BYTES);
          if (own_direct) {
            tma_load_2d(sA, &tmC.m[9], &full[s], kb * BK, tm * BMT - p.ag_self * p.ag_rows);
          } else if (!p.a_mn) {
            tma_load_2d(sA, &tmA, &full[s], kb * BK, tm * BMT);      // one box of BMT rows
          } else {
#pragma unroll
            for (int c = 0; c < BMT / 64; ++c) tma_load_2d(sA + c * 8192, &tmA, &full[s], tm * BMT + c * 64, kb * BK);
          }
          if (!p.b_mn) {
            tma_load_2d(sB, &tmB, &full[s], kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sB + c * 8192, &tmB, &full[s], tn * BN + c * 64, kb * BK);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      // descriptor halves, encoded once: per instruction only the start-address field moves
      const uint32_t a_hi = smem_desc_hi(p.a_mn ? p.mn_sbo : 1024u), b_hi = smem_desc_hi(p.b_mn ? p.mn_sbo : 1024u);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), p.a_mn ? p.mn_lbo : 16u);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem) + C_::A_BYTES, p.b_mn ? p.mn_lbo : 16u);
      const uint32_t a_k = (p.a_mn ? p.mn_kstep : (uint32_t)(UMMA_K * 2)) >> 4;
      const uint32_t b_k = (p.b_mn ? p.mn_kstep : (uint32_t)(UMMA_K * 2)) >> 4;
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;   // MT == 1: acc alternates per tile; MT == 2: slots 0/1 are the halves
      bool ok = true;
      int kcount = 0;
      // The issue loop is kept as short as it can be: this one thread has to hand the tensor core an instruction
      // every ~128 cycles.  Whether the NEXT ring slot is full is looked up (non-blocking) in the shadow of the
      // current slot's instructions, so the common case never waits for a barrier round trip.
      bool ready = false;
      WorkItem w;
      for (int wi = 0; ok && work_item(p, wi, blockIdx.x, gridDim.x, KB, ntiles, w); ++wi) {
        // the accumulator (MT == 1) or both halves (MT == 2) of an earlier tile must have been drained
        if (!mbar_wait(&tempty[MT == 2 ? 0 : acc], acc_ph ^ 1, p.ew, 200)) { ok = false; break; }
        if (MT == 2 && !mbar_wait(&tempty[1], acc_ph ^ 1, p.ew, 202)) { ok = false; break; }
        tc_fence_after();
        int fwd_tn = -1;                 // >= 0: this tile forwards its k-blocks kb % fwd_split == fwd_tn
        if (p.fwd_peers > 0) {
          int tm, tn;
          tile_coords(p, w.tile, tiles_m, BMT, tm, tn);
          if (forwards_tile(p, tm, tn, BMT)) fwd_tn = tn;
        }
        const uint32_t d0 = tmem_base + (uint32_t)((MT == 2 ? 0 : acc) * BN);
        for (int kb = 0; kb < w.k1 - w.k0; ++kb) {      // kb counts from the start of this run: a fresh accumulator
          const bool skip = (MMT_DBG & 1) && kcount++ >= kStages;
          if (!ready && !skip && !mbar_wait(&full[s], ph, p.ew, 201)) { ok = false; break; }
          const uint32_t so = (uint32_t)s * (C_::STAGE_BYTES >> 4);
          int sn = s + 1;
          uint32_t phn = ph;
          if (sn == kStages) { sn = 0; phn ^= 1; }
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t bdesc = smem_desc_join(b_hi, b_lo0 + so + (uint32_t)k * b_k);
#pragma unroll
            for (int h = 0; h < MT; ++h) {
              // half h: 128 rows further (K-major) or two 64-column chunks further (MN-major)
              const uint64_t adesc =
                  smem_desc_join(a_hi, a_lo0 + so + (uint32_t)h * ((BM * BK * 2) >> 4) + (uint32_t)k * a_k);
              tc_mma_ss(d0 + (uint32_t)(h * BN), adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            if (k == 0) ready = mbar_test(&full[sn], phn);
          }
          // the stage has landed: the forwarder may send it on
          if (fwd_tn >= 0 && (w.k0 + kb) % p.fwd_split == fwd_tn) mbar_arrive(&fwd_go[s]);
          if (!(MMT_DBG & 2)) tc_commit(&empty[s]);
          s = sn;
          ph = phn;
        }
        if (!ok) break;
        if (MT == 1) {
          tc_commit(&tfull[acc]);
          acc ^= 1;
          if (acc == 0) acc_ph ^= 1;
        } else {
          tc_commit(&tfull[0]);
          tc_commit(&tfull[1]);
          acc_ph ^= 1;
        }
      }
    }
  } else if (warp >= 2 + kEpiWarps) {
    // ------------------------------ all-gather forwarder (one thread) ----------
    if (p.fwd_peers > 0 && lane == 0) {
      uint32_t use = 0;                  // ring slots handed out so far (the TMA producer counts the same way)
      uint32_t go_parity = 0;            // per stage: parity of the next fwd_go phase
      bool ok = true;
      WorkItem w;
      for (int wi = 0; ok && work_item(p, wi, blockIdx.x, gridDim.x, KB, ntiles, w); ++wi) {
        int tm, tn;
        tile_coords(p, w.tile, tiles_m, BMT, tm, tn);
        if (!forwards_tile(p, tm, tn, BMT)) {
          use += (uint32_t)(w.k1 - w.k0);
          continue;
        }
        for (int kb = w.k0; kb < w.k1; ++kb, ++use) {
          if (kb % p.fwd_split != tn) continue;
          const uint32_t s = use % (uint32_t)kStages;
          if (!mbar_wait(&fwd_go[s], (go_parity >> s) & 1u, p.ew, 400)) { ok = false; break; }
          go_parity ^= 1u << s;
          const uint8_t* sA = smem + (size_t)s * C_::STAGE_BYTES;
          for (int q = 0; q < p.fwd_dsts; ++q) tma_store_2d(&tmC.m[1 + q], sA, kb * BK, tm * BMT);
          tma_store_commit();
          tma_store_wait_read();         // shared memory has been read; the stage may be refilled
          mbar_arrive(&fwd_done[s]);
        }
        if (!ok) break;
        tma_store_wait_all();            // this CTA's share of the row block has been written everywhere ...
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence_system();
        const int block = (tm * BMT - p.ag_self * p.ag_rows) / BMT;
        const int parts = min(p.fwd_split, tiles_n);
        if (atomicAdd(&p.fwd_counter[block], 1) == parts - 1) {
          p.fwd_counter[block] = 0;      // ready for the next launch
          __threadfence_system();
          for (int q = 0; q < p.fwd_peers; ++q)   // ... and the last share announces the block
            flag_store_release_sys(p.fwd_flag[q] + p.ag_self * kAgChunks + block, p.ag_epoch);
        }
      }
    }
  } else {
    // ------------------------------ epilogue (8 warps) -------------------------
    const int q = warp & 3;              // tensor-memory lane quadrant this warp may read
    const int half = (warp - 2) >> 2;    // which groups of 64 columns this warp takes
    uint8_t* slab = sStore + (size_t)(warp - 2) * kSlabBytes;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    WorkItem w;
    constexpr long kSlot = (long)BMT * BN;      // floats per stream-K workspace slot
    for (int wi = 0; ok && work_item(p, wi, blockIdx.x, gridDim.x, KB, ntiles, w); ++wi) {
      int tm, tn;
      tile_coords(p, w.tile, tiles_m, BMT, tm, tn);
      const int n_contrib = (w.kind == 2 && !(MMT_DBG & 32)) ? (int)blockIdx.x - w.first_contrib : 0;
      if (w.kind == 2 && !(MMT_DBG & 16)) {
        // the CTAs that did the first k-blocks of this tile have left their partial sums
        for (int c = w.first_contrib; c < (int)blockIdx.x && ok; ++c)
          ok = flag_wait_ge(&p.sk_flags[c], p.sk_epoch, MMT_WAIT_NS, p.ew, 310);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll 1
      for (int h = 0; h < MT; ++h) {
        const int slot = MT == 2 ? h : acc;
        MMT_TRACE_STAMP(1);
        ok = mbar_wait(&tfull[slot], acc_ph, p.ew, 300);
        MMT_TRACE_STAMP(2);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (w.kind == 1 && (MMT_DBG & 64)) {       // measurement only: drop the partial sums
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(smem_u32(&tempty[slot]));
        } else if (w.kind == 1) {
          epilogue_partial<BN>(tmem_base + (uint32_t)(slot * BN), p.sk_ws + (long)blockIdx.x * kSlot + (long)h * BM * BN,
                               q, half, lane, smem_u32(&tempty[slot]));
        } else {
          epilogue_any<BN>(p, tmC, false, tmem_base + (uint32_t)(slot * BN), tm * BMT + h * BM, tn * BN, q, half, lane, slab,
                             smem_u32(&tempty[slot]), p.sk_ws + (long)w.first_contrib * kSlot + (long)h * BM * BN,
                             n_contrib, kSlot);
        }
      }
      if (!ok) break;
      if (w.kind == 1) {
        // every epilogue warp has stored its part: publish "the partial sums of CTA blockIdx.x are complete"
        __threadfence();
        epi_bar_sync();
        if (warp == 2 && lane == 0) flag_store_release_sys(&p.sk_flags[blockIdx.x], p.sk_epoch);
      }
      if (MT == 1) {
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      } else {
        acc_ph ^= 1;
      }
    }
  }

  if (warp >= 2 && warp < 2 + kEpiWarps && lane == 0) {
    tma_store_wait_all();                       // every bulk store of this warp has been written out
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  if (p.rs_rows || p.sc_row) __threadfence_system();   // this thread's peer stores are visible system-wide
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C_::TMEM_COLS);
  if (MMT_CLK && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    MMT_CLK[0] = (unsigned long long)(clock64() - clk_c0);
    MMT_CLK[1] = t1 - clk_t0;
  }
  if ((p.rs_rows || p.sc_row) && threadIdx.x == 0) {
    // last CTA to finish publishes "my partial sums have landed" to every peer
    if (atomicAdd(p.rs_counter, 1) == (int)gridDim.x - 1) {
      *p.rs_counter = 0;
      __threadfence_system();
      for (int r = 0; r < p.rs_ranks; ++r) flag_store_release_sys(p.rs_flag[r], p.rs_epoch);
    }
  }
}

// ------------------------------------------------------------------------------------
// 2-CTA kernel (cta_group::2): a pair of CTAs on neighbouring SMs computes one 256 x 256 tile.
//
// Each CTA stages its own 128 rows of A and HALF of the B tile (128 of the 256 output columns), the
// leader CTA issues tcgen05.mma.cta_group::2 with M = 256, and each CTA's tensor memory receives its
// 128 x 256 half of the accumulator.  Compared with the 1-CTA kernel every B byte is read from
// shared memory once per 256 rows instead of once per 128, which is what lifts the shared-memory
// bandwidth bound of 128 x 256 tiles.  Every CTA loads exactly what it keeps (plain TMA loads only).
//
// Barriers: full[s] lives in the leader and counts the bytes of BOTH CTAs' TMA loads (the follower's
// loads signal the leader's barrier); empty[s] and tfull[a] exist in both CTAs and the leader's
// tcgen05.commit arrives on each of them; tempty[a] lives in the leader and collects the epilogue
// warps of both CTAs.
// ------------------------------------------------------------------------------------
struct PairCfg {
  static constexpr int BN = 256;                      // tile columns (128 per CTA in shared memory)
  static constexpr uint32_t A_BYTES = BM * BK * 2;    // this CTA's 128 rows of A
  static constexpr uint32_t B_BYTES = 128 * BK * 2;   // this CTA's half of the B tile
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t STORE_BYTES = kEpiWarps * kSlabBytes;
  static constexpr int kStages = 6;
  static constexpr uint32_t TMEM_COLS = 512;          // two 256-column accumulators
  static constexpr size_t SMEM = 1024 + (size_t)kStages * STAGE_BYTES + STORE_BYTES + (2 * kStages + 4) * 8 + 16;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ OutMaps tmC, const GemmParams p) {
  using C_ = PairCfg;
  constexpr int kStages = C_::kStages;
  constexpr int BN = C_::BN;
  constexpr int BMT = 2 * BM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sStore = smem + (size_t)kStages * C_::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStore + C_::STORE_BYTES);
  uint64_t* full = bars;                  // used in the leader only
  uint64_t* empty = bars + kStages;       // both CTAs
  uint64_t* tfull = bars + 2 * kStages;   // both CTAs
  uint64_t* tempty = tfull + 2;           // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  long long clk_c0 = 0;
  unsigned long long clk_t0 = 0;
  if (MMT_CLK && blockIdx.x == 0 && threadIdx.x == 0) {
    clk_c0 = clock64();
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(clk_t0));
  }
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int tiles_m = (p.M + BMT - 1) / BMT;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int ntiles = tiles_m * tiles_n;
  const int KB = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 2 * kEpiWarps);   // the epilogue warps of both CTAs
    mbar_init(&tempty[1], 2 * kEpiWarps);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, C_::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers are initialised before anybody signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      uint32_t ag_seen = p.ag_flags ? (1u << p.ag_self) : 0u;
      int kcount = 0;
      for (int tile = pair; tile < ntiles && ok; tile += npairs) {
        int tm, tn;
        tile_coords(p, tile, tiles_m, BMT, tm, tn);
        const int row0 = tm * BMT + (int)rank * BM;      // this CTA's rows of A
        const int col0 = tn * BN + (int)rank * 128;      // this CTA's half of the B tile
        if (p.ag_flags && row0 < p.M) {
          const int r1 = min(row0 + BM, p.M) - 1;
          for (int src = row0 / p.ag_rows; src <= r1 / p.ag_rows && ok; ++src) {
            if (ag_seen & (1u << src)) continue;
            ok = flag_wait_ge(&p.ag_flags[src], p.ag_epoch, MMT_WAIT_NS, p.ew, 120);
            ag_seen |= 1u << src;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < KB; ++kb) {
          if ((MMT_DBG & 1) && kcount++ >= kStages) continue;
          if (!mbar_wait(&empty[s], ph ^ 1, p.ew, 121)) { ok = false; break; }
          uint8_t* sA = smem + (size_t)s * C_::STAGE_BYTES;
          uint8_t* sB = sA + C_::A_BYTES;
          const uint32_t lbar = map_to_cta(smem_u32(&full[s]), 0);
          if (leader) mbar_expect_tx(&full[s], 2 * C_::STAGE_BYTES);   // the loads of both CTAs
          if (!p.a_mn) {
            tma_load_2d_pair(sA, &tmA, lbar, kb * BK, row0);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_pair(sA + c * 8192, &tmA, lbar, row0 + c * 64, kb * BK);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sB, &tmB, lbar, kb * BK, col0);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_pair(sB + c * 8192, &tmB, lbar, col0 + c * 64, kb * BK);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && leader) {
      // One 256 x 256 MMA per k-step.  (Splitting it into two 256 x 128 MMAs on alternating accumulators, to avoid
      // back-to-back MMAs into one accumulator, was measured and is slower: at N = 128 every CTA reads as many operand
      // bytes per MMA cycle -- its A rows, its own B rows and the partner's -- as shared memory delivers.)
      const uint32_t idesc = make_idesc_bf16(BMT, BN, p.a_mn, p.b_mn);
      const uint32_t a_hi = smem_desc_hi(p.a_mn ? p.mn_sbo : 1024u), b_hi = smem_desc_hi(p.b_mn ? p.mn_sbo : 1024u);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), p.a_mn ? p.mn_lbo : 16u);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem) + C_::A_BYTES, p.b_mn ? p.mn_lbo : 16u);
      const uint32_t a_k = (p.a_mn ? p.mn_kstep : (uint32_t)(UMMA_K * 2)) >> 4;
      const uint32_t b_k = (p.b_mn ? p.mn_kstep : (uint32_t)(UMMA_K * 2)) >> 4;
      const uint32_t empty0 = map_to_cta(smem_u32(&empty[0]), 0), empty1 = map_to_cta(smem_u32(&empty[0]), 1);
      const uint32_t tfull0 = map_to_cta(smem_u32(&tfull[0]), 0), tfull1 = map_to_cta(smem_u32(&tfull[0]), 1);
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      int kcount = 0;
      bool ready = false;   // see the 1-CTA kernel: the next slot's barrier is probed behind this slot's MMAs
      for (int tile = pair; tile < ntiles && ok; tile += npairs) {
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.ew, 220)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < KB; ++kb) {
          const bool skip = (MMT_DBG & 1) && kcount++ >= kStages;
          if (!ready && !skip && !mbar_wait(&full[s], ph, p.ew, 221)) { ok = false; break; }
          const uint32_t so = (uint32_t)s * (C_::STAGE_BYTES >> 4);
          int sn = s + 1;
          uint32_t phn = ph;
          if (sn == kStages) { sn = 0; phn ^= 1; }
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = smem_desc_join(a_hi, a_lo0 + so + (uint32_t)k * a_k);
            const uint64_t bdesc = smem_desc_join(b_hi, b_lo0 + so + (uint32_t)k * b_k);
            tc_mma_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            if (k == 0) ready = mbar_test(&full[sn], phn);
          }
          if (!(MMT_DBG & 2)) {
            tc_commit_pair(empty0 + (uint32_t)s * 8u);     // the stage is free again in both CTAs
            tc_commit_pair(empty1 + (uint32_t)s * 8u);
          }
          s = sn;
          ph = phn;
        }
        if (!ok) break;
        tc_commit_pair(tfull0 + (uint32_t)acc * 8u);       // both halves of the accumulator are complete
        tc_commit_pair(tfull1 + (uint32_t)acc * 8u);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------ epilogue (both CTAs, 8 warps each) ------------------------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint8_t* slab = sStore + (size_t)(warp - 2) * kSlabBytes;
    int acc = 0;
    uint32_t acc_ph = 0;
    for (int tile = pair; tile < ntiles; tile += npairs) {
      int tm, tn;
      tile_coords(p, tile, tiles_m, BMT, tm, tn);
      bool ok = mbar_wait(&tfull[acc], acc_ph, p.ew, 320);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      epilogue_any<BN>(p, tmC, true, tmem_base + (uint32_t)(acc * BN), tm * BMT + (int)rank * BM, tn * BN, q, half, lane,
                         slab, map_to_cta(smem_u32(&tempty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1;
    }
    if (lane == 0) {
      tma_store_wait_all();                     // every bulk store of this warp has been written out
      asm volatile("fence.proxy.async;" ::: "memory");
    }
  }

  if (p.rs_rows) __threadfence_system();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // nobody leaves (or frees tensor memory) while the peer may still touch it
  if (warp == 1) tmem_dealloc_pair(tmem_base, C_::TMEM_COLS);
  if (MMT_CLK && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    MMT_CLK[0] = (unsigned long long)(clock64() - clk_c0);
    MMT_CLK[1] = t1 - clk_t0;
  }
  if (p.rs_rows && threadIdx.x == 0) {
    if (atomicAdd(p.rs_counter, 1) == (int)gridDim.x - 1) {
      *p.rs_counter = 0;
      __threadfence_system();
      for (int r = 0; r < p.rs_ranks; ++r) flag_store_release_sys(p.rs_flag[r], p.rs_epoch);
    }
  }
}

// ------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

bool ensure_encode() {
  if (g_encode) return true;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
    return false;
  g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  return true;
}

int g_l2promo = 3;   // CUtensorMapL2promotion of operand maps: 0 none, 1 64 B, 2 128 B, 3 256 B
uint32_t g_mn_lbo = 8192, g_mn_sbo = 1024, g_mn_kstep = 2048;

template <int BN, int MT>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tc, const GemmParams& p, int sms,
           cudaStream_t st) {
  using C_ = Cfg<BN, MT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05<BN, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)C_::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tiles = ((p.M + C_::BMT - 1) / C_::BMT) * ((p.N + BN - 1) / BN);
  const int grid = (tiles < sms && p.sk_tiles == 0) ? tiles : sms;
  gemm_bf16_tcgen05<BN, MT><<<grid, kThreads, C_::SMEM, st>>>(ta, tb, tc, p);
  return (int)cudaGetLastError();
}

int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tc, const GemmParams& p, int sms,
                cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_pair, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)PairCfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + PairCfg::BN - 1) / PairCfg::BN);
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  gemm_bf16_tcgen05_pair<<<2 * pairs, kThreads, PairCfg::SMEM, st>>>(ta, tb, tc, p);
  return (int)cudaGetLastError();
}

// stream-K workspace of this process's device: one fp32 slot per CTA and one flag word per CTA
float* g_sk_ws = nullptr;
int* g_sk_flags = nullptr;
int g_sk_epoch = 0;
// Stream-K is OFF unless asked for (MMT_GEMM_STREAM_K=1 or mmt_gemm_set_stream_k(1)): on isolated GEMMs with a
// partial last wave it saves 5-17 % (e.g. 2048 x 3584 x 18944: 247 -> 204 us with 128-row tiles), but inside a
// training step at the board's power cap its extra partial-sum traffic costs as much as the idle SMs it fills
// (7B step on one B200: 204.5 ms without, 205.9 ms with).
int g_sk_mode = -1;           // 1 = on, 0 = off, -1 = not yet read from the environment
double g_mt2_const = -1.0;    // fixed cost of a 256-row tile in the tile-shape model (MMT_GEMM_MT2_CONST overrides)

void read_env_once() {
  if (g_sk_mode < 0) {
    const char* e = getenv("MMT_GEMM_STREAM_K");
    g_sk_mode = (e && e[0] == '1') ? 1 : 0;
  }
  if (g_mt2_const < 0.0) {
    const char* e = getenv("MMT_GEMM_MT2_CONST");
    g_mt2_const = e ? atof(e) : 4.06;
  }
}
cudaEvent_t g_sk_event = nullptr;
cudaStream_t g_sk_stream = nullptr;
constexpr int kSkMaxCtas = 160;

bool sk_ready() {
  if (g_sk_ws) return true;
  if (cudaMalloc(&g_sk_ws, (size_t)kSkMaxCtas * 256 * 256 * sizeof(float)) != cudaSuccess) return false;
  if (cudaMalloc(&g_sk_flags, kSkMaxCtas * sizeof(int)) != cudaSuccess) return false;
  cudaMemset(g_sk_flags, 0, kSkMaxCtas * sizeof(int));
  cudaEventCreateWithFlags(&g_sk_event, cudaEventDisableTiming);
  return true;
}

// Number of trailing tiles to cut along K (0 = none): worth it when the last wave is clearly partial and every CTA
// still gets a few k-blocks of it.
int sk_tiles_for(int tiles, long kb, int sms, int mt) {
  read_env_once();
  if (!g_sk_mode || sms > kSkMaxCtas || kb < 4) return 0;
  const int rem = tiles % sms;
  if (rem == 0 || rem > (sms * 17) / 20) return 0;
  // each CTA needs a run long enough to pay for its partial-sum traffic (128 KB per 128-row accumulator)
  if ((long)rem * kb < (mt == 2 ? 48L : 24L) * sms) return 0;
  return rem;
}

int g_force_bn = 0;   // 0 = choose, else the tile width (64 / 128 / 192 / 256) of every following GEMM
int g_force_mt = 0;   // 0 = choose, 1 / 2 = force the number of 128-row accumulators per tile, 3 = 2-CTA kernel
int g_use_pair = 0;
int g_group_m = 0;
unsigned long long* g_clk = nullptr;
int g_dbg = 0;

}  // namespace

// 2-D bf16 tensor map with 128-byte swizzle.  `inner` elements are contiguous,
// rows are `ld` elements apart; the box is box_inner x box_outer elements.
extern "C" int mmt_make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                                uint32_t box_inner, uint32_t box_outer) {
  if (!ensure_encode()) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, (CUtensorMapL2promotion)g_l2promo,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

// Encoded tensor maps are kept per (address, extents, row stride, box): a training step issues the same few hundred
// GEMMs on the same buffers every iteration, and encoding three maps per launch is host time on the launch path.
namespace {
struct TmapKey {
  uint64_t ptr, inner, outer, ld, box;
  int promo;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && ld == o.ld && box == o.box && promo == o.promo;
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapSlots = 1 << 13;
thread_local TmapSlot* g_tmap_cache = nullptr;

int cached_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                   uint32_t box_outer) {
  if (!g_tmap_cache) g_tmap_cache = static_cast<TmapSlot*>(calloc(kTmapSlots, sizeof(TmapSlot)));
  const TmapKey k{reinterpret_cast<uint64_t>(ptr), inner, outer, ld, ((uint64_t)box_inner << 32) | box_outer, g_l2promo};
  if (!g_tmap_cache) return mmt_make_tmap_2d(out, ptr, inner, outer, ld, box_inner, box_outer);
  uint64_t h = k.ptr * 0x9E3779B97F4A7C15ull ^ (k.inner * 0xC2B2AE3D27D4EB4Full) ^ (k.outer << 17) ^ (k.ld << 7) ^ k.box;
  h ^= h >> 29;
  TmapSlot& slot = g_tmap_cache[h & (kTmapSlots - 1)];
  if (slot.used && slot.key == k) {
    *out = slot.map;
    return 0;
  }
  const int r = mmt_make_tmap_2d(out, ptr, inner, outer, ld, box_inner, box_outer);
  if (r == 0) {
    slot.key = k;
    slot.map = *out;
    slot.used = true;
  }
  return r;
}
}  // namespace

// Tuning knob: 0 = choose per call, 1 = 128-row tiles, 2 = 256-row tiles in one CTA, 3 = 2-CTA kernel.
extern "C" void mmt_gemm_force_mt(int mt) { g_force_mt = mt; }
// Tuning knob: tile width of every following GEMM (0 = choose per call).
extern "C" void mmt_gemm_force_bn(int bn) { g_force_bn = bn; }
// Raster band height in m-tiles (0 = choose, -1 = one band: m-fastest over the whole matrix).
extern "C" void mmt_gemm_group_m(int g) { g_group_m = g; }
#ifdef MMT_GEMM_MEASURE
// Measurement aid: device pointer to two 64-bit words that CTA 0 of every following GEMM fills with the SM
// cycles and the nanoseconds it spent in the kernel (nullptr = off).  cycles / ns = SM clock in GHz under load.
extern "C" void mmt_gemm_set_clock_probe(unsigned long long* p) { g_clk = p; }
#endif
// Tuning knob: L2 promotion size of the tensor maps (0 none, 1 64 B, 2 128 B, 3 256 B).
extern "C" void mmt_gemm_set_l2promo(int v) { g_l2promo = v; }
#ifdef MMT_GEMM_MEASURE
// Measurement only (results are wrong): see GemmParams::dbg.
extern "C" void mmt_gemm_set_dbg(int d) { g_dbg = d; }
#endif
// Default kernel for M >= 256 and 256-wide tiles: 1 = the 2-CTA kernel, 0 = the 1-CTA kernels.
extern "C" void mmt_gemm_use_pair(int on) { g_use_pair = on; }

#ifdef MMT_GEMM_MEASURE
// Bring-up knob: descriptor constants used for MN-major shared-memory tiles.
extern "C" void mmt_gemm_set_mn_desc(uint32_t lbo, uint32_t sbo, uint32_t kstep) {
  g_mn_lbo = lbo;
  g_mn_sbo = sbo;
  g_mn_kstep = kstep;
}
#endif

// Optional collective roles of a GEMM launch (see GemmParams).
struct MmtGemmComm {
  const int* ag_flags;
  int ag_epoch, ag_rows, ag_self;
  // forwarder (fwd_peers == 0: the rows were pushed by an earlier launch): gathered buffers ([ranks * ag_rows, K],
  // row stride lda) and flag arrays of the remote peers
  unsigned long long fwd_dst[8];
  int* fwd_flag[8];
  int fwd_peers;
  // fwd_src != nullptr: this rank's rows are read from here ([ag_rows, K], row stride fwd_src_ld) and also stored to
  // its own gathered buffer A; nullptr: they are in A already
  const void* fwd_src;
  int fwd_src_ld;
  int* fwd_counter;                 // [64] ints, zero between launches
  unsigned long long rs_base[8];
  int* rs_flag[8];
  int* rs_counter;
  int rs_rows, rs_self, rs_ranks, rs_epoch;
  // column scatter (see GemmParams::sc_row): destinations rs_base[r] ([sc_rows_dst, sc_ld]), flags rs_flag / rs_epoch /
  // rs_counter, rs_ranks owners
  const int* sc_row;
  int sc_part, sc_w, sc_ld, sc_rows_dst;
  // K-slice consumer (see GemmParams::kf_flags)
  const int* kf_flags;
  int kf_epoch, kf_w, kf_self, kf_ranks;
};

// Layout of MmtGemmComm as this library was compiled: {sizeof, offsets of a few fields}.  The Python binding mirrors
// the struct with ctypes and compares itself with these numbers when it loads (a mismatch would send peer addresses
// into the wrong fields).  Returns the number of values written.
extern "C" int mmt_gemm_comm_layout(int* out, int n) {
  const int v[] = {(int)sizeof(MmtGemmComm),          (int)offsetof(MmtGemmComm, ag_flags),
                   (int)offsetof(MmtGemmComm, ag_self),     (int)offsetof(MmtGemmComm, fwd_dst),
                   (int)offsetof(MmtGemmComm, fwd_flag),    (int)offsetof(MmtGemmComm, fwd_peers),
                   (int)offsetof(MmtGemmComm, fwd_src),     (int)offsetof(MmtGemmComm, fwd_src_ld),
                   (int)offsetof(MmtGemmComm, fwd_counter), (int)offsetof(MmtGemmComm, rs_base),
                   (int)offsetof(MmtGemmComm, rs_flag),     (int)offsetof(MmtGemmComm, rs_counter),
                   (int)offsetof(MmtGemmComm, rs_rows),     (int)offsetof(MmtGemmComm, rs_epoch),
                   (int)offsetof(MmtGemmComm, sc_row),      (int)offsetof(MmtGemmComm, sc_rows_dst),
                   (int)offsetof(MmtGemmComm, kf_flags),    (int)offsetof(MmtGemmComm, kf_ranks)};
  const int count = (int)(sizeof(v) / sizeof(v[0]));
  for (int i = 0; i < count && i < n; ++i) out[i] = v[i];
  return count;
}

namespace {
const MmtGemmComm* g_comm = nullptr;
}

// Attach collective roles to the NEXT mmt_gemm_bf16 call of this thread of control (cleared by that call).
extern "C" void mmt_gemm_set_comm(const MmtGemmComm* c) { g_comm = c; }

// C = epilogue(alpha * A * B^T).  See the file header for layouts.
//   a_mn / b_mn : 0 = K-major ([rows][K], ld = row stride), 1 = MN-major ([K][rows], ld = k-row stride)
//   act         : 0 none, 1 GELU
//   bn          : 0 = choose, else one of 64/128/192/256
// Returns 0 or a CUDA / driver error code (negative: argument error).
extern "C" int mmt_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual, int M,
                             int N, int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn, int act,
                             int accumulate, int out_f32, float alpha, int bn, void* stream) {
  // collective roles belong to THIS call only: take them before any early return, so that a call that fails its
  // argument checks cannot leave them behind for an unrelated GEMM
  const MmtGemmComm* comm = g_comm;
  g_comm = nullptr;
  if (M <= 0 || N <= 0 || K <= 0) return comm ? -9 : 0;     // peers would wait for flags that an empty GEMM never sets
  if (mmt_ensure_context(A)) return -7;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7) || (residual && (ldr & 7))) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return -3;
  const int sms = mmt_sm_count();
  // Tile shape: rows = 128 (accumulator double buffered in tensor memory, epilogue hidden behind the next tile) or
  // 256 (two accumulators that share every B tile: the main loop alternates between them, which keeps the tensor pipe
  // busier than back-to-back MMAs into one accumulator, but the two fill tensor memory and the epilogue is exposed);
  // width = 192 or 256 columns (narrower only for narrow outputs: a 128-wide MMA is bound by shared-memory reads).
  // Cost of a candidate = waves x (k-blocks x c + e), in units of one 256 x 256 x 64 step, with c and e fitted (least
  // squares over 200 sustained measurements on B200: the step's text shapes, the short-K vision shapes and the
  // tensor-parallel shards, all layouts) per tile shape (rows x width: 128 x 256 c 0.568 e 0.86; 256 x 256 c 0.824
  // e 4.06; 128 x 192 c 0.507 e 0.4; 256 x 192 c 0.726 e 2.61).  What it mostly decides is how well the tile count
  // fills the 148 SMs.
  read_env_once();
  int mt = 1;
  const long kb = (K + BK - 1) / BK;
  const bool plain = comm == nullptr;
  auto cost = [&](int m, int width) {
    const long tiles = (long)((M + 128 * m - 1) / (128 * m)) * ((N + width - 1) / width);
    const long full = tiles / sms, rem = tiles % sms;
    double waves = (double)full + (rem ? 1.0 : 0.0);
    if (rem && plain && width == 256 && sk_tiles_for((int)tiles, kb, sms, m) > 0)
      waves = (double)full + (double)rem / sms + (m == 2 ? 16.0 : 8.0) / (double)kb;
    double c, e;
    if (width == 256) { c = m == 2 ? 0.824 : 0.568; e = m == 2 ? g_mt2_const : 0.86; }
    else              { c = m == 2 ? 0.726 : 0.507; e = m == 2 ? 2.61 : 0.4; }
    return waves * ((double)kb * c + e);
  };
  if (bn == 0 && g_force_bn) bn = g_force_bn;
  if (bn == 0 && N <= 192) bn = N > 128 ? 192 : (N > 64 ? 128 : 64);
  if (bn == 0) {
    double best = 1e30;
    for (int m = 1; m <= (M >= 256 ? 2 : 1); ++m) {
      if (g_force_mt == 1 || g_force_mt == 2) m = g_force_mt;
      for (int width = 192; width <= 256; width += 64) {
        const double c = cost(m, width);
        if (c < best) { best = c; mt = m; bn = width; }
      }
      if (g_force_mt == 1 || g_force_mt == 2) break;
    }
    if (M < 256) mt = 1;
  } else if (bn >= 192) {
    mt = (M >= 256 && cost(2, bn) < cost(1, bn)) ? 2 : 1;
    if (g_force_mt == 1 || g_force_mt == 2) mt = M >= 256 ? g_force_mt : 1;
  } else if (g_force_mt == 2 && M >= 256 && bn == 128) {
    mt = 2;
  }
  if (bn == 256 && M >= 256 && (g_force_mt == 3 || (g_use_pair && g_force_mt == 0)) && !(comm && (comm->fwd_peers > 0 || comm->sc_row || comm->kf_flags)))
    mt = 3;   // 2-CTA kernel
  const int bmt = mt == 3 ? BM : BM * mt;              // rows per TMA box of A
  const int bbox = mt == 3 ? 128 : bn;                 // rows per TMA box of B
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = cached_tmap_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, (uint32_t)bmt);
  else       r = cached_tmap_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK);
  if (r) return 1000 + r;
  if (!b_mn) r = cached_tmap_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, (uint32_t)bbox);
  else       r = cached_tmap_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
  if (r) return 2000 + r;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.act = act; p.accumulate = accumulate; p.out_f32 = out_f32; p.alpha = alpha;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.mn_lbo = g_mn_lbo; p.mn_sbo = g_mn_sbo; p.mn_kstep = g_mn_kstep;
  p.ew = mmt_error_word();
  p.clk = g_clk;
  p.dbg = g_dbg;  // read through MMT_DBG only
  p.tiles_n = (N + bn - 1) / bn;
  // raster bands of 2048 rows: a wave of CTAs then covers a roughly square block of C, so the A and B tiles it
  // needs are shared by many CTAs while they are in L2
  p.group_m = g_group_m > 0 ? g_group_m : (g_group_m < 0 ? 0 : 2048 / (mt == 1 ? BM : 2 * BM));
  p.ag_flags = nullptr;
  p.ag_epoch = p.ag_rows = p.ag_self = 0;
  p.fwd_peers = p.fwd_dsts = p.fwd_split = p.fwd_direct = p.ag_chunk = 0;
  p.fwd_counter = nullptr;
  for (int i = 0; i < 8; ++i) p.fwd_flag[i] = nullptr;
  p.rs_rows = p.rs_self = p.rs_ranks = p.rs_epoch = 0;
  p.rs_counter = nullptr;
  p.sc_row = nullptr;
  p.sc_part = p.sc_w = p.sc_ld = 0;
  p.kf_flags = nullptr;
  p.kf_epoch = p.kf_w = p.kf_self = p.kf_ranks = 0;
  if (comm) {
    const MmtGemmComm* c = comm;
    p.ag_flags = c->ag_flags; p.ag_epoch = c->ag_epoch; p.ag_rows = c->ag_rows; p.ag_self = c->ag_self;
    p.rs_rows = c->rs_rows; p.rs_self = c->rs_self; p.rs_ranks = c->rs_ranks; p.rs_epoch = c->rs_epoch;
    p.rs_counter = c->rs_counter;
    for (int i = 0; i < 8; ++i) { p.rs_base[i] = c->rs_base[i]; p.rs_flag[i] = c->rs_flag[i]; }
    if (p.ag_flags && (p.ag_rows <= 0 || a_mn)) return -5;
    if (c->fwd_peers) {
      // forwarder: chunk flags per tile-high block of rows, so the blocks must tile every rank's rows exactly; the
      // gathered buffers are [ranks * ag_rows, K] on every rank; the reduce-scatter role uses the same map table
      if (!p.ag_flags || c->fwd_peers < 0 || c->fwd_peers > 7 || mt == 3 || p.rs_rows || out_f32 ||
          p.ag_rows % bmt != 0 || p.ag_rows / bmt > kAgChunks || (long)M > (long)p.ag_rows * (c->fwd_peers + 1))
        return -10;
      if (!c->fwd_counter || (c->fwd_src && ((c->fwd_src_ld & 7) || (reinterpret_cast<uintptr_t>(c->fwd_src) & 15))))
        return -11;
      p.fwd_peers = c->fwd_peers;
      p.fwd_direct = c->fwd_src ? 1 : 0;
      p.fwd_dsts = p.fwd_peers + p.fwd_direct;
      p.fwd_counter = c->fwd_counter;
      // k-blocks of a row block are dealt out to (up to) eight column tiles: small enough shares that the CTAs which
      // forward are not late for their next tile, and all of them in the first wave of a raster band
      p.fwd_split = std::max(1, std::min(std::min(8, (N + bn - 1) / bn), (int)kb));
      p.ag_chunk = bmt;
      for (int i = 0; i < p.fwd_peers; ++i) {
        if (!c->fwd_dst[i] || !c->fwd_flag[i]) return -11;
        p.fwd_flag[i] = c->fwd_flag[i];
      }
    }
    if (c->sc_row) {
      // the scatter lives in the straight-line epilogue of the 1-CTA kernels; 16-byte pieces must not straddle owners
      if (p.rs_rows || p.ag_flags || out_f32 || accumulate || act || alpha != 1.0f || mt == 3 || p.rs_ranks < 1 ||
          p.rs_ranks > 8 || c->sc_w <= 0 || (c->sc_w & 7) || c->sc_part != c->sc_w * p.rs_ranks || N % c->sc_part ||
          c->sc_ld != (N / c->sc_part) * c->sc_w || !p.rs_counter || c->sc_rows_dst <= 0)
        return -12;
      p.sc_row = c->sc_row; p.sc_part = c->sc_part; p.sc_w = c->sc_w; p.sc_ld = c->sc_ld;
    }
    if (c->kf_flags) {
      if (a_mn || c->kf_w <= 0 || c->kf_ranks < 1 || c->kf_ranks > 8 || c->kf_self < 0 || c->kf_self >= c->kf_ranks ||
          (long)c->kf_w * c->kf_ranks != K || mt == 3)
        return -13;
      p.kf_flags = c->kf_flags; p.kf_epoch = c->kf_epoch; p.kf_w = c->kf_w; p.kf_self = c->kf_self;
      p.kf_ranks = c->kf_ranks;
    }
    if (p.rs_rows && (out_f32 || p.rs_ranks > 8 || p.rs_ranks < 1)) return -6;
    // every row needs an owner among the rs_ranks peers: a longer M would index past the peer table
    if (p.rs_rows && (long)M > (long)p.rs_rows * p.rs_ranks) return -8;
  }
  // stream-K for a partial last wave (plain GEMMs on the 1-CTA kernels only)
  p.sk_tiles = 0;
  p.sk_ws = nullptr;
  p.sk_flags = nullptr;
  p.sk_epoch = 0;
  bool sk_on = false;
  if (!comm && mt != 3 && !(MMT_DBG & 1)) {
    const int tiles = ((M + bmt - 1) / bmt) * ((N + bn - 1) / bn);
    const int skt = sk_tiles_for(tiles, (K + BK - 1) / BK, sms, mt);
    if (skt > 0 && sk_ready()) {
      p.sk_tiles = skt;
      p.sk_ws = g_sk_ws;
      p.sk_flags = g_sk_flags;
      p.sk_epoch = ++g_sk_epoch;
      sk_on = true;
    }
  }
  // bf16 results leave through the epilogue warps' shared-memory slabs as full 128-byte row segments
  // bf16 results leave through the epilogue warps' shared-memory slabs: as bulk stores of [32 x 64] boxes
  // (tma_store == 2; a reduce-scatter producer needs rows-per-owner to be a multiple of 32 for that, so that a slab
  // has a single owner) or else as plain 16-byte stores of full row segments (tma_store == 1)
  OutMaps tc;
  memset(&tc, 0, sizeof(tc));
  p.tma_store = 0;
  if (!out_f32) {
    p.tma_store = 1;
    if (p.sc_row) {
      p.tma_store = 2;
      for (int i = 0; i < p.rs_ranks; ++i) {
        r = cached_tmap_2d(&tc.m[i], reinterpret_cast<const void*>(p.rs_base[i]), (uint64_t)p.sc_ld,
                           (uint64_t)comm->sc_rows_dst, (uint64_t)p.sc_ld, 64, 32);
        if (r) return 3000 + r;
      }
    } else if (p.rs_rows) {
      if (p.rs_rows % 32 == 0) {
        p.tma_store = 2;
        for (int i = 0; i < p.rs_ranks; ++i) {
          const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(p.rs_base[i]) +
                                      (long)p.rs_self * p.rs_rows * ldc;
          r = cached_tmap_2d(&tc.m[i], base, (uint64_t)N, (uint64_t)p.rs_rows, (uint64_t)ldc, 64, 32);
          if (r) return 3000 + r;
        }
      }
    } else {
      p.tma_store = 2;
      r = cached_tmap_2d(&tc.m[0], C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 32);
      if (r) return 3000 + r;
    }
  }
  for (int i = 0; i < p.fwd_dsts; ++i) {
    const void* dst = i < p.fwd_peers ? reinterpret_cast<const void*>(comm->fwd_dst[i]) : A;
    r = cached_tmap_2d(&tc.m[1 + i], dst, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, (uint32_t)bmt);
    if (r) return 4000 + r;
  }
  if (p.fwd_direct) {
    r = cached_tmap_2d(&tc.m[9], comm->fwd_src, (uint64_t)K, (uint64_t)p.ag_rows, (uint64_t)comm->fwd_src_ld, BK,
                       (uint32_t)bmt);
    if (r) return 4000 + r;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // the stream-K workspace is shared: a launch on another stream than the previous user waits for that one
  if (sk_on && g_sk_stream != st && g_sk_epoch > 1) cudaStreamWaitEvent(st, g_sk_event, 0);
  int rc;
  switch (bn) {
    case 256:
      if (mt == 3) rc = launch_pair(ta, tb, tc, p, sms, st);
      else rc = mt == 2 ? launch<256, 2>(ta, tb, tc, p, sms, st) : launch<256, 1>(ta, tb, tc, p, sms, st);
      break;
    case 192: rc = mt == 2 ? launch<192, 2>(ta, tb, tc, p, sms, st) : launch<192, 1>(ta, tb, tc, p, sms, st); break;
    case 128: rc = mt == 2 ? launch<128, 2>(ta, tb, tc, p, sms, st) : launch<128, 1>(ta, tb, tc, p, sms, st); break;
    case 64:  rc = launch<64, 1>(ta, tb, tc, p, sms, st); break;
    default:  return -4;
  }
  if (sk_on) {
    cudaEventRecord(g_sk_event, st);
    g_sk_stream = st;
  }
  return rc;
}

// Tuning knob: 1 = stream-K for partial last waves, 0 = whole tiles only (default).
extern "C" void mmt_gemm_set_stream_k(int on) { g_sk_mode = on; }
