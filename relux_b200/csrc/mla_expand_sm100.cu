// Decompression of the cached MLA latents into per-head keys and values for a prompt, on the 5th-generation tensor
// cores: the first half of MLA.forwardCached's attention for seqQ > 1, where the reference multiplies ALL cached
// latent rows by W_UK and W_UV (internal/transformer/mla.go:323-326) before it scores them.  For a prompt this order is
// the cheap one: 192 + 128 multiply-adds per (query, key, head) on the expanded rows against 576 + 512 on the latent
// rows, at the price of one [tokens x 512] x [512 x 2 H 128] product per call.
//
//   Kx[h][t][0:128] = sum_c ckv[t][c] * W_UK[c][h * 128 + d]        Vx[h][t][0:128] = sum_c ckv[t][c] * W_UV[c][h * 128 + d]
//
// bf16 operands, float32 accumulation in tensor memory, bf16 results in a dense scratch array the prefill kernel reads
// with plain 2-D TMA boxes: row = h * Ttot + base[sequence] + token, Ttot = sum over sequences of the cached length
// rounded up to 256 (rows past a sequence's end are computed from whatever its last page holds and masked later).
//
// Shape: a TOKEN TILE is 256 consecutive tokens of one sequence (4 pages), an OUTPUT TILE 128 columns (one head of K or
// of V).  A worker is a CTA pair (tcgen05 cta_group::2, M = 256, N = 128): CTA r holds tokens [128 r, 128 r + 128) of the
// token tile -- 8 latent blocks of [128 tokens x 64 columns], 128 KB, straight out of the blocked pages -- and columns
// [64 r, 64 r + 64) of every weight stage ([128 latent rows x 64 columns], MN-major as the weights lie).  Worker w takes a
// contiguous run of (token tile, output tile) units in token-tile-major order, so the latent tile is loaded once per run
// (twice when the run crosses a token tile) and the 32 MB of weights stream from L2 through a four-stage ring.
// The latent tile is the A operand of every MMA of a run: it is copied once from shared memory into tensor memory (lane =
// token, two latents per 32-bit column, 256 columns), so that the MMAs read only the weight stages from shared memory.
// The accumulator is double-buffered in tensor memory: four epilogue warps convert unit n while the MMAs of unit n + 1
// run (they also make the copy of the latent tile, between two runs of units), and the bf16 rows leave through a
// swizzled shared tile and TMA stores (whole 128-byte lines instead of 16 bytes per lane at a 256-byte pitch).
// What bounds the kernel is neither of those: every token tile streams all of W_UK and W_UV (32 MB at 128 heads), 256
// flop per weight byte at 256 tokens per pair, and the L2 -> SM traffic measured 4.2 TB/s: 1.0-1.06 PFLOP/s with the latent
// tile in shared or in tensor memory, with rows stored from registers or by TMA alike.
// Warp roles per CTA: 4 epilogue warps, 1 TMA producer, 1 MMA issuer (leader CTA only).
// No TMA multicast.  The weight stages' full barriers live in the leader and count both CTAs' bytes; the latent tile's
// full barrier is each CTA's own (its epilogue warps wait on it).  Every wait is bounded, and the MMA issuer sees its
// last MMA complete before the pair frees its tensor memory.
#include <algorithm>
#include <cuda_bf16.h>

#include "common.cuh"
#include "internal.h"
#include "umma.cuh"
#include "prep_parts.cuh"

namespace relux {

namespace {

constexpr int kDC = 512, kPage = 64, kTokTile = 256;
constexpr int kBlk = 8192;                          // one [64 rows x 64 cols] bf16 box, 128-byte swizzled
constexpr int kABlock = 2 * kBlk;                   // [128 tokens x 64 latent columns]
constexpr int kABytes = (kDC / 64) * kABlock;       // 131072
constexpr int kStageBytes = 2 * kBlk;               // [128 latent rows x 64 output columns]
constexpr int kStages = 4, kStagesPerUnit = kDC / 128;
constexpr int kSmemRing = kABytes;
constexpr int kSmemOut = kSmemRing + kStages * kStageBytes;   // one output tile [128 tokens x (cols 0-63 | cols 64-127)] bf16, swizzled
constexpr int kOutBytes = 4 * kBlk;
constexpr int kSmemBar = kSmemOut + kOutBytes;                // 229376
constexpr int kSmemTotal = kSmemBar + 1024;
constexpr int kEpiWarps = 4, kThreads = 32 * (kEpiWarps + 2);
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemA = 256;                    // accumulators at columns [0, 256), the latent tile at [256, 512)

struct Bars {
  uint64_t a_full, a_empty, a_ready, b_full[kStages], b_empty[kStages], acc_full[2], acc_empty[2], drain;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
};
static_assert(sizeof(Bars) <= 1024, "barrier block too large");

struct ExpandParams {
  const int32_t* table;
  int32_t table_stride;
  const int32_t* len;
  const int32_t* seq_ids;
  const int32_t* seq_base;     // [n_seqs + 1] first dense row of every sequence (multiples of 256)
  int32_t num_pages, n_seqs, extra, H;
  int32_t n_out;               // output tiles per token tile = 2 H
  int32_t units, span;         // (token tile, output tile) units in all, and per worker
  int32_t blocks_per_page;     // 64-column blocks of one page (latent + rope)
  int64_t row0;                // first TMA row of this layer in the pool's block array
  int64_t Ttot;
  int32_t* status;
};

__device__ __noinline__ void wait_slow(uint64_t* bar, uint32_t parity, Bars* b, int32_t* status) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 255) == 255 && b->abort_flag) return;
    if (i > 512) __nanosleep(20);
  }
  b->abort_flag = 1;
  set_status(status, RELUX_ERR_TIMEOUT);
}
__device__ __forceinline__ void wait_bar(uint64_t* bar, uint32_t parity, Bars* b, int32_t* status) {
  if (!mbar_try_wait(bar, parity)) wait_slow(bar, parity, b, status);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    mla_expand_sm100_kernel(const __grid_constant__ CUtensorMap tmap_pool, const __grid_constant__ CUtensorMap tmap_wuk,
                            const __grid_constant__ CUtensorMap tmap_wuv, const __grid_constant__ CUtensorMap tmap_out,
                            const ExpandParams prm) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int worker = blockIdx.x >> 1;
  const int u0 = worker * prm.span, u1 = min(prm.units, u0 + prm.span);
  if (u0 >= u1) return;   // both CTAs of the pair leave before any pair-wide step

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) set_status(prm.status, RELUX_ERR_UNSUPPORTED);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->a_empty, kEpiWarps);       // this CTA's copy has left the shared tile
    mbar_init(&bars->a_ready, 2 * kEpiWarps);   // both CTAs' latent tiles are in tensor memory (the leader's copy is waited on)
    for (int s = 0; s < kStages; s++) { mbar_init(&bars->b_full[s], 1); mbar_init(&bars->b_empty[s], 1); }
    for (int s = 0; s < 2; s++) { mbar_init(&bars->acc_full[s], 1); mbar_init(&bars->acc_empty[s], 2 * kEpiWarps); }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc<2>(&bars->tmem_base, kTmemCols);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == kEpiWarps) {
    // =============================== producer ===============================
    const bool el = elect_one();
    if (el) {
      tma_prefetch_desc(&tmap_pool);
      tma_prefetch_desc(&tmap_wuk);
      tma_prefetch_desc(&tmap_wuv);
    }
    int cur_tt = -1, na = 0, gs = 0;
    for (int u = u0; u < u1; u++) {
      const int tt = u / prm.n_out, nt = u % prm.n_out;
      if (tt != cur_tt) {
        // the sequence that owns dense rows [256 tt, 256 tt + 256): last i with seq_base[i] <= 256 tt
        int lo = 0, hi = prm.n_seqs - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (__ldg(prm.seq_base + mid) <= tt * kTokTile) lo = mid;
          else hi = mid - 1;
        }
        const int seq = prm.seq_ids ? __ldg(prm.seq_ids + lo) : lo;
        const int T = __ldg(prm.len + seq) + prm.extra;
        const int last_slot = max(0, (T + kPage - 1) / kPage - 1);
        const int tok0 = tt * kTokTile - __ldg(prm.seq_base + lo) + 128 * (int)rank;   // this CTA's first token in the sequence
        int64_t y[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++) {
          const int slot = min(tok0 / kPage + h2, last_slot);
          int32_t pg = __ldg(prm.table + (size_t)seq * prm.table_stride + slot);
          if (pg < 0 || pg >= prm.num_pages) {   // reported, and replaced by page 0 so that no load leaves the pool
            set_status(prm.status, RELUX_ERR_BAD_PAGE);
            pg = 0;
          }
          y[h2] = prm.row0 + (int64_t)pg * prm.blocks_per_page * kPage;
        }
        if (na > 0) wait_bar(&bars->a_empty, (na - 1) & 1, bars, prm.status);
        // every CTA's latent tile reports to its OWN barrier: its epilogue warps copy it to tensor memory
        const uint32_t lead = mapa_u32(smem_u32(&bars->a_full), rank);
        if (el) {
          mbar_expect_tx(&bars->a_full, kABytes);
#pragma unroll 1
          for (int kb = 0; kb < kDC / 64; kb++) {
            tma_load_2d_2sm(smem + kb * kABlock, &tmap_pool, 0, (int32_t)(y[0] + kb * kPage), lead);
            tma_load_2d_2sm(smem + kb * kABlock + kBlk, &tmap_pool, 0, (int32_t)(y[1] + kb * kPage), lead);
          }
        }
        __syncwarp();
        na++;
        cur_tt = tt;
      }
      const CUtensorMap* wm = nt < prm.H ? &tmap_wuk : &tmap_wuv;
      const int x = (nt < prm.H ? nt : nt - prm.H) * 128 + 64 * (int)rank;
#pragma unroll 1
      for (int s = 0; s < kStagesPerUnit; s++, gs++) {
        const int st = gs % kStages, use = gs / kStages;
        if (use > 0) wait_bar(&bars->b_empty[st], (use - 1) & 1, bars, prm.status);
        const uint32_t lead = mapa_u32(smem_u32(&bars->b_full[st]), 0);
        if (el) {
          if (rank == 0) mbar_expect_tx(&bars->b_full[st], 2 * kStageBytes);   // the column halves of both CTAs
          tma_load_2d_2sm(smem + kSmemRing + st * kStageBytes, wm, x, s * 128, lead);
        }
        __syncwarp();
      }
    }
  } else if (warp == kEpiWarps + 1) {
    // =============================== MMA issuer (leader CTA only) ===============================
    const bool el = elect_one();
    if (rank == 0) {
      const uint32_t idesc = make_idesc_bf16(256, 128, false, true);
      int cur_tt = -1, na = 0, gs = 0, n = 0;
      for (int u = u0; u < u1; u++, n++) {
        const int tt = u / prm.n_out;
        if (tt != cur_tt) {
          wait_bar(&bars->a_ready, na & 1, bars, prm.status);
          na++;
          cur_tt = tt;
        }
        const int buf = n & 1;
        if (n >= 2) wait_bar(&bars->acc_empty[buf], ((n >> 1) - 1) & 1, bars, prm.status);
#pragma unroll 1
        for (int s = 0; s < kStagesPerUnit; s++, gs++) {
          const int st = gs % kStages;
          wait_bar(&bars->b_full[st], (gs / kStages) & 1, bars, prm.status);
          tc_fence_after();
          if (el) {
            const uint64_t dB = make_desc_mnmajor_sw128(smem_u32(smem + kSmemRing + st * kStageBytes), kBlk);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
              umma_ts<2>(tmem + buf * 128, tmem + kTmemA + (8 * s + ks) * 8, dB + ((uint32_t)(ks * 2048) >> 4), idesc, (s | ks) != 0);
            }
            umma_commit_mc<2>(&bars->b_empty[st], 0x3);
          }
          __syncwarp();
        }
        if (el) umma_commit_mc<2>(&bars->acc_full[buf], 0x3);
        __syncwarp();
      }
      // Nothing of this pair may be freed while an MMA is in flight.  On the ordinary path the epilogue's last wait says
      // so already; after a wait that gave up it does not, so the issuer itself sees its last MMA complete.
      if (el) umma_commit<2>(&bars->drain);
      __syncwarp();
      mbar_wait(&bars->drain, 0);
    }
  } else {
    // =============================== epilogue: accumulator -> bf16 rows ===============================
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const uint32_t lead_empty0 = mapa_u32(smem_u32(&bars->acc_empty[0]), 0), lead_empty1 = mapa_u32(smem_u32(&bars->acc_empty[1]), 0);
    const uint32_t lead_ready = mapa_u32(smem_u32(&bars->a_ready), 0);
    const int row = warp * 32 + lane;
    int n = 0, na = 0, cur_tt = -1;
    for (int u = u0; u < u1; u++, n++) {
      const int tt = u / prm.n_out, nt = u % prm.n_out;
      if (tt != cur_tt) {
        // A new latent tile.  The MMAs that read the previous one have completed (this warp has seen acc_full of the last
        // unit that used it).  Row `row` of every 64-column block -> 32 columns of this thread's lane.
        wait_bar(&bars->a_full, na & 1, bars, prm.status);
        __syncwarp();
#pragma unroll 1
        for (int kb = 0; kb < kDC / 64; kb++) {
          uint32_t w[32];
          const uint8_t* src = smem + kb * kABlock + row * 128;
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + ((j ^ (row & 7)) << 4));
            w[4 * j] = v.x;
            w[4 * j + 1] = v.y;
            w[4 * j + 2] = v.z;
            w[4 * j + 3] = v.w;
          }
          tmem_st_32x32b_x32(tmem + lane_addr + kTmemA + kb * 32, w);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->a_empty);        // the producer may fetch the next token tile into the shared tile
          mbar_arrive_cluster(lead_ready);
        }
        na++;
        cur_tt = tt;
      }
      const int buf = n & 1;
      wait_bar(&bars->acc_full[buf], (n >> 1) & 1, bars, prm.status);
      __syncwarp();   // the TMEM loads below are warp-collective
      tc_fence_after();
      // the stores of the previous unit have read the shared tile
      if (threadIdx.x == 0) tma_store_wait_read();
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
      uint8_t* orow = smem + kSmemOut + row * 128;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + buf * 128 + c, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; i++) pk[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
        // columns c .. c + 31 = 16-byte chunks (c & 63) / 8 .. + 3 of the 64-column half c / 64
#pragma unroll
        for (int i = 0; i < 4; i++)
          *reinterpret_cast<uint4*>(orow + (c >> 6) * 2 * kBlk + (((((c & 63) >> 3) + i) ^ (row & 7)) << 4)) =
              make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf ? lead_empty1 : lead_empty0);   // the accumulator is free again
      fence_proxy_async();
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
      if (threadIdx.x == 0) {
        // first row of this CTA's 128 tokens in the [2 H Ttot][128] array of expanded keys and values
        const int32_t y = (int32_t)((int64_t)nt * prm.Ttot + (int64_t)tt * kTokTile + 128 * (int)rank);
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++)
#pragma unroll
          for (int r2 = 0; r2 < 2; r2++) tma_store_2d(&tmap_out, 64 * h2, y + 64 * r2, smem + kSmemOut + h2 * 2 * kBlk + r2 * kBlk);
        tma_store_commit();
      }
    }
  }
  if (threadIdx.x == 0) tma_store_wait_all();
  __syncwarp();
  tc_fence_before();
  cluster_sync();
  if (warp == 0) tmem_dealloc<2>(tmem, kTmemCols);
}

// seq_base[i] = dense row of sequence i's first token: running sum of the cached lengths rounded up to 256 (one block,
// a block-wide scan per 256 sequences).
__global__ void mla_expand_plan_kernel(const int32_t* __restrict__ len, const int32_t* __restrict__ seq_ids, int n_seqs, int extra,
                                       int32_t* __restrict__ seq_base) {
  __shared__ int32_t s_warp[32];
  int base = 0;
  for (int i0 = 0; i0 < n_seqs; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    int rows = 0;
    if (i < n_seqs) {
      const int T = len[seq_ids ? seq_ids[i] : i] + extra;
      rows = (T + kTokTile - 1) / kTokTile * kTokTile;
    }
    int total;
    const int before = prep_block_excl_scan(rows, s_warp, &total);
    if (i < n_seqs) seq_base[i] = base + before;
    base += total;
  }
  if (threadIdx.x == 0) seq_base[n_seqs] = base;
}

int expand_workers(Pool* p) {
  static int max_clusters = 0;
  if (!max_clusters) {
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemTotal;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(mla_expand_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, mla_expand_sm100_kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = std::max(1, p->dev->sm_count / 2);
    }
    max_clusters = n;
  }
  return max_clusters;
}

}  // namespace


bool mla_expand_eligible(const Pool* p, int num_heads, int head_dim) {
  const relux_pool_params& prm = p->prm;
  return p->has_tmap && p->mla_blocked && prm.page_tokens == kPage && prm.mla_dc == kDC && prm.mla_dhr % 64 == 0 && head_dim == 128 &&
         num_heads >= 1;
}

// Dense rows the expanded keys / values of this batch need (per head): sum of the lengths rounded up to 256.
int64_t mla_expand_rows(const Pool* p, const SeqBatch& sb, int layer, int extra) {
  int64_t t = 0;
  for (int i = 0; i < sb.n_seqs; i++) {
    const int64_t T = p->h_len[(size_t)layer * p->prm.max_seqs + sb.seq[i]] + extra;
    t += (T + kTokTile - 1) / kTokTile * kTokTile;
  }
  return t;
}

// kx, vx: device bf16 [H][Ttot][128]; seq_base: device int32 [n_seqs + 1] (written here).
int32_t launch_mla_expand_sm100(Pool* p, const SeqBatch& sb, int layer, int extra, int H, const uint16_t* w_uk, const uint16_t* w_uv,
                                int64_t Ttot, uint16_t* kx, uint16_t* vx, int32_t* seq_base) {
  const relux_pool_params& prm = p->prm;
  cudaStream_t st = p->dev->stream;
  CUtensorMap t_uk, t_uv, t_out;
  if (!make_tmap_2d(&t_uk, (void*)w_uk, kDC, (uint64_t)H * 128, 64, 128) || !make_tmap_2d(&t_uv, (void*)w_uv, kDC, (uint64_t)H * 128, 64, 128)) {
    set_error("tensor maps for W_UK / W_UV could not be encoded");
    return RELUX_ERR_CUDA;
  }
  // keys and values are one array: vx must follow kx directly (row = (K: head | V: H + head) * Ttot + dense token row)
  if (vx != kx + (size_t)H * Ttot * 128 || !make_tmap_2d(&t_out, kx, (uint64_t)2 * H * Ttot, 128, 64, 64)) {
    set_error("tensor map for the expanded keys / values could not be encoded");
    return RELUX_ERR_CUDA;
  }
  const int32_t* len = p->d_len + (size_t)layer * prm.max_seqs;
  mla_expand_plan_kernel<<<1, 256, 0, st>>>(len, sb.d_seq_ids, sb.n_seqs, extra, seq_base);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  ExpandParams k{};
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.len = len;
  k.seq_ids = sb.d_seq_ids;
  k.seq_base = seq_base;
  k.num_pages = prm.num_pages;
  k.n_seqs = sb.n_seqs;
  k.extra = extra;
  k.H = H;
  k.n_out = 2 * H;
  const int64_t units = Ttot / kTokTile * k.n_out;
  if (units <= 0) return RELUX_OK;
  if (units > ((int64_t)1 << 30)) { set_error("batch too long for one expansion launch"); return RELUX_ERR_UNSUPPORTED; }
  k.units = (int32_t)units;
  const int workers = (int)std::min<int64_t>(expand_workers(p), units);
  k.span = (int32_t)((units + workers - 1) / workers);
  k.blocks_per_page = p->row_elems_a / 64;
  k.row0 = (int64_t)layer * prm.num_pages * k.blocks_per_page * kPage;
  k.Ttot = Ttot;
  k.status = p->d_status;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_expand_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  const int launched = (int)((units + k.span - 1) / k.span);
  mla_expand_sm100_kernel<<<dim3(2 * launched), kThreads, kSmemTotal, st>>>(p->tmap_mla, t_uk, t_uv, t_out, k);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux
