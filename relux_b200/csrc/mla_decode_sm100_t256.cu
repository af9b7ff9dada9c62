// Absorbed MLA flash-decode on tcgen05 / TMEM, 256-token tile variant (see mla_decode_sm100.cu for the
// 128-token-tile kernel and for why a CTA pair is used).
//
// Difference to the 128-token kernel.  `tcgen05.mma cta_group::2 M128 N128 K16` issues in 45.4 cycles (70 % of the
// tensor peak for that shape), `M128 N256 K16` in 64.4 cycles (peak).  With 256 tokens per tile (CTA r holds tile
// pages 2r and 2r+1, i.e. 128 tokens) S = Q~ K^T also runs with N = 256, which cuts the tensor time per 128 tokens
// from 36*45.4 + 16*64.4 = 2664 to 18*64.4 + 16*64.4 = 2190 cycles.  Tensor memory is then exactly full:
// O 256 columns + two S buffers of 128 columns.
//
// Shared memory per CTA: Q~ 72 KB | P 32 KB | a ring of seven 16 KB slots | barriers.  Operands stream through the
// ring in the order the MMA warp consumes them:
//   K entry (tile t, column block db): [page 2r, block db | page 2r+1, block db]  = 128 token rows x 64 columns
//   V entry (tile t, output block nb, tile page p): [page p, block 4nb+2r | page p, block 4nb+2r+1] = 64 tokens x 128 dims
// sequence: K(0) x9, then per tile t: K(t+1) x9, V(t) x8.  Entry n lives in slot n % 7; its full barrier is in the
// leader CTA (bytes of both CTAs' loads), its empty barrier in each CTA (tcgen05.commit multicast).
// No TMA multicast is used; every wait is bounded (see wait_bar).
//
// Status: selectable with RELUX_MLA_TILE=256, not the default.  At 64 sequences x 32768 tokens it takes 0.56 ms
// against 0.50 ms of the 128-token kernel: the ring holds 112 KB per CTA, seven entries = 1.8k tensor cycles of
// lead, which is less than the load latency under full HBM load, so the tensor pipe waits on full barriers
// (6.1k cycles per tile against 4.4k of MMA issue).  Pulling pages into L2 ahead of time with
// cp.async.bulk.prefetch made it slower still (0.76 ms), so kPrefetchTiles stays 0.
#include <cstdlib>
#include <cuda_bf16.h>
#include "common.cuh"
#include "internal.h"
#include "splitkv.h"
#include "umma.cuh"

namespace relux {

namespace {

constexpr int kHeads = 128, kDC = 512, kDR = 64, kRow = kDC + kDR;  // 576
constexpr int kPage = 64;
constexpr int kBlk = 8192;                  // one [64 rows x 64 cols] bf16 block, 128-byte swizzled
constexpr int kNumKB = kRow / 64;           // 9 column blocks per row
constexpr int kTilePages = 4;               // 256 tokens per tile
constexpr int kSlots = 7, kSlotBytes = 2 * kBlk;
constexpr int kSmemQ = 0;
constexpr int kSmemP = kSmemQ + kNumKB * kBlk;            // 73728; P: 4 blocks [64 rows x 64 tokens]
constexpr int kSmemRing = kSmemP + 4 * kBlk;              // 106496
constexpr int kSmemBar = kSmemRing + kSlots * kSlotBytes; // 221184
constexpr int kSmemTotal = kSmemBar + 3072;               // 224256
constexpr int kMaxChunkPages = 320;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0, kTmemS = 256;              // O: 2 x 128 columns; S: 2 buffers x 128 columns
constexpr float kRescaleThreshold = 8.0f;
constexpr int kPrefetchTiles = 0;   // L2 prefetch distance of the producer, in tiles

struct Bars {
  uint64_t full[kSlots], empty[kSlots];
  uint64_t s_full[2];
  uint64_t p_full, pv_done, q_full;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  float rowmax[2][2][64];   // [tile parity][token half][row]
  float lsum[64];
  int32_t page_row[kMaxChunkPages];
};
static_assert(sizeof(Bars) <= 3072, "barrier block too large");

struct Params {
  const WorkItem* items;
  const int32_t* table;
  int32_t table_stride;
  const int32_t* len;
  int32_t num_pages, S, extra, causal;
  int32_t layer_row0;
  float scale_log2;
  float* part_o;
  float* part_ml;
  int32_t rows_total;
  int32_t* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Bounded wait: one try_wait in the common case; on time-out the waiter records RELUX_ERR_TIMEOUT, raises the
// CTA's abort flag and returns, every later wait returns on its first failed poll, nobody leaves a loop early.
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
    mla_decode_sm100_t256_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_q,
                                 const Params prm) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int item_idx = blockIdx.x >> 1;
  const int sq = blockIdx.y;
  const WorkItem item = prm.items[item_idx];
  const int T = prm.len[item.seq] + prm.extra;
  const int limit_tok = prm.causal ? (T - prm.S + sq + 1) : T;
  const int tok_end = min(limit_tok, item.page_end * kPage);
  const int npages = item.page_end - item.page_begin;
  const int ntiles = (npages + kTilePages - 1) / kTilePages;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) set_status(prm.status, RELUX_ERR_UNSUPPORTED);
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlots; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 8);    // one arrival per softmax warp of each CTA
    mbar_init(&bars->pv_done, 1);
    mbar_init(&bars->q_full, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc<2>(&bars->tmem_base, kTmemCols);
    tmem_relinquish<2>();
  }
  for (int i = threadIdx.x; i < npages && i < kMaxChunkPages; i += blockDim.x) {
    int32_t pg = prm.table[(size_t)item.seq * prm.table_stride + item.page_begin + i];
    if (pg < 0 || pg >= prm.num_pages) {
      set_status(prm.status, RELUX_ERR_BAD_PAGE);
      pg = 0;
    }
    bars->page_row[i] = prm.layer_row0 + pg * (kNumKB * kPage);
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 4) {
    // =============================== producer ===============================
    const bool el = elect_one();
    const uint32_t lead_q = mapa_u32(smem_u32(&bars->q_full), 0);
    const int qrow = (item.seq_index * prm.S + sq) * kHeads + 64 * (int)rank;
    if (el) {
      tma_prefetch_desc(&tmap_kv);
      tma_prefetch_desc(&tmap_q);
      if (rank == 0) mbar_expect_tx(&bars->q_full, 2 * kNumKB * kBlk);
#pragma unroll
      for (int db = 0; db < kNumKB; db++) tma_load_2d_2sm(smem + kSmemQ + db * kBlk, &tmap_q, db * 64, qrow, lead_q);
    }
    __syncwarp();
    auto page_row = [&](int tile, int p) -> int32_t {   // p = page of the tile, 0..3; missing pages fall back to page 0
      int lp = kTilePages * tile + p;
      if (lp >= npages) lp = 0;
      return bars->page_row[lp];
    };
    int n = 0;  // ring entry counter, identical in both CTAs and in the MMA warp
    auto acquire = [&]() -> int {
      const int slot = n % kSlots, use = n / kSlots;
      if (use > 0) wait_bar(&bars->empty[slot], (use - 1) & 1, bars, prm.status);
      n++;
      return slot;
    };
    auto load_k = [&](int tile) {
      const int32_t ya = page_row(tile, 2 * (int)rank), yb = page_row(tile, 2 * (int)rank + 1);
#pragma unroll 1
      for (int db = 0; db < kNumKB; db++) {
        const int slot = acquire();
        const uint32_t lead = mapa_u32(smem_u32(&bars->full[slot]), 0);
        if (el) {
          if (rank == 0) mbar_expect_tx(&bars->full[slot], 2 * kSlotBytes);
          uint8_t* dst = smem + kSmemRing + slot * kSlotBytes;
          tma_load_2d_2sm(dst, &tmap_kv, 0, ya + db * kPage, lead);
          tma_load_2d_2sm(dst + kBlk, &tmap_kv, 0, yb + db * kPage, lead);
        }
        __syncwarp();
      }
    };
    auto load_v = [&](int tile) {
#pragma unroll 1
      for (int u = 0; u < 2 * kTilePages; u++) {  // u = p * 2 + nb : tile page outer, output block inner
        const int p = u >> 1, nb = u & 1;
        const int slot = acquire();
        const uint32_t lead = mapa_u32(smem_u32(&bars->full[slot]), 0);
        const int32_t y = page_row(tile, p);
        const int blk0 = 4 * nb + 2 * (int)rank;
        if (el) {
          if (rank == 0) mbar_expect_tx(&bars->full[slot], 2 * kSlotBytes);
          uint8_t* dst = smem + kSmemRing + slot * kSlotBytes;
          tma_load_2d_2sm(dst, &tmap_kv, 0, y + blk0 * kPage, lead);
          tma_load_2d_2sm(dst + kBlk, &tmap_kv, 0, y + (blk0 + 1) * kPage, lead);
        }
        __syncwarp();
      }
    };
    // The ring holds less than half a tile, too little to cover the HBM latency of the key loads; the pages of
    // tile t + kPrefetchTiles are therefore pulled into L2 ahead of time (no shared memory, no barrier).
    auto prefetch_k = [&](int tile) {
      if (tile < ntiles && el) {
        const int32_t ya = page_row(tile, 2 * (int)rank), yb = page_row(tile, 2 * (int)rank + 1);
#pragma unroll
        for (int db = 0; db < kNumKB; db++) {
          tma_prefetch_l2_2d(&tmap_kv, 0, ya + db * kPage);
          tma_prefetch_l2_2d(&tmap_kv, 0, yb + db * kPage);
        }
      }
      __syncwarp();
    };
    if (kPrefetchTiles > 0)
      for (int t = 1; t <= kPrefetchTiles; t++) prefetch_k(t);
    load_k(0);
    for (int i = 0; i < ntiles; i++) {
      if (kPrefetchTiles > 0) prefetch_k(i + 1 + kPrefetchTiles);
      if (i + 1 < ntiles) load_k(i + 1);
      load_v(i);
    }
  } else if (warp == 5) {
    // =============================== MMA issuer (leader CTA only) ===============================
    if (rank == 0) {
      const bool el = elect_one();
      const uint32_t idesc_qk = make_idesc_bf16(128, 256, false, false);
      const uint32_t idesc_pv = make_idesc_bf16(128, 256, false, true);
      const uint64_t dQ = make_desc_kmajor_sw128(smem_u32(smem + kSmemQ));
      const uint64_t dP = make_desc_kmajor_sw128(smem_u32(smem + kSmemP));
      const uint64_t dRk = make_desc_kmajor_sw128(smem_u32(smem + kSmemRing));
      const uint64_t dRv = make_desc_mnmajor_sw128(smem_u32(smem + kSmemRing), kBlk);
      wait_bar(&bars->q_full, 0, bars, prm.status);
      int n = 0;
      auto next_full = [&]() -> int {
        const int slot = n % kSlots, use = n / kSlots;
        wait_bar(&bars->full[slot], use & 1, bars, prm.status);
        n++;
        return slot;
      };
      auto issue_qk = [&](int tile) {
        const uint32_t d = tmem + kTmemS + (tile & 1) * 128;
#pragma unroll 1
        for (int db = 0; db < kNumKB; db++) {
          const int slot = next_full();
          const uint32_t soff = (uint32_t)(slot * kSlotBytes) >> 4, qoff = (uint32_t)(db * kBlk) >> 4;
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 4; kk++) umma_ss<2>(d, dQ + qoff + kk * 2, dRk + soff + kk * 2, idesc_qk, (db | kk) != 0);
            umma_commit_mc<2>(&bars->empty[slot], 0x3);
          }
          __syncwarp();
        }
        if (el) umma_commit_mc<2>(&bars->s_full[tile & 1], 0x3);
        __syncwarp();
      };
      auto issue_pv = [&](int tile) {
        wait_bar(&bars->p_full, tile & 1, bars, prm.status);
        tc_fence_after();
#pragma unroll 1
        for (int u = 0; u < 2 * kTilePages; u++) {
          const int p = u >> 1, nb = u & 1;
          const int slot = next_full();
          const uint32_t soff = (uint32_t)(slot * kSlotBytes) >> 4, poff = (uint32_t)(p * kBlk) >> 4;
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
              umma_ss<2>(tmem + kTmemO + nb * 128, dP + poff + kk * 2, dRv + soff + kk * 128, idesc_pv, (tile | p | kk) != 0);
            umma_commit_mc<2>(&bars->empty[slot], 0x3);
          }
          __syncwarp();
        }
        if (el) umma_commit_mc<2>(&bars->pv_done, 0x3);
        __syncwarp();
      };
      issue_qk(0);
      for (int i = 0; i < ntiles; i++) {
        if (i + 1 < ntiles) issue_qk(i + 1);
        issue_pv(i);
      }
    }
  } else {
    // =============================== softmax / correction / epilogue (warps 0-3) ===============================
    const int L = warp * 32 + lane;   // TMEM lane
    const int row = L & 63;           // head index inside this CTA
    const int hf = L >> 6;            // token half of the tile: tokens [128 hf, 128 hf + 128) = the pages of CTA hf
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY, l_run = 0.f;
    const uint32_t p_full_lead = mapa_u32(smem_u32(&bars->p_full), 0);
    for (int i = 0; i < ntiles; i++) {
      wait_bar(&bars->s_full[i & 1], (i >> 1) & 1, bars, prm.status);
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_addr + kTmemS + (i & 1) * 128;
      const int tok0 = (item.page_begin + kTilePages * i + 2 * hf) * kPage;
      const int nvalid = max(0, min(2 * kPage, tok_end - tok0));   // valid ones of this thread's 128 tokens
      // pass 1: row maximum of the raw scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t sv[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, sv);
        tmem_ld_wait();
        if (nvalid >= (c + 1) * 32) {
#pragma unroll
          for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(sv[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (c * 32 + j < nvalid) mx = fmaxf(mx, __uint_as_float(sv[j]));
        }
      }
      mx *= prm.scale_log2;
      bars->rowmax[i & 1][hf][row] = mx;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      mx = fmaxf(mx, bars->rowmax[i & 1][hf ^ 1][row]);
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + kRescaleThreshold) {
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
        rescale = (m_used != -INFINITY);
        m_used = mx;
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      // pass 2: p = 2^(s * scale - m) -> bf16, kept in registers (128 tokens = 64 words) until the P buffer is free
      float psum = 0.f;
      uint32_t pk[64];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        uint32_t sv[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, sv);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(sv[j]), prm.scale_log2, neg_m));
          float p1 = ex2_approx(fmaf(__uint_as_float(sv[j + 1]), prm.scale_log2, neg_m));
          if (c * 32 + j >= nvalid) p0 = 0.f;
          if (c * 32 + j + 1 >= nvalid) p1 = 0.f;
          psum += p0 + p1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          pk[c * 16 + j / 2] = *reinterpret_cast<uint32_t*>(&b2);
        }
      }
      tc_fence_before();   // last read of this S buffer
      // P(i) may overwrite the buffer, and O may be rescaled, only after PV(i-1) has completed
      if (i > 0) wait_bar(&bars->pv_done, (i - 1) & 1, bars, prm.status);
      if (rescale && i > 0) {
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
          uint32_t ov[32];
          tmem_ld_32x32b_x32(tmem + lane_addr + kTmemO + c, ov);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
          tmem_st_32x32b_x32(tmem + lane_addr + kTmemO + c, ov);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      // P blocks 2hf, 2hf+1, row `row`: 64 tokens = one 128-byte swizzled row each
#pragma unroll
      for (int c = 0; c < 4; c++) {
        uint8_t* prow = smem + kSmemP + (2 * hf + (c >> 1)) * kBlk + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; q4++) {
          const int chunk = (c & 1) * 4 + q4;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(pk[c * 16 + 4 * q4], pk[c * 16 + 4 * q4 + 1], pk[c * 16 + 4 * q4 + 2], pk[c * 16 + 4 * q4 + 3]);
        }
      }
      l_run = l_run * alpha + psum;
      fence_proxy_async();
      tc_fence_before();   // the S buffer has been read for the last time: QK(i+2) may overwrite it after P_full
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(p_full_lead);
    }
    // ---- epilogue ----
    wait_bar(&bars->pv_done, (ntiles - 1) & 1, bars, prm.status);
    const bool ok = !bars->abort_flag;
    tc_fence_after();
    if (hf == 1) bars->lsum[row] = l_run;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const size_t prow = (size_t)item_idx * prm.rows_total + (size_t)sq * kHeads + 64 * rank + row;
    if (hf == 0) {
      prm.part_ml[prow * 2] = ok ? m_used : -INFINITY;
      prm.part_ml[prow * 2 + 1] = ok ? (l_run + bars->lsum[row]) : 0.f;
    }
    float* orow = prm.part_o + prow * kDC;
#pragma unroll 1
    for (int nb = 0; nb < 2; nb++)
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t ov[32];
        if (ok && m_used != -INFINITY) {
          tmem_ld_32x32b_x32(tmem + lane_addr + kTmemO + nb * 128 + c, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) ov[j] = 0u;
        }
        float4* dst = reinterpret_cast<float4*>(orow + 256 * nb + 128 * hf + c);
#pragma unroll
        for (int j = 0; j < 8; j++)
          dst[j] = make_float4(__uint_as_float(ov[4 * j]), __uint_as_float(ov[4 * j + 1]), __uint_as_float(ov[4 * j + 2]),
                               __uint_as_float(ov[4 * j + 3]));
      }
  }
  tc_fence_before();
  cluster_sync();
  if (warp == 0) tmem_dealloc<2>(tmem, kTmemCols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

int32_t launch_mla_decode_sm100_t256(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const SplitPlan& plan, const uint16_t* q_abs) {
  const relux_pool_params& prm = p->prm;
  static EncodeTiledFn enc = nullptr;
  if (!enc) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      set_error("cuTensorMapEncodeTiled is not available");
      return RELUX_ERR_CUDA;
    }
    enc = (EncodeTiledFn)sym;
  }
  CUtensorMap tq;
  {
    const uint64_t rows = (uint64_t)sb.n_seqs * a.q_tokens * kHeads;
    cuuint64_t dims[2] = {kRow, rows};
    cuuint64_t strides[1] = {kRow * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t es[2] = {1, 1};
    if (enc(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)q_abs, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_error("tensor map for the absorbed queries could not be encoded");
      return RELUX_ERR_CUDA;
    }
  }
  Params k;
  k.items = plan.items;
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.len = p->d_len + (size_t)a.layer * prm.max_seqs;
  k.num_pages = prm.num_pages;
  k.S = a.q_tokens;
  k.extra = a.extra_tokens;
  k.causal = a.causal;
  k.layer_row0 = (int32_t)((int64_t)a.layer * prm.num_pages * kNumKB * kPage);
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.part_o = (float*)p->part_o.p;
  k.part_ml = (float*)p->part_ml.p;
  k.rows_total = a.q_tokens * kHeads;
  k.status = p->d_status;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_decode_sm100_t256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  dim3 grid(2 * plan.num_items, a.q_tokens);
  mla_decode_sm100_t256_kernel<<<grid, 192, kSmemTotal, p->dev->stream>>>(p->tmap_mla, tq, k);
  RELUX_CUDA_TRY(cudaGetLastError());
  return RELUX_OK;
}

}  // namespace relux
