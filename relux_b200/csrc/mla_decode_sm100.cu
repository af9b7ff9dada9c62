// Absorbed MLA flash-decode on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA page loads.
// Shape: 128 query heads, latent 512, rope key 64 (row = 576 bf16 = 1152 B), 64-token pages.
//
// Why a CTA PAIR per work item.  The 128 heads that share one latent row are the M dimension of both
// contractions (S = Q~ K^T, O = P C).  O alone is 128 x 512 f32 = all 512 TMEM columns of one SM, and
// Q~ (128 x 576 bf16 = 144 KB) would leave no shared memory for KV tiles.  With cta_group::2 each CTA owns
// 64 heads: Q~ is 72 KB per CTA, O is 64 x 512 f32 = 256 TMEM columns (lanes 0-63 hold output dims
// [0,128) of each 256-wide block, lanes 64-127 dims [128,256)), and the B operand (the KV rows) is split between
// the two CTAs' shared memories and read by both tensor cores.  No TMA multicast is used anywhere: each CTA
// issues its own loads (`.cta_group::2` only routes the completion bytes to the leader's mbarrier).
//
// One work item = (sequence, chunk of pages, query token).  Per 128-token tile (two pages; page r of the tile
// belongs to CTA r):
//   S[128 x 128]  = Q~[128 x 576] . K[128 tok x 576]^T      36 MMAs M128 N128 K16, K-major A and B
//   softmax warps : S from TMEM -> scaled exp2 with a lazily updated running max -> P (bf16) to shared memory
//   O[128 x 512] += P[128 x 128 tok] . C[128 tok x 512]      16 MMAs M128 N256 K16, B is MN-major (the same
//                                                              row-major page data, read "transposed" by descriptor)
// Shared memory per CTA: Q~ 72 KB | K slots 9 x 8 KB (own page, 64-dim column blocks) | V slots 4 x 16 KB
// (both pages x own 256 output dims) | P 16 KB | barriers.  Every slot has a full barrier (in the leader CTA,
// counting the bytes of both CTAs' loads) and an empty barrier (in each CTA, armed by tcgen05.commit multicast).
// Issue order of the single MMA thread: QK(0); then for each tile i: QK(i+1), PV(i) -- so the softmax of tile i+1
// overlaps PV(i) and QK(i+2).
//
// All waits are bounded; a wait that runs out sets RELUX_ERR_TIMEOUT in the status word, raises a shared abort
// flag so the other warps stop waiting too, and the CTA pair still meets at the final cluster barrier and frees
// its tensor memory.
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
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + kNumKB * kBlk;        // 73728
constexpr int kSmemV = kSmemK + kNumKB * kBlk;        // 147456
constexpr int kSmemP = kSmemV + 4 * 2 * kBlk;         // 212992
constexpr int kSmemBar = kSmemP + 2 * kBlk;           // 229376
constexpr int kSmemTotal = kSmemBar + 3072;           // 232448 = the 227 KB a CTA may use
constexpr int kMaxChunkPages = 320;                   // page ids of a chunk are cached in shared memory
constexpr int kKGroups = 3, kKPerGroup = kNumKB / kKGroups;  // K slots are armed / released in groups of 3 blocks
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0, kTmemS = 256;          // O: 2 x 128 columns; S: 2 buffers x 64 columns
constexpr int kPrefetchTiles = 0;                      // L2 prefetch distance of the producer in tiles (0 = off: measured no gain,
                                                       // the kernel is bound by the tensor pipe at the power-capped clock, not by load latency)
constexpr float kRescaleThreshold = 8.0f;             // log2 units: rescale O only when the max grew by > 2^8

struct Bars {
  uint64_t k_full[kKGroups], k_empty[kKGroups];
  uint64_t v_full[4], v_empty[4];
  uint64_t s_full[2];
  uint64_t p_full, pv_done, q_full;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  float rowmax[2][2][64];   // [tile parity][token half][row]
  float lsum[64];
  int32_t page_row[kMaxChunkPages];   // first pool row (TMA y coordinate) of every page of this chunk
#ifdef RELUX_MLA_PROF
  long long ts_k[kNumKB], ts_v[4], ts_pv;
#endif
};
static_assert(sizeof(Bars) <= 3072, "barrier block too large");

struct MlaSm100Params {
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
  long long* prof;   // optional cycle counters of cluster 0 (RELUX_MLA_PROF builds only)
  int32_t dbg;       // RELUX_MLA_PROF builds: 1 = skip V loads, 2 = skip K loads after the first tile (timing experiments, wrong results)
};

#ifdef RELUX_MLA_PROF
#define PROF_T0() long long prof_t0__ = clock64()
#define PROF_ADD(slot) do { if (prm.prof && blockIdx.x < 2 && blockIdx.y == 0) prof_acc[slot] += clock64() - prof_t0__; } while (0)
#define PROF_DECL() long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; const long long prof_start = clock64()
#define PROF_FLUSH(base) do { if (prm.prof && blockIdx.x < 2 && blockIdx.y == 0) { for (int q_ = 0; q_ < 8; q_++) prm.prof[(blockIdx.x * 4 + (base)) * 8 + q_] = prof_acc[q_]; prm.prof[100 + blockIdx.x * 4 + (base)] = clock64() - prof_start; } } while (0)
#else
#define PROF_T0()
#define PROF_ADD(slot)
#define PROF_DECL()
#define PROF_FLUSH(base)
#endif

// Bounded wait.  The common case (phase already complete) is a single try_wait.  When the bound runs out the
// waiter records RELUX_ERR_TIMEOUT, raises the CTA's abort flag and RETURNS: nobody leaves a loop early, every
// later wait sees the flag on its first failed poll and returns at once, so all warps still reach the named
// barriers and the final cluster barrier with garbage results and a non-zero status word.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

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
    mla_decode_sm100_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_q,
                            const MlaSm100Params prm) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int item_idx = blockIdx.x >> 1;
  const int sq = blockIdx.y;  // query token of this work item
  const WorkItem item = prm.items[item_idx];
  const int T = prm.len[item.seq] + prm.extra;
  const int limit_tok = prm.causal ? (T - prm.S + sq + 1) : T;             // tokens [0, limit_tok) are visible
  const int tok_end = min(limit_tok, item.page_end * kPage);
  const int npages = item.page_end - item.page_begin;
  const int ntiles = (npages + 1) >> 1;

  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled layouts need a 1024-byte aligned base
    if (threadIdx.x == 0) set_status(prm.status, RELUX_ERR_UNSUPPORTED);
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kKGroups; i++) { mbar_init(&bars->k_full[i], 1); mbar_init(&bars->k_empty[i], 1); }
    for (int i = 0; i < 4; i++) { mbar_init(&bars->v_full[i], 1); mbar_init(&bars->v_empty[i], 1); }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 8);    // one arrival per softmax warp of each CTA of the pair
    mbar_init(&bars->pv_done, 1);
    mbar_init(&bars->q_full, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc<2>(&bars->tmem_base, kTmemCols);
    tmem_relinquish<2>();
  }
  // page table slice of this chunk -> shared memory (validated once; a bad id is reported and replaced by page 0)
  for (int i = threadIdx.x; i < npages && i < kMaxChunkPages; i += blockDim.x) {
    int32_t pg = prm.table[(size_t)item.seq * prm.table_stride + item.page_begin + i];
    if (pg < 0 || pg >= prm.num_pages) {
      set_status(prm.status, RELUX_ERR_BAD_PAGE);
      pg = 0;
    }
    bars->page_row[i] = prm.layer_row0 + pg * (kNumKB * kPage);   // first TMA row of the page's block 0
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 4) {
    // =============================== producer: TMA loads into this CTA's slots ===============================
    // The whole warp stays converged and one elected lane issues: operands that every lane computes identically
    // live in uniform registers, which is what keeps the issue rate of TMA / tcgen05 instructions high.
    const bool el = elect_one();
    const uint32_t lead_q = mapa_u32(smem_u32(&bars->q_full), 0);
    const int qrow = (item.seq_index * prm.S + sq) * kHeads + 64 * (int)rank;   // Q~ rows of this CTA's 64 heads
    if (el) {
      tma_prefetch_desc(&tmap_kv);
      tma_prefetch_desc(&tmap_q);
      if (rank == 0) mbar_expect_tx(&bars->q_full, 2 * kNumKB * kBlk);
#pragma unroll
      for (int db = 0; db < kNumKB; db++) tma_load_2d_2sm(smem + kSmemQ + db * kBlk, &tmap_q, db * 64, qrow, lead_q);
    }
    __syncwarp();
    // page of the tile held by CTA r (falls back to the chunk's first page when the tile has only one page)
    auto page_row = [&](int tile, int r) -> int32_t {
      int lp = 2 * tile + r;
      if (lp >= npages) lp = 0;
      return bars->page_row[lp];
    };
    auto load_k = [&](int tile) {
      const int32_t y = page_row(tile, rank);
#pragma unroll
      for (int g = 0; g < kKGroups; g++) {
        if (tile > 0) wait_bar(&bars->k_empty[g], (tile - 1) & 1, bars, prm.status);
        const uint32_t lead = mapa_u32(smem_u32(&bars->k_full[g]), 0);
#ifdef RELUX_MLA_PROF
        if ((prm.dbg & 2) && tile > 0) {
          if (el && rank == 0) mbar_arrive(&bars->k_full[g]);
          __syncwarp();
          continue;
        }
#endif
        if (el) {
          if (rank == 0) mbar_expect_tx(&bars->k_full[g], 2 * kKPerGroup * kBlk);
#pragma unroll
          for (int j = 0; j < kKPerGroup; j++) {
            const int db = g * kKPerGroup + j;
            tma_load_2d_2sm(smem + kSmemK + db * kBlk, &tmap_kv, 0, y + db * kPage, lead);
          }
        }
        __syncwarp();
      }
    };
    auto load_v = [&](int tile) {
#pragma unroll
      for (int u = 0; u < 4; u++) {  // u = nb * 2 + kb
        const int nb = u >> 1, kb = u & 1;
        if (tile > 0) wait_bar(&bars->v_empty[u], (tile - 1) & 1, bars, prm.status);
        const int32_t y = page_row(tile, kb);
        const uint32_t lead = mapa_u32(smem_u32(&bars->v_full[u]), 0);
        const int blk0 = 4 * nb + 2 * (int)rank;   // this CTA's 128 output dims of block nb = column blocks blk0, blk0 + 1
#ifdef RELUX_MLA_PROF
        if (prm.dbg & 1) {
          if (el && rank == 0) mbar_arrive(&bars->v_full[u]);
          __syncwarp();
          continue;
        }
#endif
        if (el) {
          if (rank == 0) mbar_expect_tx(&bars->v_full[u], 4 * kBlk);
          tma_load_2d_2sm(smem + kSmemV + u * 2 * kBlk, &tmap_kv, 0, y + blk0 * kPage, lead);
          tma_load_2d_2sm(smem + kSmemV + u * 2 * kBlk + kBlk, &tmap_kv, 0, y + (blk0 + 1) * kPage, lead);
        }
        __syncwarp();
      }
    };
    // Shared memory holds a single tile, which cannot cover the HBM latency; the producer therefore pulls the
    // page of tile t + kPrefetchTiles into L2 (no shared memory, no barrier) so that the real loads hit L2.
    auto prefetch_k = [&](int tile) {
      if (tile < ntiles && el) {
        const int32_t y = page_row(tile, rank);
#pragma unroll
        for (int db = 0; db < kNumKB; db++) tma_prefetch_l2_2d(&tmap_kv, 0, y + db * kPage);
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
    // =============================== MMA issuer (leader CTA only, converged warp + elected lane) ===============================
    if (rank == 0) {
      PROF_DECL();
      const bool el = elect_one();
      const uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      const uint32_t idesc_pv = make_idesc_bf16(128, 256, false, true);
      // descriptors of the region bases; an operand at +bytes is base + (bytes >> 4) in the low word
      const uint64_t dQ = make_desc_kmajor_sw128(smem_u32(smem + kSmemQ));
      const uint64_t dK = make_desc_kmajor_sw128(smem_u32(smem + kSmemK));
      const uint64_t dP = make_desc_kmajor_sw128(smem_u32(smem + kSmemP));
      const uint64_t dV = make_desc_mnmajor_sw128(smem_u32(smem + kSmemV), kBlk);
      wait_bar(&bars->q_full, 0, bars, prm.status);
      auto issue_qk = [&](int tile) {
        const uint32_t d = tmem + kTmemS + (tile & 1) * 64;
#pragma unroll
        for (int g = 0; g < kKGroups; g++) {
          { PROF_T0();
          wait_bar(&bars->k_full[g], tile & 1, bars, prm.status);
          PROF_ADD(0); }
          if (el) {
#pragma unroll
            for (int j = 0; j < kKPerGroup * 4; j++) {
              const uint32_t off = (uint32_t)((g * kKPerGroup + (j >> 2)) * kBlk + (j & 3) * 32) >> 4;
              umma_ss<2>(d, dQ + off, dK + off, idesc_qk, (g | j) != 0);
            }
            umma_commit_mc<2>(&bars->k_empty[g], 0x3);
          }
          __syncwarp();
        }
        if (el) umma_commit_mc<2>(&bars->s_full[tile & 1], 0x3);
        __syncwarp();
      };
      auto issue_pv = [&](int tile) {
        { PROF_T0();
        wait_bar(&bars->p_full, tile & 1, bars, prm.status);
        PROF_ADD(1); }
        tc_fence_after();   // P rows and a possible O rescale were written by the softmax warps of both CTAs
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int nb = u >> 1, kb = u & 1;
          { PROF_T0();
          wait_bar(&bars->v_full[u], tile & 1, bars, prm.status);
          PROF_ADD(2); }
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
              umma_ss<2>(tmem + kTmemO + nb * 128, dP + ((uint32_t)(kb * kBlk + kk * 32) >> 4),
                         dV + ((uint32_t)(u * 2 * kBlk + kk * 2048) >> 4), idesc_pv, (tile | kb | kk) != 0);
            umma_commit_mc<2>(&bars->v_empty[u], 0x3);
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
      if (lane == 0) PROF_FLUSH(1);
    }
  } else {
    // =============================== softmax / correction / epilogue (warps 0-3) ===============================
    const int L = warp * 32 + lane;   // TMEM lane
    const int row = L & 63;           // head index inside this CTA
    const int hf = L >> 6;            // token half of the tile (= which CTA's page)
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    PROF_DECL();
    const uint32_t p_full_lead = mapa_u32(smem_u32(&bars->p_full), 0);
    for (int i = 0; i < ntiles; i++) {
      // no thread leaves this loop early: every thread must reach the same named barriers
      { PROF_T0();
      wait_bar(&bars->s_full[i & 1], (i >> 1) & 1, bars, prm.status);
      PROF_ADD(0); }
      tc_fence_after();
      PROF_T0();
      uint32_t sv[2][32];
      tmem_ld_32x32b_x32(tmem + lane_addr + kTmemS + (i & 1) * 64, sv[0]);
      tmem_ld_32x32b_x32(tmem + lane_addr + kTmemS + (i & 1) * 64 + 32, sv[1]);
      tmem_ld_wait();
      // valid tokens of this thread's 64: [0, nvalid); only the last tile(s) of a chunk are partial
      const int tok0 = (item.page_begin + 2 * i + hf) * kPage;
      const int nvalid = (item.page_begin + 2 * i + hf < item.page_end) ? max(0, min(kPage, tok_end - tok0)) : 0;
      if (nvalid < kPage) {
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++)
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (h2 * 32 + j >= nvalid) sv[h2][j] = 0xFF800000u;  // -inf
      }
      // row max of the raw scores (the softmax scale is positive, so it commutes with max)
      float mx = -INFINITY;
#pragma unroll
      for (int h2 = 0; h2 < 2; h2++)
#pragma unroll
        for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(sv[h2][j]));
      mx *= prm.scale_log2;
      bars->rowmax[i & 1][hf][row] = mx;
      PROF_ADD(1);
      { PROF_T0();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      PROF_ADD(2); }
      long long prof_t1__ = 0;
#ifdef RELUX_MLA_PROF
      prof_t1__ = clock64();
#endif
      mx = fmaxf(mx, bars->rowmax[i & 1][hf ^ 1][row]);
      // lazily updated running max: both threads of a row take the same decision
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + kRescaleThreshold) {   // also true on the first tile with a visible token (m_used = -inf)
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
        rescale = (m_used != -INFINITY);
        m_used = mx;
      }
      // p = 2^(s * scale_log2 - m): one FFMA and one MUFU.EX2 per score
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      float psum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int h2 = 0; h2 < 2; h2++)
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(sv[h2][j]), prm.scale_log2, neg_m));
          const float p1 = ex2_approx(fmaf(__uint_as_float(sv[h2][j + 1]), prm.scale_log2, neg_m));
          psum += p0 + p1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          pk[h2 * 16 + j / 2] = *reinterpret_cast<uint32_t*>(&b2);
        }
      l_run = l_run * alpha + psum;
      // P(i) may overwrite the buffer, and O may be rescaled, only after PV(i-1) has completed
#ifdef RELUX_MLA_PROF
      if (prm.prof && blockIdx.x < 2 && blockIdx.y == 0) prof_acc[3] += clock64() - prof_t1__;
#endif
      { PROF_T0();
      if (i > 0) wait_bar(&bars->pv_done, (i - 1) & 1, bars, prm.status);
      PROF_ADD(4); }
      if (rescale && i > 0) {
#ifdef RELUX_MLA_PROF
        ;
#endif
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
      // P row: 64 tokens = 128 bytes = one swizzled row of block hf
      { PROF_T0();
      uint8_t* prow = smem + kSmemP + hf * kBlk + row * 128;
#pragma unroll
      for (int c = 0; c < 8; c++)
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      PROF_ADD(6); }
      { PROF_T0();
      fence_proxy_async();
      PROF_ADD(7); }
      { PROF_T0();
      __syncwarp();
      PROF_ADD(5); }
      if (lane == 0) mbar_arrive_cluster(p_full_lead);
    }
    if (threadIdx.x == 0) PROF_FLUSH(2);
    // ---- epilogue: O (unnormalised), running max and sum of this chunk -> split-KV partial ----
    wait_bar(&bars->pv_done, (ntiles - 1) & 1, bars, prm.status);
    ok = !bars->abort_flag;
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

}  // namespace

bool mla_sm100_eligible(const Pool* p, const relux_attn_args& a) {
  const relux_pool_params& prm = p->prm;
  if (getenv("RELUX_MLA_GENERIC")) return false;
  return p->has_tmap && p->mla_blocked && prm.page_tokens == kPage && prm.mla_dc == kDC && prm.mla_dhr == kDR && a.num_heads == kHeads;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int32_t launch_mla_decode_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const SplitPlan& plan, const uint16_t* q_abs) {
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
  MlaSm100Params k;
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
  k.prof = nullptr;
  k.dbg = getenv("RELUX_MLA_DBG") ? atoi(getenv("RELUX_MLA_DBG")) : 0;
#ifdef RELUX_MLA_PROF
  static long long* d_prof = nullptr;
  if (!d_prof) cudaMalloc(&d_prof, 64 * 8 * sizeof(long long));
  cudaMemsetAsync(d_prof, 0, 64 * 8 * sizeof(long long), p->dev->stream);
  k.prof = d_prof;
#endif
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_decode_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  dim3 grid(2 * plan.num_items, a.q_tokens);
  mla_decode_sm100_kernel<<<grid, 192, kSmemTotal, p->dev->stream>>>(p->tmap_mla, tq, k);
  RELUX_CUDA_TRY(cudaGetLastError());
#ifdef RELUX_MLA_PROF
  {
    long long h[64 * 8];
    cudaStreamSynchronize(p->dev->stream);
    cudaMemcpy(h, d_prof, sizeof(h), cudaMemcpyDeviceToHost);
    const char* names[3] = {"producer [k_empty v_empty]", "mma      [k_full p_full v_full]", "softmax  [s_full math1 barmax math2 pv_done barP Pwrite fence_proxy]"};
    for (int cta = 0; cta < 2; cta++)
      for (int r = 0; r < 3; r++) {
        fprintf(stderr, "prof cta%d %s:", cta, names[r]);
        for (int q = 0; q < 8; q++) fprintf(stderr, " %lld", h[(cta * 4 + r) * 8 + q]);
        fprintf(stderr, "  total %lld\n", h[100 + cta * 4 + r]);
      }
    fprintf(stderr, "prof items=%d chunk_pages=%d stalled_k_waits=%lld\n", plan.num_items, plan.chunk_pages, h[200]);
  }
#endif
  return RELUX_OK;
}

}  // namespace relux
