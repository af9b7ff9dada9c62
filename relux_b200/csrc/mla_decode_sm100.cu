// Absorbed MLA flash-decode on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA page loads.
// Shape: 128 query heads, latent 512, rope key 64 (row = 576 bf16 = 1152 B), 64-token pages.
//
// Why a CTA PAIR per worker.  The 128 heads that share one latent row are the M dimension of both
// contractions (S = Q~ K^T, O = P C).  O alone is 128 x 512 f32 = all 512 TMEM columns of one SM, and
// Q~ (128 x 576 bf16 = 144 KB) would leave no shared memory for KV tiles.  With cta_group::2 each CTA owns
// 64 heads: Q~ is 72 KB per CTA, O is 64 x 512 f32 = 256 TMEM columns (lanes 0-63 hold output dims
// [0,128) of each 256-wide block, lanes 64-127 dims [128,256)), and the B operand (the KV rows) is split between
// the two CTAs' shared memories and read by both tensor cores.  No TMA multicast is used anywhere: each CTA
// issues its own loads (`.cta_group::2` only routes the completion bytes to the leader's mbarrier).
//
// Persistent workers over a stream partition.  The pages of all sequences of the call, laid end to end, are cut
// into as many equal ranges as CTA pairs fit on the GPU; a worker (one pair) walks its range once.  An ITEM is
// the part of one sequence inside one range, so a worker changes item (new Q~, new accumulator, one split-KV
// partial written) only where a sequence ends inside its range.  The tile pipeline does not drain at an item
// boundary: Q~ of the next item is loaded as soon as the last QK^T of the current one has completed, and the
// first QK^T of the next item is issued right behind the last PV of the current one.
//
// Per 128-token tile (two pages; page r of the tile belongs to CTA r):
//   S[128 x 128]  = Q~[128 x 576] . K[128 tok x 576]^T      36 MMAs M128 N128 K16, K-major A and B
//   softmax warps : S from TMEM -> scaled exp2 with a lazily updated running max -> P (bf16) to shared memory
//   O[128 x 512] += P[128 x 128 tok] . C[128 tok x 512]      16 MMAs M128 N256 K16, B is MN-major (the same
//                                                              row-major page data, read "transposed" by descriptor)
// Shared memory per CTA: Q~ 72 KB | K slots 9 x 8 KB (own page, 64-dim column blocks) | V slots 4 x 16 KB
// (both pages x own 256 output dims) | P 16 KB | barriers.  Every slot has a full barrier (in the leader CTA,
// counting the bytes of both CTAs' loads) and an empty barrier (in each CTA, armed by tcgen05.commit multicast).
// Tiles are numbered g = 0, 1, ... over the worker's whole range; every barrier completes one phase per tile
// (s_full[b] one per tile with g & 1 == b; q_full one per item), which gives all wait parities.
// Issue order of the MMA warp: QK(0); then for each tile g: QK(g+1), PV(g) -- so the softmax of tile g+1
// overlaps PV(g) and QK(g+2).
//
// All waits are bounded; a wait that runs out sets RELUX_ERR_TIMEOUT in the status word, raises a shared abort
// flag so the other warps stop waiting too, and the CTA pair still meets at the final cluster barrier and frees
// its tensor memory.
#include <algorithm>
#include <cstdlib>
#include <cuda_bf16.h>
#include "common.cuh"
#include "internal.h"
#include "splitkv.h"
#include "umma.cuh"

namespace relux {

namespace {

constexpr int kMaxHeads = 128, kDC = 512, kDR = 64, kRow = kDC + kDR;  // 576
constexpr int kPage = 64;
constexpr int kBlk = 8192;                  // one [64 rows x 64 cols] bf16 block, 128-byte swizzled
constexpr int kNumKB = kRow / 64;           // 9 column blocks per row
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + kNumKB * kBlk;        // 73728
constexpr int kSmemV = kSmemK + kNumKB * kBlk;        // 147456
constexpr int kSmemP = kSmemV + 4 * 2 * kBlk;         // 212992
constexpr int kSmemBar = kSmemP + 2 * kBlk;           // 229376
constexpr int kSmemTotal = kSmemBar + 2048;           // 231424 of the 232448 bytes a CTA may use
constexpr int kKGroups = 3, kKPerGroup = kNumKB / kKGroups;  // K slots are armed / released in groups of 3 blocks
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0, kTmemS = 256;          // O: 2 x 128 columns; S: 2 buffers x 64 columns
constexpr float kRescaleThreshold = 8.0f;             // log2 units: rescale O only when the max grew by > 2^8
constexpr int kMaxInterleavedQ = 8;                   // up to this many query tokens work side by side on one range

struct Bars {
  uint64_t k_full[kKGroups], k_empty[kKGroups];
  uint64_t v_full[4], v_empty[4];
  uint64_t s_full[2];
  uint64_t p_full, pv_done, q_full;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  float rowmax[2][2][64];   // [tile parity][token half][row]
  float lsum[64];
};
static_assert(sizeof(Bars) <= 2048, "barrier block too large");

struct MlaSm100Params {
  const StreamItem* items;
  const int32_t* worker_first;   // [workers + 1]
  const int32_t* table;
  int32_t table_stride;
  int32_t num_pages, S, sx, causal;   // sx: query tokens interleaved along grid x (their workers share the range through L2)
  int32_t H;                          // query heads, <= 128: the M = 128 tile is padded with whatever rows follow in q~
                                      // (finite values, computed and thrown away; rows past the end of q~ are zero-filled by TMA)
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

// Bounded wait.  The common case (phase already complete) is a single try_wait.  When the bound runs out the
// waiter records RELUX_ERR_TIMEOUT, raises the CTA's abort flag and RETURNS: nobody leaves a loop early, every
// later wait sees the flag on its first failed poll and returns at once, so all warps still reach the named
// barriers and the final cluster barrier with garbage results and a non-zero status word.
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

__device__ __forceinline__ StreamItem load_item(const StreamItem* p) {
  const int4 a = __ldg(reinterpret_cast<const int4*>(p));
  const int4 b = __ldg(reinterpret_cast<const int4*>(p) + 1);
  StreamItem it;
  it.seq_index = a.x; it.seq = a.y; it.page_begin = a.z; it.page_end = a.w;
  it.tokens = b.x; it.pad[0] = it.pad[1] = it.pad[2] = 0;
  return it;
}

// Page ids of an item as the producer warp holds them: lane l keeps the first pool row (TMA y coordinate) of
// pages 32 * blk + l (`cur`) and 32 * (blk + 1) + l (`nxt`); positions past the item's last page repeat the last page.
struct PageWin {
  int32_t cur, nxt, blk;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
    mla_decode_sm100_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_q,
                            const MlaSm100Params prm) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = blockIdx.x >> 1;
  const int worker = cluster / prm.sx;
  const int sq = blockIdx.y * prm.sx + cluster % prm.sx;   // query token of this worker
  chain_release();
  chain_wait();   // the ranges, the absorbed queries and the step's new rows come from the kernel before this one
  const int it0 = prm.worker_first[worker], it1 = prm.worker_first[worker + 1];
  if (it0 >= it1 || sq >= prm.S) return;   // an empty range: both CTAs of the pair leave before any pair-wide step

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
    if (el) {
      tma_prefetch_desc(&tmap_kv);
      tma_prefetch_desc(&tmap_q);
    }
    auto win_load = [&](const StreamItem& it, int blk) -> int32_t {
      const int lp = min(32 * blk + lane, it.page_end - it.page_begin - 1);
      int32_t pg = __ldg(prm.table + (size_t)it.seq * prm.table_stride + it.page_begin + lp);
      if (pg < 0 || pg >= prm.num_pages) {   // reported, and replaced by page 0 so that no load leaves the pool
        set_status(prm.status, RELUX_ERR_BAD_PAGE);
        pg = 0;
      }
      return prm.layer_row0 + pg * (kNumKB * kPage);
    };
    auto win_get = [&](const PageWin& w, int lp) -> int32_t {
      if ((lp >> 5) == w.blk) return __shfl_sync(0xffffffffu, w.cur, lp & 31);
      return __shfl_sync(0xffffffffu, w.nxt, lp & 31);
    };
    // g = worker-wide index of the tile being loaded
    auto load_q = [&](const StreamItem& it) {
      const int qrow = (it.seq_index * prm.S + sq) * prm.H + 64 * (int)rank;   // Q~ rows of this CTA's 64 heads
      if (el) {
        if (rank == 0) mbar_expect_tx(&bars->q_full, 2 * kNumKB * kBlk);
#pragma unroll
        for (int db = 0; db < kNumKB; db++) tma_load_2d_2sm(smem + kSmemQ + db * kBlk, &tmap_q, db * 64, qrow, lead_q);
      }
      __syncwarp();
    };
    auto load_k = [&](const PageWin& w, int tile, int g) {
      const int32_t y = win_get(w, 2 * tile + (int)rank);   // the tile's page held by this CTA
#pragma unroll
      for (int grp = 0; grp < kKGroups; grp++) {
        if (g > 0) wait_bar(&bars->k_empty[grp], (g - 1) & 1, bars, prm.status);
        const uint32_t lead = mapa_u32(smem_u32(&bars->k_full[grp]), 0);
        if (el) {
          if (rank == 0) mbar_expect_tx(&bars->k_full[grp], 2 * kKPerGroup * kBlk);
#pragma unroll
          for (int j = 0; j < kKPerGroup; j++) {
            const int db = grp * kKPerGroup + j;
            tma_load_2d_2sm(smem + kSmemK + db * kBlk, &tmap_kv, 0, y + db * kPage, lead);
          }
        }
        __syncwarp();
      }
    };
    auto load_v = [&](const PageWin& w, int tile, int g) {
      const int32_t y0 = win_get(w, 2 * tile), y1 = win_get(w, 2 * tile + 1);
#pragma unroll
      for (int u = 0; u < 4; u++) {  // u = nb * 2 + kb
        const int nb = u >> 1, kb = u & 1;
        if (g > 0) wait_bar(&bars->v_empty[u], (g - 1) & 1, bars, prm.status);
        const int32_t y = kb ? y1 : y0;
        const uint32_t lead = mapa_u32(smem_u32(&bars->v_full[u]), 0);
        const int blk0 = 4 * nb + 2 * (int)rank;   // this CTA's 128 output dims of block nb = column blocks blk0, blk0 + 1
        if (el) {
          if (rank == 0) mbar_expect_tx(&bars->v_full[u], 4 * kBlk);
          tma_load_2d_2sm(smem + kSmemV + u * 2 * kBlk, &tmap_kv, 0, y + blk0 * kPage, lead);
          tma_load_2d_2sm(smem + kSmemV + u * 2 * kBlk + kBlk, &tmap_kv, 0, y + (blk0 + 1) * kPage, lead);
        }
        __syncwarp();
      }
    };
    StreamItem cur = load_item(prm.items + it0);
    PageWin w;
    w.cur = win_load(cur, 0);
    w.nxt = win_load(cur, 1);
    w.blk = 0;
    load_q(cur);
    load_k(w, 0, 0);
    int g = 0;
    for (int it = it0; it < it1; ++it) {
      const bool has_next = it + 1 < it1;
      StreamItem nxt = cur;
      PageWin wn = w;
      if (has_next) {   // fetched now, used at the end of this item
        nxt = load_item(prm.items + it + 1);
        wn.cur = win_load(nxt, 0);
        wn.nxt = win_load(nxt, 1);
        wn.blk = 0;
      }
      const int npages = cur.page_end - cur.page_begin;
      const int ntiles = (npages + 1) >> 1;
      for (int i = 0; i < ntiles; i++, g++) {
        if (i + 1 < ntiles) {
          load_k(w, i + 1, g + 1);
        } else if (has_next) {
          // the next item's first K tile goes group by group behind QK^T(g) like any other tile; Q~ may be replaced once
          // the last QK^T of this item (tile g) has completed, which the last group's slot being free says
          load_k(wn, 0, g + 1);
          wait_bar(&bars->k_empty[kKGroups - 1], g & 1, bars, prm.status);
          load_q(nxt);
        }
        load_v(w, i, g);
        if (((2 * i + 2) >> 5) > w.blk) {
          w.cur = w.nxt;
          w.blk++;
          w.nxt = win_load(cur, w.blk + 1);
        }
      }
      cur = nxt;
      w = wn;
    }
  } else if (warp == 5) {
    // =============================== MMA issuer (leader CTA only, converged warp + elected lane) ===============================
    if (rank == 0) {
      const bool el = elect_one();
      const uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      const uint32_t idesc_pv = make_idesc_bf16(128, 256, false, true);
      // descriptors of the region bases; an operand at +bytes is base + (bytes >> 4) in the low word
      const uint64_t dQ = make_desc_kmajor_sw128(smem_u32(smem + kSmemQ));
      const uint64_t dK = make_desc_kmajor_sw128(smem_u32(smem + kSmemK));
      const uint64_t dP = make_desc_kmajor_sw128(smem_u32(smem + kSmemP));
      const uint64_t dV = make_desc_mnmajor_sw128(smem_u32(smem + kSmemV), kBlk);
      auto issue_qk = [&](int g) {
        const uint32_t d = tmem + kTmemS + (g & 1) * 64;
#pragma unroll
        for (int grp = 0; grp < kKGroups; grp++) {
          wait_bar(&bars->k_full[grp], g & 1, bars, prm.status);
          if (el) {
#pragma unroll
            for (int j = 0; j < kKPerGroup * 4; j++) {
              const uint32_t off = (uint32_t)((grp * kKPerGroup + (j >> 2)) * kBlk + (j & 3) * 32) >> 4;
              umma_ss<2>(d, dQ + off, dK + off, idesc_qk, (grp | j) != 0);
            }
            umma_commit_mc<2>(&bars->k_empty[grp], 0x3);
          }
          __syncwarp();
        }
        if (el) umma_commit_mc<2>(&bars->s_full[g & 1], 0x3);
        __syncwarp();
      };
      auto issue_pv = [&](int g, bool first) {
        wait_bar(&bars->p_full, g & 1, bars, prm.status);
        tc_fence_after();   // P rows, a possible O rescale and the previous item's O read-out were done by the softmax warps
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int nb = u >> 1, kb = u & 1;
          wait_bar(&bars->v_full[u], g & 1, bars, prm.status);
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
              umma_ss<2>(tmem + kTmemO + nb * 128, dP + ((uint32_t)(kb * kBlk + kk * 32) >> 4),
                         dV + ((uint32_t)(u * 2 * kBlk + kk * 2048) >> 4), idesc_pv, !first || (kb | kk) != 0);
            umma_commit_mc<2>(&bars->v_empty[u], 0x3);
          }
          __syncwarp();
        }
        if (el) umma_commit_mc<2>(&bars->pv_done, 0x3);
        __syncwarp();
      };
      auto tiles_of = [&](int it) -> int {
        const int4 a = __ldg(reinterpret_cast<const int4*>(prm.items + it));
        return (a.w - a.z + 1) >> 1;
      };
      int ntiles = tiles_of(it0);
      int g = 0, n = 0;
      wait_bar(&bars->q_full, 0, bars, prm.status);
      issue_qk(0);
      for (int it = it0; it < it1; ++it, ++n) {
        const bool has_next = it + 1 < it1;
        const int next_tiles = has_next ? tiles_of(it + 1) : 0;
        for (int i = 0; i < ntiles; i++, g++) {
          if (i + 1 < ntiles) {
            issue_qk(g + 1);
          }
          issue_pv(g, i == 0);
          if (i + 1 == ntiles && has_next) {
            // at an item end PV(g) goes first: the next Q~ lands a memory latency after QK^T(g), later than P(g) is ready,
            // and the softmax warps can start writing the item out as soon as PV(g) has completed
            wait_bar(&bars->q_full, (n + 1) & 1, bars, prm.status);
            issue_qk(g + 1);
          }
        }
        ntiles = next_tiles;
      }
    }
  } else {
    // =============================== softmax / correction / epilogue (warps 0-3) ===============================
    const int L = warp * 32 + lane;   // TMEM lane
    const int row = L & 63;           // head index inside this CTA
    const int hf = L >> 6;            // token half of the tile (= which CTA's page)
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const uint32_t p_full_lead = mapa_u32(smem_u32(&bars->p_full), 0);
    StreamItem cur = load_item(prm.items + it0);
    int g = 0;
    for (int it = it0; it < it1; ++it) {
      StreamItem nxt = cur;
      if (it + 1 < it1) nxt = load_item(prm.items + it + 1);   // fetched now, used after this item
      const int limit_tok = prm.causal ? (cur.tokens - prm.S + sq + 1) : cur.tokens;   // tokens [0, limit_tok) are visible
      const int tok_end = min(limit_tok, cur.page_end * kPage);
      const int ntiles = (cur.page_end - cur.page_begin + 1) >> 1;
      float m_used = -INFINITY, l_run = 0.f;
      for (int i = 0; i < ntiles; i++, g++) {
        // no thread leaves this loop early: every thread must reach the same named barriers
        wait_bar(&bars->s_full[g & 1], (g >> 1) & 1, bars, prm.status);
        tc_fence_after();
        uint32_t sv[2][32];
        tmem_ld_32x32b_x32(tmem + lane_addr + kTmemS + (g & 1) * 64, sv[0]);
        tmem_ld_32x32b_x32(tmem + lane_addr + kTmemS + (g & 1) * 64 + 32, sv[1]);
        tmem_ld_wait();
        // valid tokens of this thread's 64: [0, nvalid); only the last tile(s) of an item are partial
        const int tok0 = (cur.page_begin + 2 * i + hf) * kPage;
        const int nvalid = (cur.page_begin + 2 * i + hf < cur.page_end) ? max(0, min(kPage, tok_end - tok0)) : 0;
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
        bars->rowmax[g & 1][hf][row] = mx;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        mx = fmaxf(mx, bars->rowmax[g & 1][hf ^ 1][row]);
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
        // P(g) may overwrite the buffer, and O may be rescaled, only after PV(g-1) has completed
        if (g > 0) wait_bar(&bars->pv_done, (g - 1) & 1, bars, prm.status);
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
        // P row: 64 tokens = 128 bytes = one swizzled row of block hf
        uint8_t* prow = smem + kSmemP + hf * kBlk + row * 128;
#pragma unroll
        for (int c = 0; c < 8; c++)
          *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(p_full_lead);
      }
      // ---- item epilogue: O (unnormalised), running max and sum -> split-KV partial of this item ----
      wait_bar(&bars->pv_done, (g - 1) & 1, bars, prm.status);
      const bool ok = !bars->abort_flag;
      tc_fence_after();
      if (hf == 1) bars->lsum[row] = l_run;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const bool real_head = 64 * (int)rank + row < prm.H;   // padding rows of the tile are not written
      const size_t prow = (size_t)it * prm.rows_total + (size_t)sq * prm.H + 64 * rank + row;
      if (hf == 0 && real_head) {
        prm.part_ml[prow * 2] = ok ? m_used : -INFINITY;
        prm.part_ml[prow * 2 + 1] = ok ? (l_run + bars->lsum[row]) : 0.f;
      }
      // O leaves through the P tile (free between the item's last PV and the next item's first softmax): a thread holds
      // one row, so stores straight from its registers put 32 rows into every instruction (6-8 us per item, measured);
      // staged, 8 lanes write one 128-byte segment of a row.  16-byte chunks are swizzled by the row on both sides.
      float* obase = prm.part_o + ((size_t)it * prm.rows_total + (size_t)sq * prm.H + 64 * rank) * kDC;   // this CTA's row 0
      const int heads_here = prm.H - 64 * (int)rank;   // rows [0, heads_here) are real heads
      uint8_t* stage = smem + kSmemP;
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
          uint8_t* srow = stage + (row * 2 + hf) * 128;   // segment (row, hf): columns 256 nb + 128 hf + c .. + 31
#pragma unroll
          for (int j = 0; j < 8; j++)
            *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) = make_uint4(ov[4 * j], ov[4 * j + 1], ov[4 * j + 2], ov[4 * j + 3]);
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
          for (int k = 0; k < 8; k++) {
            const int seg = k * 16 + (L >> 3), r = seg >> 1, h2 = seg & 1, j = L & 7;
            const uint4 v = *reinterpret_cast<const uint4*>(stage + seg * 128 + ((j ^ (r & 7)) << 4));
            if (r < heads_here) *reinterpret_cast<uint4*>(obase + (size_t)r * kDC + 256 * nb + 128 * h2 + c + 4 * j) = v;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      tc_fence_before();   // the O read-out is ordered before this thread's next p_full arrival, which releases the first PV of the next item
      cur = nxt;
    }
  }
  tc_fence_before();
  cluster_sync();
  if (warp == 0) tmem_dealloc<2>(tmem, kTmemCols);
}

}  // namespace

bool mla_sm100_eligible(const Pool* p, const relux_attn_args& a) {
  const relux_pool_params& prm = p->prm;
  if (p->tune.get(RELUX_TUNE_MLA_GENERIC)) return false;
  // fewer than 128 heads run on the same M = 128 tile (padded); below 16 heads the CUDA-core kernel is the better fit
  return p->has_tmap && p->mla_blocked && prm.page_tokens == kPage && prm.mla_dc == kDC && prm.mla_dhr == kDR && a.num_heads <= kMaxHeads &&
         a.num_heads >= 16;
}


// Number of ranges the stream of pages is cut into: one per CTA pair that can be resident at the same time,
// divided among the query tokens that run side by side.
int mla_sm100_workers(Pool* p, int q_tokens) {
  static int max_clusters = 0;
  if (!max_clusters) {
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74, 1, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = kSmemTotal;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(mla_decode_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, mla_decode_sm100_kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = std::max(1, p->dev->sm_count / 2);
    }
    max_clusters = n;
  }
  int mc = max_clusters;
  if (const int ov = p->tune.get(RELUX_TUNE_MLA_WORKERS)) mc = std::max(1, ov);   // tuning knob
  if (q_tokens > kMaxInterleavedQ) {
    // A long multi-token call (a prompt) has one row of workers per query token: the rows already fill the device, so a
    // row needs only enough workers for about two waves in total, and each worker walks a long piece of the stream
    // (2048 tokens, one sequence: 3.2 ms with a full row of workers per token, 0.94 ms with one).
    return std::min(mc, std::max(1, (2 * mc + q_tokens - 1) / q_tokens));
  }
  return std::max(1, mc / q_tokens);
}

int32_t launch_mla_decode_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const SplitPlan& plan, const uint16_t* q_abs) {
  const relux_pool_params& prm = p->prm;
  if (plan.num_items == 0) return RELUX_OK;   // every sequence is empty: the merge writes zeros
  CUtensorMap tq;   // the absorbed queries [rows][576], 64 x 64 boxes
  if (!make_tmap_2d(&tq, (void*)q_abs, (uint64_t)sb.n_seqs * a.q_tokens * a.num_heads, kRow, 64, 64)) {
    set_error("tensor map for the absorbed queries could not be encoded");
    return RELUX_ERR_CUDA;
  }
  const int sx = a.q_tokens <= kMaxInterleavedQ ? a.q_tokens : 1;
  MlaSm100Params k;
  k.items = plan.stream_items;
  k.worker_first = plan.worker_first;
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.num_pages = prm.num_pages;
  k.S = a.q_tokens;
  k.sx = sx;
  k.causal = a.causal;
  k.layer_row0 = (int32_t)((int64_t)a.layer * prm.num_pages * kNumKB * kPage);
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.part_o = (float*)p->part_o.p;
  k.part_ml = (float*)p->part_ml.p;
  k.rows_total = a.q_tokens * a.num_heads;
  k.H = a.num_heads;
  k.status = p->d_status;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_decode_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  dim3 grid(2 * plan.num_workers * sx, a.q_tokens / sx);
  RELUX_CUDA_TRY(launch_chained(p->tune.get(RELUX_TUNE_CHAINED_LAUNCHES) != 0, mla_decode_sm100_kernel, grid, dim3(192), (size_t)kSmemTotal,
                                p->dev->stream, p->tmap_mla, tq, k));
  return RELUX_OK;
}

}  // namespace relux
