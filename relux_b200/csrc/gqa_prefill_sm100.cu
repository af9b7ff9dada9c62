// Paged GQA prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), for multi-token cached calls
// (a prompt, or a long verify): the kernel the decode path lacks, because a decode CTA holds at most 32 query rows.
//
// What it replaces: the attention loops of MHA.forwardCached for seqQ > 1 (internal/transformer/mha.go:318-348) with the
// online-softmax rule of flashOnlineAccum.update (internal/transformer/flash_attention.go:36-73, 99-187): running max,
// rescale of sum and output by exp(old - new), accumulate exp(s - max) * v.  Semantics are the library's (causal INSIDE
// the new tokens: query row i sees cached rows j <= T - S + i).
//
// Shape: head_dim 128, 64-token pages, g = num_heads / num_kv_heads a divisor of 128.
// A block = 128 / g query tokens of one (sequence, kv head): the g query heads that share the kv head times the tokens
// are 128 rows (M) of both contractions.  An ITEM is a pair of adjacent blocks; a WORKER is a CTA pair (cluster of 2,
// tcgen05 cta_group::2, M = 256): CTA r owns block 2p + r of the item, the two blocks share every K / V tile, and each
// CTA loads HALF of it:
//   Q tile  : own 128 rows x 128 dims bf16 (32 KB), one 3-D TMA box per 64-dim half; row = token_in_block * g + head
//   per 128-key tile (two pages of the kv head):
//     S[256 x 128] = Q K^T      8 MMAs M256 N128 K16; B = K, split by keys: CTA r holds page 2j + r (16 KB)
//     softmax warps: S from TMEM -> exp2 with a lazily updated running max -> P bf16 into a swizzled shared tile
//                    (two P tiles in turn, so the exponentials of tile j+1 run while PV(j) still reads P(j))
//     O[256 x 128] += P V       8 MMAs M256 N128 K16; B = V as it lies (MN-major), split by output dims: CTA r holds
//                               dims [64 r, 64 r + 64) of both pages (16 KB)
// Persistent workers.  As many CTA pairs as fit on the GPU are launched once; worker w takes items w, w + W, ... of a
// list ordered longest first.  One launch per block measured 16k cycles (8 us) of fixed cost per CTA pair -- launch,
// tensor-memory allocation, the latency of the first Q / K loads, pipeline fill, drain and the epilogue -- against
// 2.1k cycles per tile: at 2048-token prompts (9 tiles per item on average) that was half of the kernel.  Here the tile
// pipeline does not drain at an item boundary: tiles are numbered over the worker's whole life, Q has two buffers (the
// next item's Q is requested while the current item's last tiles are in flight), the first QK^T of the next item is
// issued ahead of the last PV of the current one like any other tile, and an item's epilogue (O read-out, normalise,
// store) overlaps the next item's first QK^T and softmax: it is ordered before the thread's next p_full arrival, which
// is what releases the next item's first PV.
// TMEM per CTA: S double-buffered (2 x 128 columns), O 128 columns; rows = TMEM lanes.  Issue order QK(g+1), PV(g).
// Warp roles per CTA: 8 softmax / epilogue warps -- a query row (TMEM lane) is shared by two threads, 64 keys (and 64
// output dims) each --, 1 TMA producer, 1 MMA issuer (leader CTA only), both converged with one elected lane.
// Barriers: full barriers live in the leader CTA and count the bytes of both CTAs' loads; empty / s_full / pv_done
// barriers live in each CTA and are armed by tcgen05.commit with mbarrier multicast (not a TMA load); p_full lives in
// the leader and counts the softmax warps of both CTAs.  No TMA multicast anywhere.
// No split-KV: the output is normalised in the epilogue and written once.
// Every wait is bounded (status RELUX_ERR_TIMEOUT, shared abort flag, all warps still reach the end and free TMEM).
#include <algorithm>
#include <cuda_bf16.h>

#include "common.cuh"
#include "internal.h"
#include "umma.cuh"

namespace relux {

namespace {

constexpr int kD = 128, kPage = 64, kTile = 128;
constexpr int kBlk = 8192;                 // one [64 rows x 64 cols] bf16 box, 128-byte swizzled
constexpr int kHalf = 2 * kBlk;            // [128 rows x 64 cols]
constexpr int kQBytes = 2 * kHalf;         // one Q tile: [dims 0-63 | dims 64-127], each 128 rows x 128 B
constexpr int kSmemQ = 0;                  // two Q tiles (items in turn)
constexpr int kSmemP = kSmemQ + 2 * kQBytes;   // two P tiles (tiles in turn) of [keys 0-63 | keys 64-127]
constexpr int kPBytes = 2 * kHalf;
constexpr int kDepth = 3;                  // K / V tiles in flight
constexpr int kStages = 2 * kDepth;        // K(g), V(g), K(g+1), V(g+1), ...
constexpr int kStageBytes = 2 * kBlk;      // 16 KB per CTA.  K: own page [dims 0-63 | dims 64-127]; V: own 64 dims [page 0 | page 1]
constexpr int kSmemRing = kSmemP + 2 * kPBytes;
constexpr int kSmemBar = kSmemRing + kStages * kStageBytes;   // 229376
constexpr int kSmemTotal = kSmemBar + 3072;                   // 232448: all a CTA may use
constexpr int kSplit = 2;                                     // threads per query row: each takes 128 / kSplit keys and output dims
constexpr int kCols = 128 / kSplit;
constexpr int kSoftmaxWarps = 4 * kSplit;
constexpr int kSoftmaxThreads = 32 * kSoftmaxWarps, kThreads = kSoftmaxThreads + 64;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemS = 0, kTmemO = 256;
constexpr float kRescaleThreshold = 8.0f;

struct Bars {
  uint64_t q_full[2], q_empty[2], kv_full[kStages], kv_empty[kStages], s_full[2], p_full, pv_done;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  float rowmax[2][kSplit][128];   // [tile parity][key slice][row]; an item's epilogue borrows the buffer of the tile that follows
                                  // for the row sums of the key slices
};
static_assert(sizeof(Bars) <= 3072, "barrier block too large");

struct PrefillParams {
  const int32_t* table;
  int32_t table_stride;
  const int32_t* len;
  const int32_t* seq_ids;
  int32_t num_pages, Hkv, H, g, S, extra, causal;
  int32_t bq;                 // query tokens per block = 128 / g
  int32_t n_qblocks, n_pairs; // blocks and block pairs per (sequence, kv head)
  int32_t n_seqs, n_items;    // items = n_pairs * Hkv * n_seqs
  int32_t krow0, vrow0;       // first TMA row of this layer's K block / V block
  float scale_log2;
  float* out;                 // [n][S][H][128] f32
  int32_t* status;
};

// One item as every warp of the pair derives it from its index: the list runs over block pairs from the last (most
// keys under the causal mask) to the first, and inside a pair index over (sequence, kv head).
struct Item {
  int32_t bi, seq, hk, pair;
  int32_t T, ntiles, last_slot;
};
__device__ __forceinline__ Item item_of(const PrefillParams& prm, int idx) {
  Item it;
  const int per = prm.Hkv * prm.n_seqs;
  it.pair = prm.n_pairs - 1 - idx / per;
  const int rem = idx % per;
  it.hk = rem % prm.Hkv;
  it.bi = rem / prm.Hkv;
  it.seq = prm.seq_ids ? __ldg(prm.seq_ids + it.bi) : it.bi;
  it.T = __ldg(prm.len + it.seq) + prm.extra;
  // keys the PAIR needs: all T without the mask, else up to the position of its last real token
  const int last_tok = min(prm.S, (2 * it.pair + 2) * prm.bq) - 1;
  const int kmax = prm.causal ? (it.T - prm.S + last_tok + 1) : it.T;
  it.ntiles = (kmax + kTile - 1) / kTile;
  it.last_slot = (it.T + kPage - 1) / kPage - 1;   // last page slot of the sequence that holds a row
  return it;
}

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

// 3-D tiled TMA load issued by either CTA of a pair into ITS OWN shared memory; the completion bytes go to an mbarrier
// given as a shared::cluster address (the pair leader's).  No multicast.
__device__ __forceinline__ void tma_load_3d_2sm(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y, int32_t z, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gqa_prefill_sm100_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_q, const PrefillParams prm) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int worker = blockIdx.x >> 1, n_workers = gridDim.x >> 1;
  if (worker >= prm.n_items) return;   // both CTAs of the pair leave before any pair-wide step

  if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled layouts need a 1024-byte aligned base (same in both CTAs of the pair)
    if (threadIdx.x == 0) set_status(prm.status, RELUX_ERR_UNSUPPORTED);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; s++) { mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); }
    for (int s = 0; s < kStages; s++) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 2 * kSoftmaxWarps);   // one arrival per softmax warp of each CTA of the pair
    mbar_init(&bars->pv_done, 1);
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

  if (warp == kSoftmaxWarps) {
    // =============================== producer: TMA loads into this CTA's slots ===============================
    // The whole warp stays converged and one elected lane issues (operands stay in uniform registers).
    const bool el = elect_one();
    if (el) {
      tma_prefetch_desc(&tmap_kv);
      tma_prefetch_desc(&tmap_q);
    }
    auto load_q = [&](const Item& it, int n) {
      // item n of this worker uses Q buffer n & 1, free again once the last QK^T of item n - 2 has completed
      if (n >= 2) wait_bar(&bars->q_empty[n & 1], ((n >> 1) - 1) & 1, bars, prm.status);
      const uint32_t lead_q = mapa_u32(smem_u32(&bars->q_full[n & 1]), 0);
      if (el) {
        const int t0 = (2 * it.pair + (int)rank) * prm.bq;
        uint8_t* dst = smem + kSmemQ + (n & 1) * kQBytes;
        if (rank == 0) mbar_expect_tx(&bars->q_full[n & 1], 2 * kQBytes);   // the Q tiles of both CTAs
        // box = [64 dims][g heads][bq tokens]: rows land as token_in_block * g + head_in_group
        tma_load_3d_2sm(dst, &tmap_q, 0, it.hk * prm.g, it.bi * prm.S + t0, lead_q);
        tma_load_3d_2sm(dst + kHalf, &tmap_q, 64, it.hk * prm.g, it.bi * prm.S + t0, lead_q);
      }
      __syncwarp();
    };
    int g = 0, n = 0;
    Item cur = item_of(prm, worker);
    load_q(cur, 0);
    for (int idx = worker; idx < prm.n_items; idx += n_workers, n++) {
      for (int j = 0; j < cur.ntiles; j++, g++) {
        int32_t y[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++) {
          const int slot = min(2 * j + h2, cur.last_slot);   // a tile's second page may lie past the sequence: its keys are masked
          int32_t pg = __ldg(prm.table + (size_t)cur.seq * prm.table_stride + slot);
          if (pg < 0 || pg >= prm.num_pages) {               // reported, and replaced by page 0 so that no load leaves the pool
            set_status(prm.status, RELUX_ERR_BAD_PAGE);
            pg = 0;
          }
          y[h2] = (pg * prm.Hkv + cur.hk) * kPage;
        }
        const int32_t y_own = rank ? y[1] : y[0];
        const int u = g / kDepth;
#pragma unroll
        for (int kv = 0; kv < 2; kv++) {
          const int st = (g % kDepth) * 2 + kv;
          if (u > 0) wait_bar(&bars->kv_empty[st], (u - 1) & 1, bars, prm.status);
          const uint32_t lead = mapa_u32(smem_u32(&bars->kv_full[st]), 0);
          if (el) {
            uint8_t* dst = smem + kSmemRing + st * kStageBytes;
            if (rank == 0) mbar_expect_tx(&bars->kv_full[st], 2 * kStageBytes);   // the halves of both CTAs
            if (kv == 0) {   // K: this CTA's page of the tile, both 64-dim halves
              tma_load_2d_2sm(dst, &tmap_kv, 0, prm.krow0 + y_own, lead);
              tma_load_2d_2sm(dst + kBlk, &tmap_kv, 64, prm.krow0 + y_own, lead);
            } else {         // V: this CTA's 64 output dims of both pages
              tma_load_2d_2sm(dst, &tmap_kv, 64 * (int)rank, prm.vrow0 + y[0], lead);
              tma_load_2d_2sm(dst + kBlk, &tmap_kv, 64 * (int)rank, prm.vrow0 + y[1], lead);
            }
          }
          __syncwarp();
        }
      }
      if (idx + n_workers < prm.n_items) {   // the next item's Q, while this item's last tiles are still in flight
        cur = item_of(prm, idx + n_workers);
        load_q(cur, n + 1);
      }
    }
  } else if (warp == kSoftmaxWarps + 1) {
    // =============================== MMA issuer (leader CTA only; converged warp + elected lane) ===============================
    const bool el = elect_one();
    if (rank == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(256, 128, false, false);
      const uint32_t idesc_pv = make_idesc_bf16(256, 128, false, true);
      const uint64_t dQ = make_desc_kmajor_sw128(smem_u32(smem + kSmemQ));
      const uint64_t dP = make_desc_kmajor_sw128(smem_u32(smem + kSmemP));
      // QK^T of tile g (worker-wide index) of item n; `first`: the item's first tile (its Q must have landed);
      // `last`: its last tile, after which the Q buffer is free
      auto issue_qk = [&](int g, int n, bool first, bool last) {
        if (first) wait_bar(&bars->q_full[n & 1], (n >> 1) & 1, bars, prm.status);
        const int st = (g % kDepth) * 2;
        wait_bar(&bars->kv_full[st], (g / kDepth) & 1, bars, prm.status);
        tc_fence_after();
        if (el) {
          const uint64_t dK = make_desc_kmajor_sw128(smem_u32(smem + kSmemRing + st * kStageBytes));
          const uint64_t dQn = dQ + ((uint32_t)((n & 1) * kQBytes) >> 4);
          const uint32_t d = tmem + kTmemS + (g & 1) * 128;
#pragma unroll
          for (int ks = 0; ks < 8; ks++) {
            const uint32_t aoff = (uint32_t)((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;   // Q: 128 rows per 64-dim half
            const uint32_t boff = (uint32_t)((ks >> 2) * kBlk + (ks & 3) * 32) >> 4;    // K: 64 rows per 64-dim half
            umma_ss<2>(d, dQn + aoff, dK + boff, idesc_qk, ks != 0);
          }
          umma_commit_mc<2>(&bars->kv_empty[st], 0x3);
          if (last) umma_commit_mc<2>(&bars->q_empty[n & 1], 0x3);
          umma_commit_mc<2>(&bars->s_full[g & 1], 0x3);
        }
        __syncwarp();
      };
      auto issue_pv = [&](int g, bool first) {
        const int st = (g % kDepth) * 2 + 1;
        wait_bar(&bars->p_full, g & 1, bars, prm.status);
        wait_bar(&bars->kv_full[st], (g / kDepth) & 1, bars, prm.status);
        tc_fence_after();   // P rows, a possible O rescale and the previous item's O read-out were done by the softmax warps of both CTAs
        if (el) {
          const uint64_t dV = make_desc_mnmajor_sw128(smem_u32(smem + kSmemRing + st * kStageBytes), kBlk);
          const uint64_t dPg = dP + ((uint32_t)((g & 1) * kPBytes) >> 4);
#pragma unroll
          for (int ks = 0; ks < 8; ks++) {
            const uint32_t aoff = (uint32_t)((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
            umma_ss<2>(tmem + kTmemO, dPg + aoff, dV + ((uint32_t)(ks * 2048) >> 4), idesc_pv, !first || ks != 0);
          }
          umma_commit_mc<2>(&bars->kv_empty[st], 0x3);
          umma_commit_mc<2>(&bars->pv_done, 0x3);
        }
        __syncwarp();
      };
      int g = 0, n = 0;
      int ntiles = item_of(prm, worker).ntiles;
      issue_qk(0, 0, true, ntiles == 1);
      for (int idx = worker; idx < prm.n_items; idx += n_workers, n++) {
        const bool has_next = idx + n_workers < prm.n_items;
        const int next_tiles = has_next ? item_of(prm, idx + n_workers).ntiles : 0;
        for (int i = 0; i < ntiles; i++, g++) {
          if (i + 1 < ntiles) issue_qk(g + 1, n, false, i + 2 == ntiles);
          else if (has_next) issue_qk(g + 1, n + 1, true, next_tiles == 1);
          issue_pv(g, i == 0);
        }
        ntiles = next_tiles;
      }
    }
  } else {
    // =============================== softmax / correction / epilogue ===============================
    // Warp w reads TMEM lanes 32 (w & 3) .. +31 (the hardware's rule); the kSplit warps that share a lane quarter take
    // one slice of kCols keys (and output dims) each.
    const int wq = warp & 3, hb = warp >> 2;
    const int r = wq * 32 + lane;                   // TMEM lane = query row
    const int tq = r / prm.g, hq = r % prm.g;       // token in block, head in group
    const uint32_t lane_addr = ((uint32_t)(wq * 32) << 16) + (uint32_t)(hb * kCols);
    const uint32_t p_full_lead = mapa_u32(smem_u32(&bars->p_full), 0);
    int g = 0;
    for (int idx = worker; idx < prm.n_items; idx += n_workers) {
      const Item it = item_of(prm, idx);
      const int t0 = (2 * it.pair + (int)rank) * prm.bq;          // first query token of this CTA's block
      const int ntok = max(0, min(prm.bq, prm.S - t0));           // its real tokens (0: the odd block of the last pair)
      const bool real = tq < ntok;
      // keys [0, t_eff) are visible to this row
      const int t_eff = prm.causal ? min(it.T, it.T - prm.S + t0 + tq + 1) : it.T;
      float m_used = -INFINITY, l_run = 0.f;
      for (int j = 0; j < it.ntiles; j++, g++) {
        wait_bar(&bars->s_full[g & 1], (g >> 1) & 1, bars, prm.status);
        __syncwarp();   // the TMEM loads below are warp-collective
        tc_fence_after();
        uint32_t sv[kCols];
#pragma unroll
        for (int c = 0; c < kCols; c += 32)
          tmem_ld_32x32b_x32(tmem + lane_addr + kTmemS + (g & 1) * 128 + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
        tmem_ld_wait();
        const int nvalid = max(0, min(kCols, t_eff - j * kTile - hb * kCols));
        if (nvalid < kCols) {
#pragma unroll
          for (int c = 0; c < kCols; c++)
            if (c >= nvalid) sv[c] = 0xFF800000u;   // -inf
        }
        // row max of the raw scores (the softmax scale is positive, so it commutes with max); four chains, not one
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < kCols; c += 4)
#pragma unroll
          for (int k = 0; k < 4; k++) mx4[k] = fmaxf(mx4[k], __uint_as_float(sv[c + k]));
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * prm.scale_log2;
        bars->rowmax[g & 1][hb][r] = mx;
        asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
#pragma unroll
        for (int k = 0; k < kSplit; k++) mx = fmaxf(mx, bars->rowmax[g & 1][k][r]);
        // lazily updated running max: all threads of a row take the same decision
        float alpha = 1.f;
        bool rescale = false;
        if (mx > m_used + kRescaleThreshold) {   // also true on the first tile with a visible key (m_used = -inf)
          alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
          rescale = (m_used != -INFINITY);
          m_used = mx;
        }
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        float ps[2] = {0.f, 0.f};
        // P(g) goes to buffer g & 1, which PV(g-2) has finished reading (QK(g) was issued after it).  32 keys at a time: one
        // FFMA + one MUFU.EX2 per score, packed to bf16, four 16-byte stores into the swizzled row of this slice's 64-key half.
        uint8_t* pbuf = smem + kSmemP + (g & 1) * kPBytes + r * 128;
#pragma unroll
        for (int q2 = 0; q2 < kCols / 32; q2++) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(sv[q2 * 32 + c]), prm.scale_log2, neg_m));
            const float p1 = ex2_approx(fmaf(__uint_as_float(sv[q2 * 32 + c + 1]), prm.scale_log2, neg_m));
            ps[0] += p0;
            ps[1] += p1;
            __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
            pk[c >> 1] = *reinterpret_cast<uint32_t*>(&b2);
          }
          const int key0 = hb * kCols + q2 * 32;   // first key of these 32 inside the tile
          uint8_t* prow = pbuf + (key0 >> 6) * kHalf;
#pragma unroll
          for (int c = 0; c < 4; c++)
            *reinterpret_cast<uint4*>(prow + (((((key0 & 63) >> 3) + c) ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        }
        l_run = l_run * alpha + (ps[0] + ps[1]);
        // O may be rescaled only after PV(g-1) has completed
        if (j > 0) wait_bar(&bars->pv_done, (g - 1) & 1, bars, prm.status);
        __syncwarp();
        // The TMEM loads and stores are warp-collective: the decision is taken for the whole warp, and the rows that keep
        // their maximum multiply by one.  This thread's slice of the row: output dims kCols hb .. +kCols-1.
        if (j > 0 && __any_sync(0xffffffffu, rescale)) {
          const float a_row = rescale ? alpha : 1.f;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < kCols; c += 32) {
            uint32_t ov[32];
            tmem_ld_32x32b_x32(tmem + lane_addr + kTmemO + c, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * a_row);
            tmem_st_32x32b_x32(tmem + lane_addr + kTmemO + c, ov);
          }
          tmem_st_wait();
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(p_full_lead);
      }
      // ---- item epilogue: O / l -> out ----
      if (it.ntiles > 0) {
        wait_bar(&bars->pv_done, (g - 1) & 1, bars, prm.status);
        __syncwarp();
        tc_fence_after();
      }
      // the row sum is the sum of its key slices (exchanged through the row-maximum buffer of the tile that follows, which
      // nobody touches before the barrier at the end of this epilogue)
      float(*lsum)[128] = bars->rowmax[g & 1];
      lsum[hb][r] = l_run;
      asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
      l_run = 0.f;
#pragma unroll
      for (int k = 0; k < kSplit; k++) l_run += lsum[k][r];
      // warp-uniform: the TMEM loads below are warp-collective
      const bool ok = it.ntiles > 0 && !__any_sync(0xffffffffu, bars->abort_flag != 0);
      const float inv = (ok && l_run > 0.f) ? 1.f / l_run : 0.f;
      float* orow = prm.out + (((size_t)it.bi * prm.S + t0 + (real ? tq : 0)) * prm.H + (size_t)it.hk * prm.g + hq) * kD + hb * kCols;
#pragma unroll 1
      for (int c = 0; c < kCols; c += 32) {
        uint32_t ov[32];
        if (ok) {
          tmem_ld_32x32b_x32(tmem + lane_addr + kTmemO + c, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) ov[i] = 0u;
        }
        if (real) {   // rows past the prompt's last token are padding: computed, never written
          float4* dst = reinterpret_cast<float4*>(orow + c);
#pragma unroll
          for (int i = 0; i < 8; i++)
            dst[i] = make_float4(__uint_as_float(ov[4 * i]) * inv, __uint_as_float(ov[4 * i + 1]) * inv, __uint_as_float(ov[4 * i + 2]) * inv,
                                 __uint_as_float(ov[4 * i + 3]) * inv);
        }
      }
      // the O read-out is ordered before this thread's next p_full arrival, which releases the first PV of the next
      // item; the row sums are read by every thread before the barrier of the next tile's row maxima
      tc_fence_before();
      asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
    }
  }
  __syncwarp();
  tc_fence_before();
  cluster_sync();
  if (warp == 0) tmem_dealloc<2>(tmem, kTmemCols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// CTA pairs that can be resident at the same time (one CTA per SM: the kernel uses all of its shared memory).
int prefill_workers(Pool* p) {
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
    if (cudaFuncSetAttribute(gqa_prefill_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, gqa_prefill_sm100_kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = std::max(1, p->dev->sm_count / 2);
    }
    max_clusters = n;
  }
  return max_clusters;
}

}  // namespace

// g query heads per kv head must tile the 128 rows of the block exactly.
bool gqa_prefill_eligible(const Pool* p, const relux_attn_args& a) {
  const relux_pool_params& prm = p->prm;
  if (!p->has_tmap || prm.page_tokens != kPage || prm.gqa_head_dim != kD) return false;
  const int g = a.num_heads / prm.gqa_num_kv_heads;
  return g >= 1 && g <= 32 && (128 % g) == 0;
}

// q: device bf16 [n][S][H][128] token-major.  out: device f32, same shape.
int32_t launch_gqa_prefill_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const uint16_t* d_q, float* d_out) {
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
  const int g = a.num_heads / prm.gqa_num_kv_heads, bq = 128 / g, S = a.q_tokens, H = a.num_heads;
  CUtensorMap tq;
  {
    cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)H, (cuuint64_t)sb.n_seqs * S};
    cuuint64_t strides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)H * kD * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)g, (cuuint32_t)bq};
    cuuint32_t es[3] = {1, 1, 1};
    if (enc(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)d_q, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_error("tensor map for the prompt's queries could not be encoded");
      return RELUX_ERR_CUDA;
    }
  }
  PrefillParams k{};
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.len = p->d_len + (size_t)a.layer * prm.max_seqs;
  k.seq_ids = sb.d_seq_ids;
  k.num_pages = prm.num_pages;
  k.Hkv = prm.gqa_num_kv_heads;
  k.H = H;
  k.g = g;
  k.S = S;
  k.extra = a.extra_tokens;
  k.causal = a.causal;
  k.bq = bq;
  k.n_qblocks = (S + bq - 1) / bq;
  k.n_pairs = (k.n_qblocks + 1) / 2;
  k.n_seqs = sb.n_seqs;
  const int64_t items = (int64_t)k.n_pairs * prm.gqa_num_kv_heads * sb.n_seqs;
  if (items > ((int64_t)1 << 30)) { set_error("prompt too long for one prefill launch"); return RELUX_ERR_UNSUPPORTED; }
  k.n_items = (int32_t)items;
  const int64_t rows_per_block = (int64_t)prm.num_pages * prm.gqa_num_kv_heads * kPage;
  k.krow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block);
  k.vrow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block + rows_per_block);
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.out = d_out;
  k.status = p->d_status;
  cudaStream_t st = p->dev->stream;
  const int workers = (int)std::min<int64_t>(prefill_workers(p), items);
  RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_prefill_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  dim3 grid(2 * workers, 1, 1);   // CTA pairs
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), st));
  gqa_prefill_sm100_kernel<<<grid, kThreads, kSmemTotal, st>>>(p->tmap_gqa, tq, k);
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), st));
  p->timed_calls++;
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux
