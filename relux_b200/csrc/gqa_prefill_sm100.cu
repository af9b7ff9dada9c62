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
//     softmax warps: S from TMEM -> exp2 with a lazily updated running max -> P packed to bf16 and written back to
//                    tensor memory over the first 64 columns of the S tile just read (P never touches shared memory)
//     O[256 x 128] += P V       8 MMAs M256 N128 K16; A = P from tensor memory; B = V as it lies (MN-major), split by
//                               output dims: CTA r holds dims [64 r, 64 r + 64) of both pages (16 KB)
// Persistent workers.  As many CTA pairs as fit on the GPU are launched once and walk a static list of items (see
// Cursor below for its order).  One launch per block measured 16k cycles (8 us) of fixed cost per CTA pair -- launch,
// tensor-memory allocation, the latency of the first Q / K loads, pipeline fill, drain and the epilogue -- against
// 2.1k cycles per tile: at 2048-token prompts (9 tiles per item on average) that was half of the kernel.  Here the tile
// pipeline does not drain at an item boundary: tiles are numbered over the worker's whole life, Q has two buffers (the
// next item's Q is requested while the current item's last tiles are in flight), the first QK^T of the next item is
// issued ahead of the last PV of the current one like any other tile, O has two accumulators (items in turn), and an
// item's read-out (O / row sum -> out) is the work of four warps of its own while the softmax warps are already on the
// next item.
// TMEM per CTA: S double-buffered (2 x 128 columns, P over the first 64 of each), O double-buffered (2 x 128 columns);
// rows = TMEM lanes.  Issue order QK(g+1), PV(g): QK(g+2), which overwrites the S / P buffer of tile g, is issued behind
// PV(g), and the tensor pipe executes in issue order.
// Warp roles per CTA: 8 softmax warps -- a query row (TMEM lane) is shared by two threads, 64 keys (and 64 output dims
// of a rescale) each --, 1 TMA producer, 1 MMA issuer (leader CTA only), both converged with one elected lane, 4 read-out
// warps.  The softmax warps are the busiest part: per tile and SM 16384 scores through max, scale, exp2, sum and pack.
// The special-function unit delivers 16 exponentials per clock and SM (1024 clocks per tile, as long as the tile's
// MMAs), so three pairs of every eight take a cubic on the FMA pipe instead, arithmetic runs two lanes per instruction
// (fma.f32x2, add.f32x2) and the row maximum takes two scores per instruction (three-input max).
// Barriers: full barriers live in the leader CTA and count the bytes of both CTAs' loads; empty / s_full / pv_done /
// o_full barriers live in each CTA and are armed by tcgen05.commit with mbarrier multicast (not a TMA load); p_full and
// o_empty live in the leader and count warps of both CTAs.  No TMA multicast anywhere.
// No split-KV: the output is normalised in the read-out and written once.
// Every wait is bounded (status RELUX_ERR_TIMEOUT, shared abort flag, all warps still reach the end and free TMEM).
//
// The same kernel serves MLA prompts (template parameter kMla): MLA.forwardCached for seqQ > 1 expands every cached
// latent row into per-head keys and values first (internal/transformer/mla.go:323-326; here mla_expand_sm100.cu, bf16
// rows in a dense scratch array) and then runs ordinary attention with 128 + 64 score dims (mla.go:328-377).  For this
// kernel that is the group size 1 case with three changes: the Q tile and every K stage carry a third 64-column block
// (the RoPE part: of the query from its own array, of the key from the pool's pages, shared by all heads), QK^T is 12
// K-steps instead of 8, and the expanded keys / values are addressed densely (head * Ttot + first row of the sequence +
// token) instead of through the page table.
// Every wait is bounded (status RELUX_ERR_TIMEOUT, shared abort flag, all warps still reach the end and free TMEM).
#include <algorithm>
#include <cuda_bf16.h>

#include "common.cuh"
#include "internal.h"
#include "umma.cuh"
#include "softmax_parts.cuh"

namespace relux {

namespace {

constexpr int kD = 128, kPage = 64, kTile = 128;
constexpr int kBlk = 8192;                 // one [64 rows x 64 cols] bf16 box, 128-byte swizzled
constexpr int kHalf = 2 * kBlk;            // [128 rows x 64 cols]
constexpr int kVBytes = 2 * kBlk;          // V stage, 16 KB per CTA: own 64 output dims of [keys 0-63 | keys 64-127]
constexpr int kMaxDepth = 4;

// Shared-memory plan of the two variants.
//   GQA (kMla = false): score width 128.  Q tile [dims 0-63 | dims 64-127] x 2 buffers (items in turn), K stage = own
//     page [dims 0-63 | dims 64-127] (16 KB), four K and four V stages: 64 + 64 + 64 = 192 KB.
//   MLA (kMla = true): score width 192 = 128 expanded key dims + 64 shared RoPE dims.  Q tile [nope 0-63 | nope 64-127 |
//     rope] (48 KB) x 2 buffers, K stage = own 64 keys [nope 0-63 | nope 64-127 | rope] (24 KB), three K and three V
//     stages: 96 + 72 + 48 = 216 KB.
// P never touches shared memory: the softmax warps write it, packed to bf16, over the first 64 columns of the S tile they
// have just read, and PV takes its A operand from tensor memory.
template <bool kMla>
struct Plan {
  static constexpr int kQHalves = kMla ? 3 : 2;
  static constexpr int kQBytes = kQHalves * kHalf;
  static constexpr int kQBufs = 2;
  static constexpr int kKBytes = (kMla ? 3 : 2) * kBlk;
  static constexpr int kDepthK = kMla ? 3 : 4, kDepthV = kMla ? 3 : 4;
  static constexpr int kKSteps = kMla ? 12 : 8;            // K = 16 slices of the score contraction
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemK = kSmemQ + kQBufs * kQBytes;
  static constexpr int kSmemV = kSmemK + kDepthK * kKBytes;
  static constexpr int kSmemBar = kSmemV + kDepthV * kVBytes;
  static constexpr int kSmemTotal = kSmemBar + 3072;
  static_assert(kSmemTotal <= 232448, "more shared memory than a CTA may use");
};
constexpr int kSplit = 2;                                     // threads per query row: each takes 128 / kSplit keys and output dims
constexpr int kCols = 128 / kSplit;
constexpr int kSoftmaxWarps = 4 * kSplit;
constexpr int kEpiWarps = 4;                                  // read-out warps: one per TMEM lane quarter
constexpr int kSoftmaxThreads = 32 * kSoftmaxWarps, kThreads = kSoftmaxThreads + 64 + 32 * kEpiWarps;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemS = 0, kTmemO = 256;                  // S(g) at kTmemS + 128 (g & 1); O of item n at kTmemO + 128 (n & 1)
constexpr float kRescaleThreshold = 8.0f;
#ifndef RELUX_PREFILL_POLY_PAIRS
#define RELUX_PREFILL_POLY_PAIRS 3
#endif
constexpr int kPolyPairsOf8 = RELUX_PREFILL_POLY_PAIRS;   // score pairs out of every eight whose exponential runs on the FMA pipe

struct Bars {
  uint64_t q_full[2], q_empty[2], k_full[kMaxDepth], k_empty[kMaxDepth], v_full[kMaxDepth], v_empty[kMaxDepth], s_full[2], p_full, pv_done;
  uint64_t o_full[2], o_empty[2], l_full, l_empty, drain;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  float rowmax[2][kSplit][128];   // [tile parity][key slice][row]; at the end of an item the buffer of the tile that follows
                                  // carries the row sums of the key slices from one slice's thread to the other's
  float lsum[128];                // an item's row sums, handed to the read-out warps
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
  int32_t n_half, n_couples;  // couples per (sequence, kv head) = ceil(n_pairs / 2), and in all
  int32_t krow0, vrow0;       // first TMA row of this layer's K block / V block (MLA: of the expanded keys / values)
  // MLA only: expanded rows are dense, row = head * Ttot + seq_base[sequence] + token; the RoPE part of a key is read from
  // the pool's pages (block rope_block of blocks_per_page 64-column blocks per page, first row of the layer pool_row0)
  const int32_t* seq_base;
  int32_t Ttot, rope_block, blocks_per_page;
  int64_t pool_row0;
  float scale_log2;
  float* out;                 // [n][S][H][128] f32
  int32_t* status;
};

// The order of the work.  Under the causal mask block pair p of a stream (a sequence's kv head) needs 2 (p + 1) key tiles:
// pairs p and n_pairs - 1 - p together always need the same number, so the unit handed to a worker is that COUPLE, the
// long member first.  Couples are numbered stream by stream and worker w takes couples w, w + W, ...: every worker gets
// the same amount of work, and the workers that run at the same time read the keys and values of a few streams only,
// which then come out of L2 (with 128 heads and long prompts the streams of one call are far larger than L2 together).
struct Cursor {
  int32_t c, m;   // couple, member (0: pair n_pairs - 1 - k, 1: pair k, for couple k of its stream)
};
__device__ __forceinline__ bool cursor_valid(const PrefillParams& prm, Cursor u) { return u.c < prm.n_couples; }
__device__ __forceinline__ Cursor cursor_next(const PrefillParams& prm, Cursor u, int n_workers) {
  const int k = u.c % prm.n_half;
  if (u.m == 0 && prm.n_pairs - 1 - k != k) return Cursor{u.c, 1};
  return Cursor{u.c + n_workers, 0};
}

// One item as every warp of the pair derives it from the cursor.
struct Item {
  int32_t bi, seq, hk, pair;
  int32_t T, ntiles, last_slot, base;
};
template <bool kMla>
__device__ __forceinline__ Item item_of(const PrefillParams& prm, Cursor u) {
  Item it;
  const int stream = u.c / prm.n_half, k = u.c % prm.n_half;
  it.pair = u.m ? k : prm.n_pairs - 1 - k;
  it.hk = stream % prm.Hkv;
  it.bi = stream / prm.Hkv;
  it.seq = prm.seq_ids ? __ldg(prm.seq_ids + it.bi) : it.bi;
  it.T = __ldg(prm.len + it.seq) + prm.extra;
  // keys the PAIR needs: all T without the mask, else up to the position of its last real token
  const int last_tok = min(prm.S, (2 * it.pair + 2) * prm.bq) - 1;
  const int kmax = prm.causal ? (it.T - prm.S + last_tok + 1) : it.T;
  it.ntiles = max(1, (kmax + kTile - 1) / kTile);
  it.last_slot = (it.T + kPage - 1) / kPage - 1;   // last page slot of the sequence that holds a row
  it.base = 0;
  if constexpr (kMla) it.base = __ldg(prm.seq_base + it.bi);
  return it;
}

// exp2(score * scale - max) for this thread's kCols scores of one row: bf16 P values, two per 32-bit word in key order,
// into pw; returns the two partial row sums.  (The caller stores pw to tensor memory: that store is warp-collective and
// this function is called under a per-row condition.)
template <bool kPoly>
__device__ __forceinline__ uint64_t exp_rows(const uint32_t (&sv)[kCols], uint64_t scale2, uint64_t neg_m2, uint32_t (&pw)[kCols / 2]) {
  static_assert(kCols == 64, "one 32-column store per thread");
  uint64_t ps2 = pack2(0.f, 0.f);
#pragma unroll
  for (int q2 = 0; q2 < kCols / 32; q2++) {
    uint32_t* pk = pw + 16 * q2;
#pragma unroll
    for (int c = 0; c < 32; c += 2) {
      const uint64_t x2 = fma2(pack2(__uint_as_float(sv[q2 * 32 + c]), __uint_as_float(sv[q2 * 32 + c + 1])), scale2, neg_m2);
      uint64_t p2;
      if (kPoly && ((c >> 1) & 7) < kPolyPairsOf8) {
        p2 = ex2_poly2(x2);
      } else {
        float x0, x1;
        unpack2(x2, x0, x1);
        p2 = pack2(ex2_approx(x0), ex2_approx(x1));
      }
      ps2 = add2(ps2, p2);
      float p0, p1;
      unpack2(p2, p0, p1);
      __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
      pk[c >> 1] = *reinterpret_cast<uint32_t*>(&b2);
    }
  }
  return ps2;
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

// tmap_kv: GQA the pool's K / V rows; MLA the expanded keys / values.  tmap_q: the queries (MLA: their nope part).
// tmap_qr, tmap_rope (MLA only): the queries' RoPE part, and the pool's 64-column blocks.
template <bool kMla>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    prefill_sm100_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_q,
                         const __grid_constant__ CUtensorMap tmap_qr, const __grid_constant__ CUtensorMap tmap_rope, const PrefillParams prm) {
  using PL = Plan<kMla>;
  constexpr int kQBytes = PL::kQBytes, kQBufs = PL::kQBufs, kKBytes = PL::kKBytes, kDepthK = PL::kDepthK, kDepthV = PL::kDepthV;
  constexpr int kSmemQ = PL::kSmemQ, kSmemK = PL::kSmemK, kSmemV = PL::kSmemV;
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + PL::kSmemBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int worker = blockIdx.x >> 1, n_workers = gridDim.x >> 1;
  if (worker >= prm.n_couples) return;   // both CTAs of the pair leave before any pair-wide step

  if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled layouts need a 1024-byte aligned base (same in both CTAs of the pair)
    if (threadIdx.x == 0) set_status(prm.status, RELUX_ERR_UNSUPPORTED);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; s++) { mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); }
    for (int s = 0; s < kMaxDepth; s++) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 2 * kSoftmaxWarps);   // one arrival per softmax warp of each CTA of the pair
    mbar_init(&bars->pv_done, 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(&bars->o_full[s], 1);
      mbar_init(&bars->o_empty[s], 2 * kEpiWarps);   // the read-out warps of both CTAs (leader's copy is the one waited on)
    }
    mbar_init(&bars->l_full, kSoftmaxWarps / kSplit);
    mbar_init(&bars->l_empty, kEpiWarps);
    mbar_init(&bars->drain, 1);
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
      if constexpr (kMla) {
        tma_prefetch_desc(&tmap_qr);
        tma_prefetch_desc(&tmap_rope);
      }
    }
    auto load_q = [&](const Item& it, int n) {
      // item n of this worker uses Q buffer n % kQBufs, free again once the last QK^T of item n - kQBufs has completed
      const int qb = n % kQBufs, use = n / kQBufs;
      if (use > 0) wait_bar(&bars->q_empty[qb], (use - 1) & 1, bars, prm.status);
      const uint32_t lead_q = mapa_u32(smem_u32(&bars->q_full[qb]), 0);
      if (el) {
        const int t0 = (2 * it.pair + (int)rank) * prm.bq;
        uint8_t* dst = smem + kSmemQ + qb * kQBytes;
        if (rank == 0) mbar_expect_tx(&bars->q_full[qb], 2 * kQBytes);   // the Q tiles of both CTAs
        // box = [64 dims][g heads][bq tokens]: rows land as token_in_block * g + head_in_group
        tma_load_3d_2sm(dst, &tmap_q, 0, it.hk * prm.g, it.bi * prm.S + t0, lead_q);
        tma_load_3d_2sm(dst + kHalf, &tmap_q, 64, it.hk * prm.g, it.bi * prm.S + t0, lead_q);
        if constexpr (kMla) tma_load_3d_2sm(dst + 2 * kHalf, &tmap_qr, 0, it.hk, it.bi * prm.S + t0, lead_q);
      }
      __syncwarp();
    };
    int g = 0, n = 0;
    Cursor cu{worker, 0};
    Item cur = item_of<kMla>(prm, cu);
    load_q(cur, 0);
    for (; cursor_valid(prm, cu); n++) {
      for (int j = 0; j < cur.ntiles; j++, g++) {
        // rows of the tile's two 64-key halves in tmap_kv (relative to krow0 / vrow0), and for MLA the pool row of the
        // RoPE block of this CTA's half
        int32_t y[2], y_rope = 0;
        if constexpr (kMla) {
          y[0] = cur.hk * prm.Ttot + cur.base + j * kTile;
          y[1] = y[0] + kPage;
          const int slot = min(2 * j + (int)rank, cur.last_slot);
          int32_t pg = __ldg(prm.table + (size_t)cur.seq * prm.table_stride + slot);
          if (pg < 0 || pg >= prm.num_pages) {
            set_status(prm.status, RELUX_ERR_BAD_PAGE);
            pg = 0;
          }
          y_rope = (int32_t)(prm.pool_row0 + ((int64_t)pg * prm.blocks_per_page + prm.rope_block) * kPage);
        } else {
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
        }
        const int32_t y_own = rank ? y[1] : y[0];
        {   // K: this CTA's 64 keys of the tile, every 64-dim block of the score contraction
          const int st = g % kDepthK, u = g / kDepthK;
          if (u > 0) wait_bar(&bars->k_empty[st], (u - 1) & 1, bars, prm.status);
          const uint32_t lead = mapa_u32(smem_u32(&bars->k_full[st]), 0);
          if (el) {
            uint8_t* dst = smem + kSmemK + st * kKBytes;
            if (rank == 0) mbar_expect_tx(&bars->k_full[st], 2 * kKBytes);   // the halves of both CTAs
            tma_load_2d_2sm(dst, &tmap_kv, 0, prm.krow0 + y_own, lead);
            tma_load_2d_2sm(dst + kBlk, &tmap_kv, 64, prm.krow0 + y_own, lead);
            if constexpr (kMla) tma_load_2d_2sm(dst + 2 * kBlk, &tmap_rope, 0, y_rope, lead);
          }
          __syncwarp();
        }
        {   // V: this CTA's 64 output dims of both halves
          const int st = g % kDepthV, u = g / kDepthV;
          if (u > 0) wait_bar(&bars->v_empty[st], (u - 1) & 1, bars, prm.status);
          const uint32_t lead = mapa_u32(smem_u32(&bars->v_full[st]), 0);
          if (el) {
            uint8_t* dst = smem + kSmemV + st * kVBytes;
            if (rank == 0) mbar_expect_tx(&bars->v_full[st], 2 * kVBytes);
            tma_load_2d_2sm(dst, &tmap_kv, 64 * (int)rank, prm.vrow0 + y[0], lead);
            tma_load_2d_2sm(dst + kBlk, &tmap_kv, 64 * (int)rank, prm.vrow0 + y[1], lead);
          }
          __syncwarp();
        }
      }
      cu = cursor_next(prm, cu, n_workers);
      if (cursor_valid(prm, cu)) {   // the next item's Q, while this item's last tiles are still in flight
        cur = item_of<kMla>(prm, cu);
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
      // QK^T of tile g (worker-wide index) of item n; `first`: the item's first tile (its Q must have landed);
      // `last`: its last tile, after which the Q buffer is free
      auto issue_qk = [&](int g, int n, bool first, bool last) {
        const int qb = n % kQBufs;
        if (first) wait_bar(&bars->q_full[qb], (n / kQBufs) & 1, bars, prm.status);
        const int st = g % kDepthK;
        wait_bar(&bars->k_full[st], (g / kDepthK) & 1, bars, prm.status);
        tc_fence_after();
        if (el) {
          const uint64_t dK = make_desc_kmajor_sw128(smem_u32(smem + kSmemK + st * kKBytes));
          const uint64_t dQn = dQ + ((uint32_t)(qb * kQBytes) >> 4);
          const uint32_t d = tmem + kTmemS + (g & 1) * 128;
#pragma unroll
          for (int ks = 0; ks < PL::kKSteps; ks++) {
            const uint32_t aoff = (uint32_t)((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;   // Q: 128 rows per 64-dim block
            const uint32_t boff = (uint32_t)((ks >> 2) * kBlk + (ks & 3) * 32) >> 4;    // K: 64 rows per 64-dim block
            umma_ss<2>(d, dQn + aoff, dK + boff, idesc_qk, ks != 0);
          }
          umma_commit_mc<2>(&bars->k_empty[st], 0x3);
          if (last) umma_commit_mc<2>(&bars->q_empty[qb], 0x3);
          umma_commit_mc<2>(&bars->s_full[g & 1], 0x3);
        }
        __syncwarp();
      };
      // PV of tile g of item n; `first`: the item's first tile (O is overwritten: the read-out of item n - 2 must have left
      // the buffer); `last`: its last tile, after which the read-out warps take the buffer
      auto issue_pv = [&](int g, int n, bool first, bool last) {
        const int st = g % kDepthV;
        if (first && n >= 2) wait_bar(&bars->o_empty[n & 1], ((n >> 1) - 1) & 1, bars, prm.status);
        wait_bar(&bars->p_full, g & 1, bars, prm.status);
        wait_bar(&bars->v_full[st], (g / kDepthV) & 1, bars, prm.status);
        tc_fence_after();   // P rows, a possible O rescale and the previous item's O read-out were done by the softmax warps of both CTAs
        if (el) {
          const uint64_t dV = make_desc_mnmajor_sw128(smem_u32(smem + kSmemV + st * kVBytes), kBlk);
          const uint32_t tP = tmem + kTmemS + (g & 1) * 128;   // P(g) lies over the first 64 columns of S(g)
#pragma unroll
          for (int ks = 0; ks < 8; ks++)
            umma_ts<2>(tmem + kTmemO + (n & 1) * 128, tP + ks * 8, dV + ((uint32_t)(ks * 2048) >> 4), idesc_pv, !first || ks != 0);
          umma_commit_mc<2>(&bars->v_empty[st], 0x3);
          umma_commit_mc<2>(&bars->pv_done, 0x3);
          if (last) umma_commit_mc<2>(&bars->o_full[n & 1], 0x3);
        }
        __syncwarp();
      };
      int g = 0, n = 0;
      Cursor cu{worker, 0};
      int ntiles = item_of<kMla>(prm, cu).ntiles;
      issue_qk(0, 0, true, ntiles == 1);
      for (; cursor_valid(prm, cu); n++) {
        cu = cursor_next(prm, cu, n_workers);
        const bool has_next = cursor_valid(prm, cu);
        const int next_tiles = has_next ? item_of<kMla>(prm, cu).ntiles : 0;
        for (int i = 0; i < ntiles; i++, g++) {
          if (i + 1 < ntiles) {
            issue_qk(g + 1, n, false, i + 2 == ntiles);
            issue_pv(g, n, i == 0, false);
          } else if (has_next && kQBufs > 1) {
            issue_qk(g + 1, n + 1, true, next_tiles == 1);
            issue_pv(g, n, i == 0, true);
          } else {
            // one Q buffer: the next item's Q is requested when this item's last QK^T has completed, so its first QK^T
            // goes behind this item's last PV instead of waiting for the load in front of it
            issue_pv(g, n, i == 0, true);
            if (has_next) issue_qk(g + 1, n + 1, true, next_tiles == 1);
          }
        }
        ntiles = next_tiles;
      }
      // Nothing of this pair may be freed while an MMA is in flight.  On the ordinary path the read-out's last wait says
      // so already; after a wait that gave up it does not, so the issuer itself sees its last MMA complete.
      if (el) umma_commit<2>(&bars->drain);
      __syncwarp();
      mbar_wait(&bars->drain, 0);
    }
  } else if (warp < kSoftmaxWarps) {
    // =============================== softmax / correction ===============================
    // Warp w reads TMEM lanes 32 (w & 3) .. +31 (the hardware's rule); the kSplit warps that share a lane quarter take
    // one slice of kCols keys (and output dims) each.
    const int wq = warp & 3, hb = warp >> 2;
    const int r = wq * 32 + lane;                   // TMEM lane = query row
    const int tq = r / prm.g;                       // token in block
    const uint32_t lane_addr = ((uint32_t)(wq * 32) << 16) + (uint32_t)(hb * kCols);
    const uint32_t p_full_lead = mapa_u32(smem_u32(&bars->p_full), 0);
    int g = 0, n = 0;
    for (Cursor cu{worker, 0}; cursor_valid(prm, cu); cu = cursor_next(prm, cu, n_workers), n++) {
      const Item it = item_of<kMla>(prm, cu);
      const int t0 = (2 * it.pair + (int)rank) * prm.bq;          // first query token of this CTA's block
      // keys [0, t_eff) are visible to this row
      const int t_eff = prm.causal ? min(it.T, it.T - prm.S + t0 + tq + 1) : it.T;
      const uint32_t tmem_o = tmem + lane_addr + kTmemO + (n & 1) * 128;
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
        // row max of the raw scores (the softmax scale is positive, so it commutes with max); four chains of three-input
        // maxima, two scores per instruction
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < kCols; c += 8)
#pragma unroll
          for (int k = 0; k < 4; k++) mx4[k] = max3(mx4[k], __uint_as_float(sv[c + 2 * k]), __uint_as_float(sv[c + 2 * k + 1]));
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
        const uint64_t scale2 = pack2(prm.scale_log2, prm.scale_log2), neg_m2 = pack2(neg_m, neg_m);
        // P(g), packed to bf16, goes over the first 64 columns of S(g): every slice of the row has read its S columns (the
        // barrier above came after the loads), and QK(g+2), which writes this S buffer again, is issued behind PV(g).
        // kPolyPairsOf8 pairs of every eight take the polynomial; a thread with a masked key in its slice (the diagonal
        // tiles only) keeps to ex2(-inf) = 0 exactly.
        uint32_t pw[kCols / 2];
        uint64_t ps2;
        if (nvalid == kCols) ps2 = exp_rows<true>(sv, scale2, neg_m2, pw);
        else ps2 = exp_rows<false>(sv, scale2, neg_m2, pw);
        __syncwarp();   // the store is warp-collective
        tmem_st_32x32b_x32(tmem + ((uint32_t)(wq * 32) << 16) + kTmemS + (g & 1) * 128 + hb * (kCols / 2), pw);
        float ps0, ps1;
        unpack2(ps2, ps0, ps1);
        l_run = l_run * alpha + (ps0 + ps1);
        // O may be rescaled only after PV(g-1) has completed.  The wait is made on an item's first tile too (PV(g-1) is then
        // the previous item's last one): PV(g-1) was issued behind the completion of p_full's phase g-1, so no warp arrives
        // for tile g before every warp OF BOTH CTAs has arrived for tile g-1.  Without it the softmax warps of one CTA,
        // which after an item's last tile wait for nothing but S of the next item's first tile (computed ahead), could
        // arrive twice while a warp of the other CTA was still writing P(g-1): p_full's phase g-1 completed early and the
        // item's last PV read an unfinished P.
        if (g > 0) wait_bar(&bars->pv_done, (g - 1) & 1, bars, prm.status);
        __syncwarp();
        // The TMEM loads and stores are warp-collective: the decision is taken for the whole warp, and the rows that keep
        // their maximum multiply by one.  This thread's slice of the row: output dims kCols hb .. +kCols-1.
        if (j > 0 && __any_sync(0xffffffffu, rescale)) {
          const float a_row = rescale ? alpha : 1.f;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < kCols; c += 32) {
            uint32_t ov[32];
            tmem_ld_32x32b_x32(tmem_o + c, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * a_row);
            tmem_st_32x32b_x32(tmem_o + c, ov);
          }
          tmem_st_wait();
        }
        tmem_st_wait();   // P, and a rescaled O
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(p_full_lead);
      }
      // ---- end of the item: the row sum (the sum of its key slices) goes to the read-out warps ----
      // The slices meet in the row-maximum buffer of the tile that follows; nobody writes it before the second barrier.
      float(*lx)[128] = bars->rowmax[g & 1];
      lx[hb][r] = l_run;
      asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
      if (hb == 0) {
        float l = 0.f;
#pragma unroll
        for (int k = 0; k < kSplit; k++) l += lx[k][r];
        if (n > 0) wait_bar(&bars->l_empty, (n - 1) & 1, bars, prm.status);   // the read-out of the previous item has taken its sums
        bars->lsum[r] = l;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->l_full);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
    }
  } else {
    // =============================== read-out: O / l -> out ===============================
    // One warp per TMEM lane quarter; item n's accumulator is O buffer n & 1, handed over by the commit behind the
    // item's last PV and handed back (to the first PV of item n + 2) when the row has been read.
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int tq = r / prm.g, hq = r % prm.g;       // token in block, head in group
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const uint32_t o_empty_lead[2] = {mapa_u32(smem_u32(&bars->o_empty[0]), 0), mapa_u32(smem_u32(&bars->o_empty[1]), 0)};
    int n = 0;
    for (Cursor cu{worker, 0}; cursor_valid(prm, cu); cu = cursor_next(prm, cu, n_workers), n++) {
      const Item it = item_of<kMla>(prm, cu);
      const int t0 = (2 * it.pair + (int)rank) * prm.bq;          // first query token of this CTA's block
      const int ntok = max(0, min(prm.bq, prm.S - t0));           // its real tokens (0: the odd block of the last pair)
      const bool real = tq < ntok;                                 // rows past the prompt's last token are padding: computed, never written
      wait_bar(&bars->l_full, n & 1, bars, prm.status);
      const float l_row = bars->lsum[r];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->l_empty);
      wait_bar(&bars->o_full[n & 1], (n >> 1) & 1, bars, prm.status);
      __syncwarp();   // the TMEM loads below are warp-collective
      tc_fence_after();
      const bool ok = !__any_sync(0xffffffffu, bars->abort_flag != 0);
      const float inv = (ok && l_row > 0.f) ? 1.f / l_row : 0.f;
      float* orow = prm.out + (((size_t)it.bi * prm.S + t0 + (real ? tq : 0)) * prm.H + (size_t)it.hk * prm.g + hq) * kD;
#pragma unroll 1
      for (int c = 0; c < kD; c += 32) {
        uint32_t ov[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + kTmemO + (n & 1) * 128 + c, ov);
        tmem_ld_wait();
        if (real) {
          float4* dst = reinterpret_cast<float4*>(orow + c);
#pragma unroll
          for (int i = 0; i < 8; i++)
            dst[i] = make_float4(__uint_as_float(ov[4 * i]) * inv, __uint_as_float(ov[4 * i + 1]) * inv, __uint_as_float(ov[4 * i + 2]) * inv,
                                 __uint_as_float(ov[4 * i + 3]) * inv);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster((n & 1) ? o_empty_lead[1] : o_empty_lead[0]);
    }
  }
  __syncwarp();
  tc_fence_before();
  cluster_sync();
  if (warp == 0) tmem_dealloc<2>(tmem, kTmemCols);
}


}  // namespace
namespace {

// CTA pairs that can be resident at the same time (one CTA per SM: the kernel uses all of its shared memory).
template <bool kMla>
int prefill_workers(Pool* p) {
  static int max_clusters = 0;
  constexpr int kSmemTotal = Plan<kMla>::kSmemTotal;
  auto gqa_prefill_sm100_kernel = prefill_sm100_kernel<kMla>;
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
  const int g = a.num_heads / prm.gqa_num_kv_heads, bq = 128 / g, S = a.q_tokens, H = a.num_heads;
  CUtensorMap tq;   // queries [n * S][H][128]: a box is the g heads of one KV head for bq tokens
  if (!make_tmap_3d(&tq, (void*)d_q, (uint64_t)sb.n_seqs * S, (uint64_t)H, kD, 64, (uint32_t)g, (uint32_t)bq)) {
    set_error("tensor map for the prompt's queries could not be encoded");
    return RELUX_ERR_CUDA;
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
  k.n_half = (k.n_pairs + 1) / 2;
  k.n_couples = k.n_half * prm.gqa_num_kv_heads * sb.n_seqs;
  const int64_t rows_per_block = (int64_t)prm.num_pages * prm.gqa_num_kv_heads * kPage;
  k.krow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block);
  k.vrow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block + rows_per_block);
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.out = d_out;
  k.status = p->d_status;
  cudaStream_t st = p->dev->stream;
  const int workers = std::min(prefill_workers<false>(p), k.n_couples);
  constexpr int kSmemTotal = Plan<false>::kSmemTotal;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(prefill_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  dim3 grid(2 * workers, 1, 1);   // CTA pairs
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), st));
  prefill_sm100_kernel<false><<<grid, kThreads, kSmemTotal, st>>>(p->tmap_gqa, tq, tq, p->tmap_gqa, k);
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), st));
  p->timed_calls++;
  count_launch(p->dev);
  return RELUX_OK;
}

// ---- MLA prompts ---------------------------------------------------------------------------------------------------
bool mla_expand_eligible(const Pool* p, int num_heads, int head_dim);
int64_t mla_expand_rows(const Pool* p, const SeqBatch& sb, int layer, int extra);
int32_t launch_mla_expand_sm100(Pool* p, const SeqBatch& sb, int layer, int extra, int H, const uint16_t* w_uk, const uint16_t* w_uv,
                                int64_t Ttot, uint16_t* kx, uint16_t* vx, int32_t* seq_base);

// Bytes of scratch the expanded keys and values of this batch take: 2 x H x Ttot rows of 128 bf16.
static int64_t mla_prefill_scratch_bytes(int64_t Ttot, int H) { return 2 * (int64_t)H * Ttot * 128 * 2; }

// A prompt goes to the expand + prefill pair when the calls' shapes fit the kernels, the prompt is long enough for the
// expansion to pay (its cost is per cached row, the saving per query row), and the scratch stays within the limit.
bool mla_prefill_eligible(const Pool* p, const SeqBatch& sb, const relux_attn_args& a) {
  const relux_pool_params& prm = p->prm;
  if (p->compat || a.mode != RELUX_ATTN_FAST || !mla_expand_eligible(p, a.num_heads, a.head_dim) || prm.mla_dhr != 64) return false;
  const int min_tokens = p->tune.get(RELUX_TUNE_MLA_PROMPT_MIN_TOKENS);
  if (min_tokens < 0 || a.q_tokens < std::max(2, min_tokens)) return false;
  const int64_t Ttot = mla_expand_rows(p, sb, a.layer, a.extra_tokens);
  if (2 * (int64_t)a.num_heads * Ttot >= ((int64_t)1 << 31)) return false;   // TMA row coordinates are 32-bit
  // absorbed scores cost 1088 multiply-adds per (query row, key), expanded ones 320 plus 512 * 256 per key and head
  // for the expansion: the expansion pays from about 170 query tokens per sequence
  const int64_t limit = (int64_t)p->tune.get(RELUX_TUNE_MLA_PROMPT_SCRATCH_MB) << 20;
  return mla_prefill_scratch_bytes(Ttot, a.num_heads) <= limit;
}

// q: device bf16 [n][S][H][128], q_rope: device bf16 [n][S][H][64], token-major.  out: device f32 [n][S][H][128].
int32_t launch_mla_prefill_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const uint16_t* d_q, const uint16_t* d_qr, float* d_out) {
  const relux_pool_params& prm = p->prm;
  const int S = a.q_tokens, H = a.num_heads;
  const int64_t Ttot = mla_expand_rows(p, sb, a.layer, a.extra_tokens);
  const size_t x_bytes = (size_t)mla_prefill_scratch_bytes(Ttot, H);
  int32_t rc = grow(p->dev, p->expand_buf, x_bytes + sizeof(int32_t) * ((size_t)sb.n_seqs + 1) + 256);
  if (rc) return rc;
  uint16_t* kx = (uint16_t*)p->expand_buf.p;
  uint16_t* vx = kx + (size_t)H * Ttot * 128;
  int32_t* seq_base = (int32_t*)((char*)p->expand_buf.p + ((x_bytes + 255) & ~(size_t)255));
  rc = launch_mla_expand_sm100(p, sb, a.layer, a.extra_tokens, H, (const uint16_t*)a.w_uk, (const uint16_t*)a.w_uv, Ttot, kx, vx, seq_base);
  if (rc) return rc;
  CUtensorMap tq, tqr, tx;
  // queries [n * S][H][128] and their rope parts [n * S][H][64]: a box is one head for 128 tokens
  if (!make_tmap_3d(&tq, (void*)d_q, (uint64_t)sb.n_seqs * S, (uint64_t)H, kD, 64, 1, 128) ||
      !make_tmap_3d(&tqr, (void*)d_qr, (uint64_t)sb.n_seqs * S, (uint64_t)H, 64, 64, 1, 128)) {
    set_error("tensor map for the prompt's queries could not be encoded");
    return RELUX_ERR_CUDA;
  }
  if (!make_tmap_2d(&tx, kx, (uint64_t)2 * H * Ttot, kD, 64, 64)) {
    set_error("tensor map for the expanded keys / values could not be encoded");
    return RELUX_ERR_CUDA;
  }
  PrefillParams k{};
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.len = p->d_len + (size_t)a.layer * prm.max_seqs;
  k.seq_ids = sb.d_seq_ids;
  k.num_pages = prm.num_pages;
  k.Hkv = H;
  k.H = H;
  k.g = 1;
  k.S = S;
  k.extra = a.extra_tokens;
  k.causal = a.causal;
  k.bq = 128;
  k.n_qblocks = (S + 127) / 128;
  k.n_pairs = (k.n_qblocks + 1) / 2;
  k.n_seqs = sb.n_seqs;
  const int64_t items = (int64_t)k.n_pairs * H * sb.n_seqs;
  if (items > ((int64_t)1 << 30)) { set_error("prompt too long for one prefill launch"); return RELUX_ERR_UNSUPPORTED; }
  k.n_items = (int32_t)items;
  k.n_half = (k.n_pairs + 1) / 2;
  k.n_couples = k.n_half * H * sb.n_seqs;
  k.krow0 = 0;
  k.vrow0 = (int32_t)((int64_t)H * Ttot);
  k.seq_base = seq_base;
  k.Ttot = (int32_t)Ttot;
  k.blocks_per_page = p->row_elems_a / 64;
  k.rope_block = prm.mla_dc / 64;
  k.pool_row0 = (int64_t)a.layer * prm.num_pages * k.blocks_per_page * kPage;
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.out = d_out;
  k.status = p->d_status;
  cudaStream_t st = p->dev->stream;
  const int workers = std::min(prefill_workers<true>(p), k.n_couples);
  constexpr int kSmemTotal = Plan<true>::kSmemTotal;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(prefill_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  dim3 grid(2 * workers, 1, 1);   // CTA pairs
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), st));
  prefill_sm100_kernel<true><<<grid, kThreads, kSmemTotal, st>>>(tx, tq, tqr, p->tmap_mla, k);
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), st));
  p->timed_calls++;
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux
