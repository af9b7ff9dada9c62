// Paged GQA prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), for multi-token cached calls
// (a prompt, or a long verify): the kernel the decode path lacks, because a decode CTA holds at most 32 query rows.
//
// What it replaces: the attention loops of MHA.forwardCached for seqQ > 1 (internal/transformer/mha.go:318-348) with the
// online-softmax rule of flashOnlineAccum.update (internal/transformer/flash_attention.go:36-73, 99-187): running max,
// rescale of sum and output by exp(old - new), accumulate exp(s - max) * v.  Semantics are the library's (causal INSIDE
// the new tokens: query row i sees cached rows j <= T - S + i).
//
// Shape: head_dim 128, 64-token pages, g = num_heads / num_kv_heads a divisor of 128.
// One CTA = one (sequence, kv head, block of 128 / g query tokens): the g query heads that share the kv head times the
// tokens of the block are the 128 rows (M) of both contractions, so every K / V tile is read once for all of them.
//   Q tile  : 128 rows x 128 dims bf16 (32 KB), one 3-D TMA box per 64-dim half; row = token_in_block * g + head_in_group
//   per 128-key tile (two pages of the kv head, 32 KB of K and 32 KB of V through a 4-stage TMA ring):
//     S[128 x 128] = Q K^T            8 MMAs M128 N128 K16, A and B K-major
//     softmax warps: S from TMEM -> exp2 with a lazily updated running max -> P bf16 into a swizzled shared tile
//                    (two P tiles in turn, so the exponentials of tile j+1 run while PV(j) still reads P(j))
//     O[128 x 128] += P V             8 MMAs M128 N128 K16, B = the V pages as they lie (MN-major by descriptor)
// TMEM: S double-buffered (2 x 128 columns), O 128 columns.  Issue order QK(j+1), PV(j): the softmax of tile j
// overlaps QK(j+1), the softmax of tile j+1 overlaps PV(j).
// Warp roles: 8 softmax / epilogue warps -- a query row (TMEM lane) is shared by two threads, 64 keys (and 64 output
// dims) each, because four warps alone, one per scheduler, leave the exponentials and their dependent chains exposed
// (measured: tensor pipe 26 % busy with four, the softmax being the period of the pipeline) --, 1 TMA producer, 1 MMA issuer.
// No split-KV: a prompt has (tokens x kv heads x sequences) / (128 / g) CTAs, which fills the device; the output is
// normalised in the epilogue and written once.  Blocks are numbered so that the longest (last) blocks start first.
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
constexpr int kSmemQ = 0;                  // [dims 0-63 | dims 64-127], each 128 rows x 128 B
constexpr int kSmemP = kSmemQ + 2 * kHalf; // two buffers of [keys 0-63 | keys 64-127]
constexpr int kPBytes = 2 * kHalf;
constexpr int kStages = 4;                 // K(j), V(j), K(j+1), V(j+1)
constexpr int kStageBytes = 2 * kHalf;     // 32 KB: [dims 0-63: page 0 | page 1][dims 64-127: page 0 | page 1]
constexpr int kSmemRing = kSmemP + 2 * kPBytes;
constexpr int kSmemBar = kSmemRing + kStages * kStageBytes;   // 229376
constexpr int kSmemTotal = kSmemBar + 3072;                   // 232448: all a CTA may use
constexpr int kSoftmaxThreads = 256, kThreads = kSoftmaxThreads + 64;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemS = 0, kTmemO = 256;
constexpr float kRescaleThreshold = 8.0f;

struct Bars {
  uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full[2], p_full, pv_done;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  float rowmax[2][2][128];   // [tile parity][key half][row]
  float lsum[128];           // row sums of the second key half, for the epilogue
};
static_assert(sizeof(Bars) <= 3072, "barrier block too large");

struct PrefillParams {
  const int32_t* table;
  int32_t table_stride;
  const int32_t* len;
  const int32_t* seq_ids;
  int32_t num_pages, Hkv, H, g, S, extra, causal;
  int32_t bq;                 // query tokens per block = 128 / g
  int32_t n_qblocks;
  int32_t krow0, vrow0;       // first TMA row of this layer's K block / V block
  float scale_log2;
  float* out;                 // [n][S][H][128] f32
  int32_t* status;
};

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

// 3-D tiled TMA load global -> shared (no multicast), completion on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y, int32_t z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
    gqa_prefill_sm100_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_q, const PrefillParams prm) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = prm.n_qblocks - 1 - (int)blockIdx.x;   // the blocks that see the most keys start first
  const int hk = blockIdx.y, bi = blockIdx.z;
  const int seq = prm.seq_ids ? prm.seq_ids[bi] : bi;
  const int T = prm.len[seq] + prm.extra;
  const int t0 = qb * prm.bq;                                  // first query token of the block
  const int ntok = min(prm.bq, prm.S - t0);                    // its real tokens
  // keys the block needs: all T without the mask, else up to the position of its last real token
  const int kmax = prm.causal ? (T - prm.S + t0 + ntok) : T;
  const int ntiles = (kmax + kTile - 1) / kTile;
  const int last_slot = (T + kPage - 1) / kPage - 1;           // last page slot of the sequence that holds a row

  if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled layouts need a 1024-byte aligned base
    if (threadIdx.x == 0) set_status(prm.status, RELUX_ERR_UNSUPPORTED);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kStages; s++) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 8);   // one arrival per softmax warp
    mbar_init(&bars->pv_done, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc<1>(&bars->tmem_base, kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 8) {
    // =============================== producer ===============================
    // The whole warp stays converged and one elected lane issues (operands stay in uniform registers).
    const bool el = elect_one();
    if (ntiles > 0) {
      if (el) {
        tma_prefetch_desc(&tmap_kv);
        tma_prefetch_desc(&tmap_q);
        mbar_expect_tx(&bars->q_full, 2 * kHalf);
        // box = [64 dims][g heads][bq tokens]: rows land as token_in_block * g + head_in_group
        tma_load_3d(smem + kSmemQ, &tmap_q, 0, hk * prm.g, bi * prm.S + t0, &bars->q_full);
        tma_load_3d(smem + kSmemQ + kHalf, &tmap_q, 64, hk * prm.g, bi * prm.S + t0, &bars->q_full);
      }
      __syncwarp();
      for (int j = 0; j < ntiles; j++) {
        int32_t y[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++) {
          const int slot = min(2 * j + h2, last_slot);   // a tile's second page may lie past the sequence: its keys are masked
          int32_t pg = __ldg(prm.table + (size_t)seq * prm.table_stride + slot);
          if (pg < 0 || pg >= prm.num_pages) {           // reported, and replaced by page 0 so that no load leaves the pool
            set_status(prm.status, RELUX_ERR_BAD_PAGE);
            pg = 0;
          }
          y[h2] = (pg * prm.Hkv + hk) * kPage;
        }
        const int u = j >> 1;
#pragma unroll
        for (int kv = 0; kv < 2; kv++) {
          const int st = (j & 1) * 2 + kv;
          if (u > 0) wait_bar(&bars->kv_empty[st], (u - 1) & 1, bars, prm.status);
          if (el) {
            uint8_t* dst = smem + kSmemRing + st * kStageBytes;
            const int32_t row0 = kv ? prm.vrow0 : prm.krow0;
            mbar_expect_tx(&bars->kv_full[st], kStageBytes);
#pragma unroll
            for (int cb = 0; cb < 2; cb++)
#pragma unroll
              for (int h2 = 0; h2 < 2; h2++) tma_load_2d(dst + cb * kHalf + h2 * kBlk, &tmap_kv, cb * 64, row0 + y[h2], &bars->kv_full[st]);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 9) {
    // =============================== MMA issuer (converged warp + elected lane) ===============================
    const bool el = elect_one();
    if (ntiles > 0) {
      const uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      const uint32_t idesc_pv = make_idesc_bf16(128, 128, false, true);
      const uint64_t dQ = make_desc_kmajor_sw128(smem_u32(smem + kSmemQ));
      const uint64_t dP = make_desc_kmajor_sw128(smem_u32(smem + kSmemP));
      auto issue_qk = [&](int j) {
        const int st = (j & 1) * 2;
        wait_bar(&bars->kv_full[st], (j >> 1) & 1, bars, prm.status);
        tc_fence_after();
        if (el) {
          const uint64_t dK = make_desc_kmajor_sw128(smem_u32(smem + kSmemRing + st * kStageBytes));
          const uint32_t d = tmem + kTmemS + (j & 1) * 128;
#pragma unroll
          for (int ks = 0; ks < 8; ks++) {
            const uint32_t off = (uint32_t)((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
            umma_ss<1>(d, dQ + off, dK + off, idesc_qk, ks != 0);
          }
          umma_commit<1>(&bars->kv_empty[st]);
          umma_commit<1>(&bars->s_full[j & 1]);
        }
        __syncwarp();
      };
      auto issue_pv = [&](int j) {
        const int st = (j & 1) * 2 + 1;
        wait_bar(&bars->p_full, j & 1, bars, prm.status);
        wait_bar(&bars->kv_full[st], (j >> 1) & 1, bars, prm.status);
        tc_fence_after();   // P rows and a possible O rescale were done by the softmax warps
        if (el) {
          const uint64_t dV = make_desc_mnmajor_sw128(smem_u32(smem + kSmemRing + st * kStageBytes), kHalf);
          const uint64_t dPj = dP + ((uint32_t)((j & 1) * kPBytes) >> 4);
#pragma unroll
          for (int ks = 0; ks < 8; ks++) {
            const uint32_t aoff = (uint32_t)((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
            umma_ss<1>(tmem + kTmemO, dPj + aoff, dV + ((uint32_t)(ks * 2048) >> 4), idesc_pv, j > 0 || ks != 0);
          }
          umma_commit<1>(&bars->kv_empty[st]);
          umma_commit<1>(&bars->pv_done);
        }
        __syncwarp();
      };
      wait_bar(&bars->q_full, 0, bars, prm.status);
      issue_qk(0);
      for (int j = 0; j < ntiles; j++) {
        if (j + 1 < ntiles) issue_qk(j + 1);
        issue_pv(j);
      }
    }
  } else {
    // =============================== softmax / correction / epilogue (warps 0-7) ===============================
    // Warp w reads TMEM lanes 32 (w & 3) .. +31 (the hardware's rule); warps 0-3 take keys / output dims 0-63 of
    // their rows, warps 4-7 take 64-127.
    const int wq = warp & 3, hb = warp >> 2;
    const int r = wq * 32 + lane;                   // TMEM lane = query row
    const int tq = r / prm.g, hq = r % prm.g;       // token in block, head in group
    const bool real = tq < ntok;
    const uint32_t lane_addr = ((uint32_t)(wq * 32) << 16) + (uint32_t)(hb * 64);
    // keys [0, t_eff) are visible to this row
    const int t_eff = prm.causal ? min(T, T - prm.S + t0 + tq + 1) : T;
    float m_used = -INFINITY, l_run = 0.f;
    for (int j = 0; j < ntiles; j++) {
      wait_bar(&bars->s_full[j & 1], (j >> 1) & 1, bars, prm.status);
      __syncwarp();   // the TMEM loads below are warp-collective
      tc_fence_after();
      uint32_t sv[64];
      tmem_ld_32x32b_x32(tmem + lane_addr + kTmemS + (j & 1) * 128, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld_32x32b_x32(tmem + lane_addr + kTmemS + (j & 1) * 128 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_wait();
      const int nvalid = max(0, min(64, t_eff - j * kTile - hb * 64));
      if (nvalid < 64) {
#pragma unroll
        for (int c = 0; c < 64; c++)
          if (c >= nvalid) sv[c] = 0xFF800000u;   // -inf
      }
      // row max of the raw scores (the softmax scale is positive, so it commutes with max); four chains, not one
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 64; c += 4)
#pragma unroll
        for (int k = 0; k < 4; k++) mx4[k] = fmaxf(mx4[k], __uint_as_float(sv[c + k]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * prm.scale_log2;
      bars->rowmax[j & 1][hb][r] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(mx, bars->rowmax[j & 1][hb ^ 1][r]);
      // lazily updated running max: both threads of a row take the same decision
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + kRescaleThreshold) {   // also true on the first tile with a visible key (m_used = -inf)
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
        rescale = (m_used != -INFINITY);
        m_used = mx;
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      float ps[2] = {0.f, 0.f};
      // P(j) goes to buffer j & 1, which PV(j-2) has finished reading (QK(j) was issued after it).  32 keys at a time:
      // one FFMA + one MUFU.EX2 per score, packed to bf16, four 16-byte stores into the swizzled row of key half hb.
      uint8_t* prow = smem + kSmemP + (j & 1) * kPBytes + hb * kHalf + r * 128;
#pragma unroll
      for (int q2 = 0; q2 < 2; q2++) {
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
#pragma unroll
        for (int c = 0; c < 4; c++)
          *reinterpret_cast<uint4*>(prow + (((q2 * 4 + c) ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      l_run = l_run * alpha + (ps[0] + ps[1]);
      // O may be rescaled only after PV(j-1) has completed
      if (j > 0) wait_bar(&bars->pv_done, (j - 1) & 1, bars, prm.status);
      __syncwarp();
      // The TMEM loads and stores are warp-collective: the decision is taken for the whole warp, and the rows that keep
      // their maximum multiply by one.  This thread's half of the row: output dims 64 hb .. +63.
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
        const float a_row = rescale ? alpha : 1.f;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 64; c += 32) {
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
      if (lane == 0) mbar_arrive(&bars->p_full);
    }
    // ---- epilogue: O / l -> out ----
    if (ntiles > 0) {
      wait_bar(&bars->pv_done, (ntiles - 1) & 1, bars, prm.status);
      __syncwarp();
      tc_fence_after();
    }
    // the row sum is the sum of its two key halves
    if (hb == 1) bars->lsum[r] = l_run;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (hb == 0) bars->lsum[r] = l_run + bars->lsum[r];
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l_run = bars->lsum[r];
    // warp-uniform: the TMEM loads below are warp-collective
    const bool ok = ntiles > 0 && !__any_sync(0xffffffffu, bars->abort_flag != 0);
    const float inv = (ok && l_run > 0.f) ? 1.f / l_run : 0.f;
    float* orow = prm.out + (((size_t)bi * prm.S + t0 + (real ? tq : 0)) * prm.H + (size_t)hk * prm.g + hq) * kD + hb * 64;
#pragma unroll 1
    for (int c = 0; c < 64; c += 32) {
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
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<1>(tmem, kTmemCols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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
  const int64_t rows_per_block = (int64_t)prm.num_pages * prm.gqa_num_kv_heads * kPage;
  k.krow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block);
  k.vrow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block + rows_per_block);
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.out = d_out;
  k.status = p->d_status;
  if (k.n_qblocks > 65535 * 32 || sb.n_seqs > 65535) { set_error("prompt too long for one launch"); return RELUX_ERR_UNSUPPORTED; }
  cudaStream_t st = p->dev->stream;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_prefill_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
  dim3 grid(k.n_qblocks, prm.gqa_num_kv_heads, sb.n_seqs);
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), st));
  gqa_prefill_sm100_kernel<<<grid, kThreads, kSmemTotal, st>>>(p->tmap_gqa, tq, k);
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), st));
  p->timed_calls++;
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux
