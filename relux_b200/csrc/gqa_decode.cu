// GQA flash-decode / speculative verify over the paged bf16 K/V pool (RELUX_ATTN_FAST).
//
// Bound: HBM bandwidth.  Every cached token costs Hkv * D * 2 (K,V) * 2 B = 4096 B at Hkv=8, D=128,
// against about 16 flop/B of work, so the kernel is organised around keeping TMA loads in flight:
//   * one CTA per (sequence chunk, kv head); warp 4 is the producer, warps 0-3 consume;
//   * the producer streams each 64-token page of this head as four 8 KB TMA boxes (K and V, two 64-wide
//     halves each, 128-byte swizzle) through a ring of kStages stages guarded by full/empty mbarriers;
//   * the g query heads sharing the kv head times the S query tokens form the 16-row M dimension of
//     mma.sync m16n8k16 (bf16 in, f32 accumulate); each consumer warp owns 16 tokens of every page and
//     keeps its own online-softmax state, so warps never wait on each other inside the loop;
//   * at the end the four warps' (max, sum, O) are combined through shared memory and written as one
//     split-KV partial; merge_splits_kernel combines the chunks of a sequence.
// All mbarrier waits are bounded; a wait that runs out records RELUX_ERR_TIMEOUT and the CTA leaves.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <vector>
#include "common.cuh"
#include "internal.h"
#include "splitkv.h"

namespace relux {

namespace {

constexpr int kStages = 5;
constexpr int kPageTok = 64;
constexpr int kD = 128;
constexpr int kStageBytes = 4 * 8192;  // K lo, K hi, V lo, V hi
constexpr int kQStride = kD + 8;       // bf16 elements per Q row in shared memory (272 B, conflict-free ldmatrix)
constexpr int kConsumerWarps = 4;

struct GqaParams {
  const WorkItem* items;
  const int32_t* table;
  int32_t table_stride;
  const int32_t* len;
  int32_t num_pages, Hkv, H, g, S, R, extra, causal;
  int32_t krow0, vrow0;  // first TMA row of this layer's K block / V block
  float scale_log2;
  const void* q;
  int32_t q_bf16;
  float* part_o;
  float* part_ml;
  int32_t rows_total;  // S * H
  int32_t q_tokens_total, q_token0;   // the S query tokens of this launch are tokens [q_token0, q_token0 + S) of a call with q_tokens_total
  // Grouped launch (a prompt): grid.z slices the call's query tokens into groups of group_tokens; slice z handles tokens
  // [(group0 + z) * group_tokens, ...) and S, R, extra above describe the whole call.  0 = one group, described by S / R / extra.
  int32_t group_tokens, group0;
  int64_t part_group_rows;            // partial rows (work items x rows_total) between two slices
  int32_t* status;
};

template <int MT>
__global__ void __launch_bounds__(160, 1) gqa_decode_kernel(const __grid_constant__ CUtensorMap tmap, const GqaParams prm) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: stages (1024-aligned) | Q | barriers
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = smem;
  uint16_t* qs = (uint16_t*)(smem + kStages * kStageBytes);
  uint64_t* full = (uint64_t*)(qs + 16 * MT * kQStride);
  uint64_t* empty = full + kStages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WorkItem item = prm.items[blockIdx.x];
  const int kvh = blockIdx.y;
  int S = prm.S, R = prm.R, extra = prm.extra, q_token0 = prm.q_token0;
  size_t part_row0 = 0;
  if (prm.group_tokens) {
    // With the causal mask a group of tokens sees the cache as if it ended with its own last token.
    q_token0 = (prm.group0 + (int)blockIdx.z) * prm.group_tokens;
    S = min(prm.group_tokens, prm.q_tokens_total - q_token0);
    R = S * prm.g;
    if (prm.causal) extra = prm.extra - (prm.q_tokens_total - q_token0 - S);
    part_row0 = (size_t)blockIdx.z * (size_t)prm.part_group_rows;
  }
  const int T = prm.len[item.seq] + extra;
  // pages of this chunk that hold tokens below T (a later group's chunk can lie wholly past an earlier group's end)
  const int npages = max(0, min(item.page_end - item.page_begin, (T - item.page_begin * kPageTok + kPageTok - 1) / kPageTok));

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    fence_mbar_init();
  }
  // Q rows of this kv head -> shared memory as bf16; row r = s * g + hq, rows >= R are zero.
  for (int e = threadIdx.x; e < 16 * MT * (kD / 2); e += blockDim.x) {
    const int r = e / (kD / 2), c = (e % (kD / 2)) * 2;
    uint32_t w = 0;
    if (r < R) {
      const int s = r / prm.g, hq = r % prm.g;
      const size_t off = (((size_t)item.seq_index * prm.q_tokens_total + q_token0 + s) * prm.H + (size_t)kvh * prm.g + hq) * kD + c;
      if (prm.q_bf16) w = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(prm.q) + off);
      else {
        float2 f = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(prm.q) + off);
        w = pack_bf16x2(f.x, f.y);
      }
    }
    *reinterpret_cast<uint32_t*>(qs + r * kQStride + c) = w;
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap);
      bool ok = true;
      for (int it = 0; it < npages && ok; it++) {
        const int st = it % kStages, k = it / kStages;
        if (k > 0 && !mbar_wait(&empty[st], (k - 1) & 1)) {
          set_status(prm.status, RELUX_ERR_TIMEOUT);
          ok = false;
          break;
        }
        int32_t pg = prm.table[(size_t)item.seq * prm.table_stride + item.page_begin + it];
        if (pg < 0 || pg >= prm.num_pages) {
          set_status(prm.status, RELUX_ERR_BAD_PAGE);
          pg = 0;  // keep the pipeline protocol intact; the status word reports the fault
        }
        uint8_t* sb = stages + st * kStageBytes;
        const int32_t krow = prm.krow0 + (pg * prm.Hkv + kvh) * kPageTok;
        const int32_t vrow = prm.vrow0 + (pg * prm.Hkv + kvh) * kPageTok;
        mbar_expect_tx(&full[st], kStageBytes);
        tma_load_2d(sb, &tmap, 0, krow, &full[st]);
        tma_load_2d(sb + 8192, &tmap, 64, krow, &full[st]);
        tma_load_2d(sb + 16384, &tmap, 0, vrow, &full[st]);
        tma_load_2d(sb + 24576, &tmap, 64, vrow, &full[st]);
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  uint32_t qa[MT][8][4];
#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
      const int m = lane >> 3;
      const int row = mt * 16 + (m & 1) * 8 + (lane & 7);
      const int col = ks * 16 + (m >> 1) * 8;
      ldmatrix_x4(qa[mt][ks][0], qa[mt][ks][1], qa[mt][ks][2], qa[mt][ks][3], smem_u32(qs + row * kQStride + col));
    }

  float oacc[MT][16][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
#pragma unroll
    for (int nt = 0; nt < 16; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) oacc[mt][nt][e] = 0.f;
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
  }
  const int tb = warp * 16;  // this warp's tokens inside every page
  bool alive = true;

  for (int it = 0; it < npages; it++) {
    const int st = it % kStages;
    if (!mbar_wait(&full[st], (it / kStages) & 1)) {
      set_status(prm.status, RELUX_ERR_TIMEOUT);
      alive = false;
      break;
    }
    const uint32_t kt = smem_u32(stages + st * kStageBytes);
    const uint32_t vt = kt + 16384;
    float sacc[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) sacc[mt][nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
      const int m = lane >> 3;
      const uint32_t row = tb + (m >> 1) * 8 + (lane & 7);
      const uint32_t chunk = (ks & 3) * 2 + (m & 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, kt + (ks >> 2) * 8192 + swz128(row, chunk));
#pragma unroll
      for (int mt = 0; mt < MT; mt++) {
        mma_bf16_16816(sacc[mt][0], qa[mt][ks], b0, b1);
        mma_bf16_16816(sacc[mt][1], qa[mt][ks], b2, b3);
      }
    }
    // scale to the log2 domain, mask the tail of the sequence and the causal part of the draft
    const int tok0 = (item.page_begin + it) * kPageTok + tb;
    const bool need_mask = (tok0 + 16 > T - (prm.causal ? S : 0));
    uint32_t pa[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        const int row = mt * 16 + hf * 8 + (lane >> 2);
        const int limit = prm.causal ? (T - S + row / prm.g) : (T - 1);  // last visible token
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            float v = sacc[mt][nt][hf * 2 + e] * prm.scale_log2;
            if (need_mask) {
              const int tok = tok0 + nt * 8 + 2 * (lane & 3) + e;
              if (tok > limit || tok >= T) v = -INFINITY;
            }
            sacc[mt][nt][hf * 2 + e] = v;
            mx = fmaxf(mx, v);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[mt][hf], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run[mt][hf] - m_use);
        m_run[mt][hf] = m_new;
        float ps = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const float pv = exp2f(sacc[mt][nt][hf * 2 + e] - m_use);
            sacc[mt][nt][hf * 2 + e] = pv;
            ps += pv;
          }
        l_run[mt][hf] = l_run[mt][hf] * alpha + ps;
#pragma unroll
        for (int nt = 0; nt < 16; nt++) {
          oacc[mt][nt][hf * 2] *= alpha;
          oacc[mt][nt][hf * 2 + 1] *= alpha;
        }
      }
      pa[mt][0] = pack_bf16x2(sacc[mt][0][0], sacc[mt][0][1]);
      pa[mt][1] = pack_bf16x2(sacc[mt][0][2], sacc[mt][0][3]);
      pa[mt][2] = pack_bf16x2(sacc[mt][1][0], sacc[mt][1][1]);
      pa[mt][3] = pack_bf16x2(sacc[mt][1][2], sacc[mt][1][3]);
    }
    // O += P V
#pragma unroll
    for (int n2 = 0; n2 < 8; n2++) {
      const int m = lane >> 3;
      const uint32_t row = tb + (m & 1) * 8 + (lane & 7);
      const uint32_t chunk = n2 * 2 + (m >> 1);  // 16 chunks of 8 dims
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vt + (chunk >> 3) * 8192 + swz128(row, chunk & 7));
#pragma unroll
      for (int mt = 0; mt < MT; mt++) {
        mma_bf16_16816(oacc[mt][2 * n2], pa[mt], b0, b1);
        mma_bf16_16816(oacc[mt][2 * n2 + 1], pa[mt], b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[st]);
  }

  // ---------------- combine the four warps, write the split-KV partial ----------------
  // every load this CTA issued has completed once all consumers passed their last full-barrier wait
  asm volatile("bar.sync 1, 128;" ::: "memory");
  constexpr int kMStride = kD + 2;
  float* mb = reinterpret_cast<float*>(stages);  // [4 warps][16*MT rows][kD + 2]
#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
      float l = l_run[mt][hf];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int row = mt * 16 + hf * 8 + (lane >> 2);
      float* dst = mb + ((size_t)warp * 16 * MT + row) * kMStride;
#pragma unroll
      for (int nt = 0; nt < 16; nt++) {
        dst[nt * 8 + 2 * (lane & 3)] = oacc[mt][nt][hf * 2];
        dst[nt * 8 + 2 * (lane & 3) + 1] = oacc[mt][nt][hf * 2 + 1];
      }
      if ((lane & 3) == 0) {
        dst[kD] = alive ? m_run[mt][hf] : -INFINITY;
        dst[kD + 1] = alive ? l : 0.f;
      }
    }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  const int d = threadIdx.x;  // 128 consumer threads, one output dim each
  for (int r = 0; r < R; r++) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; w++) M = fmaxf(M, mb[((size_t)w * 16 * MT + r) * kMStride + kD]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; w++) {
      const float* src = mb + ((size_t)w * 16 * MT + r) * kMStride;
      const float f = (src[kD] == -INFINITY) ? 0.f : exp2f(src[kD] - M);
      L += src[kD + 1] * f;
      O += src[d] * f;
    }
    const int s = r / prm.g, hq = r % prm.g;
    const size_t grow = part_row0 + (size_t)blockIdx.x * prm.rows_total + (size_t)s * prm.H + (size_t)kvh * prm.g + hq;
    prm.part_o[grow * kD + d] = O;
    if (d == 0) {
      prm.part_ml[grow * 2] = M;
      prm.part_ml[grow * 2 + 1] = L;
    }
  }
}

template <int MT>
constexpr size_t gqa_smem_bytes() {
  return 1024 + (size_t)kStages * kStageBytes + (size_t)16 * MT * kQStride * 2 + 2 * kStages * 8 + 64;
}

}  // namespace

// One launch of the decode kernel + merge for query tokens [s0, s0 + Sg) of a call with a.q_tokens tokens.
// With the causal mask a group of tokens sees the cache as if it ended with its own last token, so the group is
// exactly a call with q_tokens = Sg on a cache shortened by the tokens that follow it (extra_g <= a.extra_tokens).
static int32_t launch_gqa_group(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const void* d_q, void* d_out, int s0, int Sg) {
  const relux_pool_params& prm = p->prm;
  const int g = a.num_heads / prm.gqa_num_kv_heads, R = g * Sg;
  const int extra_g = a.causal ? a.extra_tokens - (a.q_tokens - s0 - Sg) : a.extra_tokens;
  SplitPlan plan;
  int32_t rc = plan_splitkv(p, sb, a.layer, extra_g, prm.gqa_num_kv_heads, 2, 1, 0, &plan);
  if (rc) return rc;
  const int rows_total = Sg * a.num_heads;
  rc = grow(p->dev, p->part_o, (size_t)plan.num_items * rows_total * kD * sizeof(float));
  if (rc) return rc;
  rc = grow(p->dev, p->part_ml, (size_t)plan.num_items * rows_total * 2 * sizeof(float));
  if (rc) return rc;
  GqaParams k{};
  k.items = plan.items;
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.len = p->d_len + (size_t)a.layer * prm.max_seqs;
  k.num_pages = prm.num_pages;
  k.Hkv = prm.gqa_num_kv_heads;
  k.H = a.num_heads;
  k.g = g;
  k.S = Sg;
  k.R = R;
  k.extra = extra_g;
  k.causal = a.causal;
  k.q_tokens_total = a.q_tokens;
  k.q_token0 = s0;
  const int64_t rows_per_block = (int64_t)prm.num_pages * prm.gqa_num_kv_heads * kPageTok;
  k.krow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block);
  k.vrow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block + rows_per_block);
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.q = d_q;
  k.q_bf16 = a.q_dtype == RELUX_DTYPE_BF16;
  k.part_o = (float*)p->part_o.p;
  k.part_ml = (float*)p->part_ml.p;
  k.rows_total = rows_total;
  k.status = p->d_status;
  dim3 grid(plan.num_items, prm.gqa_num_kv_heads);
  cudaStream_t st = p->dev->stream;
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), st));
  if (R <= 16) {
    constexpr size_t smem = gqa_smem_bytes<1>();
    RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gqa_decode_kernel<1><<<grid, 160, smem, st>>>(p->tmap_gqa, k);
  } else {
    constexpr size_t smem = gqa_smem_bytes<2>();
    RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gqa_decode_kernel<2><<<grid, 160, smem, st>>>(p->tmap_gqa, k);
  }
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), st));
  p->timed_calls++;
  count_launch(p->dev);
  return launch_merge_rows(p, plan, sb.n_seqs, rows_total, kD, (float*)d_out, a.q_tokens * a.num_heads, s0 * a.num_heads);
}

// A multi-token call longer than one group (a prompt): one work list for the whole call, the groups of `per_group`
// query tokens as z slices of the decode grid and of the merge grid.  Slice z sees the cache as if it ended with its own
// last token (causal), so its chunks past that point load nothing and leave neutral partials.  The partials of all
// slices of a launch are alive at once; launches are cut so that they stay within 256 MiB.
static int32_t launch_gqa_prompt(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const void* d_q, void* d_out, int per_group) {
  const relux_pool_params& prm = p->prm;
  const int g = a.num_heads / prm.gqa_num_kv_heads;
  const int groups = (a.q_tokens + per_group - 1) / per_group;
  // every work item becomes groups x kv heads CTAs, so the planner may keep the chunks long: a prompt fills the SMs
  // through its slices, and a CTA that streams many pages amortises its prologue
  SplitPlan plan;
  int32_t rc = plan_splitkv(p, sb, a.layer, a.extra_tokens, prm.gqa_num_kv_heads * groups, 2, 1, 0, &plan);
  if (rc) return rc;
  const int rows_total = per_group * a.num_heads;
  const size_t group_rows = (size_t)plan.num_items * rows_total;
  const size_t group_bytes = group_rows * kD * sizeof(float);
  const size_t budget = (size_t)std::max(1, p->tune.get(RELUX_TUNE_GQA_PROMPT_PARTIAL_MB)) << 20;   // tuning / test knob
  const int zmax = (int)std::max<size_t>(1, std::min<size_t>({(size_t)groups, (size_t)65535, budget / std::max<size_t>(1, group_bytes)}));
  rc = grow(p->dev, p->part_o, (size_t)zmax * group_bytes);
  if (rc) return rc;
  rc = grow(p->dev, p->part_ml, (size_t)zmax * group_rows * 2 * sizeof(float));
  if (rc) return rc;
  GqaParams k{};
  k.items = plan.items;
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.len = p->d_len + (size_t)a.layer * prm.max_seqs;
  k.num_pages = prm.num_pages;
  k.Hkv = prm.gqa_num_kv_heads;
  k.H = a.num_heads;
  k.g = g;
  k.S = a.q_tokens;                 // the whole call; every slice derives its own S, R and extra
  k.R = per_group * g;
  k.extra = a.extra_tokens;
  k.causal = a.causal;
  k.q_tokens_total = a.q_tokens;
  k.q_token0 = 0;
  k.group_tokens = per_group;
  k.part_group_rows = (int64_t)group_rows;
  const int64_t rows_per_block = (int64_t)prm.num_pages * prm.gqa_num_kv_heads * kPageTok;
  k.krow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block);
  k.vrow0 = (int32_t)((int64_t)a.layer * 2 * rows_per_block + rows_per_block);
  k.scale_log2 = a.scale * 1.4426950408889634f;
  k.q = d_q;
  k.q_bf16 = a.q_dtype == RELUX_DTYPE_BF16;
  k.part_o = (float*)p->part_o.p;
  k.part_ml = (float*)p->part_ml.p;
  k.rows_total = rows_total;
  k.status = p->d_status;
  cudaStream_t st = p->dev->stream;
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), st));
  for (int z0 = 0; z0 < groups; z0 += zmax) {
    const int nz = std::min(zmax, groups - z0);
    k.group0 = z0;
    dim3 grid(plan.num_items, prm.gqa_num_kv_heads, nz);
    if (per_group * g <= 16) {
      constexpr size_t smem = gqa_smem_bytes<1>();
      RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      gqa_decode_kernel<1><<<grid, 160, smem, st>>>(p->tmap_gqa, k);
    } else {
      constexpr size_t smem = gqa_smem_bytes<2>();
      RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      gqa_decode_kernel<2><<<grid, 160, smem, st>>>(p->tmap_gqa, k);
    }
    RELUX_CUDA_TRY(cudaGetLastError());
    count_launch(p->dev);
    rc = launch_merge_rows(p, plan, sb.n_seqs, rows_total, kD, (float*)d_out, a.q_tokens * a.num_heads, z0 * rows_total, nz,
                           (long long)group_rows);
    if (rc) return rc;
  }
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), st));
  p->timed_calls++;
  return RELUX_OK;
}

bool gqa_prefill_eligible(const Pool* p, const relux_attn_args& a);
int32_t launch_gqa_prefill_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const uint16_t* d_q, float* d_out);

bool gqa_prompt_wants_bf16(const Pool* p, const relux_attn_args& a) {
  const int g = a.num_heads / std::max(1, p->prm.gqa_num_kv_heads);
  return g >= 1 && a.q_tokens > std::max(1, 32 / g) && !p->tune.get(RELUX_TUNE_GQA_PROMPT_SLICES) && gqa_prefill_eligible(p, a);
}

int32_t launch_gqa_decode_fast(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const void* d_q, void* d_out) {
  const relux_pool_params& prm = p->prm;
  const int g = a.num_heads / prm.gqa_num_kv_heads;
  if (!p->has_tmap || prm.page_tokens != kPageTok || prm.gqa_head_dim != kD || g > 32) {
    set_error("GQA FAST kernel needs page_tokens=64, head_dim=128 and num_heads/num_kv_heads <= 32 "
              "(got page_tokens=%d head_dim=%d group=%d); use RELUX_ATTN_REFERENCE for other shapes",
              prm.page_tokens, prm.gqa_head_dim, g);
    return RELUX_ERR_UNSUPPORTED;
  }
  // the kernel holds (num_heads / num_kv_heads) * q_tokens <= 32 query rows per kv head; longer multi-token calls
  // (a prompt) are cut into groups of tokens that run as the z slices of one grid
  const int per_group = std::max(1, 32 / g);
  if (a.q_tokens <= per_group) return launch_gqa_group(p, sb, a, d_q, d_out, 0, a.q_tokens);
  // a prompt: 128 query rows per CTA on the tcgen05 prefill kernel; the grid slices of the decode kernel serve the
  // group sizes that do not tile 128 rows, and stay selectable as a tuning knob
  if (a.q_dtype == RELUX_DTYPE_BF16 && gqa_prompt_wants_bf16(p, a)) return launch_gqa_prefill_sm100(p, sb, a, (const uint16_t*)d_q, (float*)d_out);
  return launch_gqa_prompt(p, sb, a, d_q, d_out, per_group);
}

// ---------------------------------------------------------------------------------------------------------
// relux_gqa_decode_noalloc: the same split-KV flash-decode for callers that must not allocate device memory
// (see include/relux_cuda.h).  Its work list and split-KV partials live in one fixed array in device memory.
// ---------------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocScratchBytes = (size_t)16 << 20;  // 16 MiB, held by every GPU that loads the library
constexpr int kNoAllocMaxItems = 4096;
constexpr int kNoAllocMaxSeqs = 4096;
constexpr int kNoAllocMaxDevices = 64;

// In host code this name is only a handle for cudaGetSymbolAddress; the kernels get the resolved device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct NoAllocSlot {
  bool ready = false;
  unsigned char* base = nullptr;
};
NoAllocSlot g_noalloc_slot[kNoAllocMaxDevices];
std::mutex g_noalloc_mu;

constexpr size_t kNaItemsOff = 0;
constexpr size_t kNaChunkOff = kNaItemsOff + sizeof(WorkItem) * kNoAllocMaxItems;                         // 64 KiB
constexpr size_t kNaPartOff = (kNaChunkOff + sizeof(int32_t) * (kNoAllocMaxSeqs + 1) + 255) & ~(size_t)255;
constexpr size_t kNaPartBytes = kNoAllocScratchBytes - kNaPartOff;
constexpr size_t kNaBytesPerRow = (size_t)(kD + 2) * sizeof(float);  // one partial row: D accumulators + (max, sum)

}  // namespace

}  // namespace relux

extern "C" __attribute__((visibility("default"))) int32_t relux_gqa_decode_noalloc(relux_pool_t handle, const relux_attn_args* a) {
  using namespace relux;
  Pool* p = as_pool(handle);
  if (!p) { set_error("bad pool handle"); return RELUX_ERR_BAD_HANDLE; }
  Device* dev = p->dev;
  std::unique_lock<std::mutex> lk(dev->mu);
  RELUX_CUDA_TRY(cudaSetDevice(dev->index));
  const relux_pool_params& prm = p->prm;
  if (!a) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  if (prm.kind != RELUX_POOL_GQA) { set_error("relux_gqa_decode_noalloc needs a GQA pool"); return RELUX_ERR_INVALID_ARG; }
  if (a->layer < 0 || a->layer >= prm.num_layers) { set_error("layerIdx=%d out of range [0, %d)", a->layer, prm.num_layers); return RELUX_ERR_INVALID_ARG; }
  if (!a->q || !a->out || a->q_tokens <= 0 || a->extra_tokens < 0 || a->num_heads <= 0 || a->head_dim != prm.gqa_head_dim ||
      a->num_heads % prm.gqa_num_kv_heads != 0) {
    set_error("relux_gqa_decode_noalloc: bad attention arguments");
    return RELUX_ERR_INVALID_ARG;
  }
  // Nothing may be staged or converted here, because staging buffers are grown with cudaMalloc.
  if (a->mode != RELUX_ATTN_FAST || a->q_mem != RELUX_MEM_DEVICE || a->out_mem != RELUX_MEM_DEVICE || a->out_dtype != RELUX_DTYPE_F32 ||
      (a->q_dtype != RELUX_DTYPE_F32 && a->q_dtype != RELUX_DTYPE_BF16) ||
      (a->q_tokens > 1 && (a->q_layout != RELUX_LAYOUT_TOKEN_MAJOR || a->out_layout != RELUX_LAYOUT_TOKEN_MAJOR))) {
    set_error("relux_gqa_decode_noalloc takes device-resident token-major q (f32 or bf16) and writes device-resident f32 output, FAST mode only");
    return RELUX_ERR_UNSUPPORTED;
  }
  {
    int32_t rca;
    if ((rca = check_dev_align(a->q, "q")) || (rca = check_dev_align(a->out, "out"))) return rca;
  }
  const int g = a->num_heads / prm.gqa_num_kv_heads, R = g * a->q_tokens;
  if (!p->has_tmap || prm.page_tokens != kPageTok || prm.gqa_head_dim != kD || R > 32) {
    set_error("relux_gqa_decode_noalloc needs page_tokens=64, head_dim=128 and (num_heads/num_kv_heads)*q_tokens <= 32");
    return RELUX_ERR_UNSUPPORTED;
  }
  if (a->n_seqs > kNoAllocMaxSeqs) {
    set_error("relux_gqa_decode_noalloc: n_seqs=%d exceeds the fixed scratch limit of %d sequences", a->n_seqs, kNoAllocMaxSeqs);
    return RELUX_ERR_UNSUPPORTED;
  }
  SeqBatch sb;  // uses the pool's pre-allocated pinned staging only
  int32_t rc = stage_batch(p, a->n_seqs, a->seq_ids, nullptr, a->q_tokens, &sb);
  if (rc) return rc;
  const int rows_total = a->q_tokens * a->num_heads;
  long total_pages = 0;
  int max_pages = 1;
  std::vector<int> pages(sb.n_seqs);
  for (int i = 0; i < sb.n_seqs; i++) {
    const int s = sb.seq[i];
    const int T = p->h_len[(size_t)a->layer * prm.max_seqs + s] + a->extra_tokens;
    if (T < a->q_tokens || T > p->seq_pages[s] * prm.page_tokens) {
      set_error("sequence %d: %d cached rows cannot serve %d query tokens within its capacity", s, T, a->q_tokens);
      return RELUX_ERR_INVALID_ARG;
    }
    pages[i] = (T + kPageTok - 1) / kPageTok;
    total_pages += pages[i];
    max_pages = std::max(max_pages, pages[i]);
  }
  // Chunk length: about four waves of CTAs, then lengthened until the partials fit the fixed scratch.
  const long max_items_by_bytes = (long)(kNaPartBytes / (kNaBytesPerRow * (size_t)rows_total));
  const long item_cap = std::min<long>(kNoAllocMaxItems, max_items_by_bytes);
  const long target = std::max(1L, 4L * dev->sm_count / prm.gqa_num_kv_heads);
  int chunk = std::max(2, (int)((total_pages + target - 1) / target));
  chunk = std::min(chunk, max_pages);
  long items = 0;
  for (;;) {
    items = 0;
    for (int i = 0; i < sb.n_seqs; i++) items += (pages[i] + chunk - 1) / chunk;
    if (items <= item_cap || chunk >= max_pages) break;
    chunk = std::min(max_pages, chunk + std::max(1, chunk / 8));
  }
  if (items > item_cap) {
    set_error("relux_gqa_decode_noalloc: %ld work items x %d query rows need %zu bytes of partials; the fixed scratch holds %zu "
              "(limits: %d items, %d sequences, 16 MiB in total)",
              items, rows_total, (size_t)items * rows_total * kNaBytesPerRow, kNaPartBytes, kNoAllocMaxItems, kNoAllocMaxSeqs);
    return RELUX_ERR_UNSUPPORTED;
  }
  // First call on this device: resolve the device address of the scratch array (the device is current here).
  if (dev->index < 0 || dev->index >= kNoAllocMaxDevices) { set_error("device index %d beyond %d", dev->index, kNoAllocMaxDevices); return RELUX_ERR_UNSUPPORTED; }
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> g2(g_noalloc_mu);
    NoAllocSlot& slot = g_noalloc_slot[dev->index];
    if (!slot.ready) {
      void* ptr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess || !ptr) return cuda_fail(e != cudaSuccess ? e : cudaErrorInvalidSymbol, "cudaGetSymbolAddress(g_noalloc_scratch)");
      slot.base = (unsigned char*)ptr;
      slot.ready = true;
    }
    base = slot.base;
  }
  WorkItem* d_items = (WorkItem*)(base + kNaItemsOff);
  int32_t* d_chunk_off = (int32_t*)(base + kNaChunkOff);
  float* d_part_ml = (float*)(base + kNaPartOff);
  float* d_part_o = d_part_ml + (size_t)items * rows_total * 2;
  cudaStream_t st = dev->stream;
  const int32_t* len = p->d_len + (size_t)a->layer * prm.max_seqs;
  rc = launch_build_worklist_raw(st, len, sb.d_seq_ids, sb.n_seqs, a->extra_tokens, prm.page_tokens, chunk, d_items, d_chunk_off);
  if (rc) return rc;
  count_launch(dev);
  GqaParams k{};
  k.items = d_items;
  k.table = p->d_table;
  k.table_stride = prm.max_pages_per_seq;
  k.len = len;
  k.num_pages = prm.num_pages;
  k.Hkv = prm.gqa_num_kv_heads;
  k.H = a->num_heads;
  k.g = g;
  k.S = a->q_tokens;
  k.R = R;
  k.extra = a->extra_tokens;
  k.causal = a->causal;
  k.q_tokens_total = a->q_tokens;
  k.q_token0 = 0;
  const int64_t rows_per_block = (int64_t)prm.num_pages * prm.gqa_num_kv_heads * kPageTok;
  k.krow0 = (int32_t)((int64_t)a->layer * 2 * rows_per_block);
  k.vrow0 = (int32_t)((int64_t)a->layer * 2 * rows_per_block + rows_per_block);
  k.scale_log2 = a->scale * 1.4426950408889634f;
  k.q = a->q;
  k.q_bf16 = a->q_dtype == RELUX_DTYPE_BF16;
  k.part_o = d_part_o;
  k.part_ml = d_part_ml;
  k.rows_total = rows_total;
  k.status = p->d_status;
  dim3 grid((unsigned)items, prm.gqa_num_kv_heads);
  if (R <= 16) {
    constexpr size_t smem = gqa_smem_bytes<1>();
    RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gqa_decode_kernel<1><<<grid, 160, smem, st>>>(p->tmap_gqa, k);
  } else {
    constexpr size_t smem = gqa_smem_bytes<2>();
    RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gqa_decode_kernel<2><<<grid, 160, smem, st>>>(p->tmap_gqa, k);
  }
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(dev);
  rc = launch_merge_raw(st, d_part_o, d_part_ml, d_chunk_off, sb.n_seqs, rows_total, kD, (float*)a->out);
  if (rc) return rc;
  count_launch(dev);
  return RELUX_OK;
}
