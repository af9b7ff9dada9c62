// Absorbed MLA flash-decode over the paged latent cache (RELUX_ATTN_FAST): host-side pipeline and
// the shape-generic CUDA-core kernels.
//
//   q~[row][h] = [ W_UK_h q_nope[row][h]  |  q_rope[row][h] ]          (mla_absorb_kernel)
//   split-KV:   scores = q~ . [c^KV | k^R]^T * scale, online softmax, O_lat += P c^KV
//               (mla_decode_sm100.cu when the shape is the tensor-core one, else mla_decode_generic_kernel)
//   merge the chunks of every sequence                                   (merge_splits_kernel)
//   out[row][h] = W_UV_h^T O_lat[row][h]                                  (mla_vup_kernel)
//
// This replaces the reference's "decompress every cached latent, then attend" (mla.go:323-377): the cache
// row (dC + dHR values, shared by all heads) is read once per token instead of being expanded to
// 2 * H * head_dim values.
#include <cstdlib>
#include "common.cuh"
#include "internal.h"
#include "splitkv.h"
#include "prep_parts.cuh"

namespace relux {

int32_t launch_mla_decode_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const SplitPlan& plan, const uint16_t* q_abs);
bool mla_sm100_eligible(const Pool* p, const relux_attn_args& a);
int mla_sm100_workers(Pool* p, int q_tokens);
bool mla_proj_mma_eligible(int Dh, int dC);
bool mla_prep_fits(int n_seqs, int H, int dC);
int32_t launch_mla_prefill_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const uint16_t* d_q, const uint16_t* d_qr, float* d_out);
int32_t launch_mla_prep(Device* dev, const void* q_nope, const void* q_rope, int q_bf16, const uint16_t* W_UK, uint16_t* q_abs, int rows,
                        int H, int dC, int dHR, const PrepAppend& ap, const PrepPlan& pl, bool chained);
int32_t launch_mla_absorb_mma(Device* dev, const void* q_nope, const void* q_rope, int q_bf16, const uint16_t* W_UK, uint16_t* q_abs,
                              int rows, int H, int dC, int dHR);
int32_t launch_mla_vup_mma(Device* dev, const uint16_t* o_lat, const uint16_t* W_UV, float* out, int rows, int H, int dC);
int32_t launch_mla_merge_vup_mma(Device* dev, const float* part_o, const float* part_ml, const int32_t* chunk_off, const uint16_t* W_UV,
                                 float* out, int rows, int S, int H, int dC, int32_t* status, bool chained);

namespace {

// ---- q absorption -----------------------------------------------------------------------------
// grid (H, dC/64, ceil(rows/16)), 256 threads.  q_nope [rows][H][Dh] (f32 or bf16), W_UK [dC][H*Dh] bf16,
// q_abs [rows][H][dC+dHR] bf16.  The blockIdx.y == 0 slice also copies q_rope into the tail of the row.
__global__ void mla_absorb_kernel(const void* __restrict__ q_nope, const void* __restrict__ q_rope, int q_bf16,
                                  const uint16_t* __restrict__ W_UK, uint16_t* __restrict__ q_abs, int rows, int H, int Dh, int dC,
                                  int dHR) {
  extern __shared__ float sm[];
  const int h = blockIdx.x, c0 = blockIdx.y * 64, r0 = blockIdx.z * 16;
  float* ws = sm;                 // [64][Dh + 1]
  float* qs = sm + 64 * (Dh + 1); // [16][Dh]
  const int tid = threadIdx.x;
  for (int e = tid; e < 64 * Dh; e += blockDim.x) {
    const int c = e / Dh, d = e % Dh;
    ws[c * (Dh + 1) + d] = (c0 + c < dC) ? f32_from_bf16_bits(W_UK[(size_t)(c0 + c) * H * Dh + (size_t)h * Dh + d]) : 0.f;
  }
  for (int e = tid; e < 16 * Dh; e += blockDim.x) {
    const int r = e / Dh, d = e % Dh;
    float v = 0.f;
    if (r0 + r < rows) {
      const size_t off = ((size_t)(r0 + r) * H + h) * Dh + d;
      v = q_bf16 ? f32_from_bf16_bits(reinterpret_cast<const uint16_t*>(q_nope)[off]) : reinterpret_cast<const float*>(q_nope)[off];
    }
    qs[r * Dh + d] = v;
  }
  __syncthreads();
  const int row_w = dC + dHR;
  for (int e = tid; e < 16 * 64; e += blockDim.x) {
    const int r = e / 64, c = e % 64;
    if (r0 + r >= rows || c0 + c >= dC) continue;
    float acc = 0.f;
    for (int d = 0; d < Dh; d++) acc += qs[r * Dh + d] * ws[c * (Dh + 1) + d];
    q_abs[((size_t)(r0 + r) * H + h) * row_w + c0 + c] = bf16_bits_from_f32(acc);
  }
  if (blockIdx.y == 0) {
    for (int e = tid; e < 16 * dHR; e += blockDim.x) {
      const int r = e / dHR, d = e % dHR;
      if (r0 + r >= rows) continue;
      const size_t off = ((size_t)(r0 + r) * H + h) * dHR + d;
      const uint16_t b = q_bf16 ? reinterpret_cast<const uint16_t*>(q_rope)[off] : bf16_bits_from_f32(reinterpret_cast<const float*>(q_rope)[off]);
      q_abs[((size_t)(r0 + r) * H + h) * row_w + dC + d] = b;
    }
  }
}

// ---- value up-projection ------------------------------------------------------------------------
// grid (H, ceil(rows/8)), Dh threads.  o_lat [rows][H][dC] f32, W_UV [dC][H*Dh] bf16, out [rows][H][Dh] f32.
__global__ void mla_vup_kernel(const float* __restrict__ o_lat, const uint16_t* __restrict__ W_UV, float* __restrict__ out, int rows,
                               int H, int Dh, int dC) {
  extern __shared__ float os[];  // [8][dC]
  const int h = blockIdx.x, r0 = blockIdx.y * 8, d = threadIdx.x;
  for (int e = threadIdx.x; e < 8 * dC; e += blockDim.x) {
    const int r = e / dC, c = e % dC;
    os[e] = (r0 + r < rows) ? o_lat[((size_t)(r0 + r) * H + h) * dC + c] : 0.f;
  }
  __syncthreads();
  if (d >= Dh) return;
  float acc[8];
#pragma unroll
  for (int r = 0; r < 8; r++) acc[r] = 0.f;
  for (int c = 0; c < dC; c++) {
    const float w = f32_from_bf16_bits(W_UV[(size_t)c * H * Dh + (size_t)h * Dh + d]);
#pragma unroll
    for (int r = 0; r < 8; r++) acc[r] += os[r * dC + c] * w;
  }
#pragma unroll
  for (int r = 0; r < 8; r++)
    if (r0 + r < rows) out[((size_t)(r0 + r) * H + h) * Dh + d] = acc[r];
}

// ---- shape-generic split-KV decode on CUDA cores ---------------------------------------------------
// grid (items, ceil(S*H / kRowsPerCta)); 8 warps, each warp owns kRpw query rows (a row = one (token, head)).
// Per 32-token tile: the tile is staged in shared memory; lane = token for the scores, lane = latent slice
// for P*C.  Meant for shapes the tensor-core kernel does not cover (small models), not for speed.
struct MlaGenParams {
  const WorkItem* items;
  const int32_t* table;
  int32_t table_stride;
  const int32_t* len;
  int32_t num_pages, page_tokens, H, S, extra, causal, dHR, blocked;
  const uint16_t* base;
  const uint16_t* q_abs;
  float scale_log2;
  float* part_o;
  float* part_ml;
  int32_t rows_total;
  int32_t* status;
};

template <int DC, int kRpw>
__global__ void __launch_bounds__(256) mla_decode_generic_kernel(const MlaGenParams prm) {
  constexpr int kTile = 32, kWarps = 8, kRows = kWarps * kRpw, kPerLane = DC / 32;
  extern __shared__ uint32_t smw[];
  const int roww = DC + prm.dHR;       // elements per cache row
  const int stride_w = roww / 2 + 1;   // 32-bit words per staged row, odd -> conflict-free column walks
  uint32_t* tile = smw;                              // [kTile][stride_w]
  uint32_t* qsm = smw + kTile * stride_w;            // [kRows][roww/2]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WorkItem item = prm.items[blockIdx.x];
  const int T = prm.len[item.seq] + prm.extra;
  const int row_base = blockIdx.y * kRows;
  for (int e = threadIdx.x; e < kRows * (roww / 2); e += blockDim.x) {
    const int r = e / (roww / 2), w = e % (roww / 2);
    const int grow = row_base + r;
    qsm[e] = (grow < prm.rows_total)
                 ? reinterpret_cast<const uint32_t*>(prm.q_abs + ((size_t)item.seq_index * prm.rows_total + grow) * roww)[w]
                 : 0u;
  }
  float o[kRpw][kPerLane];
  float m_run[kRpw], l_run[kRpw];
#pragma unroll
  for (int r = 0; r < kRpw; r++) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; i++) o[r][i] = 0.f;
  }
  const int tok_begin = item.page_begin * prm.page_tokens;
  const int tok_end = min(T, item.page_end * prm.page_tokens);
  for (int t0 = tok_begin; t0 < tok_end; t0 += kTile) {
    __syncthreads();
    // stage kTile rows (16-byte global loads, 4-byte shared stores)
    const int vec_per_row = roww / 8;
    for (int e = threadIdx.x; e < kTile * vec_per_row; e += blockDim.x) {
      const int r = e / vec_per_row, v = e % vec_per_row;
      const int tok = t0 + r;
      uint4 x = make_uint4(0, 0, 0, 0);
      if (tok < tok_end) {
        int32_t pg;
        if (page_of(prm.table, prm.table_stride, item.seq, tok / prm.page_tokens, prm.num_pages, prm.status, &pg))
          x = *reinterpret_cast<const uint4*>(prm.base + (size_t)pg * prm.page_tokens * roww +
                                              mla_page_off(prm.blocked != 0, prm.page_tokens, roww, tok % prm.page_tokens, v * 8));
      }
      uint32_t* dst = tile + r * stride_w + v * 4;
      dst[0] = x.x; dst[1] = x.y; dst[2] = x.z; dst[3] = x.w;
    }
    __syncthreads();
    const int tok = t0 + lane;
#pragma unroll
    for (int r = 0; r < kRpw; r++) {
      const int lrow = warp * kRpw + r, grow = row_base + lrow;
      if (grow >= prm.rows_total) continue;
      const uint32_t* qrow = qsm + lrow * (roww / 2);
      const uint32_t* krow = tile + lane * stride_w;
      float acc = 0.f;
      for (int w = 0; w < roww / 2; w++) {
        const uint32_t qv = qrow[w], kv = krow[w];
        acc = fmaf(bf16_lo(qv), bf16_lo(kv), acc);
        acc = fmaf(bf16_hi(qv), bf16_hi(kv), acc);
      }
      float s = acc * prm.scale_log2;
      const int srow = grow / prm.H;  // query token index of this row
      const int limit = prm.causal ? (T - prm.S + srow) : (T - 1);
      if (tok >= tok_end || tok > limit) s = -INFINITY;
      const float mx = warp_max(s);
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run[r] - m_use);
      m_run[r] = m_new;
      const float pv = exp2f(s - m_use);
      l_run[r] = l_run[r] * alpha + warp_sum(pv);
#pragma unroll
      for (int i = 0; i < kPerLane; i++) o[r][i] *= alpha;
      // O += p_t * C[t][:]: lane owns latent words lane + 32*i (two values each)
      for (int t = 0; t < kTile; t++) {
        const float pt = __shfl_sync(0xffffffffu, pv, t);
        if (pt == 0.f) continue;
        const uint32_t* crow = tile + t * stride_w;
#pragma unroll
        for (int i = 0; i < kPerLane / 2; i++) {
          const uint32_t cv = crow[lane + 32 * i];
          o[r][2 * i] = fmaf(pt, bf16_lo(cv), o[r][2 * i]);
          o[r][2 * i + 1] = fmaf(pt, bf16_hi(cv), o[r][2 * i + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRpw; r++) {
    const int grow = row_base + warp * kRpw + r;
    if (grow >= prm.rows_total) continue;
    const size_t prow = (size_t)blockIdx.x * prm.rows_total + grow;
#pragma unroll
    for (int i = 0; i < kPerLane / 2; i++) {
      float2 v = make_float2(o[r][2 * i], o[r][2 * i + 1]);
      *reinterpret_cast<float2*>(prm.part_o + prow * DC + 2 * (lane + 32 * i)) = v;
    }
    if (lane == 0) {
      prm.part_ml[prow * 2] = m_run[r];
      prm.part_ml[prow * 2 + 1] = l_run[r];
    }
  }
}

template <int DC>
int32_t launch_generic(Pool* p, const MlaGenParams& k, int items, cudaStream_t st) {
  constexpr int kRpw = (DC >= 512) ? 2 : 4;
  constexpr int kRows = 8 * kRpw;
  const int roww = DC + k.dHR;
  const size_t smem = ((size_t)32 * (roww / 2 + 1) + (size_t)kRows * (roww / 2)) * 4;
  auto kern = mla_decode_generic_kernel<DC, kRpw>;
  if (smem > 48 * 1024) RELUX_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(items, (k.rows_total + kRows - 1) / kRows);
  kern<<<grid, 256, smem, st>>>(k);
  RELUX_CUDA_TRY(cudaGetLastError());
  return RELUX_OK;
}

}  // namespace

bool mla_step_fusable(Pool* p, const relux_attn_args& a, int n_seqs) {
  const relux_pool_params& prm = p->prm;
  return !p->compat && a.mode == RELUX_ATTN_FAST && a.extra_tokens == 0 && mla_sm100_eligible(p, a) &&
         mla_proj_mma_eligible(a.head_dim, prm.mla_dc) && mla_prep_fits(n_seqs, a.num_heads, prm.mla_dc);
}

int32_t launch_mla_decode_fast(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const void* d_q, const void* d_qr,
                               void* d_out, const StepAppend* step) {
  const relux_pool_params& prm = p->prm;
  const int H = a.num_heads, Dh = a.head_dim, dC = prm.mla_dc, dHR = prm.mla_dhr, S = a.q_tokens;
  const int rows = sb.n_seqs * S, rows_total = S * H, roww = dC + dHR;
  if (!(dC == 64 || dC == 128 || dC == 256 || dC == 512)) {
    set_error("MLA FAST kernels cover dC in {64,128,256,512} (got %d); use RELUX_ATTN_REFERENCE", dC);
    return RELUX_ERR_UNSUPPORTED;
  }
  // a prompt: expand the cached latents into per-head keys / values once, then ordinary attention on the prefill kernel
  if (!step && a.q_dtype == RELUX_DTYPE_BF16 && mla_prefill_eligible(p, sb, a))
    return launch_mla_prefill_sm100(p, sb, a, (const uint16_t*)d_q, (const uint16_t*)d_qr, (float*)d_out);
  cudaStream_t st = p->dev->stream;
  int32_t rc = grow(p->dev, p->q_abs, (size_t)rows * H * roww * 2);
  if (rc) return rc;
  const bool sm100 = mla_sm100_eligible(p, a);
  SplitPlan plan;
  // The stream partition depends on the cached lengths only, the absorb on the queries only: the one-block builder
  // runs on the side stream next to the absorb kernel and is joined before the decode kernel.
  cudaStream_t side = p->dev->side_stream;
  const bool fused_prep = step != nullptr;   // the caller checked mla_step_fusable
  const bool fork = sm100 && side != nullptr && !fused_prep;
  if (fused_prep) {
    // one launch: absorb + the step's append + the stream partition (the host lengths already count the new rows)
    rc = plan_stream(p, sb, a.layer, a.extra_tokens, mla_sm100_workers(p, S), 2, &plan, st, false);
    if (rc) return rc;
    PrepAppend ap;
    ap.table = p->d_table;
    ap.table_stride = prm.max_pages_per_seq;
    ap.len = p->d_len + (size_t)a.layer * prm.max_seqs;
    ap.seq_ids = sb.d_seq_ids;
    ap.row_off = step->d_row_off;
    ap.num_pages = prm.num_pages;
    ap.page_tokens = prm.page_tokens;
    ap.max_pages_per_seq = prm.max_pages_per_seq;
    ap.n_seqs = sb.n_seqs;
    ap.status = p->d_status;
    ap.done = reinterpret_cast<uint32_t*>(p->d_status + 1);
    ap.layer_base = p->storage + (size_t)a.layer * p->layer_elems;
    ap.ckv = step->ckv;
    ap.kr = step->kr;
    ap.f32 = step->dtype == RELUX_DTYPE_F32;
    ap.dC = dC;
    ap.dHR = dHR;
    ap.blocked = p->mla_blocked ? 1 : 0;
    PrepPlan pl;
    pl.extra = a.extra_tokens;
    pl.G = plan.chunk_pages;
    pl.workers = plan.num_workers;
    pl.items = plan.stream_items;
    pl.chunk_off = plan.chunk_off;
    pl.worker_first = plan.worker_first;
    rc = launch_mla_prep(p->dev, d_q, d_qr, a.q_dtype == RELUX_DTYPE_BF16, (const uint16_t*)a.w_uk, (uint16_t*)p->q_abs.p, rows, H, dC, dHR, ap,
                         pl, p->tune.get(RELUX_TUNE_CHAINED_LAUNCHES) != 0);
    if (rc) return rc;
  }
  if (fork) {
    RELUX_CUDA_TRY(cudaEventRecord(p->dev->ev_fork, st));
    RELUX_CUDA_TRY(cudaStreamWaitEvent(side, p->dev->ev_fork, 0));
    rc = plan_stream(p, sb, a.layer, a.extra_tokens, mla_sm100_workers(p, S), 2, &plan, side);
    if (rc) return rc;
    RELUX_CUDA_TRY(cudaEventRecord(p->dev->ev_join, side));
  }
  const bool proj_mma = mla_proj_mma_eligible(Dh, dC);
  if (fused_prep) {
    // absorbed queries, appended rows and the partition are already queued
  } else if (proj_mma) {
    rc = launch_mla_absorb_mma(p->dev, d_q, d_qr, a.q_dtype == RELUX_DTYPE_BF16, (const uint16_t*)a.w_uk, (uint16_t*)p->q_abs.p, rows, H, dC,
                               dHR);
    if (rc) return rc;
  } else {
    dim3 grid(H, (dC + 63) / 64, (rows + 15) / 16);
    size_t smem = ((size_t)64 * (Dh + 1) + (size_t)16 * Dh) * 4;
    if (smem > 48 * 1024) RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_absorb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mla_absorb_kernel<<<grid, 256, smem, st>>>(d_q, d_qr, a.q_dtype == RELUX_DTYPE_BF16, (const uint16_t*)a.w_uk, (uint16_t*)p->q_abs.p,
                                               rows, H, Dh, dC, dHR);
    RELUX_CUDA_TRY(cudaGetLastError());
    count_launch(p->dev);
  }
  if (fused_prep) {
  } else if (fork)
    RELUX_CUDA_TRY(cudaStreamWaitEvent(st, p->dev->ev_join, 0));
  else if (sm100)   // persistent CTA pairs over a stream partition; ranges are whole 128-token tiles
    rc = plan_stream(p, sb, a.layer, a.extra_tokens, mla_sm100_workers(p, S), 2, &plan, st);
  else
    rc = plan_splitkv(p, sb, a.layer, a.extra_tokens, std::max(1, rows_total / 16), 1, 1, 0, &plan);
  if (rc) return rc;
  rc = grow(p->dev, p->part_o, (size_t)plan.num_items * rows_total * dC * sizeof(float));
  if (rc) return rc;
  rc = grow(p->dev, p->part_ml, (size_t)plan.num_items * rows_total * 2 * sizeof(float));
  if (rc) return rc;
  const bool fused_merge = proj_mma && dC <= 512;
  if (!fused_merge) {   // the unfused paths hand the merged latent output to the up-projection through this buffer
    rc = grow(p->dev, p->o_lat, (size_t)rows * H * dC * sizeof(float));
    if (rc) return rc;
  }
  // the event pair around the decode kernel: on every call, or on every Nth (the records are not free: they sit
  // between this launch and its neighbours)
  const int stride = std::max(1, p->tune.get(RELUX_TUNE_KERNEL_TIMING_STRIDE));
  const bool timed = (p->attn_calls++ % (uint64_t)stride) == 0;
  if (timed) RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), st));
  if (sm100) {
    rc = launch_mla_decode_sm100(p, sb, a, plan, (const uint16_t*)p->q_abs.p);
    if (rc) return rc;
  } else {
    MlaGenParams k;
    k.items = plan.items;
    k.table = p->d_table;
    k.table_stride = prm.max_pages_per_seq;
    k.len = p->d_len + (size_t)a.layer * prm.max_seqs;
    k.num_pages = prm.num_pages;
    k.page_tokens = prm.page_tokens;
    k.H = H;
    k.S = S;
    k.extra = a.extra_tokens;
    k.causal = a.causal;
    k.dHR = dHR;
    k.blocked = p->mla_blocked ? 1 : 0;
    k.base = p->storage + (size_t)a.layer * p->layer_elems;
    k.q_abs = (const uint16_t*)p->q_abs.p;
    k.scale_log2 = a.scale * 1.4426950408889634f;
    k.part_o = (float*)p->part_o.p;
    k.part_ml = (float*)p->part_ml.p;
    k.rows_total = rows_total;
    k.status = p->d_status;
    switch (dC) {
      case 64: rc = launch_generic<64>(p, k, plan.num_items, st); break;
      case 128: rc = launch_generic<128>(p, k, plan.num_items, st); break;
      case 256: rc = launch_generic<256>(p, k, plan.num_items, st); break;
      default: rc = launch_generic<512>(p, k, plan.num_items, st); break;
    }
    if (rc) return rc;
  }
  if (timed) {
    RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), st));
    p->timed_calls++;
  }
  count_launch(p->dev);
  if (fused_merge) {
    // split-KV merge fused into the up-projection: the merged latent output never touches HBM
    rc = launch_mla_merge_vup_mma(p->dev, (const float*)p->part_o.p, (const float*)p->part_ml.p, plan.chunk_off, (const uint16_t*)a.w_uv,
                                  (float*)d_out, rows, S, H, dC, p->d_status, p->tune.get(RELUX_TUNE_CHAINED_LAUNCHES) != 0);
    if (rc) return rc;
  } else if (proj_mma) {
    // merged latent output goes to the up-projection as bf16 (tensor-core operand)
    rc = launch_merge(p, plan, sb.n_seqs, rows_total, dC, nullptr, (uint16_t*)p->o_lat.p);
    if (rc) return rc;
    rc = launch_mla_vup_mma(p->dev, (const uint16_t*)p->o_lat.p, (const uint16_t*)a.w_uv, (float*)d_out, rows, H, dC);
    if (rc) return rc;
  } else {
    rc = launch_merge(p, plan, sb.n_seqs, rows_total, dC, (float*)p->o_lat.p, nullptr);
    if (rc) return rc;
    dim3 grid(H, (rows + 7) / 8);
    size_t smem = (size_t)8 * dC * 4;
    int threads = ((Dh + 31) / 32) * 32;
    mla_vup_kernel<<<grid, threads, smem, st>>>((const float*)p->o_lat.p, (const uint16_t*)a.w_uv, (float*)d_out, rows, H, Dh, dC);
    RELUX_CUDA_TRY(cudaGetLastError());
    count_launch(p->dev);
  }
  return RELUX_OK;
}

}  // namespace relux
