// Split-KV scheduling shared by the FAST attention kernels.
//
// A sequence's cached rows are cut into chunks of `chunk_pages` pages; every (sequence, chunk)
// is one work item handled by one CTA (or CTA pair), so a handful of long sequences still fills
// all SMs.  The list is built on the device from the device-resident lengths; the host computes
// only the item COUNT from its shadow lengths, so no host->device copy is needed per step.
#include <cstdlib>
#include "common.cuh"
#include "internal.h"
#include "splitkv.h"

namespace relux {

__global__ void build_worklist_kernel(const int32_t* __restrict__ len, const int32_t* __restrict__ seq_ids, int n_seqs, int extra,
                                      int page_tokens, int chunk_pages, WorkItem* __restrict__ items, int32_t* __restrict__ chunk_off) {
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < n_seqs; i++) {
      chunk_off[i] = acc;
      int seq = seq_ids ? seq_ids[i] : i;
      int T = len[seq] + extra;
      int pages = (T + page_tokens - 1) / page_tokens;
      acc += (pages + chunk_pages - 1) / chunk_pages;
    }
    chunk_off[n_seqs] = acc;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_seqs; i += blockDim.x) {
    int seq = seq_ids ? seq_ids[i] : i;
    int T = len[seq] + extra;
    int pages = (T + page_tokens - 1) / page_tokens;
    int c0 = chunk_off[i], nc = chunk_off[i + 1] - c0;
    for (int c = 0; c < nc; c++) {
      WorkItem w;
      w.seq_index = i;
      w.seq = seq;
      w.page_begin = c * chunk_pages;
      w.page_end = min(pages, (c + 1) * chunk_pages);
      items[c0 + c] = w;
    }
  }
}

int32_t plan_splitkv(Pool* p, const SeqBatch& sb, int layer, int extra, int ctas_per_item, int min_chunk_pages, int chunk_multiple,
                     int max_chunk_pages, SplitPlan* plan) {
  const relux_pool_params& prm = p->prm;
  long total_pages = 0;
  int max_pages = 0;
  for (int i = 0; i < sb.n_seqs; i++) {
    int T = p->h_len[(size_t)layer * prm.max_seqs + sb.seq[i]] + extra;
    int pages = (T + prm.page_tokens - 1) / prm.page_tokens;
    total_pages += pages;
    max_pages = std::max(max_pages, pages);
  }
  long target_items = std::max(1L, 4L * p->dev->sm_count / std::max(1, ctas_per_item));
  int chunk = (int)((total_pages + target_items - 1) / target_items);
  chunk = std::max(chunk, min_chunk_pages);
  chunk = std::max(1, std::min(chunk, std::max(1, max_pages)));
  if (const char* ov = getenv("RELUX_CHUNK_PAGES")) chunk = std::max(1, atoi(ov));  // tuning aid
  chunk = (chunk + chunk_multiple - 1) / chunk_multiple * chunk_multiple;
  if (max_chunk_pages > 0) chunk = std::min(chunk, max_chunk_pages / chunk_multiple * chunk_multiple);
  int items = 0;
  for (int i = 0; i < sb.n_seqs; i++) {
    int T = p->h_len[(size_t)layer * prm.max_seqs + sb.seq[i]] + extra;
    int pages = (T + prm.page_tokens - 1) / prm.page_tokens;
    items += (pages + chunk - 1) / chunk;
  }
  plan->chunk_pages = chunk;
  plan->num_items = items;
  size_t bytes = sizeof(WorkItem) * (size_t)items + sizeof(int32_t) * ((size_t)sb.n_seqs + 1) + 64;
  int32_t rc = grow(p->dev, p->work, bytes);
  if (rc) return rc;
  plan->items = (WorkItem*)p->work.p;
  size_t off = (sizeof(WorkItem) * (size_t)items + 15) & ~(size_t)15;
  plan->chunk_off = (int32_t*)((char*)p->work.p + off);
  const int32_t* len = p->d_len + (size_t)layer * prm.max_seqs;
  build_worklist_kernel<<<1, 256, 0, p->dev->stream>>>(len, sb.d_seq_ids, sb.n_seqs, extra, prm.page_tokens, chunk, plan->items,
                                                       plan->chunk_off);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

// Combines the partial results of every chunk of a sequence:
//   M = max_c m_c,  L = sum_c l_c 2^(m_c - M),  O = sum_c O_c 2^(m_c - M) / L
// part_o [item][rows][width] f32 holds UNNORMALISED accumulators, part_ml [item][rows][2] = (m, l) with m in
// the log2 domain.  grid (rows, n_seqs); out row stride and placement given by the caller.
__global__ void merge_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int32_t* __restrict__ chunk_off, int rows, int width, float* __restrict__ out,
                                    uint16_t* __restrict__ out_bf16) {
  const int r = blockIdx.x, i = blockIdx.y;
  const int c0 = chunk_off[i], c1 = chunk_off[i + 1];
  float M = -INFINITY;
  for (int c = c0; c < c1; c++) M = fmaxf(M, part_ml[((size_t)c * rows + r) * 2]);
  float L = 0.f;
  for (int c = c0; c < c1; c++) {
    const float* ml = part_ml + ((size_t)c * rows + r) * 2;
    L += ml[1] * exp2f(ml[0] - M);
  }
  const float inv = (L > 0.f) ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float acc = 0.f;
    for (int c = c0; c < c1; c++) {
      const float m = part_ml[((size_t)c * rows + r) * 2];
      acc += part_o[((size_t)c * rows + r) * width + d] * exp2f(m - M);
    }
    const size_t o = ((size_t)i * rows + r) * width + d;
    if (out) out[o] = acc * inv;
    if (out_bf16) out_bf16[o] = bf16_bits_from_f32(acc * inv);
  }
}

int32_t launch_merge(Pool* p, const SplitPlan& plan, int n_seqs, int rows, int width, float* out, uint16_t* out_bf16) {
  dim3 grid(rows, n_seqs);
  merge_splits_kernel<<<grid, 128, 0, p->dev->stream>>>((const float*)p->part_o.p, (const float*)p->part_ml.p, plan.chunk_off, rows,
                                                        width, out, out_bf16);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux
