// Split-KV scheduling shared by the FAST attention kernels.
//
// A sequence's cached rows are cut into chunks of `chunk_pages` pages; every (sequence, chunk)
// is one work item handled by one CTA (or CTA pair), so a handful of long sequences still fills
// all SMs.  The list is built on the device from the device-resident lengths; the host computes
// only the item COUNT from its shadow lengths, so no host->device copy is needed per step.
#include <cstdlib>
#include <vector>
#include "common.cuh"
#include "internal.h"
#include "splitkv.h"

namespace relux {

// One block of 256 threads: every thread counts the chunks of its sequences, a block-wide exclusive scan gives the
// offsets, then every thread writes the items of its sequences.
__global__ void build_worklist_kernel(const int32_t* __restrict__ len, const int32_t* __restrict__ seq_ids, int n_seqs, int extra,
                                      int page_tokens, int chunk_pages, WorkItem* __restrict__ items, int32_t* __restrict__ chunk_off) {
  __shared__ int32_t s_warp[8];
  __shared__ int32_t s_base;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i0 = 0; i0 < n_seqs; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    int seq = 0, pages = 0, nc = 0;
    if (i < n_seqs) {
      seq = seq_ids ? seq_ids[i] : i;
      const int T = len[seq] + extra;
      pages = (T + page_tokens - 1) / page_tokens;
      nc = (pages + chunk_pages - 1) / chunk_pages;
    }
    int incl = nc;   // inclusive scan inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int wbase = 0;
    for (int w = 0; w < warp; w++) wbase += s_warp[w];
    const int c0 = s_base + wbase + incl - nc;
    if (i < n_seqs) {
      chunk_off[i] = c0;
      for (int c = 0; c < nc; c++) {
        WorkItem w;
        w.seq_index = i;
        w.seq = seq;
        w.page_begin = c * chunk_pages;
        w.page_end = min(pages, (c + 1) * chunk_pages);
        items[c0 + c] = w;
      }
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) s_base = c0 + nc;   // running total after this batch of sequences
    __syncthreads();
  }
  if (threadIdx.x == 0) chunk_off[n_seqs] = s_base;
}

// Chooses the chunk length.  CTAs are scheduled in waves over the SMs, so the step time is about
//   waves(chunk) * (chunk + overhead),  waves = ceil(items(chunk) * ctas_per_item / sm_count),
// in units of "time to stream one page"; `overhead` stands for the prologue (query load, TMEM set-up) and
// epilogue (partial write + its share of the merge) of one item.  All candidates are evaluated and the
// cheapest wins, which avoids a nearly empty last wave (e.g. 4.3 waves costing 5).
int32_t plan_splitkv(Pool* p, const SeqBatch& sb, int layer, int extra, int ctas_per_item, int min_chunk_pages, int chunk_multiple,
                     int max_chunk_pages, SplitPlan* plan) {
  const relux_pool_params& prm = p->prm;
  std::vector<int> pages(sb.n_seqs);
  int max_pages = 1;
  for (int i = 0; i < sb.n_seqs; i++) {
    int T = p->h_len[(size_t)layer * prm.max_seqs + sb.seq[i]] + extra;
    pages[i] = (T + prm.page_tokens - 1) / prm.page_tokens;
    max_pages = std::max(max_pages, pages[i]);
  }
  const int mult = std::max(1, chunk_multiple);
  int lo = std::max(std::max(1, min_chunk_pages), mult);
  lo = (lo + mult - 1) / mult * mult;
  int hi = (max_pages + mult - 1) / mult * mult;
  if (max_chunk_pages > 0) hi = std::min(hi, max_chunk_pages / mult * mult);
  hi = std::max(hi, lo);
  const double overhead = 6.0;
  const int sms = std::max(1, p->dev->sm_count);
  int chunk = hi;
  double best = 1e300;
  const int step = std::max(mult, (hi - lo) / 512 / mult * mult);
  for (int c = lo; c <= hi; c += step) {
    long items_c = 0;
    for (int i = 0; i < sb.n_seqs; i++) items_c += (pages[i] + c - 1) / c;
    const long waves = (items_c * ctas_per_item + sms - 1) / sms;
    const double cost = (double)waves * (c + overhead);
    if (cost < best - 1e-9 || (cost < best + 1e-9 && c > chunk)) {
      best = cost;
      chunk = c;
    }
  }
  if (const int ov = p->tune.get(RELUX_TUNE_CHUNK_PAGES)) {  // tuning knob
    chunk = std::max(1, ov);
    chunk = (chunk + mult - 1) / mult * mult;
    if (max_chunk_pages > 0) chunk = std::min(chunk, max_chunk_pages / mult * mult);
  }
  int items = 0;
  for (int i = 0; i < sb.n_seqs; i++) items += (pages[i] + chunk - 1) / chunk;
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

// Exclusive prefix sum over the block (blockDim.x = 256); *total receives the block's sum.
__device__ __forceinline__ int block_excl_scan(int v, int32_t* s_warp, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();   // s_warp may still be read from the previous call
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int base = 0, sum = 0;
  for (int w = 0; w < 8; w++) {
    if (w < warp) base += s_warp[w];
    sum += s_warp[w];
  }
  *total = sum;
  return base + incl - v;
}

// Stream partition (see plan_stream): sequence i occupies pages [start_i, start_i + pages_i) of the stream and
// is cut at every multiple of G; items are numbered in stream order, so the items of a sequence and the items of
// a worker are both contiguous.
__global__ void build_stream_kernel(const int32_t* __restrict__ len, const int32_t* __restrict__ seq_ids, int n_seqs, int extra,
                                    int page_tokens, int G, int workers, StreamItem* __restrict__ items, int32_t* __restrict__ chunk_off,
                                    int32_t* __restrict__ worker_first) {
  __shared__ int32_t s_warp[8];
  int page_base = 0, item_base = 0;
  for (int i0 = 0; i0 < n_seqs; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    int seq = 0, pages = 0, tokens = 0;
    if (i < n_seqs) {
      seq = seq_ids ? seq_ids[i] : i;
      tokens = len[seq] + extra;
      pages = (tokens + page_tokens - 1) / page_tokens;
    }
    int tot_pages, tot_items;
    const int start = page_base + block_excl_scan(pages, s_warp, &tot_pages);
    const int w0 = start / G;
    const int nc = pages > 0 ? (start + pages - 1) / G - w0 + 1 : 0;
    const int c0 = item_base + block_excl_scan(nc, s_warp, &tot_items);
    if (i < n_seqs) {
      chunk_off[i] = c0;
      for (int c = 0; c < nc; c++) {
        const int lo = max(start, (w0 + c) * G), hi = min(start + pages, (w0 + c + 1) * G);
        StreamItem w;
        w.seq_index = i;
        w.seq = seq;
        w.page_begin = lo - start;
        w.page_end = hi - start;
        w.tokens = tokens;
        w.pad[0] = w.pad[1] = w.pad[2] = 0;
        items[c0 + c] = w;
        if (lo == (w0 + c) * G) worker_first[w0 + c] = c0 + c;   // the item that holds the first page of a range
      }
    }
    page_base += tot_pages;
    item_base += tot_items;
  }
  if (threadIdx.x == 0) chunk_off[n_seqs] = item_base;
  // ranges past the end of the stream are empty
  for (int w = (page_base + G - 1) / G + threadIdx.x; w <= workers; w += blockDim.x) worker_first[w] = item_base;
}

// Host statement of the stream partition: range length G and the counts that follow from it.  The device builder
// (build_stream_kernel) applies the same arithmetic to the device-resident lengths.
void stream_partition_shape(const int* pages, int n_seqs, int workers, int page_multiple, long chunk_override, long* G_out,
                            int* workers_out, int* items_out) {
  long total = 0;
  for (int i = 0; i < n_seqs; i++) total += pages[i];
  workers = std::max(1, workers);
  const int mult = std::max(1, page_multiple);
  long G = (total + workers - 1) / workers;
  G = std::max<long>((G + mult - 1) / mult * mult, 2L * mult);   // at least two tiles per range
  if (chunk_override > 0) G = std::max<long>(mult, (chunk_override + mult - 1) / mult * mult);
  int items = 0;
  long start = 0;
  for (int i = 0; i < n_seqs; i++) {
    if (pages[i] > 0) items += (int)((start + pages[i] - 1) / G - start / G + 1);
    start += pages[i];
  }
  *G_out = G;
  *workers_out = (int)std::max<long>(1, (total + G - 1) / G);
  *items_out = items;
}

int32_t plan_stream(Pool* p, const SeqBatch& sb, int layer, int extra, int workers, int page_multiple, SplitPlan* plan, cudaStream_t st,
                    bool launch_builder) {
  const relux_pool_params& prm = p->prm;
  std::vector<int> pages(sb.n_seqs);
  for (int i = 0; i < sb.n_seqs; i++) {
    const int T = p->h_len[(size_t)layer * prm.max_seqs + sb.seq[i]] + extra;
    pages[i] = (T + prm.page_tokens - 1) / prm.page_tokens;
  }
  long G = 0;
  int items = 0;
  stream_partition_shape(pages.data(), sb.n_seqs, workers, page_multiple, (long)p->tune.get(RELUX_TUNE_CHUNK_PAGES), &G, &workers, &items);
  plan->chunk_pages = (int)G;
  plan->num_items = items;
  plan->num_workers = workers;
  const size_t off_chunk = sizeof(StreamItem) * (size_t)items;
  const size_t off_worker = (off_chunk + sizeof(int32_t) * ((size_t)sb.n_seqs + 1) + 15) & ~(size_t)15;
  int32_t rc = grow(p->dev, p->work, off_worker + sizeof(int32_t) * ((size_t)workers + 1) + 64);
  if (rc) return rc;
  plan->items = nullptr;
  plan->stream_items = (StreamItem*)p->work.p;
  plan->chunk_off = (int32_t*)((char*)p->work.p + off_chunk);
  plan->worker_first = (int32_t*)((char*)p->work.p + off_worker);
  if (!launch_builder) return RELUX_OK;
  const int32_t* len = p->d_len + (size_t)layer * prm.max_seqs;
  build_stream_kernel<<<1, 256, 0, st>>>(len, sb.d_seq_ids, sb.n_seqs, extra, prm.page_tokens, (int)G, workers,
                                                     plan->stream_items, plan->chunk_off, plan->worker_first);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux

// The stream partition computed on the host from page counts (no device involved): what the persistent MLA decode
// kernel's planner produces for sequences of pages[i] pages.  items_out receives n_items x {seq_index, page_begin,
// page_end, worker}; worker_first [workers_out + 1]; chunk_off [n_seqs + 1].  Returns the number of items, or -1 when
// `cap` items are not enough.  Scheduling aid for callers and tests; no counterpart in the reference.
extern "C" __attribute__((visibility("default"))) int32_t relux_stream_partition(const relux_stream_partition_args* args) {
  if (!args) return -1;
  const int32_t* pages = args->pages;
  const int32_t n_seqs = args->n_seqs, workers = args->workers, page_multiple = args->page_multiple, cap = args->cap;
  int32_t *range_pages_out = args->range_pages_out, *workers_out = args->workers_out, *items_out = args->items_out;
  int32_t *worker_first = args->worker_first, *chunk_off = args->chunk_off;
  if (!pages || n_seqs <= 0 || !range_pages_out || !workers_out) return -1;
  long G = 0;
  int W = 0, items = 0;
  std::vector<int> pg(pages, pages + n_seqs);
  relux::stream_partition_shape(pg.data(), n_seqs, workers, page_multiple, 0, &G, &W, &items);
  *range_pages_out = (int32_t)G;
  *workers_out = W;
  if (items > cap) return -1;
  long start = 0;
  int n = 0;
  if (worker_first)
    for (int w = 0; w <= W; w++) worker_first[w] = items;
  for (int i = 0; i < n_seqs; i++) {
    if (chunk_off) chunk_off[i] = n;
    if (pages[i] > 0) {
      const long w0 = start / G, w1 = (start + pages[i] - 1) / G;
      for (long w = w0; w <= w1; w++) {
        const long lo = std::max(start, w * G), hi = std::min(start + pages[i], (w + 1) * G);
        if (items_out) {
          items_out[4 * n] = i;
          items_out[4 * n + 1] = (int32_t)(lo - start);
          items_out[4 * n + 2] = (int32_t)(hi - start);
          items_out[4 * n + 3] = (int32_t)w;
        }
        if (worker_first && lo == w * G) worker_first[w] = n;
        n++;
      }
    }
    start += pages[i];
  }
  if (chunk_off) chunk_off[n_seqs] = n;
  return n;
}

namespace relux {

// Combines the partial results of every chunk of a sequence:
//   M = max_c m_c,  L = sum_c l_c 2^(m_c - M),  O = sum_c O_c 2^(m_c - M) / L
// part_o [item][rows][width] f32 holds UNNORMALISED accumulators, part_ml [item][rows][2] = (m, l) with m in
// the log2 domain.  grid (rows, n_seqs); out row stride and placement given by the caller.
// The rows of sequence i land at out row i * out_rows + out_row0 + r (out_rows = rows, out_row0 = 0 unless the launch
// covers only some of a call's query tokens).
__global__ void merge_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int32_t* __restrict__ chunk_off, int rows, int width, float* __restrict__ out,
                                    uint16_t* __restrict__ out_bf16, int out_rows, int out_row0, long long part_group_rows) {
  // grid.z > 1: slices of a grouped launch, `rows` output rows and part_group_rows partial rows apart
  const int r = blockIdx.x, i = blockIdx.y;
  out_row0 += (int)blockIdx.z * rows;
  if (out_row0 + r >= out_rows) return;      // the last group of a prompt may be short
  const size_t z0 = (size_t)blockIdx.z * (size_t)part_group_rows;
  const int c0 = chunk_off[i], c1 = chunk_off[i + 1];
  float M = -INFINITY;
  for (int c = c0; c < c1; c++) M = fmaxf(M, part_ml[(z0 + (size_t)c * rows + r) * 2]);
  float L = 0.f;
  for (int c = c0; c < c1; c++) {
    const float* ml = part_ml + (z0 + (size_t)c * rows + r) * 2;
    L += ml[1] * exp2f(ml[0] - M);
  }
  const float inv = (L > 0.f) ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float acc = 0.f;
    for (int c = c0; c < c1; c++) {
      const float m = part_ml[(z0 + (size_t)c * rows + r) * 2];
      acc += part_o[(z0 + (size_t)c * rows + r) * width + d] * exp2f(m - M);
    }
    const size_t o = ((size_t)i * out_rows + out_row0 + r) * width + d;
    if (out) out[o] = acc * inv;
    if (out_bf16) out_bf16[o] = bf16_bits_from_f32(acc * inv);
  }
}

int32_t launch_merge(Pool* p, const SplitPlan& plan, int n_seqs, int rows, int width, float* out, uint16_t* out_bf16) {
  dim3 grid(rows, n_seqs);
  merge_splits_kernel<<<grid, 128, 0, p->dev->stream>>>((const float*)p->part_o.p, (const float*)p->part_ml.p, plan.chunk_off, rows,
                                                        width, out, out_bf16, rows, 0, 0);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

int32_t launch_merge_rows(Pool* p, const SplitPlan& plan, int n_seqs, int rows, int width, float* out, int out_rows, int out_row0,
                          int slices, long long part_group_rows) {
  dim3 grid(rows, n_seqs, slices);
  merge_splits_kernel<<<grid, 128, 0, p->dev->stream>>>((const float*)p->part_o.p, (const float*)p->part_ml.p, plan.chunk_off, rows,
                                                        width, out, nullptr, out_rows, out_row0, part_group_rows);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

// Raw launchers on caller-provided buffers (no pool scratch involved).
int32_t launch_build_worklist_raw(cudaStream_t st, const int32_t* len, const int32_t* seq_ids, int n_seqs, int extra, int page_tokens,
                                  int chunk_pages, WorkItem* items, int32_t* chunk_off) {
  build_worklist_kernel<<<1, 256, 0, st>>>(len, seq_ids, n_seqs, extra, page_tokens, chunk_pages, items, chunk_off);
  RELUX_CUDA_TRY(cudaGetLastError());
  return RELUX_OK;
}
int32_t launch_merge_raw(cudaStream_t st, const float* part_o, const float* part_ml, const int32_t* chunk_off, int n_seqs, int rows,
                         int width, float* out) {
  dim3 grid(rows, n_seqs);
  merge_splits_kernel<<<grid, 128, 0, st>>>(part_o, part_ml, chunk_off, rows, width, out, nullptr, rows, 0, 0);
  RELUX_CUDA_TRY(cudaGetLastError());
  return RELUX_OK;
}

}  // namespace relux
