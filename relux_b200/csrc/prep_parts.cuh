// Device parts of the fused MLA decode-step preparation (one launch instead of three): the append of the step's new
// rows, and the stream partition the persistent decode kernel walks.  They run as extra blocks of the query-absorb grid
// (mla_proj.cu); the stand-alone kernels in append.cu and splitkv.cu do the same work for the unfused calls.
#pragma once

#include "common.cuh"
#include "splitkv.h"

namespace relux {

struct PrepAppend {
  const int32_t* table;
  int32_t table_stride;
  int32_t* len;                // this layer's [max_seqs]
  const int32_t* seq_ids;
  const int32_t* row_off;      // nullptr = one new row per sequence
  int32_t num_pages, page_tokens, max_pages_per_seq, n_seqs;
  int32_t* status;
  uint32_t* done;              // zero between launches; counts the blocks that have finished with the lengths
  uint16_t* layer_base;
  const void* ckv;
  const void* kr;
  int32_t f32, dC, dHR, blocked;
};

struct PrepPlan {
  int32_t extra, G, workers;
  StreamItem* items;
  int32_t* chunk_off;
  int32_t* worker_first;
};

// 8 consecutive source elements -> one uint4 of bf16 bits (float32 sources rounded with the reference's rule).
__device__ __forceinline__ uint4 prep_load8(const void* src, size_t elem_off, bool f32) {
  if (f32) {
    const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + elem_off);
    const float4 a = s[0], b = s[1];
    return make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
  }
  return *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(src) + elem_off);
}

// Every block that reads the lengths arrives here once it is done with them; the last one to arrive advances all
// lengths by the rows appended (MLACache.Append: total += newLen, mla_cache.go:178) and re-arms the counter.
__device__ __forceinline__ void prep_arrive_and_advance(const PrepAppend& g, uint32_t expected) {
  __shared__ bool s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(g.done, 1u) == expected - 1;
  }
  __syncthreads();
  if (!s_last) return;
  for (int i = threadIdx.x; i < g.n_seqs; i += blockDim.x) {
    const int seq = g.seq_ids ? g.seq_ids[i] : i;
    g.len[seq] += g.row_off ? g.row_off[i + 1] - g.row_off[i] : 1;
  }
  if (threadIdx.x == 0) *g.done = 0u;
}

// All new rows of sequence i (MLA row = [dC | dHR] fused; 16-byte stores).
__device__ __forceinline__ void prep_append_seq(const PrepAppend& g, int i) {
  const int seq = g.seq_ids ? g.seq_ids[i] : i;
  const int r0 = g.row_off ? g.row_off[i] : i;
  const int nrows = g.row_off ? g.row_off[i + 1] - r0 : 1;
  const int base_len = g.len[seq];
  const int row_elems = g.dC + g.dHR, vec_per_row = row_elems / 8, vc = g.dC / 8;
  for (int r = 0; r < nrows; r++) {
    const int pos = base_len + r;
    const int slot = pos / g.page_tokens;
    int32_t pg;
    if (slot >= g.max_pages_per_seq || !page_of(g.table, g.table_stride, seq, slot, g.num_pages, g.status, &pg)) {
      if (slot >= g.max_pages_per_seq) set_status(g.status, RELUX_ERR_OVERFLOW);
      continue;
    }
    uint16_t* page = g.layer_base + (size_t)pg * g.page_tokens * row_elems;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      const uint4 w = (v < vc) ? prep_load8(g.ckv, (size_t)(r0 + r) * g.dC + (size_t)v * 8, g.f32 != 0)
                               : prep_load8(g.kr, (size_t)(r0 + r) * g.dHR + (size_t)(v - vc) * 8, g.f32 != 0);
      *reinterpret_cast<uint4*>(page + mla_page_off(g.blocked != 0, g.page_tokens, row_elems, pos % g.page_tokens, v * 8)) = w;
    }
  }
}

// Exclusive prefix sum over a block of up to 1024 threads; *total receives the block's sum.
__device__ __forceinline__ int prep_block_excl_scan(int v, int32_t* s_warp, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
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
  for (int w = 0; w < nw; w++) {
    if (w < warp) base += s_warp[w];
    sum += s_warp[w];
  }
  *total = sum;
  return base + incl - v;
}

// The stream partition over the lengths AFTER this step's append (the append of the same launch has not advanced them
// yet: every sequence counts its cached rows + its new rows + extra).  Same arithmetic as build_stream_kernel.
__device__ __forceinline__ void prep_build_stream(const PrepAppend& g, const PrepPlan& pl) {
  __shared__ int32_t s_warp[32];
  int page_base = 0, item_base = 0;
  for (int i0 = 0; i0 < g.n_seqs; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    int seq = 0, pages = 0, tokens = 0;
    if (i < g.n_seqs) {
      seq = g.seq_ids ? g.seq_ids[i] : i;
      tokens = g.len[seq] + (g.row_off ? g.row_off[i + 1] - g.row_off[i] : 1) + pl.extra;
      pages = (tokens + g.page_tokens - 1) / g.page_tokens;
    }
    int tot_pages, tot_items;
    const int start = page_base + prep_block_excl_scan(pages, s_warp, &tot_pages);
    const int w0 = start / pl.G;
    const int nc = pages > 0 ? (start + pages - 1) / pl.G - w0 + 1 : 0;
    const int c0 = item_base + prep_block_excl_scan(nc, s_warp, &tot_items);
    if (i < g.n_seqs) {
      pl.chunk_off[i] = c0;
      for (int c = 0; c < nc; c++) {
        const int lo = max(start, (w0 + c) * pl.G), hi = min(start + pages, (w0 + c + 1) * pl.G);
        StreamItem w;
        w.seq_index = i;
        w.seq = seq;
        w.page_begin = lo - start;
        w.page_end = hi - start;
        w.tokens = tokens;
        w.pad[0] = w.pad[1] = w.pad[2] = 0;
        pl.items[c0 + c] = w;
        if (lo == (w0 + c) * pl.G) pl.worker_first[w0 + c] = c0 + c;   // the item that holds the first page of a range
      }
    }
    page_base += tot_pages;
    item_base += tot_items;
  }
  if (threadIdx.x == 0) pl.chunk_off[g.n_seqs] = item_base;
  // ranges past the end of the stream are empty
  for (int w = (page_base + pl.G - 1) / pl.G + threadIdx.x; w <= pl.workers; w += blockDim.x) pl.worker_first[w] = item_base;
}

}  // namespace relux
