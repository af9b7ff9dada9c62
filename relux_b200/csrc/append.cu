// Cache-append, length bookkeeping, row gather and activation layout kernels.
//
// Append is pure byte movement (HBM-write bound, a few KB per step): each thread moves one
// 16-byte bf16 vector (8 elements) so every row segment is written with coalesced 16-byte
// stores.  float32 inputs are rounded with the reference's own rule (dtype_convert.go:15-24).
#include "common.cuh"
#include "internal.h"

namespace relux {

// 8 consecutive source elements -> one uint4 of bf16 bits.
template <bool kF32>
__device__ __forceinline__ uint4 load8_as_bf16(const void* src, size_t elem_off) {
  if constexpr (kF32) {
    const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + elem_off);
    float4 a = s[0], b = s[1];
    return make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
  } else {
    return *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(src) + elem_off);
  }
}

struct AppendGeom {
  const int32_t* table;
  int32_t table_stride;
  int32_t* len;        // this layer's [max_seqs]
  const int32_t* seq_ids;
  const int32_t* row_off;
  int32_t num_pages, page_tokens, max_pages_per_seq;
  int32_t* status;
  int32_t advance;
  uint32_t* done;      // zero between launches; counts finished blocks of the running append
};

// Length bookkeeping fused into the append: every block reads its sequence's length before it arrives here, so the
// last block to arrive may advance all lengths (and re-arm the counter for the next launch).  grid.x = n_seqs.
__device__ __forceinline__ void advance_lengths_by_last_block(const AppendGeom& g) {
  if (!g.advance) return;
  __shared__ bool s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(g.done, 1u) == gridDim.x * gridDim.y - 1;
  }
  __syncthreads();
  if (!s_last) return;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
    const int seq = g.seq_ids ? g.seq_ids[i] : i;
    g.len[seq] += g.row_off ? g.row_off[i + 1] - g.row_off[i] : 1;
  }
  if (threadIdx.x == 0) *g.done = 0u;
}

// grid (n_seqs, row_slices).  One sequence's new rows are spread over blockIdx.y.
// MLA row = [dC | dHR] fused, dC and dHR multiples of 8.
// `shadow` (reference-compat pools only, else null): this layer's float32 copy of the rows, [page][token][dC + dHR] -- the
// reference's MLA cache holds float32 (mla_cache.go:46-52, 171-176).
template <bool kF32>
__global__ void mla_append_kernel(AppendGeom g, uint16_t* __restrict__ layer_base, const void* __restrict__ ckv,
                                  const void* __restrict__ kr, int dC, int dHR, int blocked, float* __restrict__ shadow) {
  const int i = blockIdx.x;
  const int seq = g.seq_ids ? g.seq_ids[i] : i;
  const int r0 = g.row_off ? g.row_off[i] : i;
  const int nrows = g.row_off ? g.row_off[i + 1] - r0 : 1;
  const int base_len = g.len[seq];
  const int row_elems = dC + dHR, vec_per_row = row_elems / 8, vc = dC / 8;
  for (int r = blockIdx.y; r < nrows; r += gridDim.y) {
    const int pos = base_len + r;
    const int slot = pos / g.page_tokens;
    int32_t pg;
    if (slot >= g.max_pages_per_seq || !page_of(g.table, g.table_stride, seq, slot, g.num_pages, g.status, &pg)) {
      if (slot >= g.max_pages_per_seq) set_status(g.status, RELUX_ERR_OVERFLOW);
      continue;
    }
    uint16_t* page = layer_base + (size_t)pg * g.page_tokens * row_elems;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      uint4 w = (v < vc) ? load8_as_bf16<kF32>(ckv, (size_t)(r0 + r) * dC + (size_t)v * 8)
                         : load8_as_bf16<kF32>(kr, (size_t)(r0 + r) * dHR + (size_t)(v - vc) * 8);
      *reinterpret_cast<uint4*>(page + mla_page_off(blocked != 0, g.page_tokens, row_elems, pos % g.page_tokens, v * 8)) = w;
      if (shadow) {
        float* srow = shadow + ((size_t)pg * g.page_tokens + pos % g.page_tokens) * row_elems + v * 8;
        const void* sp = (v < vc) ? ckv : kr;
        const size_t so = (v < vc) ? (size_t)(r0 + r) * dC + (size_t)v * 8 : (size_t)(r0 + r) * dHR + (size_t)(v - vc) * 8;
#pragma unroll
        for (int e = 0; e < 8; e++)
          srow[e] = kF32 ? reinterpret_cast<const float*>(sp)[so + e] : f32_from_bf16_bits(reinterpret_cast<const uint16_t*>(sp)[so + e]);
      }
    }
  }
  advance_lengths_by_last_block(g);
}

// GQA: source rows K,V [tok][Hkv][D] (token-major) or [Hkv][n_new][D] per sequence (head-major);
// destination pages [Hkv][page_tokens][D], K block then V block per layer.
template <bool kF32>
__global__ void gqa_append_kernel(AppendGeom g, uint16_t* __restrict__ k_base, uint16_t* __restrict__ v_base,
                                  const void* __restrict__ ksrc, const void* __restrict__ vsrc, int Hkv, int D, int head_major) {
  const int i = blockIdx.x;
  const int seq = g.seq_ids ? g.seq_ids[i] : i;
  const int r0 = g.row_off ? g.row_off[i] : i;
  const int nrows = g.row_off ? g.row_off[i + 1] - r0 : 1;
  const int base_len = g.len[seq];
  const int vec_per_head = D / 8, vec_per_tok = Hkv * vec_per_head;
  for (int r = blockIdx.y; r < nrows; r += gridDim.y) {
    const int pos = base_len + r;
    const int slot = pos / g.page_tokens;
    int32_t pg;
    if (slot >= g.max_pages_per_seq || !page_of(g.table, g.table_stride, seq, slot, g.num_pages, g.status, &pg)) {
      if (slot >= g.max_pages_per_seq) set_status(g.status, RELUX_ERR_OVERFLOW);
      continue;
    }
    const size_t page_off = (size_t)pg * Hkv * g.page_tokens * D;
    for (int v = threadIdx.x; v < 2 * vec_per_tok; v += blockDim.x) {
      const int which = v / vec_per_tok, vv = v % vec_per_tok;
      const int h = vv / vec_per_head, c = vv % vec_per_head;
      const size_t src_off = head_major ? ((size_t)r0 * Hkv * D + ((size_t)h * nrows + r) * D + (size_t)c * 8)
                                        : (((size_t)(r0 + r) * Hkv + h) * D + (size_t)c * 8);
      uint4 w = load8_as_bf16<kF32>(which ? vsrc : ksrc, src_off);
      uint16_t* dst = (which ? v_base : k_base) + page_off + ((size_t)h * g.page_tokens + (pos % g.page_tokens)) * D + (size_t)c * 8;
      *reinterpret_cast<uint4*>(dst) = w;
    }
  }
  advance_lengths_by_last_block(g);
}

__global__ void set_len_kernel(int32_t* len, const int32_t* seq_ids, const int32_t* new_len, int n_seqs) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_seqs) return;
  len[seq_ids ? seq_ids[i] : i] = new_len[i];
}

static AppendGeom make_geom(Pool* p, const SeqBatch& sb, int layer, int advance) {
  AppendGeom g;
  g.table = p->d_table;
  g.table_stride = p->prm.max_pages_per_seq;
  g.len = p->d_len + (size_t)layer * p->prm.max_seqs;
  g.seq_ids = sb.d_seq_ids;
  g.row_off = sb.d_row_off;
  g.num_pages = p->prm.num_pages;
  g.page_tokens = p->prm.page_tokens;
  g.max_pages_per_seq = p->prm.max_pages_per_seq;
  g.status = p->d_status;
  g.advance = advance;
  g.done = reinterpret_cast<uint32_t*>(p->d_status + 1);
  return g;
}

static int32_t finish_append(Pool* p) {
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

int32_t launch_mla_append(Pool* p, const SeqBatch& sb, int layer, const void* ckv, const void* kr, int dtype, int advance) {
  AppendGeom g = make_geom(p, sb, layer, advance);
  uint16_t* base = p->storage + (size_t)layer * p->layer_elems;
  dim3 grid(sb.n_seqs, std::min(std::max(sb.max_rows, 1), 64));
  int threads = 96;  // 72 vectors per 576-element row
  float* shadow = p->shadow_f32 ? p->shadow_f32 + (size_t)layer * p->layer_elems : nullptr;
  if (dtype == RELUX_DTYPE_F32)
    mla_append_kernel<true><<<grid, threads, 0, p->dev->stream>>>(g, base, ckv, kr, p->prm.mla_dc, p->prm.mla_dhr, p->mla_blocked, shadow);
  else
    mla_append_kernel<false><<<grid, threads, 0, p->dev->stream>>>(g, base, ckv, kr, p->prm.mla_dc, p->prm.mla_dhr, p->mla_blocked, shadow);
  return finish_append(p);
}

int32_t launch_gqa_append(Pool* p, const SeqBatch& sb, int layer, const void* k, const void* v, int dtype, int layout,
                          int advance) {
  AppendGeom g = make_geom(p, sb, layer, advance);
  uint16_t* kb = p->storage + (size_t)layer * p->layer_elems;
  uint16_t* vb = kb + p->page_elems * p->prm.num_pages;
  dim3 grid(sb.n_seqs, std::min(std::max(sb.max_rows, 1), 64));
  int threads = 256;
  int hm = layout == RELUX_LAYOUT_HEAD_MAJOR;
  if (dtype == RELUX_DTYPE_F32)
    gqa_append_kernel<true><<<grid, threads, 0, p->dev->stream>>>(g, kb, vb, k, v, p->prm.gqa_num_kv_heads, p->prm.gqa_head_dim, hm);
  else
    gqa_append_kernel<false><<<grid, threads, 0, p->dev->stream>>>(g, kb, vb, k, v, p->prm.gqa_num_kv_heads, p->prm.gqa_head_dim, hm);
  return finish_append(p);
}

int32_t launch_set_len(Pool* p, const SeqBatch& sb, int layer, const int32_t* d_new_len) {
  int32_t* len = p->d_len + (size_t)layer * p->prm.max_seqs;
  set_len_kernel<<<(sb.n_seqs + 127) / 128, 128, 0, p->dev->stream>>>(len, sb.d_seq_ids, d_new_len, sb.n_seqs);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

// Logical rows [tok0, tok0+n) of one sequence -> dense buffers (the View of the reference caches).
__global__ void gather_rows_kernel(const uint16_t* __restrict__ layer_base, const int32_t* __restrict__ table, int table_stride,
                                   int seq, int tok0, int n, int num_pages, int page_tokens, int kind, int dC, int dHR, int Hkv, int D,
                                   size_t v_off, uint16_t* __restrict__ da, uint16_t* __restrict__ db, int32_t* status, int blocked) {
  const int r = blockIdx.x;
  if (r >= n) return;
  const int pos = tok0 + r;
  int32_t pg;
  if (!page_of(table, table_stride, seq, pos / page_tokens, num_pages, status, &pg)) return;
  const int in_pg = pos % page_tokens;
  if (kind == RELUX_POOL_MLA) {
    const uint16_t* page = layer_base + (size_t)pg * page_tokens * (dC + dHR);
    for (int e = threadIdx.x; e < dC + dHR; e += blockDim.x) {
      const uint16_t x = page[mla_page_off(blocked != 0, page_tokens, dC + dHR, in_pg, e)];
      if (e < dC) da[(size_t)r * dC + e] = x;
      else db[(size_t)r * dHR + (e - dC)] = x;
    }
  } else {
    for (int e = threadIdx.x; e < Hkv * D; e += blockDim.x) {
      const int h = e / D, d = e % D;
      const size_t off = (size_t)pg * Hkv * page_tokens * D + ((size_t)h * page_tokens + in_pg) * D + d;
      da[(size_t)r * Hkv * D + e] = layer_base[off];
      db[(size_t)r * Hkv * D + e] = layer_base[v_off + off];
    }
  }
}

int32_t launch_gather_rows(Pool* p, int layer, int seq, int tok0, int n, uint16_t* d_a, uint16_t* d_b) {
  const relux_pool_params& prm = p->prm;
  const uint16_t* base = p->storage + (size_t)layer * p->layer_elems;
  gather_rows_kernel<<<n, 128, 0, p->dev->stream>>>(base, p->d_table, prm.max_pages_per_seq, seq, tok0, n, prm.num_pages,
                                                    prm.page_tokens, prm.kind, prm.mla_dc, prm.mla_dhr, prm.gqa_num_kv_heads,
                                                    prm.gqa_head_dim, p->page_elems * prm.num_pages, d_a, d_b, p->d_status, p->mla_blocked);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

// Activation relayout / dtype conversion: [n][S][H][D] <-> [n][H][S][D], f32 <-> bf16.
__global__ void convert_layout_kernel(const void* __restrict__ src, void* __restrict__ dst, int S, int H, int D, int src_bf16,
                                      int dst_bf16, int src_hm, int dst_hm, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    // i indexes the canonical token-major order
    const int d = (int)(i % D);
    size_t t = i / D;
    const int h = (int)(t % H);
    t /= H;
    const int s = (int)(t % S);
    const size_t b = t / S;
    const size_t hm = ((b * H + h) * S + s) * D + d;
    const size_t si = src_hm ? hm : i, di = dst_hm ? hm : i;
    float v = src_bf16 ? f32_from_bf16_bits(reinterpret_cast<const uint16_t*>(src)[si]) : reinterpret_cast<const float*>(src)[si];
    if (dst_bf16) reinterpret_cast<uint16_t*>(dst)[di] = src_bf16 ? reinterpret_cast<const uint16_t*>(src)[si] : bf16_bits_from_f32(v);
    else reinterpret_cast<float*>(dst)[di] = v;
  }
}

int32_t convert_layout(Device* dev, const void* src, void* dst, int n, int S, int H, int D, int src_dtype, int dst_dtype,
                       int src_layout, int dst_layout) {
  size_t total = (size_t)n * S * H * D;
  if (total == 0) return RELUX_OK;
  int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 8);
  convert_layout_kernel<<<blocks, 256, 0, dev->stream>>>(src, dst, S, H, D, src_dtype == RELUX_DTYPE_BF16, dst_dtype == RELUX_DTYPE_BF16,
                                                         src_layout == RELUX_LAYOUT_HEAD_MAJOR && S > 1,
                                                         dst_layout == RELUX_LAYOUT_HEAD_MAJOR && S > 1, total);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(dev);
  return RELUX_OK;
}

}  // namespace relux
