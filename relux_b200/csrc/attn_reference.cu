// RELUX_ATTN_REFERENCE: cached attention in float32 on CUDA cores with the reference's own
// operation order, so that its results can be compared bit for bit with a CPU restatement:
//   * every dot product is a k-ascending chain of unfused multiply-then-add
//     (internal/transformer/matmul.go:15-44),
//   * scores are scaled, masked with -Inf, then softmaxRows (mha.go:837-861): exact row max,
//     weights fastexp32(v - max) with the < -20 cut-off, j-ascending sum, multiply by 1/sum,
//   * O = P V with j ascending,
//   * MLA decompresses each latent row with W_UK / W_UV first (mla.go:323-326) instead of absorbing.
// One CTA per (head, sequence); the score rows live in shared memory, which bounds q_tokens * T.
// Meant for the small models where greedy token ids are compared, not for speed.
//
// RELUX_ATTN_REFERENCE_FAITHFUL adds the reference's own indexing on top of the same arithmetic:
//   GQA  the cache stream is written chunk by chunk (one chunk per Append, head-major inside the chunk,
//        kvcache.go:407-438) and read as [numKVHeads][T][headDim] (mha.go:299-312): logical (kv head h, position j)
//        is stream row r = h*T + j, which lies in the chunk c with Hkv*P_c <= r < Hkv*P_(c+1) and holds the row that
//        chunk's head (r - Hkv*P_c) / len_c wrote for token P_c + (r - Hkv*P_c) % len_c;
//   MLA  kcAll / vAll are [T][H][headDim] but indexed as [H][T][headDim] (mla.go:323-326 vs :348, 351): logical
//        (head h, position j) reads token (h*T + j) / H with the up-projection columns of head (h*T + j) % H; the
//        rope part is indexed correctly (mla.go:329-336); latent rows are the float32 values that were appended;
//   mask only when q_tokens == T (mha.go:340, mla.go:368).
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "internal.h"

namespace relux {

struct RefGeom {
  const int32_t* table;
  int32_t table_stride;
  const int32_t* len;
  const int32_t* seq_ids;
  int32_t num_pages, page_tokens;
  int32_t* status;
  int32_t S, extra, causal, H;
  float scale;
  int32_t blocked;   // MLA page layout (see mla_page_off)
  // RELUX_ATTN_REFERENCE_FAITHFUL
  int32_t faithful;
  const int32_t* chunk_tab;   // GQA: per sequence of the call [count, P_0 .. P_(count-1)]
  int32_t chunk_stride;
  const float* shadow;        // MLA: float32 rows of this layer, [page][token][dC + dHR]
};

// Masked under the intended rule (row s of the S new rows sees positions <= T - S + s); the reference's own rule applies
// that mask only when the call covers the whole cache (S == T).
__device__ __forceinline__ bool ref_masked(const RefGeom& g, int T, int S, int s, int j) {
  if (!g.causal) return false;
  if (g.faithful && S != T) return false;
  return j > T - S + s;
}

// Shared tail: softmaxRows over w[S][T] and nothing else; all threads of the CTA call it.
__device__ void softmax_rows_ref(float* w, int S, int T, float* red) {
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int s = 0; s < S; s++) {
    float* row = w + (size_t)s * T;
    float m = -INFINITY;
    for (int j = tid; j < T; j += nt) m = fmaxf(m, row[j]);
    m = warp_max(m);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    if (tid < 32) {
      float v = (tid < (nt + 31) / 32) ? red[tid] : -INFINITY;
      v = warp_max(v);
      if (tid == 0) red[0] = v;
    }
    __syncthreads();
    m = red[0];
    __syncthreads();
    for (int j = tid; j < T; j += nt) {
      float diff = __fsub_rn(row[j], m);
      row[j] = (diff < -20.0f) ? 0.0f : fastexp32_ref(diff);
    }
    __syncthreads();
    if (tid == 0) {
      float sum = 0.0f;
      for (int j = 0; j < T; j++) sum = __fadd_rn(sum, row[j]);
      red[0] = __fdiv_rn(1.0f, sum);
    }
    __syncthreads();
    const float inv = red[0];
    for (int j = tid; j < T; j += nt) row[j] = __fmul_rn(row[j], inv);
    __syncthreads();
  }
}

// grid (H, n_seqs).  q, out: [n][S][H][D] f32 token-major.
__global__ void gqa_reference_kernel(RefGeom g, const uint16_t* __restrict__ k_base, const uint16_t* __restrict__ v_base,
                                     const float* __restrict__ q, float* __restrict__ out, int Hkv, int D) {
  extern __shared__ float smem[];
  __shared__ float red[32];
  const int h = blockIdx.x, i = blockIdx.y;
  const int seq = g.seq_ids ? g.seq_ids[i] : i;
  const int T = g.len[seq] + g.extra;
  const int S = g.S, kvh = h / (g.H / Hkv);
  float* w = smem;  // [S][T]
  int32_t* src = reinterpret_cast<int32_t*>(smem + (size_t)S * T);   // [T] physical (kv head << 20 | token) of logical position j
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int j = tid; j < T; j += nt) {
    int ph = kvh, pt = j;
    if (g.faithful) {
      const int32_t* ct = g.chunk_tab + (size_t)i * g.chunk_stride;
      const int nc = ct[0];
      const int r = kvh * T + j;
      int lo = 0, hi = nc - 1;   // last chunk whose first stream row Hkv * P_c is <= r
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (Hkv * ct[1 + mid] <= r) lo = mid; else hi = mid - 1;
      }
      const int P = ct[1 + lo], len = ((lo + 1 < nc) ? ct[2 + lo] : T) - P;
      const int rr = r - Hkv * P;
      ph = rr / len;
      pt = P + rr % len;
    }
    src[j] = (ph << 20) | pt;
  }
  __syncthreads();
  for (int j = tid; j < T; j += nt) {
    const int ph = src[j] >> 20, pt = src[j] & 0xFFFFF;
    int32_t pg;
    bool ok = page_of(g.table, g.table_stride, seq, pt / g.page_tokens, g.num_pages, g.status, &pg);
    const uint16_t* kr = k_base + (size_t)(ok ? pg : 0) * Hkv * g.page_tokens * D + ((size_t)ph * g.page_tokens + (pt % g.page_tokens)) * D;
    for (int s = 0; s < S; s++) {
      const float* qv = q + (((size_t)i * S + s) * g.H + h) * D;
      float sum = 0.0f;
      for (int d = 0; d < D; d++) sum = __fadd_rn(sum, __fmul_rn(qv[d], f32_from_bf16_bits(kr[d])));
      float v = __fmul_rn(sum, g.scale);
      if (ref_masked(g, T, S, s, j)) v = -INFINITY;
      w[(size_t)s * T + j] = ok ? v : -INFINITY;
    }
  }
  __syncthreads();
  softmax_rows_ref(w, S, T, red);
  for (int e = tid; e < S * D; e += nt) {
    const int s = e / D, d = e % D;
    float o = 0.0f;
    for (int j = 0; j < T; j++) {
      const int ph = src[j] >> 20, pt = src[j] & 0xFFFFF;
      int32_t pg = g.table[(size_t)seq * g.table_stride + pt / g.page_tokens];
      if (pg < 0 || pg >= g.num_pages) continue;
      const uint16_t* vr = v_base + (size_t)pg * Hkv * g.page_tokens * D + ((size_t)ph * g.page_tokens + (pt % g.page_tokens)) * D;
      o = __fadd_rn(o, __fmul_rn(w[(size_t)s * T + j], f32_from_bf16_bits(vr[d])));
    }
    out[(((size_t)i * S + s) * g.H + h) * D + d] = o;
  }
}

// grid (H, n_seqs).  qc/out: [n][S][H][Dh], qr: [n][S][H][dHR], W_UK/W_UV: [dC][H*Dh] bf16.
__global__ void mla_reference_kernel(RefGeom g, const uint16_t* __restrict__ base, const float* __restrict__ qc,
                                     const float* __restrict__ qr, const uint16_t* __restrict__ W_UK,
                                     const uint16_t* __restrict__ W_UV, float* __restrict__ out, int Dh, int dC, int dHR) {
  extern __shared__ float smem[];
  __shared__ float red[32];
  const int h = blockIdx.x, i = blockIdx.y;
  const int seq = g.seq_ids ? g.seq_ids[i] : i;
  const int T = g.len[seq] + g.extra;
  const int S = g.S, H = g.H, row = dC + dHR;
  float* w = smem;  // [S][T]
  const int tid = threadIdx.x, nt = blockDim.x;
  const size_t wstride = (size_t)H * Dh;
  const bool blk = g.blocked != 0;
  // value of column c of the cached row of token t: the bf16 page, or the float32 copy in faithful mode
  auto cached = [&](int32_t pg, int t, int c) -> float {
    const int tk = t % g.page_tokens;
    if (g.shadow) return g.shadow[((size_t)pg * g.page_tokens + tk) * row + c];
    return f32_from_bf16_bits(base[(size_t)pg * g.page_tokens * row + mla_page_off(blk, g.page_tokens, row, tk, c)]);
  };
  for (int j = tid; j < T; j += nt) {
    // content part: logical (h, j) -> physical (token tp, head hp)
    const int r = h * T + j;
    const int tp = g.faithful ? r / H : j, hp = g.faithful ? r % H : h;
    int32_t pg, pgc;
    bool ok = page_of(g.table, g.table_stride, seq, j / g.page_tokens, g.num_pages, g.status, &pg);
    ok = page_of(g.table, g.table_stride, seq, tp / g.page_tokens, g.num_pages, g.status, &pgc) && ok;
    if (!ok) pg = pgc = 0;
    for (int s = 0; s < S; s++) {
      const float* qcv = qc + (((size_t)i * S + s) * H + h) * Dh;
      const float* qrv = qr + (((size_t)i * S + s) * H + h) * dHR;
      // Qc . Kc^T with Kc[j][d] = sum_c C[j][c] * W_UK[c][h*Dh+d]   (mla.go:325, 355)
      float a = 0.0f;
      for (int d = 0; d < Dh; d++) {
        float kc = 0.0f;
        for (int c = 0; c < dC; c++)
          kc = __fadd_rn(kc, __fmul_rn(cached(pgc, tp, c), f32_from_bf16_bits(W_UK[(size_t)c * wstride + (size_t)hp * Dh + d])));
        a = __fadd_rn(a, __fmul_rn(qcv[d], kc));
      }
      float rsum = 0.0f;
      for (int d = 0; d < dHR; d++) rsum = __fadd_rn(rsum, __fmul_rn(qrv[d], cached(pg, j, dC + d)));
      float v = __fmul_rn(__fadd_rn(a, rsum), g.scale);
      if (ref_masked(g, T, S, s, j)) v = -INFINITY;
      w[(size_t)s * T + j] = ok ? v : -INFINITY;
    }
  }
  __syncthreads();
  softmax_rows_ref(w, S, T, red);
  for (int e = tid; e < S * Dh; e += nt) {
    const int s = e / Dh, d = e % Dh;
    float o = 0.0f;
    for (int j = 0; j < T; j++) {
      const int r = h * T + j;
      const int tp = g.faithful ? r / H : j, hp = g.faithful ? r % H : h;
      int32_t pg = g.table[(size_t)seq * g.table_stride + tp / g.page_tokens];
      if (pg < 0 || pg >= g.num_pages) continue;
      float vv = 0.0f;
      for (int c = 0; c < dC; c++)
        vv = __fadd_rn(vv, __fmul_rn(cached(pg, tp, c), f32_from_bf16_bits(W_UV[(size_t)c * wstride + (size_t)hp * Dh + d])));
      o = __fadd_rn(o, __fmul_rn(w[(size_t)s * T + j], vv));
    }
    out[(((size_t)i * S + s) * H + h) * Dh + d] = o;
  }
}

static int32_t ref_geom(Pool* p, const SeqBatch& sb, const relux_attn_args& a, RefGeom* g, size_t* smem_bytes) {
  const relux_pool_params& prm = p->prm;
  int maxT = 0;
  for (int i = 0; i < sb.n_seqs; i++) maxT = std::max(maxT, p->h_len[(size_t)a.layer * prm.max_seqs + sb.seq[i]] + a.extra_tokens);
  size_t need = ((size_t)a.q_tokens + 1) * maxT * sizeof(float);   // scores, and one index per position (GQA)
  if (need > 200 * 1024) {
    set_error("RELUX_ATTN_REFERENCE keeps q_tokens*T=%d*%d scores in shared memory; the limit is 51200", a.q_tokens, maxT);
    return RELUX_ERR_UNSUPPORTED;
  }
  *smem_bytes = need;
  g->table = p->d_table;
  g->table_stride = prm.max_pages_per_seq;
  g->len = p->d_len + (size_t)a.layer * prm.max_seqs;
  g->seq_ids = sb.d_seq_ids;
  g->num_pages = prm.num_pages;
  g->page_tokens = prm.page_tokens;
  g->status = p->d_status;
  g->S = a.q_tokens;
  g->extra = a.extra_tokens;
  g->causal = a.causal;
  g->H = a.num_heads;
  g->scale = a.scale;
  g->blocked = p->mla_blocked ? 1 : 0;
  g->faithful = a.mode == RELUX_ATTN_REFERENCE_FAITHFUL ? 1 : 0;
  g->chunk_tab = nullptr;
  g->chunk_stride = 0;
  g->shadow = nullptr;
  return RELUX_OK;
}

// Chunk starts of the call's sequences -> device, [n_seqs][1 + max chunks]: count, then P_0 .. P_(count-1).
static int32_t stage_chunks(Pool* p, const SeqBatch& sb, int layer, RefGeom* g) {
  size_t most = 1;
  for (int i = 0; i < sb.n_seqs; i++) most = std::max(most, p->chunks[(size_t)layer * p->prm.max_seqs + sb.seq[i]].size());
  const size_t stride = most + 1;
  std::vector<int32_t> tab((size_t)sb.n_seqs * stride, 0);
  for (int i = 0; i < sb.n_seqs; i++) {
    const std::vector<int32_t>& c = p->chunks[(size_t)layer * p->prm.max_seqs + sb.seq[i]];
    if (c.empty() || c[0] != 0) {
      set_error("sequence %d has cached rows that no Append call of this pool wrote; the chunk history needed by "
                "RELUX_ATTN_REFERENCE_FAITHFUL is incomplete", sb.seq[i]);
      return RELUX_ERR_INVALID_ARG;
    }
    tab[i * stride] = (int32_t)c.size();
    std::copy(c.begin(), c.end(), tab.begin() + i * stride + 1);
  }
  int32_t rc = grow(p->dev, p->chunk_tab, tab.size() * 4);
  if (rc) return rc;
  RELUX_CUDA_TRY(cudaMemcpyAsync(p->chunk_tab.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, p->dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(p->dev->stream));   // `tab` is pageable and goes out of scope
  g->chunk_tab = (const int32_t*)p->chunk_tab.p;
  g->chunk_stride = (int32_t)stride;
  return RELUX_OK;
}

int32_t launch_attn_reference_gqa(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const float* d_q, float* d_out) {
  RefGeom g;
  size_t smem;
  int32_t rc = ref_geom(p, sb, a, &g, &smem);
  if (rc) return rc;
  if (g.faithful && (rc = stage_chunks(p, sb, a.layer, &g))) return rc;
  const uint16_t* kb = p->storage + (size_t)a.layer * p->layer_elems;
  const uint16_t* vb = kb + p->page_elems * p->prm.num_pages;
  if (smem > 48 * 1024) RELUX_CUDA_TRY(cudaFuncSetAttribute(gqa_reference_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(a.num_heads, sb.n_seqs);
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), p->dev->stream));
  gqa_reference_kernel<<<grid, 128, smem, p->dev->stream>>>(g, kb, vb, d_q, d_out, p->prm.gqa_num_kv_heads, p->prm.gqa_head_dim);
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), p->dev->stream));
  p->timed_calls++;
  count_launch(p->dev);
  return RELUX_OK;
}

int32_t launch_attn_reference_mla(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const float* d_q, const float* d_qr,
                                  float* d_out) {
  RefGeom g;
  size_t smem;
  int32_t rc = ref_geom(p, sb, a, &g, &smem);
  if (rc) return rc;
  const uint16_t* base = p->storage + (size_t)a.layer * p->layer_elems;
  if (g.faithful) g.shadow = p->shadow_f32 + (size_t)a.layer * p->layer_elems;
  if (smem > 48 * 1024) RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_reference_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(a.num_heads, sb.n_seqs);
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), p->dev->stream));
  mla_reference_kernel<<<grid, 128, smem, p->dev->stream>>>(g, base, d_q, d_qr, (const uint16_t*)a.w_uk, (const uint16_t*)a.w_uv, d_out,
                                                            a.head_dim, p->prm.mla_dc, p->prm.mla_dhr);
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), p->dev->stream));
  p->timed_calls++;
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux
