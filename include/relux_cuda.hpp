// relux_cuda.hpp -- header-only C++ host mirror of relux's cache objects over the C ABI of relux_cuda.h.
//
// relux is Go; where no Go toolchain exists the host side above the C ABI is this header.  The classes keep the
// reference's names, argument meaning and error behaviour:
//   relux::KVCache   <- transformer.KVCache   (internal/transformer/kvcache.go:34-49; NewKVCacheSized :66-93,
//                       Append :240-316, View :363-380, TotalLen :383-388, Reset :174-202, DType :169-172)
//   relux::MLACache  <- transformer.MLACache  (internal/transformer/mla_cache.go:21-59, Append :152-182,
//                       View :222-233, TotalLen :236-241, Reset :118-133)
// plus Attend(), the replacement of the attention loops of MHA.forwardCached (mha.go:292-348) and
// MLA.forwardCached (mla.go:317-377), and ForwardCached(), the whole of those two functions (layer input in,
// layer output out) with the weight matrices resident on the device.  Where the reference panics, these throw relux::Panic with the same wording.
// One object = one sequence, every layer, exactly like the reference's caches; batched serving uses the pool-level
// C functions directly.
#ifndef RELUX_CUDA_HPP_
#define RELUX_CUDA_HPP_

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "relux_cuda.h"

namespace relux {

struct Panic : std::runtime_error {
  int32_t status;
  Panic(int32_t s, const std::string& m) : std::runtime_error(m), status(s) {}
};

inline void check(int32_t rc) {
  if (rc != RELUX_OK) {
    char buf[512];
    relux_cuda_last_error(buf, sizeof(buf));
    throw Panic(rc, std::string(buf));
  }
}

enum class DType { Float32 = RELUX_DTYPE_F32, BFloat16 = RELUX_DTYPE_BF16 };

class Device {
 public:
  explicit Device(int index = 0) { check(relux_cuda_device_open(index, &h_)); }
  ~Device() { if (h_) relux_cuda_device_close(h_); }
  Device(const Device&) = delete;
  Device& operator=(const Device&) = delete;
  relux_device_t handle() const { return h_; }
  void Sync() { check(relux_cuda_sync(h_)); }
  void* Upload(const void* host, size_t bytes) {
    void* d = nullptr;
    check(relux_cuda_dev_alloc(h_, bytes, &d));
    check(relux_cuda_h2d(h_, d, host, bytes));
    check(relux_cuda_sync(h_));
    return d;
  }
  void Free(void* d) { check(relux_cuda_dev_free(h_, d)); }

 private:
  relux_device_t h_ = nullptr;
};

// K / V tensors follow the reference's shape [1, numKVHeads, newLen, headDim], float32.
class KVCache {
 public:
  // NewKVCacheSized(numLayers, maxLen, numKVHeads, headDim, BFloat16)
  KVCache(Device& dev, int numLayers, int maxLen, int numKVHeads, int headDim, int pageTokens = 64)
      : layers_(numLayers), hkv_(numKVHeads), d_(headDim) {
    if (numLayers <= 0) throw Panic(RELUX_ERR_INVALID_ARG, "NewKVCacheSized: numLayers=" + std::to_string(numLayers) + ", must be > 0");
    if (maxLen <= 0) throw Panic(RELUX_ERR_INVALID_ARG, "NewKVCacheSized: maxLen=" + std::to_string(maxLen) + ", must be > 0");
    relux_pool_params p{};
    p.kind = RELUX_POOL_GQA;
    p.num_layers = numLayers;
    p.page_tokens = pageTokens;
    p.num_pages = (maxLen + pageTokens - 1) / pageTokens;
    p.max_seqs = 1;
    p.max_pages_per_seq = p.num_pages;
    p.gqa_num_kv_heads = numKVHeads;
    p.gqa_head_dim = headDim;
    check(relux_pool_create(dev.handle(), &p, &pool_));
    check(relux_seq_alloc(pool_, maxLen, &seq_));
  }
  ~KVCache() { if (pool_) relux_pool_destroy(pool_); }
  KVCache(const KVCache&) = delete;
  KVCache& operator=(const KVCache&) = delete;

  DType GetDType() const { return DType::BFloat16; }
  int TotalLen(int layerIdx) const {
    int32_t n = 0;
    check(relux_seq_len(pool_, layerIdx, seq_, &n));
    return n;
  }
  void Append(int layerIdx, const float* newK, const float* newV, int newLen) {
    if (layerIdx < 0 || layerIdx >= layers_)
      throw Panic(RELUX_ERR_INVALID_ARG, "KVCache.Append: layerIdx=" + std::to_string(layerIdx) + " out of range [0, " + std::to_string(layers_) + ")");
    relux_append_args a{};
    a.layer = layerIdx;
    a.n_seqs = 1;
    a.seq_ids = &seq_;
    int32_t n = newLen;
    a.n_new = &n;
    a.a = newK;
    a.b = newV;
    a.dtype = RELUX_DTYPE_F32;
    a.mem = RELUX_MEM_HOST;
    a.layout = RELUX_LAYOUT_HEAD_MAJOR;
    a.advance = 1;
    check(relux_gqa_append(pool_, &a));
  }
  // View: bf16 bit patterns of K and V as [numKVHeads][total][headDim]; false when the layer is empty (nil view).
  bool View(int layerIdx, std::vector<uint16_t>* k, std::vector<uint16_t>* v) const {
    const int t = TotalLen(layerIdx);
    if (t == 0) return false;
    std::vector<uint16_t> kt((size_t)t * hkv_ * d_), vt(kt.size());
    relux_read_rows_args rr{};
    rr.layer = layerIdx; rr.seq_id = seq_; rr.tok0 = 0; rr.n_tokens = t; rr.dst_a = kt.data(); rr.dst_b = vt.data();
    check(relux_pool_read_rows(pool_, &rr));
    k->resize(kt.size());
    v->resize(vt.size());
    for (int tok = 0; tok < t; tok++)
      for (int h = 0; h < hkv_; h++)
        for (int e = 0; e < d_; e++) {
          (*k)[((size_t)h * t + tok) * d_ + e] = kt[((size_t)tok * hkv_ + h) * d_ + e];
          (*v)[((size_t)h * t + tok) * d_ + e] = vt[((size_t)tok * hkv_ + h) * d_ + e];
        }
    return true;
  }
  void Reset() {
    int32_t zero = 0;
    check(relux_seq_set_len(pool_, -1, 1, &seq_, &zero));
  }
  // q, out: [1, numHeads, seqQ, headDim] float32; the seqQ query rows are the last seqQ cached rows.
  void Attend(int layerIdx, const float* q, float* out, int numHeads, int seqQ, float scale, bool causal,
              int mode = RELUX_ATTN_FAST) {
    relux_attn_args a{};
    a.layer = layerIdx;
    a.n_seqs = 1;
    a.seq_ids = &seq_;
    a.q_tokens = seqQ;
    a.causal = causal ? 1 : 0;
    a.num_heads = numHeads;
    a.head_dim = d_;
    a.scale = scale;
    a.q = q;
    a.q_dtype = RELUX_DTYPE_F32;
    a.q_mem = RELUX_MEM_HOST;
    a.q_layout = RELUX_LAYOUT_HEAD_MAJOR;
    a.out = out;
    a.out_dtype = RELUX_DTYPE_F32;
    a.out_mem = RELUX_MEM_HOST;
    a.out_layout = RELUX_LAYOUT_HEAD_MAJOR;
    a.mode = mode;
    check(relux_gqa_decode(pool_, &a));
  }
  // MHA.forwardCached (mha.go:245-369): x, out [1, seqQ, dModel] float32; w = device copies of Wq, Wk, Wv, Wo.
  void ForwardCached(int layerIdx, const float* x, float* out, const relux_gqa_layer_weights& w, int dModel, int numHeads, int seqQ,
                     bool causal, bool rope, float ropeBase = 10000.f, int mode = RELUX_ATTN_FAST) {
    relux_gqa_layer_args a{};
    a.layer = layerIdx;
    a.n_seqs = 1;
    a.seq_ids = &seq_;
    a.q_tokens = seqQ;
    a.causal = causal ? 1 : 0;
    a.d_model = dModel;
    a.num_heads = numHeads;
    a.rope = rope ? 1 : 0;
    a.rope_base = ropeBase;
    a.advance = 1;
    a.mode = mode;
    a.x = x;
    a.x_dtype = RELUX_DTYPE_F32;
    a.x_mem = RELUX_MEM_HOST;
    a.out = out;
    a.out_mem = RELUX_MEM_HOST;
    a.w = &w;
    check(relux_gqa_forward_cached(pool_, &a));
  }
  // Sampler.Sample (internal/transformer/sampler.go:73-218) on one row of logits: `draw` is the uniform number the
  // reference would take from its generator; previousTokens / nPrevious as in the reference (nullptr: no repetition
  // control).  Uses this cache's pool for the device work; the cache itself is not touched.
  int Sample(const float* logits, int vocab, float draw, const relux_sampler_params& sampling, const int32_t* previousTokens = nullptr,
             int nPrevious = 0, float repeatPenalty = 0.f, float frequencyPenalty = 0.f, float presencePenalty = 0.f, int repeatWindow = 0,
             int mode = RELUX_ATTN_FAST) {
    relux_sample_args a{};
    int32_t tok = -1, len = nPrevious;
    a.n_rows = 1;
    a.vocab = vocab;
    a.mem = RELUX_MEM_HOST;
    a.mode = mode;
    a.logits = logits;
    a.draws = &draw;
    a.sampler = sampling;
    a.repeat_penalty = repeatPenalty;
    a.frequency_penalty = frequencyPenalty;
    a.presence_penalty = presencePenalty;
    a.repeat_window = repeatWindow;
    a.prev_tokens = previousTokens;
    a.prev_len = previousTokens ? &len : nullptr;
    a.prev_stride = nPrevious;
    a.tokens = &tok;
    check(relux_sampler_sample(pool_, &a));
    return tok;
  }
  // SpeculativeDecoder.acceptPhase (speculative.go:211-253) for this cache's sequence: draftLogits [k][vocab],
  // targetLogits [k + 1][vocab], draws [k + 1] = the uniform numbers the reference would take from its generator, in
  // order.  Returns the number of accepted draft tokens, *resampled receives the resampled / bonus token.  commit:
  // the rows a verify call left past the cursor become part of the sequence (nAccepted + 1 of them).
  int AcceptPhase(const int32_t* draftTokens, const float* draftLogits, const float* targetLogits, int k, int vocab,
                  const float* draws, const relux_sampler_params& sampling, int* resampled, bool commit = true,
                  int mode = RELUX_ATTN_FAST) {
    relux_spec_accept_args a{};
    int32_t nAcc = 0, next = 0;
    a.n_seqs = 1;
    a.k = k;
    a.vocab = vocab;
    a.mem = RELUX_MEM_HOST;
    a.draft_tokens = draftTokens;
    a.draft_logits = draftLogits;
    a.target_logits = targetLogits;
    a.draws = draws;
    a.sampler = sampling;
    a.mode = mode;
    a.commit = commit ? 1 : 0;
    a.seq_ids = &seq_;
    a.n_accepted = &nAcc;
    a.next_token = &next;
    check(relux_spec_accept(pool_, &a));
    *resampled = next;
    return nAcc;
  }

 private:
  relux_pool_t pool_ = nullptr;
  int32_t seq_ = 0;
  int layers_, hkv_, d_;
};

// newC [1, newLen, dC], newKR [1, newLen, dHR] float32 (k^R already rotated), like mla.go:309-312.
class MLACache {
 public:
  MLACache(Device& dev, int numLayers, int maxLen, int dC, int dHR, int pageTokens = 64) : layers_(numLayers), dc_(dC), dhr_(dHR) {
    if (numLayers <= 0) throw Panic(RELUX_ERR_INVALID_ARG, "NewMLACache: numLayers=" + std::to_string(numLayers) + ", must be > 0");
    if (maxLen <= 0) throw Panic(RELUX_ERR_INVALID_ARG, "NewMLACache: maxLen=" + std::to_string(maxLen) + ", must be > 0");
    relux_pool_params p{};
    p.kind = RELUX_POOL_MLA;
    p.num_layers = numLayers;
    p.page_tokens = pageTokens;
    p.num_pages = (maxLen + pageTokens - 1) / pageTokens;
    p.max_seqs = 1;
    p.max_pages_per_seq = p.num_pages;
    p.mla_dc = dC;
    p.mla_dhr = dHR;
    check(relux_pool_create(dev.handle(), &p, &pool_));
    check(relux_seq_alloc(pool_, maxLen, &seq_));
  }
  ~MLACache() { if (pool_) relux_pool_destroy(pool_); }
  MLACache(const MLACache&) = delete;
  MLACache& operator=(const MLACache&) = delete;

  int TotalLen(int layerIdx) const {
    int32_t n = 0;
    check(relux_seq_len(pool_, layerIdx, seq_, &n));
    return n;
  }
  void Append(int layerIdx, const float* newC, const float* newKR, int newLen) {
    if (layerIdx < 0 || layerIdx >= layers_)
      throw Panic(RELUX_ERR_INVALID_ARG, "MLACache.Append: layerIdx=" + std::to_string(layerIdx) + " out of range [0, " + std::to_string(layers_) + ")");
    relux_append_args a{};
    a.layer = layerIdx;
    a.n_seqs = 1;
    a.seq_ids = &seq_;
    int32_t n = newLen;
    a.n_new = &n;
    a.a = newC;
    a.b = newKR;
    a.dtype = RELUX_DTYPE_F32;
    a.mem = RELUX_MEM_HOST;
    a.advance = 1;
    check(relux_mla_append(pool_, &a));
  }
  bool View(int layerIdx, std::vector<uint16_t>* c, std::vector<uint16_t>* kr) const {
    const int t = TotalLen(layerIdx);
    if (t == 0) return false;
    c->resize((size_t)t * dc_);
    kr->resize((size_t)t * dhr_);
    relux_read_rows_args rr{};
    rr.layer = layerIdx; rr.seq_id = seq_; rr.tok0 = 0; rr.n_tokens = t; rr.dst_a = c->data(); rr.dst_b = kr->data();
    check(relux_pool_read_rows(pool_, &rr));
    return true;
  }
  void Reset() {
    int32_t zero = 0;
    check(relux_seq_set_len(pool_, -1, 1, &seq_, &zero));
  }
  // qc [1,H,seqQ,Dh], qr [1,H,seqQ,dHR], out [1,H,seqQ,Dh] float32; wUK / wUV: device copies of the bf16 weights.
  void Attend(int layerIdx, const float* qc, const float* qr, const void* wUK, const void* wUV, float* out, int numHeads,
              int headDim, int seqQ, float scale, bool causal, int mode = RELUX_ATTN_FAST) {
    relux_attn_args a{};
    a.layer = layerIdx;
    a.n_seqs = 1;
    a.seq_ids = &seq_;
    a.q_tokens = seqQ;
    a.causal = causal ? 1 : 0;
    a.num_heads = numHeads;
    a.head_dim = headDim;
    a.scale = scale;
    a.q = qc;
    a.q_rope = qr;
    a.q_dtype = RELUX_DTYPE_F32;
    a.q_mem = RELUX_MEM_HOST;
    a.q_layout = RELUX_LAYOUT_HEAD_MAJOR;
    a.w_uk = wUK;
    a.w_uv = wUV;
    a.out = out;
    a.out_dtype = RELUX_DTYPE_F32;
    a.out_mem = RELUX_MEM_HOST;
    a.out_layout = RELUX_LAYOUT_HEAD_MAJOR;
    a.mode = mode;
    check(relux_mla_decode(pool_, &a));
  }
  // One decode step in one call: Append of one row, then Attend with one query token (relux_mla_step; mla.go:309-377).
  void Step(int layerIdx, const float* newC, const float* newKR, const float* qc, const float* qr, const void* wUK, const void* wUV,
            float* out, int numHeads, int headDim, float scale, int mode = RELUX_ATTN_FAST) {
    relux_append_args ap{};
    ap.layer = layerIdx;
    ap.n_seqs = 1;
    ap.seq_ids = &seq_;
    ap.a = newC;
    ap.b = newKR;
    ap.dtype = RELUX_DTYPE_F32;
    ap.mem = RELUX_MEM_HOST;
    ap.advance = 1;
    relux_attn_args a{};
    a.layer = layerIdx;
    a.n_seqs = 1;
    a.seq_ids = &seq_;
    a.q_tokens = 1;
    a.causal = 1;
    a.num_heads = numHeads;
    a.head_dim = headDim;
    a.scale = scale;
    a.q = qc;
    a.q_rope = qr;
    a.q_dtype = RELUX_DTYPE_F32;
    a.q_mem = RELUX_MEM_HOST;
    a.q_layout = RELUX_LAYOUT_HEAD_MAJOR;
    a.w_uk = wUK;
    a.w_uv = wUV;
    a.out = out;
    a.out_dtype = RELUX_DTYPE_F32;
    a.out_mem = RELUX_MEM_HOST;
    a.out_layout = RELUX_LAYOUT_HEAD_MAJOR;
    a.mode = mode;
    check(relux_mla_step(pool_, &ap, &a));
  }
  // MLA.forwardCached (mla.go:272-397): x, out [1, seqQ, dModel] float32; w = device copies of the seven matrices.
  void ForwardCached(int layerIdx, const float* x, float* out, const relux_mla_layer_weights& w, int dModel, int numHeads, int seqQ,
                     bool causal, float ropeBase = 10000.f, int mode = RELUX_ATTN_FAST) {
    relux_mla_layer_args a{};
    a.layer = layerIdx;
    a.n_seqs = 1;
    a.seq_ids = &seq_;
    a.q_tokens = seqQ;
    a.causal = causal ? 1 : 0;
    a.d_model = dModel;
    a.num_heads = numHeads;
    a.rope_base = ropeBase;
    a.mode = mode;
    a.x = x;
    a.x_dtype = RELUX_DTYPE_F32;
    a.x_mem = RELUX_MEM_HOST;
    a.out = out;
    a.out_mem = RELUX_MEM_HOST;
    a.w = &w;
    check(relux_mla_forward_cached(pool_, &a));
  }

 private:
  relux_pool_t pool_ = nullptr;
  int32_t seq_ = 0;
  int layers_, dc_, dhr_;
};

}  // namespace relux

#endif  // RELUX_CUDA_HPP_
