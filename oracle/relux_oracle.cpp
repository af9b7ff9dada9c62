// relux_oracle.cpp -- TEST INFRASTRUCTURE ONLY.
//
// A CPU restatement, in C++, of the KV-cache / cached-attention path of the
// pure-Go framework xDarkicex/relux.  It is the checker for the CUDA library:
// only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
// load it.  Nothing in the product path links, imports or calls this file.
//
// The Go toolchain is not available where this was written, so the reference
// itself could not be executed.  Pinning status:
//   * bf16 conversion, KVCache layout/grow/reset, RoPE tables and rotation,
//     RMSNorm, greedy argmax: PINNED against the known-answer tests the
//     reference ships (kvcache_test.go, dtype_test.go, rope_test.go,
//     rmsnorm_test.go, sampler_test.go) -- see tests/test_oracle_pins.py.
//   * cached attention outputs (MHA.forwardCached, MLA.forwardCached, MLACache,
//     speculative verify): PARITY UNPINNED -- the reference has no test that
//     computes or compares them, and it cannot be run here.
//
// Float semantics mirrored from Go on amd64: every float32 `sum += a*b` is an
// unfused multiply followed by an add, so this file must be compiled with
// -ffp-contract=off and without -ffast-math.  Loops are ordered so that each
// output element sees exactly the reference's k-ascending summation order.
//
// Each function names the reference file:line (paths relative to the relux
// repository root) whose behaviour it restates.

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <algorithm>
#include <limits>
#ifdef _OPENMP
#include <omp.h>
#endif

#define RO_API extern "C" __attribute__((visibility("default")))

// ----------------------------------------------------------------------------
// bf16 <-> f32      internal/transformer/dtype_convert.go:15-24, 32-35
// ----------------------------------------------------------------------------
static inline uint16_t bf16_from_f32(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  uint32_t bias = 0x7FFFu + ((u >> 16) & 1u);   // round-to-nearest-even, no NaN special case
  u += bias;
  return (uint16_t)(u >> 16);
}
static inline float f32_from_bf16(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
RO_API uint16_t ro_bf16_from_f32(float x) { return bf16_from_f32(x); }
RO_API float ro_f32_from_bf16(uint16_t b) { return f32_from_bf16(b); }
RO_API void ro_bf16_slice_from_f32(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = bf16_from_f32(src[i]);
}
RO_API void ro_f32_slice_from_bf16(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = f32_from_bf16(src[i]);
}
// BF16SliceFromF64: float64 -> float32 -> bf16   dtype_convert.go:71-80
RO_API void ro_bf16_slice_from_f64(const double* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = bf16_from_f32((float)src[i]);
}

// ----------------------------------------------------------------------------
// matmul helpers    internal/transformer/matmul.go:15-27, 32-44
//                   internal/transformer/mha.go:759-785 (matmulBatched3D, pure-Go branch)
// ----------------------------------------------------------------------------
// C[M,N] = A[M,K] @ B[K,N].  Loop order (i,k,j) keeps every C[i,j]'s additions in
// k-ascending order starting from +0, which is bit-identical to the reference's
// (i,j,k) order, and lets the compiler vectorise over j.
static void matmul_f32(float* out, const float* a, const float* b, int M, int K, int N) {
  for (int i = 0; i < M; i++) {
    float* o = out + (size_t)i * N;
    for (int j = 0; j < N; j++) o[j] = 0.0f;
    for (int k = 0; k < K; k++) {
      const float av = a[(size_t)i * K + k];
      const float* br = b + (size_t)k * N;
      for (int j = 0; j < N; j++) o[j] = o[j] + av * br[j];
    }
  }
}
// C[M,N] = A[M,K] @ B[N,K]^T
static void matmul_f32_transb(float* out, const float* a, const float* b, int M, int K, int N) {
  for (int i = 0; i < M; i++) {
    const float* ar = a + (size_t)i * K;
    for (int j = 0; j < N; j++) {
      const float* br = b + (size_t)j * K;
      float sum = 0.0f;
      for (int k = 0; k < K; k++) sum = sum + ar[k] * br[k];
      out[(size_t)i * N + j] = sum;
    }
  }
}
// A [M,K] f32, B [K,N] bf16 (widened on the fly), C [M,N] f32.
static void matmul_a_f32_b_bf16(float* out, const float* a, const uint16_t* b, int M, int K, int N) {
  std::vector<float> brow((size_t)N);
  for (int i = 0; i < M; i++) {
    float* o = out + (size_t)i * N;
    for (int j = 0; j < N; j++) o[j] = 0.0f;
    for (int k = 0; k < K; k++) {
      const float av = a[(size_t)i * K + k];
      const uint16_t* br = b + (size_t)k * N;
      for (int j = 0; j < N; j++) brow[j] = f32_from_bf16(br[j]);
      for (int j = 0; j < N; j++) o[j] = o[j] + av * brow[j];
    }
  }
}
RO_API void ro_matmul(float* out, const float* a, const float* b, int M, int K, int N) { matmul_f32(out, a, b, M, K, N); }
RO_API void ro_matmul_transb(float* out, const float* a, const float* b, int M, int K, int N) { matmul_f32_transb(out, a, b, M, K, N); }
RO_API void ro_matmul_batched3d(float* out, const float* a, const uint16_t* b, int batch, int seq, int inDim, int outDim) {
  matmul_a_f32_b_bf16(out, a, b, batch * seq, inDim, outDim);
}

// ----------------------------------------------------------------------------
// fastexp32 + softmaxRows     internal/transformer/mha.go:823-833, 837-861
// ----------------------------------------------------------------------------
// The Go constants float32(1<<23)/0.6931471805599453 and 127.0*float32(1<<23)-405000 round
// to 12102203.0f and 1064948224.0f whichever way the constant folding is ordered.
static inline float fastexp_factor() { return (float)(8388608.0 / 0.6931471805599453); }
static inline float fastexp32_go(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 87.0f) return std::numeric_limits<float>::infinity();
  const float factor = fastexp_factor();
  const float bias = (float)(127.0 * 8388608.0 - 405000.0);
  float t = factor * x;
  t = t + bias;
  int32_t i = (int32_t)t;
  uint32_t u = (uint32_t)i;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}
RO_API float ro_fastexp32(float x) { return fastexp32_go(x); }

// Test-only switch: 1 replaces fastexp32 by libm exp (no -20 cut-off) inside softmaxRows, giving the
// exact softmax.  It separates "the kernel's indexing/masking is right" from "the reference's 3 %
// exp approximation", which dominates the difference at short contexts.  Default 0 = reference.
static int g_exact_exp = 0;
RO_API void ro_set_exact_exp(int on) { g_exact_exp = on; }

static void softmax_rows(float* m, int rows, int cols) {
  if (g_exact_exp) {
    for (int r = 0; r < rows; r++) {
      float* row = m + (size_t)r * cols;
      float maxV = row[0];
      for (int j = 1; j < cols; j++)
        if (row[j] > maxV) maxV = row[j];
      double sum = 0.0;
      for (int j = 0; j < cols; j++) {
        double e = std::exp((double)row[j] - (double)maxV);
        row[j] = (float)e;
        sum += e;
      }
      for (int j = 0; j < cols; j++) row[j] = (float)((double)row[j] / sum);
    }
    return;
  }
  for (int r = 0; r < rows; r++) {
    float* row = m + (size_t)r * cols;
    float maxV = row[0];
    for (int j = 1; j < cols; j++)
      if (row[j] > maxV) maxV = row[j];
    float sum = 0.0f;
    for (int j = 0; j < cols; j++) {
      float diff = row[j] - maxV;
      if (diff < -20.0f) row[j] = 0.0f;
      else row[j] = fastexp32_go(diff);
      sum = sum + row[j];
    }
    float invSum = 1.0f / sum;
    for (int j = 0; j < cols; j++) row[j] = row[j] * invSum;
  }
}
RO_API void ro_softmax_rows(float* m, int rows, int cols) { softmax_rows(m, rows, cols); }

// ----------------------------------------------------------------------------
// RoPE      internal/transformer/rope.go:50-75 (tables), 130-180 (Apply)
// ----------------------------------------------------------------------------
struct Rope {
  int headDim = 0, maxSeqLen = 0;
  float base = 0;
  std::vector<float> cosT, sinT;
};
static void rope_fill(Rope& r, int from, int to) {
  int half = r.headDim / 2;
  for (int pos = from; pos < to; pos++)
    for (int i = 0; i < half; i++) {
      float theta = 1.0f / (float)std::pow((double)r.base, (double)(2 * i) / (double)r.headDim);
      float angle = (float)((double)pos * (double)theta);
      r.cosT[(size_t)pos * half + i] = (float)std::cos((double)angle);
      r.sinT[(size_t)pos * half + i] = (float)std::sin((double)angle);
    }
}
static void rope_init(Rope& r, int headDim, float base, int maxSeqLen) {
  r.headDim = headDim; r.base = base; r.maxSeqLen = maxSeqLen;
  r.cosT.assign((size_t)maxSeqLen * (headDim / 2), 0.f);
  r.sinT.assign((size_t)maxSeqLen * (headDim / 2), 0.f);
  rope_fill(r, 0, maxSeqLen);
}
// rowPosMode 0 = reference rule (rope.go:151-158: startPos>0 -> every row gets startPos;
//                                else row % seqLen, or 0 for rank-1 input)
// rowPosMode 1 = intended rule: position = startPos + (row % seqLen)
// Returns 0, or -1 where the reference panics (position >= maxSeqLen).
static int rope_apply(const Rope& r, const float* x, float* out, int64_t rows, int seqLen, bool rank1,
                      int startPos, int rowPosMode) {
  int half = r.headDim / 2;
  for (int64_t row = 0; row < rows; row++) {
    int64_t base = row * r.headDim;
    int pos;
    if (rowPosMode == 1) pos = startPos + (rank1 ? 0 : (int)(row % seqLen));
    else if (startPos > 0) pos = startPos;
    else if (rank1) pos = 0;
    else pos = (int)(row % seqLen);
    if (pos >= r.maxSeqLen) return -1;
    const float* c = &r.cosT[(size_t)pos * half];
    const float* s = &r.sinT[(size_t)pos * half];
    for (int i = 0; i < half; i++) {
      float x0 = x[base + 2 * i], x1 = x[base + 2 * i + 1];
      float a = x0 * c[i], b = x1 * s[i];
      out[base + 2 * i] = a - b;
      float d = x1 * c[i], e = x0 * s[i];
      out[base + 2 * i + 1] = d + e;
    }
  }
  return 0;
}
RO_API void* ro_rope_new(int headDim, float base, int maxSeqLen) {
  if (headDim <= 0 || headDim % 2 != 0 || maxSeqLen <= 0) return nullptr;  // reference panics
  Rope* r = new Rope();
  rope_init(*r, headDim, base, maxSeqLen);
  return r;
}
RO_API void ro_rope_free(void* p) { delete (Rope*)p; }
RO_API const float* ro_rope_cos(void* p) { return ((Rope*)p)->cosT.data(); }
RO_API const float* ro_rope_sin(void* p) { return ((Rope*)p)->sinT.data(); }
RO_API int ro_rope_max_seq_len(void* p) { return ((Rope*)p)->maxSeqLen; }
// ExtendMaxSeqLen   rope.go:93-116   (returns -1 where the reference panics)
RO_API int ro_rope_extend(void* p, int newMax) {
  Rope* r = (Rope*)p;
  if (newMax <= r->maxSeqLen || newMax <= 0) return -1;
  int half = r->headDim / 2, old = r->maxSeqLen;
  r->cosT.resize((size_t)newMax * half);
  r->sinT.resize((size_t)newMax * half);
  r->maxSeqLen = newMax;
  rope_fill(*r, old, newMax);
  return 0;
}
RO_API int ro_rope_apply(void* p, const float* x, float* out, int64_t rows, int seqLen, int rank1,
                         int startPos, int rowPosMode) {
  return rope_apply(*(Rope*)p, x, out, rows, seqLen, rank1 != 0, startPos, rowPosMode);
}

// ----------------------------------------------------------------------------
// KVCache    internal/transformer/kvcache.go:34-49 (struct), 52-93 (constructors),
//            174-202 (Reset), 240-316 (Append), 363-380 (View), 407-438 (copyInto)
// ----------------------------------------------------------------------------
// The stream is kept exactly as the reference keeps it: Append copies
// newLen * rowSize source elements linearly to element offset total * rowSize,
// where rowSize = product of the source dims between batch and seq, times headDim
// (kvcache.go:414-416 skips the batch dim).  View re-labels the same buffer
// [1, Hkv, total, D].
struct LayerKV {
  bool present = false;
  std::vector<float> kf, vf;       // float32 storage
  std::vector<uint16_t> kb, vb;    // bf16 storage
  std::vector<int> shape;          // shape of the stored tensor (legacy) / full shape (sized)
  int total = 0, capacity = 0;
};
struct KVCache {
  std::vector<LayerKV> layers;
  int dtype = 0;  // 0 = float32, 1 = bfloat16
  int maxLen = 0, numKVHeads = 0, headDim = 0;
};
RO_API void* ro_kvcache_new(int numLayers, int dtype) {
  if (numLayers <= 0) return nullptr;
  KVCache* c = new KVCache();
  c->layers.resize(numLayers);
  c->dtype = dtype;
  return c;
}
RO_API void* ro_kvcache_new_sized(int numLayers, int maxLen, int numKVHeads, int headDim, int dtype) {
  if (numLayers <= 0 || maxLen <= 0) return nullptr;
  KVCache* c = new KVCache();
  c->layers.resize(numLayers);
  c->dtype = dtype; c->maxLen = maxLen; c->numKVHeads = numKVHeads; c->headDim = headDim;
  size_t n = (size_t)numKVHeads * maxLen * headDim;
  for (auto& l : c->layers) {
    l.present = true; l.capacity = maxLen;
    l.shape = {1, numKVHeads, maxLen, headDim};
    if (dtype == 1) { l.kb.assign(n, 0); l.vb.assign(n, 0); }
    else { l.kf.assign(n, 0.f); l.vf.assign(n, 0.f); }
  }
  return c;
}
RO_API void ro_kvcache_free(void* p) { delete (KVCache*)p; }
RO_API int ro_kvcache_dtype(void* p) { return ((KVCache*)p)->dtype; }
RO_API int ro_kvcache_total_len(void* p, int layer) {
  KVCache* c = (KVCache*)p;
  if (layer < 0 || layer >= (int)c->layers.size()) return 0;
  return c->layers[layer].total;
}
static int64_t row_size_of(const int* shape, int rank) {
  int seqAxis = rank - 2;
  int64_t rowSize = shape[rank - 1];
  for (int i = 1; i < seqAxis; i++) rowSize *= shape[i];
  return rowSize;
}
static void copy_into(KVCache* c, LayerKV& l, bool isK, const float* src, const int* shape, int rank,
                      int startRow, int seqLen) {
  int64_t rowSize = row_size_of(shape, rank);
  for (int r = 0; r < seqLen; r++) {
    int64_t dstRow = (int64_t)(startRow + r) * rowSize, srcRow = (int64_t)r * rowSize;
    for (int64_t j = 0; j < rowSize; j++) {
      if (c->dtype == 1) (isK ? l.kb : l.vb)[dstRow + j] = bf16_from_f32(src[srcRow + j]);
      else (isK ? l.kf : l.vf)[dstRow + j] = src[srcRow + j];
    }
  }
}
// Returns 0; -1 layer out of range; -2 rank < 3; -3 overflow (all panics in the reference).
RO_API int ro_kvcache_append(void* p, int layer, const float* newK, const float* newV, const int* shape, int rank) {
  KVCache* c = (KVCache*)p;
  if (layer < 0 || layer >= (int)c->layers.size()) return -1;
  if (rank < 3) return -2;
  int seqAxis = rank - 2, headDim = shape[rank - 1], newLen = shape[seqAxis];
  LayerKV& cur = c->layers[layer];
  int64_t other = 1;
  for (int i = 0; i < seqAxis; i++) other *= shape[i];
  if (!cur.present) {
    // legacy path: allocate exactly newLen   kvcache.go:260-276
    LayerKV nl;
    nl.present = true; nl.total = newLen; nl.capacity = 0;
    nl.shape.assign(shape, shape + rank);
    size_t n = (size_t)other * newLen * headDim;
    if (c->dtype == 1) { nl.kb.assign(n, 0); nl.vb.assign(n, 0); } else { nl.kf.assign(n, 0.f); nl.vf.assign(n, 0.f); }
    copy_into(c, nl, true, newK, shape, rank, 0, newLen);
    copy_into(c, nl, false, newV, shape, rank, 0, newLen);
    cur = nl;
    return 0;
  }
  if (cur.capacity > 0) {
    if (cur.total + newLen > cur.capacity) return -3;
    copy_into(c, cur, true, newK, shape, rank, cur.total, newLen);
    copy_into(c, cur, false, newV, shape, rank, cur.total, newLen);
    cur.total += newLen;
    return 0;
  }
  // legacy grow: new buffer, copy old rows then new rows   kvcache.go:293-316
  int oldTotal = cur.total;
  int newTotal = oldTotal + newLen;
  LayerKV nl;
  nl.present = true; nl.total = newTotal; nl.capacity = 0;
  nl.shape.assign(shape, shape + rank);
  nl.shape[seqAxis] = newTotal;
  size_t n = (size_t)other * newTotal * headDim;
  if (c->dtype == 1) { nl.kb.assign(n, 0); nl.vb.assign(n, 0); } else { nl.kf.assign(n, 0.f); nl.vf.assign(n, 0.f); }
  // copyInto(newKT, cur.K, 0, oldTotal): source is the old cache tensor (widened to f32)
  {
    std::vector<int> oshape = cur.shape;
    size_t on = (c->dtype == 1) ? cur.kb.size() : cur.kf.size();
    std::vector<float> ok(on), ov(on);
    for (size_t i = 0; i < on; i++) {
      ok[i] = (c->dtype == 1) ? f32_from_bf16(cur.kb[i]) : cur.kf[i];
      ov[i] = (c->dtype == 1) ? f32_from_bf16(cur.vb[i]) : cur.vf[i];
    }
    copy_into(c, nl, true, ok.data(), oshape.data(), (int)oshape.size(), 0, oldTotal);
    copy_into(c, nl, false, ov.data(), oshape.data(), (int)oshape.size(), 0, oldTotal);
  }
  copy_into(c, nl, true, newK, shape, rank, oldTotal, newLen);
  copy_into(c, nl, false, newV, shape, rank, oldTotal, newLen);
  cur = nl;
  return 0;
}
// View: writes the view shape (rank <= 8) and returns the number of elements the view
// covers (0 = nil view).  kvcache.go:363-380
RO_API int64_t ro_kvcache_view_shape(void* p, int layer, int* shapeOut, int* rankOut) {
  KVCache* c = (KVCache*)p;
  if (layer < 0 || layer >= (int)c->layers.size()) return -1;
  LayerKV& cur = c->layers[layer];
  if (!cur.present) { *rankOut = 0; return 0; }
  std::vector<int> s = cur.shape;
  if (cur.capacity > 0) s[s.size() - 2] = cur.total;
  int64_t n = 1;
  for (size_t i = 0; i < s.size(); i++) { shapeOut[i] = s[i]; n *= s[i]; }
  *rankOut = (int)s.size();
  return n;
}
// Copies the first n elements of the layer's backing buffers widened to f32 (what
// Tensor.ToF32 / DataF32 expose; tensor.go:134-153).
RO_API void ro_kvcache_read_f32(void* p, int layer, float* kOut, float* vOut, int64_t n) {
  KVCache* c = (KVCache*)p;
  LayerKV& cur = c->layers[layer];
  for (int64_t i = 0; i < n; i++) {
    kOut[i] = (c->dtype == 1) ? f32_from_bf16(cur.kb[i]) : cur.kf[i];
    vOut[i] = (c->dtype == 1) ? f32_from_bf16(cur.vb[i]) : cur.vf[i];
  }
}
RO_API void ro_kvcache_read_bf16(void* p, int layer, uint16_t* kOut, uint16_t* vOut, int64_t n) {
  KVCache* c = (KVCache*)p;
  LayerKV& cur = c->layers[layer];
  for (int64_t i = 0; i < n; i++) { kOut[i] = cur.kb[i]; vOut[i] = cur.vb[i]; }
}
RO_API void ro_kvcache_reset(void* p) {
  KVCache* c = (KVCache*)p;
  for (auto& l : c->layers) {
    if (l.capacity > 0) {
      l.total = 0;
      std::fill(l.kb.begin(), l.kb.end(), 0); std::fill(l.vb.begin(), l.vb.end(), 0);
      std::fill(l.kf.begin(), l.kf.end(), 0.f); std::fill(l.vf.begin(), l.vf.end(), 0.f);
    } else {
      l = LayerKV();
    }
  }
}

// ----------------------------------------------------------------------------
// MLACache   internal/transformer/mla_cache.go:21-59, 118-133, 152-182, 222-233
// float32 storage in the reference; `roundBF16` stores BF16FromF32(row) widened back,
// which is what a bf16 paged pool holds.
// ----------------------------------------------------------------------------
struct MLALayer { std::vector<float> c, kr; int total = 0, capacity = 0; };
struct MLACache { std::vector<MLALayer> layers; int maxLen = 0, dC = 0, dHR = 0; bool roundBF16 = false; };
RO_API void* ro_mlacache_new(int numLayers, int maxLen, int dC, int dHR, int roundBF16) {
  if (numLayers <= 0 || maxLen <= 0) return nullptr;
  MLACache* c = new MLACache();
  c->layers.resize(numLayers);
  c->maxLen = maxLen; c->dC = dC; c->dHR = dHR; c->roundBF16 = roundBF16 != 0;
  for (auto& l : c->layers) {
    l.c.assign((size_t)maxLen * dC, 0.f);
    l.kr.assign((size_t)maxLen * dHR, 0.f);
    l.capacity = maxLen;
  }
  return c;
}
RO_API void ro_mlacache_free(void* p) { delete (MLACache*)p; }
RO_API int ro_mlacache_total_len(void* p, int layer) {
  MLACache* c = (MLACache*)p;
  if (layer < 0 || layer >= (int)c->layers.size()) return 0;
  return c->layers[layer].total;
}
// newC holds nElemsC values, newKR nElemsKR values, newLen = shape[rank-2] of newC.
// The reference copies ALL source elements (mla_cache.go:171-172) but advances the
// cursor by newLen only.  Returns -1 bad layer, -3 overflow.
RO_API int ro_mlacache_append(void* p, int layer, const float* newC, int64_t nElemsC, const float* newKR,
                              int64_t nElemsKR, int newLen) {
  MLACache* c = (MLACache*)p;
  if (layer < 0 || layer >= (int)c->layers.size()) return -1;
  MLALayer& cur = c->layers[layer];
  if (cur.total + newLen > cur.capacity) return -3;
  int64_t roomC = (int64_t)cur.c.size() - (int64_t)cur.total * c->dC;
  int64_t roomR = (int64_t)cur.kr.size() - (int64_t)cur.total * c->dHR;
  int64_t nc = std::min(nElemsC, roomC), nr = std::min(nElemsKR, roomR);  // Go copy() clamps to dst length
  for (int64_t i = 0; i < nc; i++) {
    float v = newC[i];
    cur.c[(size_t)cur.total * c->dC + i] = c->roundBF16 ? f32_from_bf16(bf16_from_f32(v)) : v;
  }
  for (int64_t i = 0; i < nr; i++) {
    float v = newKR[i];
    cur.kr[(size_t)cur.total * c->dHR + i] = c->roundBF16 ? f32_from_bf16(bf16_from_f32(v)) : v;
  }
  cur.total += newLen;
  return 0;
}
RO_API void ro_mlacache_read(void* p, int layer, float* cOut, float* krOut) {
  MLACache* c = (MLACache*)p;
  MLALayer& cur = c->layers[layer];
  std::memcpy(cOut, cur.c.data(), (size_t)cur.total * c->dC * 4);
  std::memcpy(krOut, cur.kr.data(), (size_t)cur.total * c->dHR * 4);
}
RO_API void ro_mlacache_reset(void* p) {
  MLACache* c = (MLACache*)p;
  for (auto& l : c->layers) {
    l.total = 0;
    std::fill(l.c.begin(), l.c.end(), 0.f);
    std::fill(l.kr.begin(), l.kr.end(), 0.f);
  }
}

// ----------------------------------------------------------------------------
// layout helpers     internal/transformer/mha.go:789-819
// ----------------------------------------------------------------------------
static void rearrange_bsnh(float* out, const float* src, int batch, int seq, int nh, int hd) {
  int rowSize = nh * hd;
  for (int b = 0; b < batch; b++)
    for (int s = 0; s < seq; s++)
      for (int h = 0; h < nh; h++)
        std::memcpy(out + ((size_t)(b * nh + h) * seq + s) * hd, src + (size_t)b * seq * rowSize + (size_t)s * rowSize + h * hd,
                    (size_t)hd * 4);
}
static void rearrange_bhsn(float* out, const float* src, int batch, int nh, int seq, int hd) {
  for (int b = 0; b < batch; b++)
    for (int h = 0; h < nh; h++)
      for (int s = 0; s < seq; s++)
        std::memcpy(out + (size_t)b * seq * nh * hd + (size_t)s * nh * hd + h * hd, src + ((size_t)(b * nh + h) * seq + s) * hd,
                    (size_t)hd * 4);
}

// ----------------------------------------------------------------------------
// Semantics switches
// ----------------------------------------------------------------------------
// RO_FAITHFUL : reproduce the reference exactly, including its layout/position quirks:
//   Q1 GQA cache written chunk-linear, read head-major (kvcache.go:407-438 vs mha.go:299-312)
//   Q2 cached MLA reads token-major kcAll/vAll as head-major (mla.go:323-326 vs :348,351)
//   Q3 RoPE startPos>0 gives every row the same position (rope.go:151-153)
//   Q4 no causal mask inside a multi-token cached call (mha.go:340, mla.go:368)
// RO_INTENDED : textbook indexing with the same arithmetic primitives: per-head cache rows,
//   token-major decompressed K/V read as such, per-row RoPE positions, causal mask inside a
//   multi-token cached call (row i sees cached rows plus new rows 0..i).
enum { RO_FAITHFUL = 0, RO_INTENDED = 1 };
enum { RO_FLAG_MLA_BF16_CACHE = 1 };  // MLA cache rows rounded to bf16 (what the paged pool stores)

// Hooks let a test run the reference forward with the cache+attention core swapped out.
// MHA: q [H,S,D], k,v [Hkv,S,D] (post-RoPE, f32) -> out [H,S,D].  startPos = tokens already cached.
typedef int (*ro_mha_hook)(void* user, int layer, int S, int startPos, const float* q, const float* k, const float* v,
                           float* out);
// MLA: qc [H,S,Dh], qr [H,S,dHR] (post-RoPE), ckv [S,dC], kr [S,dHR] (post-RoPE) -> out [H,S,Dh]
typedef int (*ro_mla_hook)(void* user, int layer, int S, int startPos, const float* qc, const float* qr,
                           const float* ckv, const float* kr, float* out);
// Whole attention layer (MHA.forwardCached / MLA.forwardCached): x [S, dModel] -> out [S, dModel].
typedef int (*ro_layer_hook)(void* user, int layer, int S, const float* x, float* out);

// ----------------------------------------------------------------------------
// Attention core shared by the cached paths: per head, S = QK^T * scale (+mask),
// softmaxRows, O = P V.     mha.go:318-348, mla.go:339-377
// kExp / vExp are [H, T, D] f32 exactly as the reference builds them.
// maskMode 0: reference rule (mask j>i only when seqQ == T);  1: intended (mask j > T-seqQ+i)
// ----------------------------------------------------------------------------
static void attend_heads(float* attnOut, const float* q, const float* kExp, const float* vExp, const float* qr,
                         const float* krExp, int H, int seqQ, int T, int D, int dR, int Dv, float scale, bool causal,
                         int maskMode) {
  std::vector<float> w((size_t)seqQ * T), w2;
  if (qr) w2.resize((size_t)seqQ * T);
  for (int h = 0; h < H; h++) {
    matmul_f32_transb(w.data(), q + (size_t)h * seqQ * D, kExp + (size_t)h * T * D, seqQ, D, T);
    if (qr) {
      matmul_f32_transb(w2.data(), qr + (size_t)h * seqQ * dR, krExp + (size_t)h * T * dR, seqQ, dR, T);
      for (size_t i = 0; i < (size_t)seqQ * T; i++) w[i] = w[i] + w2[i];
    }
    for (int i = 0; i < seqQ; i++)
      for (int j = 0; j < T; j++) {
        w[(size_t)i * T + j] = w[(size_t)i * T + j] * scale;
        bool masked;
        if (maskMode == 0) masked = causal && seqQ == T && j > i;
        else masked = causal && j > (T - seqQ + i);
        if (masked) w[(size_t)i * T + j] = -std::numeric_limits<float>::infinity();
      }
    softmax_rows(w.data(), seqQ, T);
    matmul_f32(attnOut + (size_t)h * seqQ * Dv, w.data(), vExp + (size_t)h * T * Dv, seqQ, T, Dv);
  }
}

// ----------------------------------------------------------------------------
// Decoder model (forward only)
//   transformer.go:178-245 (construction), 269-281 (Forward), 887-966 (Generate)
//   embedding.go:60-91, rmsnorm.go:69-97, linear.go:65-104, mlp.go:103-176,462-464,
//   transformer_block.go:60-84,119-142, sampler.go:53-66
// Weights are injected by the caller as one flat bf16 buffer (the reference's own init
// is a fixed arithmetic pattern, mha.go:84-94); norm gammas are 1 and all biases 0 as
// the reference constructors leave them (rmsnorm.go:51-54, mlp.go:70-78, linear.go:54-58).
// Flat order: embed[V,D]; per layer { MHA: Wq[D,H*hd] Wk[D,Hkv*hd] Wv[D,Hkv*hd] Wo[H*hd,D]
//   | MLA: W_Q[D,H*hd] W_DKV[D,dC] W_UK[dC,H*hd] W_UV[dC,H*hd] W_KR[D,dHR] W_QR[D,H*dHR] W_O[H*hd,D] }
//   W1[D,F] (WGate[D,F] if swiglu) W2[F,D]; lmHead[D,V].
// ----------------------------------------------------------------------------
struct ModelCfg {
  int32_t vocab, dModel, numHeads, numKVHeads, numLayers, dFF, maxSeqLen;
  float ropeBase;
  int32_t causal, swiglu, mla, dC, dHR;
};
struct LayerW {
  const uint16_t *Wq = 0, *Wk = 0, *Wv = 0, *Wo = 0;
  const uint16_t *W_Q = 0, *W_DKV = 0, *W_UK = 0, *W_UV = 0, *W_KR = 0, *W_QR = 0, *W_O = 0;
  const uint16_t *W1 = 0, *WGate = 0, *W2 = 0;
};
struct Model {
  ModelCfg cfg;
  int headDim;
  std::vector<uint16_t> weights;
  const uint16_t* embed; const uint16_t* lmHead;
  std::vector<LayerW> L;
  Rope rope, ropeKR;
  // runtime
  int mode = RO_FAITHFUL, flags = 0;
  KVCache* kv = nullptr; MLACache* mc = nullptr;
  // intended-mode caches: per layer [Hkv][maxLen][D] bf16 for K and V
  std::vector<std::vector<uint16_t>> ik, iv; std::vector<int> ilen;
  ro_mha_hook mhaHook = nullptr; ro_mla_hook mlaHook = nullptr; void* hookUser = nullptr;
  ro_layer_hook layerHook = nullptr;
  int status = 0;
};
RO_API int64_t ro_model_weight_count(const ModelCfg* c) {
  int64_t hd = c->dModel / c->numHeads, n = (int64_t)c->vocab * c->dModel;
  for (int l = 0; l < c->numLayers; l++) {
    if (c->mla) {
      n += (int64_t)c->dModel * c->numHeads * hd + (int64_t)c->dModel * c->dC + 2 * (int64_t)c->dC * c->numHeads * hd +
           (int64_t)c->dModel * c->dHR + (int64_t)c->dModel * c->numHeads * c->dHR + (int64_t)c->numHeads * hd * c->dModel;
    } else {
      n += (int64_t)c->dModel * c->numHeads * hd + 2 * (int64_t)c->dModel * c->numKVHeads * hd +
           (int64_t)c->numHeads * hd * c->dModel;
    }
    n += (int64_t)c->dModel * c->dFF * (c->swiglu ? 2 : 1) + (int64_t)c->dFF * c->dModel;
  }
  n += (int64_t)c->dModel * c->vocab;
  return n;
}
RO_API void* ro_model_new(const ModelCfg* c, const uint16_t* flatWeights) {
  if (c->vocab <= 0 || c->dModel <= 0 || c->numHeads <= 0 || c->numKVHeads <= 0 || c->numLayers <= 0 || c->dFF <= 0 ||
      c->maxSeqLen <= 0 || c->dModel % c->numHeads != 0 || c->numHeads % c->numKVHeads != 0)
    return nullptr;
  Model* m = new Model();
  m->cfg = *c;
  if (m->cfg.ropeBase == 0) m->cfg.ropeBase = 10000.f;
  m->headDim = c->dModel / c->numHeads;
  if (m->cfg.mla) {
    if (m->cfg.dC <= 0) m->cfg.dC = 4 * m->headDim;
    if (m->cfg.dHR <= 0) m->cfg.dHR = m->headDim / 2;
  }
  int64_t n = ro_model_weight_count(&m->cfg);
  m->weights.assign(flatWeights, flatWeights + n);
  const uint16_t* p = m->weights.data();
  auto take = [&](int64_t cnt) { const uint16_t* r = p; p += cnt; return r; };
  int D = c->dModel, H = c->numHeads, Hkv = c->numKVHeads, hd = m->headDim, F = c->dFF;
  m->embed = take((int64_t)c->vocab * D);
  m->L.resize(c->numLayers);
  for (auto& l : m->L) {
    if (m->cfg.mla) {
      l.W_Q = take((int64_t)D * H * hd); l.W_DKV = take((int64_t)D * m->cfg.dC);
      l.W_UK = take((int64_t)m->cfg.dC * H * hd); l.W_UV = take((int64_t)m->cfg.dC * H * hd);
      l.W_KR = take((int64_t)D * m->cfg.dHR); l.W_QR = take((int64_t)D * H * m->cfg.dHR);
      l.W_O = take((int64_t)H * hd * D);
    } else {
      l.Wq = take((int64_t)D * H * hd); l.Wk = take((int64_t)D * Hkv * hd); l.Wv = take((int64_t)D * Hkv * hd);
      l.Wo = take((int64_t)H * hd * D);
    }
    l.W1 = take((int64_t)D * F);
    if (c->swiglu) l.WGate = take((int64_t)D * F);
    l.W2 = take((int64_t)F * D);
  }
  m->lmHead = take((int64_t)D * c->vocab);
  // transformer.go:200-201: shared RoPE over headDim; MLA builds its own over dHR with
  // base fixed at 10000 and maxSeqLen taken from the shared one (transformer_block.go:70-75)
  rope_init(m->rope, hd, m->cfg.ropeBase, c->maxSeqLen);
  if (m->cfg.mla) rope_init(m->ropeKR, m->cfg.dHR, 10000.f, c->maxSeqLen);
  return m;
}
RO_API void ro_model_free(void* p) {
  Model* m = (Model*)p;
  delete m->kv; delete m->mc;
  delete m;
}
RO_API void ro_model_set_mode(void* p, int mode, int flags) { Model* m = (Model*)p; m->mode = mode; m->flags = flags; }
RO_API void ro_model_set_hooks(void* p, ro_mha_hook a, ro_mla_hook b, void* user) {
  Model* m = (Model*)p; m->mhaHook = a; m->mlaHook = b; m->hookUser = user;
}
RO_API void ro_model_set_layer_hook(void* p, ro_layer_hook h) { ((Model*)p)->layerHook = h; }
RO_API int ro_model_status(void* p) { return ((Model*)p)->status; }

// rmsnorm.go:69-97 with gamma = 1 (stored bf16 1.0), eps = 1e-5 fixed in blocks
// (transformer_block.go:62-63); the final norm uses cfg.NormEps whose default is 1e-5.
static void rmsnorm(float* out, const float* x, int rows, int D, float eps) {
  for (int r = 0; r < rows; r++) {
    const float* xr = x + (size_t)r * D;
    float sumSq = 0.f;
    for (int j = 0; j < D; j++) { float v = xr[j]; sumSq = sumSq + v * v; }
    float meanSq = sumSq / (float)D;
    float rstd = (float)(1.0 / std::sqrt((double)(meanSq + eps)));
    for (int j = 0; j < D; j++) out[(size_t)r * D + j] = xr[j] * rstd * 1.0f;
  }
}
RO_API void ro_rmsnorm(float* out, const float* x, int rows, int D, float eps) { rmsnorm(out, x, rows, D, eps); }
static inline float gelu_exact(float x) { return 0.5f * x * (1.0f + (float)std::erf((double)x / 1.4142135623730951)); }
static inline float silu(float x) { return x / (1.0f + (float)std::exp((double)(-x))); }
RO_API float ro_gelu(float x) { return gelu_exact(x); }

// mlp.go:103-176
static void mlp_forward(const Model* m, const LayerW& l, float* y, const float* x, int n) {
  int D = m->cfg.dModel, F = m->cfg.dFF;
  std::vector<float> h((size_t)n * F);
  if (m->cfg.swiglu) {
    std::vector<float> up((size_t)n * F), gated((size_t)n * F);
    matmul_a_f32_b_bf16(up.data(), x, l.W1, n, D, F);
    matmul_a_f32_b_bf16(gated.data(), x, l.WGate, n, D, F);
    for (size_t i = 0; i < (size_t)n * F; i++) h[i] = silu(up[i]) * gated[i];
    matmul_a_f32_b_bf16(y, h.data(), l.W2, n, F, D);
  } else {
    std::vector<float> pre((size_t)n * F);
    matmul_a_f32_b_bf16(pre.data(), x, l.W1, n, D, F);
    for (size_t i = 0; i < (size_t)n * F; i++) { pre[i] = pre[i] + 0.0f; h[i] = gelu_exact(pre[i]); }
    matmul_a_f32_b_bf16(y, h.data(), l.W2, n, F, D);
    for (size_t i = 0; i < (size_t)n * D; i++) y[i] = y[i] + 0.0f;
  }
}

// MHA.forwardCached   mha.go:245-369  (batch is always 1 on this path, transformer.go:951,960)
static int mha_forward_cached(Model* m, int layer, float* out, const float* x, int seqQ) {
  const LayerW& l = m->L[layer];
  int D = m->cfg.dModel, H = m->cfg.numHeads, Hkv = m->cfg.numKVHeads, hd = m->headDim;
  std::vector<float> qd((size_t)seqQ * H * hd), kd((size_t)seqQ * Hkv * hd), vd((size_t)seqQ * Hkv * hd);
  matmul_a_f32_b_bf16(qd.data(), x, l.Wq, seqQ, D, H * hd);
  matmul_a_f32_b_bf16(kd.data(), x, l.Wk, seqQ, D, Hkv * hd);
  matmul_a_f32_b_bf16(vd.data(), x, l.Wv, seqQ, D, Hkv * hd);
  int cacheLen;
  if (m->mhaHook) cacheLen = m->ilen[layer];
  else cacheLen = (m->mode == RO_FAITHFUL) ? m->kv->layers[layer].total : m->ilen[layer];
  std::vector<float> q((size_t)H * seqQ * hd), k((size_t)Hkv * seqQ * hd), v((size_t)Hkv * seqQ * hd), tmp;
  rearrange_bsnh(q.data(), qd.data(), 1, seqQ, H, hd);
  rearrange_bsnh(k.data(), kd.data(), 1, seqQ, Hkv, hd);
  rearrange_bsnh(v.data(), vd.data(), 1, seqQ, Hkv, hd);
  int posMode = (m->mode == RO_FAITHFUL) ? 0 : 1;
  tmp.resize(q.size());
  if (rope_apply(m->rope, q.data(), tmp.data(), (int64_t)H * seqQ, seqQ, false, cacheLen, posMode)) return -4;
  q = tmp;
  tmp.resize(k.size());
  if (rope_apply(m->rope, k.data(), tmp.data(), (int64_t)Hkv * seqQ, seqQ, false, cacheLen, posMode)) return -4;
  k = tmp;
  std::vector<float> attnOut((size_t)H * seqQ * hd);
  float scale = (float)(1.0 / std::sqrt((double)hd));
  if (m->mhaHook) {
    int rc = m->mhaHook(m->hookUser, layer, seqQ, cacheLen, q.data(), k.data(), v.data(), attnOut.data());
    if (rc) return rc;
    m->ilen[layer] += seqQ;
  } else {
    int T;
    std::vector<float> kExp, vExp;
    int g = H / Hkv;
    if (m->mode == RO_FAITHFUL) {
      int shape[4] = {1, Hkv, seqQ, hd};
      if (ro_kvcache_append(m->kv, layer, k.data(), v.data(), shape, 4)) return -3;
      LayerKV& cur = m->kv->layers[layer];
      T = cur.total;
      // View + ToF32: the buffer read as [1,Hkv,T,hd] with head stride T*hd (Q1)
      kExp.resize((size_t)H * T * hd); vExp.resize((size_t)H * T * hd);
      for (int h = 0; h < H; h++) {
        int kvH = h / g;
        for (size_t i = 0; i < (size_t)T * hd; i++) {
          kExp[(size_t)h * T * hd + i] = f32_from_bf16(cur.kb[(size_t)kvH * T * hd + i]);
          vExp[(size_t)h * T * hd + i] = f32_from_bf16(cur.vb[(size_t)kvH * T * hd + i]);
        }
      }
    } else {
      int cap = m->cfg.maxSeqLen;
      if (cacheLen + seqQ > cap) return -3;
      for (int h = 0; h < Hkv; h++)
        for (int s = 0; s < seqQ; s++)
          for (int d = 0; d < hd; d++) {
            m->ik[layer][((size_t)h * cap + cacheLen + s) * hd + d] = bf16_from_f32(k[((size_t)h * seqQ + s) * hd + d]);
            m->iv[layer][((size_t)h * cap + cacheLen + s) * hd + d] = bf16_from_f32(v[((size_t)h * seqQ + s) * hd + d]);
          }
      m->ilen[layer] += seqQ;
      T = m->ilen[layer];
      kExp.resize((size_t)H * T * hd); vExp.resize((size_t)H * T * hd);
      for (int h = 0; h < H; h++) {
        int kvH = h / g;
        for (size_t i = 0; i < (size_t)T * hd; i++) {
          kExp[(size_t)h * T * hd + i] = f32_from_bf16(m->ik[layer][(size_t)kvH * cap * hd + i]);
          vExp[(size_t)h * T * hd + i] = f32_from_bf16(m->iv[layer][(size_t)kvH * cap * hd + i]);
        }
      }
    }
    attend_heads(attnOut.data(), q.data(), kExp.data(), vExp.data(), nullptr, nullptr, H, seqQ, T, hd, 0, hd, scale,
                 m->cfg.causal != 0, m->mode == RO_FAITHFUL ? 0 : 1);
  }
  std::vector<float> back((size_t)seqQ * H * hd);
  rearrange_bhsn(back.data(), attnOut.data(), 1, H, seqQ, hd);
  matmul_a_f32_b_bf16(out, back.data(), l.Wo, seqQ, H * hd, D);
  return 0;
}

// MLA.forwardCached   mla.go:272-397
static int mla_forward_cached(Model* m, int layer, float* out, const float* x, int seqQ) {
  const LayerW& l = m->L[layer];
  int D = m->cfg.dModel, H = m->cfg.numHeads, hd = m->headDim, dC = m->cfg.dC, dHR = m->cfg.dHR;
  int n = seqQ;
  std::vector<float> qcF((size_t)n * H * hd), qrF((size_t)n * H * dHR), ckv((size_t)n * dC), kr((size_t)n * dHR);
  matmul_a_f32_b_bf16(qcF.data(), x, l.W_Q, n, D, H * hd);
  matmul_a_f32_b_bf16(qrF.data(), x, l.W_QR, n, D, H * dHR);
  matmul_a_f32_b_bf16(ckv.data(), x, l.W_DKV, n, D, dC);
  matmul_a_f32_b_bf16(kr.data(), x, l.W_KR, n, D, dHR);
  std::vector<float> qc((size_t)H * n * hd), qr((size_t)H * n * dHR), tmp;
  rearrange_bsnh(qc.data(), qcF.data(), 1, seqQ, H, hd);
  rearrange_bsnh(qr.data(), qrF.data(), 1, seqQ, H, dHR);
  int cacheLen = m->mlaHook ? m->ilen[layer] : m->mc->layers[layer].total;
  int posMode = (m->mode == RO_FAITHFUL) ? 0 : 1;
  tmp.resize(qr.size());
  if (rope_apply(m->ropeKR, qr.data(), tmp.data(), (int64_t)H * seqQ, seqQ, false, cacheLen, posMode)) return -4;
  qr = tmp;
  tmp.resize(kr.size());
  if (rope_apply(m->ropeKR, kr.data(), tmp.data(), n, n, false, cacheLen, posMode)) return -4;
  kr = tmp;
  std::vector<float> attnOut((size_t)H * seqQ * hd);
  float scale = (float)(1.0 / std::sqrt((double)(hd + dHR)));
  if (m->mlaHook) {
    int rc = m->mlaHook(m->hookUser, layer, seqQ, cacheLen, qc.data(), qr.data(), ckv.data(), kr.data(), attnOut.data());
    if (rc) return rc;
    m->ilen[layer] += seqQ;
  } else {
    if (ro_mlacache_append(m->mc, layer, ckv.data(), (int64_t)n * dC, kr.data(), (int64_t)n * dHR, seqQ)) return -3;
    MLALayer& cur = m->mc->layers[layer];
    int T = cur.total;
    // decompress every cached latent: [T, H*hd] token-major   mla.go:323-326
    std::vector<float> kcAll((size_t)T * H * hd), vAll((size_t)T * H * hd);
    matmul_a_f32_b_bf16(kcAll.data(), cur.c.data(), l.W_UK, T, dC, H * hd);
    matmul_a_f32_b_bf16(vAll.data(), cur.c.data(), l.W_UV, T, dC, H * hd);
    std::vector<float> krAll((size_t)H * T * dHR);
    for (int h = 0; h < H; h++) std::memcpy(&krAll[(size_t)h * T * dHR], cur.kr.data(), (size_t)T * dHR * 4);
    if (m->mode == RO_FAITHFUL) {
      // Q2: the flat [T,H,hd] buffers are indexed as if [H,T,hd]
      attend_heads(attnOut.data(), qc.data(), kcAll.data(), vAll.data(), qr.data(), krAll.data(), H, seqQ, T, hd, dHR, hd,
                   scale, m->cfg.causal != 0, 0);
    } else {
      std::vector<float> kcH((size_t)H * T * hd), vH((size_t)H * T * hd);
      rearrange_bsnh(kcH.data(), kcAll.data(), 1, T, H, hd);
      rearrange_bsnh(vH.data(), vAll.data(), 1, T, H, hd);
      attend_heads(attnOut.data(), qc.data(), kcH.data(), vH.data(), qr.data(), krAll.data(), H, seqQ, T, hd, dHR, hd, scale,
                   m->cfg.causal != 0, 1);
    }
  }
  std::vector<float> back((size_t)seqQ * H * hd);
  rearrange_bhsn(back.data(), attnOut.data(), 1, H, seqQ, hd);
  matmul_a_f32_b_bf16(out, back.data(), l.W_O, seqQ, H * hd, D);
  return 0;
}

// Transformer.Forward with batchSize 1   transformer.go:269-281, transformer_block.go:119-142
static int model_forward(Model* m, const int* tokens, int seq, float* logits) {
  int D = m->cfg.dModel, V = m->cfg.vocab;
  std::vector<float> h((size_t)seq * D), normed((size_t)seq * D), attn((size_t)seq * D), post((size_t)seq * D),
      mlp((size_t)seq * D);
  for (int i = 0; i < seq; i++) {
    if (tokens[i] < 0 || tokens[i] >= V) return -5;
    for (int j = 0; j < D; j++) h[(size_t)i * D + j] = f32_from_bf16(m->embed[(size_t)tokens[i] * D + j]);
  }
  for (int l = 0; l < m->cfg.numLayers; l++) {
    rmsnorm(normed.data(), h.data(), seq, D, 1e-5f);
    int rc = m->layerHook ? m->layerHook(m->hookUser, l, seq, normed.data(), attn.data())
             : m->cfg.mla ? mla_forward_cached(m, l, attn.data(), normed.data(), seq)
                          : mha_forward_cached(m, l, attn.data(), normed.data(), seq);
    if (rc) return rc;
    for (size_t i = 0; i < (size_t)seq * D; i++) post[i] = h[i] + attn[i];
    rmsnorm(normed.data(), post.data(), seq, D, 1e-5f);
    mlp_forward(m, m->L[l], mlp.data(), normed.data(), seq);
    for (size_t i = 0; i < (size_t)seq * D; i++) h[i] = post[i] + mlp[i];
  }
  rmsnorm(normed.data(), h.data(), seq, D, 1e-5f);
  matmul_a_f32_b_bf16(logits, normed.data(), m->lmHead, seq, D, V);
  for (size_t i = 0; i < (size_t)seq * V; i++) logits[i] = logits[i] + 0.0f;  // zero bias, linear.go:94-96
  return 0;
}
// Sampler.Greedy: first index wins on ties   sampler.go:53-66
static int greedy(const float* logits, int n) {
  int best = 0; float bv = logits[0];
  for (int i = 1; i < n; i++) if (logits[i] > bv) { bv = logits[i]; best = i; }
  return best;
}
RO_API int ro_greedy(const float* logits, int n) { return greedy(logits, n); }

static void model_begin(Model* m) {
  delete m->kv; delete m->mc; m->kv = nullptr; m->mc = nullptr;
  int Lr = m->cfg.numLayers;
  m->ilen.assign(Lr, 0);
  if (m->cfg.mla) {
    m->mc = (MLACache*)ro_mlacache_new(Lr, m->cfg.maxSeqLen, m->cfg.dC, m->cfg.dHR, (m->flags & RO_FLAG_MLA_BF16_CACHE) ? 1 : 0);
  } else if (m->mode == RO_FAITHFUL) {
    m->kv = (KVCache*)ro_kvcache_new_sized(Lr, m->cfg.maxSeqLen, m->cfg.numKVHeads, m->headDim, 1);
  } else {
    size_t n = (size_t)m->cfg.numKVHeads * m->cfg.maxSeqLen * m->headDim;
    m->ik.assign(Lr, std::vector<uint16_t>(n, 0));
    m->iv.assign(Lr, std::vector<uint16_t>(n, 0));
  }
}
// Starts a cached session (what Generate does at transformer.go:907-947).
RO_API void ro_model_begin(void* p) { model_begin((Model*)p); }
// The attention module of one layer alone on the session's caches: MHA.Forward / MLA.Forward in Inference mode with a
// cache attached (mha.go:126-128, mla.go:130-132 -> forwardCached).  x [seq, dModel] -> out [seq, dModel].
RO_API int ro_model_attention_forward(void* p, int layer, const float* x, int seq, float* out) {
  Model* m = (Model*)p;
  if (layer < 0 || layer >= m->cfg.numLayers || (m->cfg.mla ? m->mc == nullptr : (m->mode == RO_FAITHFUL && m->kv == nullptr))) return -7;
  return m->cfg.mla ? mla_forward_cached(m, layer, out, x, seq) : mha_forward_cached(m, layer, out, x, seq);
}
// One cached Forward over `seq` tokens; logits [seq, vocab].
RO_API int ro_model_forward(void* p, const int* tokens, int seq, float* logits) {
  Model* m = (Model*)p;
  int rc = model_forward(m, tokens, seq, logits);
  m->status = rc;
  return rc;
}
// Generate with greedy selection (temperature <= 0, topK = 1 in the reference resolves to the
// argmax unless two logits tie exactly; ties are reported through *ties).
// out receives len(prompt)+maxNew ids.  margins (optional, maxNew floats) = top1-top2 logit gap.
RO_API int ro_model_generate(void* p, const int* prompt, int nPrompt, int maxNew, int* out, float* margins, int* ties) {
  Model* m = (Model*)p;
  if (maxNew <= 0 || nPrompt <= 0) return -6;
  model_begin(m);
  int V = m->cfg.vocab;
  std::vector<float> logits((size_t)nPrompt * V);
  int rc = model_forward(m, prompt, nPrompt, logits.data());
  if (rc) { m->status = rc; return rc; }
  auto pick = [&](const float* lg, int step) {
    int b = greedy(lg, V);
    float second = -std::numeric_limits<float>::infinity();
    int nt = 0;
    for (int i = 0; i < V; i++) {
      if (i != b && lg[i] > second) second = lg[i];
      if (i != b && lg[i] == lg[b]) nt++;
    }
    if (margins) margins[step] = lg[b] - second;
    if (ties && nt) (*ties)++;
    return b;
  };
  if (ties) *ties = 0;
  for (int i = 0; i < nPrompt; i++) out[i] = prompt[i];
  int next = pick(&logits[(size_t)(nPrompt - 1) * V], 0);
  out[nPrompt] = next;
  for (int i = 1; i < maxNew; i++) {
    rc = model_forward(m, &next, 1, logits.data());
    if (rc) { m->status = rc; return rc; }
    next = pick(logits.data(), i);
    out[nPrompt + i] = next;
  }
  return 0;
}

// ----------------------------------------------------------------------------
// Standalone attention ops at arbitrary shapes (INTENDED indexing, reference arithmetic:
// f32 k-ascending dot products, full-row softmaxRows with fastexp32, f32 P*V).
// Inputs are the logical, unpaged caches as bf16.
// ----------------------------------------------------------------------------
// MLA, the reference way: decompress every latent with W_UK / W_UV, then attend.
//   ckv  [B][Tmax][dC] bf16, kr [B][Tmax][dHR] bf16, ctx[B] (rows valid, INCLUDING the S new rows)
//   qc   [B][S][H][Dh] f32, qr [B][S][H][dHR] f32, W_UK/W_UV [dC][H*Dh] bf16
//   out  [B][S][H][Dh] f32.   causal: row i of S sees cached rows j <= ctx-S+i.
RO_API void ro_mla_attend_decompress(int B, int S, int H, int Dh, int dC, int dHR, int Tmax, const int* ctx,
                                     const uint16_t* ckv, const uint16_t* kr, const float* qc, const float* qr,
                                     const uint16_t* W_UK, const uint16_t* W_UV, float scale, int causal, float* out,
                                     int nThreads) {
#ifdef _OPENMP
  if (nThreads > 0) omp_set_num_threads(nThreads);
#endif
#pragma omp parallel for schedule(dynamic, 1)
  for (int b = 0; b < B; b++) {
    int T = ctx[b];
    std::vector<float> c((size_t)T * dC), kcAll((size_t)T * H * Dh), vAll((size_t)T * H * Dh);
    for (size_t i = 0; i < (size_t)T * dC; i++) c[i] = f32_from_bf16(ckv[(size_t)b * Tmax * dC + i]);
    matmul_a_f32_b_bf16(kcAll.data(), c.data(), W_UK, T, dC, H * Dh);
    matmul_a_f32_b_bf16(vAll.data(), c.data(), W_UV, T, dC, H * Dh);
    std::vector<float> kcH((size_t)H * T * Dh), vH((size_t)H * T * Dh), krAll((size_t)H * T * dHR);
    rearrange_bsnh(kcH.data(), kcAll.data(), 1, T, H, Dh);
    rearrange_bsnh(vH.data(), vAll.data(), 1, T, H, Dh);
    for (int h = 0; h < H; h++)
      for (size_t i = 0; i < (size_t)T * dHR; i++) krAll[(size_t)h * T * dHR + i] = f32_from_bf16(kr[(size_t)b * Tmax * dHR + i]);
    std::vector<float> qch((size_t)H * S * Dh), qrh((size_t)H * S * dHR), o((size_t)H * S * Dh);
    rearrange_bsnh(qch.data(), qc + (size_t)b * S * H * Dh, 1, S, H, Dh);
    rearrange_bsnh(qrh.data(), qr + (size_t)b * S * H * dHR, 1, S, H, dHR);
    attend_heads(o.data(), qch.data(), kcH.data(), vH.data(), qrh.data(), krAll.data(), H, S, T, Dh, dHR, Dh, scale,
                 causal != 0, 1);
    rearrange_bhsn(out + (size_t)b * S * H * Dh, o.data(), 1, H, S, Dh);
  }
}
// MLA, absorbed algebra in f32 (same softmax primitive): q~ = W_UK[h] q_c, scores over the
// latent, O_lat = P C, out = W_UV[h]^T O_lat.  Mathematically equal to the routine above,
// rounding differs; used where decompression is too slow to run.
RO_API void ro_mla_attend_absorbed(int B, int S, int H, int Dh, int dC, int dHR, int Tmax, const int* ctx,
                                   const uint16_t* ckv, const uint16_t* kr, const float* qc, const float* qr,
                                   const uint16_t* W_UK, const uint16_t* W_UV, float scale, int causal, float* out,
                                   int nThreads) {
#ifdef _OPENMP
  if (nThreads > 0) omp_set_num_threads(nThreads);
#endif
  std::vector<float> wuk((size_t)dC * H * Dh), wuv((size_t)dC * H * Dh);
  for (size_t i = 0; i < wuk.size(); i++) { wuk[i] = f32_from_bf16(W_UK[i]); wuv[i] = f32_from_bf16(W_UV[i]); }
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < B; b++)
    for (int h = 0; h < H; h++) {
      int T = ctx[b];
      std::vector<float> qt((size_t)S * dC), w((size_t)S * T), olat((size_t)S * dC);
      for (int s = 0; s < S; s++)
        for (int c = 0; c < dC; c++) {
          float sum = 0.f;
          const float* q = qc + (((size_t)b * S + s) * H + h) * Dh;
          for (int d = 0; d < Dh; d++) sum = sum + q[d] * wuk[(size_t)c * H * Dh + (size_t)h * Dh + d];
          qt[(size_t)s * dC + c] = sum;
        }
      for (int s = 0; s < S; s++)
        for (int j = 0; j < T; j++) {
          const uint16_t* cr = ckv + ((size_t)b * Tmax + j) * dC;
          const uint16_t* rr = kr + ((size_t)b * Tmax + j) * dHR;
          const float* q = qr + (((size_t)b * S + s) * H + h) * dHR;
          float a = 0.f, r = 0.f;
          for (int c = 0; c < dC; c++) a = a + qt[(size_t)s * dC + c] * f32_from_bf16(cr[c]);
          for (int d = 0; d < dHR; d++) r = r + q[d] * f32_from_bf16(rr[d]);
          float v = (a + r) * scale;
          if (causal && j > T - S + s) v = -std::numeric_limits<float>::infinity();
          w[(size_t)s * T + j] = v;
        }
      softmax_rows(w.data(), S, T);
      for (int s = 0; s < S; s++) {
        float* o = &olat[(size_t)s * dC];
        for (int c = 0; c < dC; c++) o[c] = 0.f;
        for (int j = 0; j < T; j++) {
          float p = w[(size_t)s * T + j];
          const uint16_t* cr = ckv + ((size_t)b * Tmax + j) * dC;
          for (int c = 0; c < dC; c++) o[c] = o[c] + p * f32_from_bf16(cr[c]);
        }
        float* od = out + (((size_t)b * S + s) * H + h) * Dh;
        for (int d = 0; d < Dh; d++) {
          float sum = 0.f;
          for (int c = 0; c < dC; c++) sum = sum + o[c] * wuv[(size_t)c * H * Dh + (size_t)h * Dh + d];
          od[d] = sum;
        }
      }
    }
}
// GQA decode / verify:  K,V [B][Tmax][Hkv][D] bf16 (token-major logical cache), q [B][S][H][D] f32,
// out [B][S][H][D] f32.  mha.go:318-348 arithmetic, intended indexing.
RO_API void ro_gqa_attend(int B, int S, int H, int Hkv, int D, int Tmax, const int* ctx, const uint16_t* K,
                          const uint16_t* V, const float* q, float scale, int causal, float* out, int nThreads) {
#ifdef _OPENMP
  if (nThreads > 0) omp_set_num_threads(nThreads);
#endif
  int g = H / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < B; b++)
    for (int h = 0; h < H; h++) {
      int T = ctx[b], kvH = h / g;
      std::vector<float> w((size_t)S * T);
      for (int s = 0; s < S; s++) {
        const float* qv = q + (((size_t)b * S + s) * H + h) * D;
        for (int j = 0; j < T; j++) {
          const uint16_t* kr = K + (((size_t)b * Tmax + j) * Hkv + kvH) * D;
          float sum = 0.f;
          for (int d = 0; d < D; d++) sum = sum + qv[d] * f32_from_bf16(kr[d]);
          float v = sum * scale;
          if (causal && j > T - S + s) v = -std::numeric_limits<float>::infinity();
          w[(size_t)s * T + j] = v;
        }
      }
      softmax_rows(w.data(), S, T);
      for (int s = 0; s < S; s++) {
        float* o = out + (((size_t)b * S + s) * H + h) * D;
        for (int d = 0; d < D; d++) o[d] = 0.f;
        for (int j = 0; j < T; j++) {
          float p = w[(size_t)s * T + j];
          const uint16_t* vr = V + (((size_t)b * Tmax + j) * Hkv + kvH) * D;
          for (int d = 0; d < D; d++) o[d] = o[d] + p * f32_from_bf16(vr[d]);
        }
      }
    }
}
// The reference's own GQA decode cost model for the CPU baseline: widen the whole capacity
// buffer bf16->f32 (tensor.go:134-153), expand Hkv->H by copy (mha.go:299-316), then attend.
// Same results as ro_gqa_attend; only the work done differs.  capacity >= ctx.
RO_API void ro_gqa_attend_reference_cost(int B, int S, int H, int Hkv, int D, int Tmax, int capacity, const int* ctx,
                                         const uint16_t* K, const uint16_t* V, const float* q, float scale, int causal,
                                         float* out, int nThreads) {
#ifdef _OPENMP
  if (nThreads > 0) omp_set_num_threads(nThreads);
#endif
  int g = H / Hkv;
#pragma omp parallel for schedule(dynamic, 1)
  for (int b = 0; b < B; b++) {
    int T = ctx[b];
    std::vector<float> kf((size_t)Hkv * capacity * D, 0.f), vf((size_t)Hkv * capacity * D, 0.f);
    for (int j = 0; j < T; j++)
      for (int kh = 0; kh < Hkv; kh++)
        for (int d = 0; d < D; d++) {
          kf[((size_t)kh * capacity + j) * D + d] = f32_from_bf16(K[(((size_t)b * Tmax + j) * Hkv + kh) * D + d]);
          vf[((size_t)kh * capacity + j) * D + d] = f32_from_bf16(V[(((size_t)b * Tmax + j) * Hkv + kh) * D + d]);
        }
    std::vector<float> kExp((size_t)H * T * D), vExp((size_t)H * T * D);
    for (int h = 0; h < H; h++) {
      std::memcpy(&kExp[(size_t)h * T * D], &kf[(size_t)(h / g) * capacity * D], (size_t)T * D * 4);
      std::memcpy(&vExp[(size_t)h * T * D], &vf[(size_t)(h / g) * capacity * D], (size_t)T * D * 4);
    }
    std::vector<float> qh((size_t)H * S * D), o((size_t)H * S * D);
    rearrange_bsnh(qh.data(), q + (size_t)b * S * H * D, 1, S, H, D);
    attend_heads(o.data(), qh.data(), kExp.data(), vExp.data(), nullptr, nullptr, H, S, T, D, 0, D, scale, causal != 0, 1);
    rearrange_bhsn(out + (size_t)b * S * H * D, o.data(), 1, H, S, D);
  }
}
RO_API int ro_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// ----------------------------------------------------------------------------
// Sampler.Sample and the speculative accept step   sampler.go:73-300, speculative.go:211-295, 346-368
// ----------------------------------------------------------------------------
#include "relux_oracle_sampling.inc"
