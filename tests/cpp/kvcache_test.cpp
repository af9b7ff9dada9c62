// The reference's own KVCache tests (internal/transformer/kvcache_test.go) replayed through the C++ host mirror
// (include/relux_cuda.hpp) on the device cache, plus the panics the reference raises on misuse.
// Prints one line per test; exit code 0 = all passed.  Built and run by tests/test_gpu_cpp_mirror.py.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "relux_cuda.hpp"

static int failures = 0;
#define EXPECT(cond, name)                                        \
  do {                                                            \
    if (!(cond)) { printf("FAIL %s: %s\n", name, #cond); failures++; } \
  } while (0)

static uint16_t bf16_from_f32(float f) {   // round to nearest even (dtype_convert.go:15-24)
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float f32_from_bf16(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

int main() {
  relux::Device dev(0);
  {  // TestKVCache_NewEmpty  kvcache_test.go:9-14
    relux::KVCache c(dev, 4, 16, 2, 8);
    EXPECT(c.TotalLen(0) == 0, "NewEmpty");
    std::vector<uint16_t> k, v;
    EXPECT(!c.View(0, &k, &v), "NewEmpty nil view");
  }
  {  // TestKVCache_AppendFirst  kvcache_test.go:16-40   (head dim widened to 8: rows are 16-byte vectors here)
    relux::KVCache c(dev, 2, 16, 2, 8);
    std::vector<float> k(16), v(16);
    for (int i = 0; i < 16; i++) { k[i] = (float)(i + 1); v[i] = (float)(i + 17); }
    c.Append(0, k.data(), v.data(), 1);
    EXPECT(c.TotalLen(0) == 1, "AppendFirst len");
    EXPECT(c.TotalLen(1) == 0, "AppendFirst other layer");
    std::vector<uint16_t> ck, cv;
    EXPECT(c.View(0, &ck, &cv), "AppendFirst view");
    bool same = ck.size() == 16;
    for (int i = 0; same && i < 16; i++) same = f32_from_bf16(ck[i]) == k[i] && f32_from_bf16(cv[i]) == v[i];
    EXPECT(same, "AppendFirst data");
  }
  {  // TestKVCache_AppendGrows  kvcache_test.go:42-66: 1 head, 1 token then 2 tokens -> concatenation
    relux::KVCache c(dev, 1, 16, 1, 8);
    std::vector<float> a(8), b(16);
    for (int i = 0; i < 8; i++) a[i] = (float)(i + 1);
    for (int i = 0; i < 16; i++) b[i] = (float)(i + 9);
    c.Append(0, a.data(), a.data(), 1);
    EXPECT(c.TotalLen(0) == 1, "AppendGrows len 1");
    c.Append(0, b.data(), b.data(), 2);
    EXPECT(c.TotalLen(0) == 3, "AppendGrows len 3");
    std::vector<uint16_t> ck, cv;
    c.View(0, &ck, &cv);
    bool same = ck.size() == 24;
    for (int i = 0; same && i < 24; i++) same = f32_from_bf16(ck[i]) == (float)(i + 1);
    EXPECT(same, "AppendGrows data");
    // TestKVCache_Reset  kvcache_test.go:68-85
    c.Reset();
    EXPECT(c.TotalLen(0) == 0, "Reset len");
    EXPECT(!c.View(0, &ck, &cv), "Reset nil view");
  }
  {  // TestKVCache_BFloat16  kvcache_test.go:87-107
    relux::KVCache c(dev, 1, 16, 1, 8);
    EXPECT(c.GetDType() == relux::DType::BFloat16, "dtype");
    std::vector<float> k = {1, 2, 3, 4, 5, 6, 7, 8};
    c.Append(0, k.data(), k.data(), 1);
    std::vector<uint16_t> ck, cv;
    c.View(0, &ck, &cv);
    bool ok = true;
    for (int i = 0; i < 8; i++) ok = ok && std::fabs(f32_from_bf16(ck[i]) - (float)(i + 1)) <= 0.01f;
    EXPECT(ok, "BFloat16 round trip");
  }
  {  // panics: layer out of range (kvcache.go:241-243), overflow (kvcache.go:282-285)
    relux::KVCache c(dev, 1, 64, 1, 8);
    std::vector<float> k(8 * 64, 1.f);
    bool threw = false;
    try { c.Append(3, k.data(), k.data(), 1); } catch (const relux::Panic& e) { threw = strstr(e.what(), "out of range") != nullptr; }
    EXPECT(threw, "layer out of range panics");
    c.Append(0, k.data(), k.data(), 64);
    threw = false;
    try { c.Append(0, k.data(), k.data(), 1); } catch (const relux::Panic& e) { threw = e.status == RELUX_ERR_OVERFLOW && strstr(e.what(), "overflow") != nullptr; }
    EXPECT(threw, "overflow panics");
  }
  {  // MLACache: append two chunks, view, reset  (mla_cache.go:152-182, 222-233)
    relux::MLACache c(dev, 2, 128, 64, 16);
    std::vector<float> cc(3 * 64), kr(3 * 16);
    for (size_t i = 0; i < cc.size(); i++) cc[i] = (float)(i % 97) * 0.5f;
    for (size_t i = 0; i < kr.size(); i++) kr[i] = (float)(i % 31) - 15.f;
    c.Append(1, cc.data(), kr.data(), 2);
    c.Append(1, cc.data() + 2 * 64, kr.data() + 2 * 16, 1);
    EXPECT(c.TotalLen(1) == 3 && c.TotalLen(0) == 0, "MLACache len");
    std::vector<uint16_t> vc, vk;
    EXPECT(c.View(1, &vc, &vk), "MLACache view");
    bool same = vc.size() == cc.size() && vk.size() == kr.size();
    for (size_t i = 0; same && i < cc.size(); i++) same = f32_from_bf16(vc[i]) == cc[i];
    for (size_t i = 0; same && i < kr.size(); i++) same = f32_from_bf16(vk[i]) == kr[i];
    EXPECT(same, "MLACache data");
    c.Reset();
    EXPECT(c.TotalLen(1) == 0, "MLACache reset");
  }
  {  // MLACache.Step = Append + Attend: the same bits from two caches fed the same rows (16 heads x 128, latent 512, rope 64)
    const int H = 16, Dh = 128, dC = 512, dHR = 64;
    relux::MLACache c1(dev, 1, 256, dC, dHR), c2(dev, 1, 256, dC, dHR);
    uint32_t state = 777u;
    auto next = [&]() { state = state * 1664525u + 1013904223u; return (float)(state >> 8) / 16777216.0f - 0.5f; };
    std::vector<uint16_t> wuk((size_t)dC * H * Dh), wuv((size_t)dC * H * Dh);
    for (auto& v : wuk) v = bf16_from_f32(next() * 0.05f);
    for (auto& v : wuv) v = bf16_from_f32(next() * 0.05f);
    void* d_uk = dev.Upload(wuk.data(), wuk.size() * 2);
    void* d_uv = dev.Upload(wuv.data(), wuv.size() * 2);
    std::vector<float> rows_c((size_t)70 * dC), rows_r((size_t)70 * dHR);
    for (auto& v : rows_c) v = next();
    for (auto& v : rows_r) v = next();
    c1.Append(0, rows_c.data(), rows_r.data(), 70);
    c2.Append(0, rows_c.data(), rows_r.data(), 70);
    bool same = true;
    for (int step = 0; step < 3 && same; step++) {
      std::vector<float> nc(dC), nr(dHR), qc((size_t)H * Dh), qr((size_t)H * dHR), o1((size_t)H * Dh, -1.f), o2((size_t)H * Dh, -2.f);
      for (auto& v : nc) v = next();
      for (auto& v : nr) v = next();
      for (auto& v : qc) v = next();
      for (auto& v : qr) v = next();
      c1.Append(0, nc.data(), nr.data(), 1);
      c1.Attend(0, qc.data(), qr.data(), d_uk, d_uv, o1.data(), H, Dh, 1, 0.0722f, true);
      c2.Step(0, nc.data(), nr.data(), qc.data(), qr.data(), d_uk, d_uv, o2.data(), H, Dh, 0.0722f);
      for (size_t i = 0; same && i < o1.size(); i++) same = o1[i] == o2[i];
      same = same && c1.TotalLen(0) == c2.TotalLen(0);
    }
    EXPECT(same, "MLACache Step equals Append + Attend");
    dev.Free(d_uk); dev.Free(d_uv);
  }
  {  // attention through the mirror: one cached row -> the output is that V row (softmax of one score = 1)
    relux::KVCache c(dev, 1, 64, 1, 128);
    std::vector<float> k(128), v(128), q(128, 0.25f), out(128, -1.f);
    for (int i = 0; i < 128; i++) { k[i] = 0.5f; v[i] = (float)(i % 8); }
    c.Append(0, k.data(), v.data(), 1);
    c.Attend(0, q.data(), out.data(), 1, 1, 0.0884f, true);
    bool same = true;
    for (int i = 0; i < 128; i++) same = same && std::fabs(out[i] - v[i]) < 1e-3f;
    EXPECT(same, "Attend single row");
  }
  {  // the whole layer through the mirror: with Wv = Wo = identity blocks and one cached row the output is x itself
    // (softmax of a single score is 1, so o = v = x Wv = x, out = o Wo = x); dModel 128, one head, no RoPE.
    const int D = 128;
    relux::KVCache c(dev, 1, 64, 1, D);
    std::vector<uint16_t> ident((size_t)D * D, 0), zero((size_t)D * D, 0);
    for (int i = 0; i < D; i++) ident[(size_t)i * D + i] = 0x3F80;   // bf16 1.0
    relux_gqa_layer_weights w;
    w.w_q = dev.Upload(zero.data(), zero.size() * 2);
    w.w_k = dev.Upload(zero.data(), zero.size() * 2);
    w.w_v = dev.Upload(ident.data(), ident.size() * 2);
    w.w_o = dev.Upload(ident.data(), ident.size() * 2);
    std::vector<float> x(D), out(D, -1.f);
    for (int i = 0; i < D; i++) x[i] = (float)(i % 16) * 0.25f;     // exactly representable in bf16
    c.ForwardCached(0, x.data(), out.data(), w, D, 1, 1, true, false, 10000.f, RELUX_ATTN_REFERENCE);
    bool same = c.TotalLen(0) == 1;
    for (int i = 0; i < D; i++) same = same && out[i] == x[i];
    EXPECT(same, "ForwardCached identity layer");
    dev.Free((void*)w.w_q); dev.Free((void*)w.w_k); dev.Free((void*)w.w_v); dev.Free((void*)w.w_o);
  }
  {  // acceptPhase through the mirror: a draft equal to the target is accepted whole, a near-zero temperature makes
    // the bonus token the argmax of the last row, and the commit advances the cache by k + 1 rows; a target without
    // mass on the first draft token rejects it and resamples another token (speculative.go:211-253).
    const int k = 3, V = 512, D = 16;
    relux::KVCache c(dev, 1, 64, 1, D);
    std::vector<float> dl((size_t)k * V), tl((size_t)(k + 1) * V);
    uint32_t state = 12345u;
    auto next = [&]() { state = state * 1664525u + 1013904223u; return (float)(state >> 8) / 16777216.0f; };
    for (auto& v : dl) v = next() * 8.f - 4.f;
    for (int i = 0; i < k * V; i++) tl[i] = dl[i];
    int best = 0;
    for (int j = 0; j < V; j++) { tl[(size_t)k * V + j] = next() * 8.f - 4.f; if (tl[(size_t)k * V + j] > tl[(size_t)k * V + best]) best = j; }
    int32_t toks[k] = {7, 400, 33};
    float draws[k + 1] = {0.3f, 0.9f, 0.5f, 0.7f};
    relux_sampler_params sp{1e-10f, 0, 1.0f, 0.0f};
    int tok = -1;
    int n = c.AcceptPhase(toks, dl.data(), tl.data(), k, V, draws, sp, &tok);
    EXPECT(n == k && tok == best && c.TotalLen(0) == k + 1, "AcceptPhase accepts an identical draft and commits k + 1 rows");
    // Sampler.Sample through the mirror: near-zero temperature is the argmax; a presence penalty on the argmax moves it
    int32_t prevTok[2] = {best, best};
    relux_sampler_params greedy{1e-10f, 0, 1.0f, 0.0f};
    const float* last = tl.data() + (size_t)k * V;
    int second = best == 0 ? 1 : 0;
    for (int j = 0; j < V; j++) if (j != best && last[j] > last[second]) second = j;
    EXPECT(c.Sample(last, V, 0.4f, greedy) == best, "Sample at temperature -> 0 is the argmax");
    EXPECT(c.Sample(last, V, 0.4f, greedy, prevTok, 2, 0.f, 0.f, 100.f) == second, "a presence penalty removes the seen argmax");
    tl[toks[0]] = -90.f;
    n = c.AcceptPhase(toks, dl.data(), tl.data(), k, V, draws, sp, &tok, false);
    EXPECT(n == 0 && tok != toks[0] && tok >= 0 && tok < V && c.TotalLen(0) == k + 1, "AcceptPhase rejects a token the target excludes");
  }
  if (failures == 0) printf("ALL PASSED\n");
  return failures ? 1 : 0;
}
