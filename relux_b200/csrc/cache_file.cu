// One sequence's cache <-> a file in the layout of the reference's file-backed caches, so that a cache can be
// checkpointed and picked up again (the reference maps such files with MAP_SHARED for crash recovery):
//   KV cache   NewKVCacheFile  (internal/transformer/kvcache.go:104-166): per layer the K tensor
//              [1, numKVHeads, maxLen, headDim] followed by the V tensor of the same shape, bf16;
//   MLA cache  NewMLACacheFile (internal/transformer/mla_cache.go:63-113): per layer C_KV [1, maxLen, dC] followed by
//              K_R [1, maxLen, dHR], float32 (the pool's bf16 rows are widened on the way out and rounded with the
//              reference's rule on the way in).
// Rows past a layer's length are written as zeros.  Like the reference's files these carry no lengths: the cursor
// lives with the caller, which passes the per-layer lengths back in when it loads.
// Host-side code over the library's own entry points (relux_pool_read_rows, relux_*_append, relux_seq_set_len).
#include <cstdio>
#include <vector>
#include "internal.h"

namespace relux {
namespace {
struct FileCloser {
  FILE* f;
  ~FileCloser() { if (f) fclose(f); }
};
}  // namespace
}  // namespace relux

using namespace relux;

extern "C" __attribute__((visibility("default"))) int32_t relux_seq_save_file(relux_pool_t h, int32_t seq, const char* path, int32_t max_len) {
  Pool* p = (Pool*)h;
  if (!p || p->magic != kPoolMagic) { set_error("bad pool handle"); return RELUX_ERR_BAD_HANDLE; }
  const relux_pool_params& prm = p->prm;
  if (!path || max_len <= 0) { set_error("save_file: nil path or maxLen=%d, must be > 0", max_len); return RELUX_ERR_INVALID_ARG; }
  std::vector<int32_t> len(prm.num_layers);
  for (int l = 0; l < prm.num_layers; l++) {
    int32_t rc = relux_seq_len(h, l, seq, &len[l]);
    if (rc) return rc;
    if (len[l] > max_len) {
      set_error("save_file: layer %d holds %d rows, more than maxLen=%d", l, len[l], max_len);
      return RELUX_ERR_OVERFLOW;
    }
  }
  FileCloser fc{fopen(path, "wb")};
  if (!fc.f) { set_error("save_file: cannot open %s for writing", path); return RELUX_ERR_INVALID_ARG; }
  const bool mla = prm.kind == RELUX_POOL_MLA;
  const int wa = mla ? prm.mla_dc : prm.gqa_num_kv_heads * prm.gqa_head_dim;
  const int wb = mla ? prm.mla_dhr : wa;
  std::vector<uint16_t> a, b;
  for (int l = 0; l < prm.num_layers; l++) {
    const int n = len[l];
    a.assign((size_t)n * wa, 0);
    b.assign((size_t)n * wb, 0);
    if (n > 0) {
      relux_read_rows_args rr{};
      rr.layer = l; rr.seq_id = seq; rr.tok0 = 0; rr.n_tokens = n; rr.dst_a = a.data(); rr.dst_b = b.data();
      int32_t rc = relux_pool_read_rows(h, &rr);
      if (rc) return rc;
    }
    if (mla) {
      for (int which = 0; which < 2; which++) {
        const std::vector<uint16_t>& src = which ? b : a;
        const int w = which ? wb : wa;
        std::vector<float> out((size_t)max_len * w, 0.f);
        for (size_t i = 0; i < (size_t)n * w; i++) {
          const uint32_t u = (uint32_t)src[i] << 16;
          memcpy(&out[i], &u, 4);
        }
        if (fwrite(out.data(), 4, out.size(), fc.f) != out.size()) { set_error("save_file: short write to %s", path); return RELUX_ERR_INVALID_ARG; }
      }
    } else {
      const int Hkv = prm.gqa_num_kv_heads, D = prm.gqa_head_dim;
      for (int which = 0; which < 2; which++) {
        const std::vector<uint16_t>& src = which ? b : a;   // [n][Hkv][D]
        std::vector<uint16_t> out((size_t)Hkv * max_len * D, 0);
        for (int t = 0; t < n; t++)
          for (int hh = 0; hh < Hkv; hh++)
            memcpy(&out[((size_t)hh * max_len + t) * D], &src[((size_t)t * Hkv + hh) * D], (size_t)D * 2);
        if (fwrite(out.data(), 2, out.size(), fc.f) != out.size()) { set_error("save_file: short write to %s", path); return RELUX_ERR_INVALID_ARG; }
      }
    }
  }
  return RELUX_OK;
}

extern "C" __attribute__((visibility("default"))) int32_t relux_seq_load_file(relux_pool_t h, int32_t seq, const char* path, int32_t max_len,
                                                                            const int32_t* layer_len) {
  Pool* p = (Pool*)h;
  if (!p || p->magic != kPoolMagic) { set_error("bad pool handle"); return RELUX_ERR_BAD_HANDLE; }
  const relux_pool_params& prm = p->prm;
  if (!path || !layer_len || max_len <= 0) { set_error("load_file: nil argument or maxLen=%d, must be > 0", max_len); return RELUX_ERR_INVALID_ARG; }
  for (int l = 0; l < prm.num_layers; l++)
    if (layer_len[l] < 0 || layer_len[l] > max_len) {
      set_error("load_file: layer %d length %d outside [0, maxLen=%d]", l, layer_len[l], max_len);
      return RELUX_ERR_INVALID_ARG;
    }
  FileCloser fc{fopen(path, "rb")};
  if (!fc.f) { set_error("load_file: cannot open %s", path); return RELUX_ERR_INVALID_ARG; }
  const bool mla = prm.kind == RELUX_POOL_MLA;
  const int32_t zero = 0;
  int32_t rc = relux_seq_set_len(h, -1, 1, &seq, &zero);
  if (rc) return rc;
  for (int l = 0; l < prm.num_layers; l++) {
    const int n = layer_len[l];
    relux_append_args ap;
    memset(&ap, 0, sizeof(ap));
    ap.layer = l;
    ap.n_seqs = 1;
    ap.seq_ids = &seq;
    ap.n_new = &n;
    ap.mem = RELUX_MEM_HOST;
    ap.layout = RELUX_LAYOUT_TOKEN_MAJOR;
    ap.advance = 1;
    if (mla) {
      std::vector<float> c((size_t)max_len * prm.mla_dc), kr((size_t)max_len * prm.mla_dhr);
      if (fread(c.data(), 4, c.size(), fc.f) != c.size() || fread(kr.data(), 4, kr.size(), fc.f) != kr.size()) {
        set_error("load_file: %s is shorter than %d layers of maxLen=%d", path, prm.num_layers, max_len);
        return RELUX_ERR_INVALID_ARG;
      }
      if (n == 0) continue;
      ap.a = c.data();
      ap.b = kr.data();
      ap.dtype = RELUX_DTYPE_F32;
      rc = relux_mla_append(h, &ap);
      if (rc) return rc;
      rc = relux_cuda_sync((relux_device_t)p->dev);   // the host vectors go out of scope
      if (rc) return rc;
    } else {
      const int Hkv = prm.gqa_num_kv_heads, D = prm.gqa_head_dim;
      std::vector<uint16_t> in((size_t)Hkv * max_len * D), k((size_t)n * Hkv * D), v((size_t)n * Hkv * D);
      for (int which = 0; which < 2; which++) {
        if (fread(in.data(), 2, in.size(), fc.f) != in.size()) {
          set_error("load_file: %s is shorter than %d layers of maxLen=%d", path, prm.num_layers, max_len);
          return RELUX_ERR_INVALID_ARG;
        }
        std::vector<uint16_t>& dst = which ? v : k;
        for (int t = 0; t < n; t++)
          for (int hh = 0; hh < Hkv; hh++)
            memcpy(&dst[((size_t)t * Hkv + hh) * D], &in[((size_t)hh * max_len + t) * D], (size_t)D * 2);
      }
      if (n == 0) continue;
      ap.a = k.data();
      ap.b = v.data();
      ap.dtype = RELUX_DTYPE_BF16;
      rc = relux_gqa_append(h, &ap);
      if (rc) return rc;
      rc = relux_cuda_sync((relux_device_t)p->dev);
      if (rc) return rc;
    }
  }
  return RELUX_OK;
}
