"""Shared builders for the GPU parity tests: seeded logical caches, permuted page tables, tolerances."""
import numpy as np

# north_star tolerance for bf16 attention outputs
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def have_gpu():
    try:
        from relux_b200 import lib as L
        import ctypes as C
        n = C.c_int32()
        return L.load().relux_cuda_device_count(C.byref(n)) == 0 and n.value > 0
    except Exception:
        return False


def check_attention(got, ref, what="", bf16_output=False, max_tol=MAX_ABS_TOL, mean_tol=MEAN_ABS_TOL):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    if bf16_output:
        # an output stored as bf16 carries half an ulp (2^-8 relative) of its own magnitude
        err = np.maximum(err - np.abs(ref) * 2.0 ** -8, 0.0)
    rel = np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30)
    assert np.isfinite(got).all(), "%s: non-finite output" % what
    assert err.max() <= max_tol, "%s: max-abs %g > %g (rel %g)" % (what, err.max(), max_tol, rel)
    assert err.mean() <= mean_tol, "%s: mean-abs %g > %g (rel %g)" % (what, err.mean(), mean_tol, rel)
    # the outputs are small numbers; the relative error gives the check teeth
    assert rel <= 5e-2, "%s: relative error %g" % (what, rel)
    return err.max(), err.mean(), rel


def permuted_tables(rng, n_seqs, pages_per_seq, num_pages=None):
    num_pages = num_pages or n_seqs * pages_per_seq
    perm = rng.permutation(num_pages).astype(np.int32)
    return perm[: n_seqs * pages_per_seq].reshape(n_seqs, pages_per_seq)


def ragged_to_padded(rows, lens, width_shape):
    """rows: [sum(lens), ...] -> [B, max(lens), ...] zero padded."""
    B, Tm = len(lens), int(max(lens))
    out = np.zeros((B, Tm) + tuple(width_shape), rows.dtype)
    o = 0
    for b, n in enumerate(lens):
        out[b, :n] = rows[o:o + n]
        o += n
    return out


# ---- the two CPU-runnable model configurations ------------------------------------------------
def model_config(name):
    from oracle import binding as orc
    if name == "config1":
        return orc.ModelCfg(vocab=100, dModel=64, numHeads=4, numKVHeads=2, numLayers=2, dFF=128, maxSeqLen=64, ropeBase=10000.0,
                            causal=1, swiglu=1, mla=0, dC=0, dHR=0)
    if name == "config2":
        # 8 heads x (content 32 + rope 16), value dim 32, latent 64; the benchmark names no FFN type: GELU, the reference default
        return orc.ModelCfg(vocab=1024, dModel=256, numHeads=8, numKVHeads=8, numLayers=4, dFF=512, maxSeqLen=512, ropeBase=10000.0,
                            causal=1, swiglu=0, mla=1, dC=64, dHR=16)
    raise KeyError(name)


def model_weights(cfg, seed=0, std=0.02):
    from oracle import binding as orc
    n = orc.Model.weight_count(cfg)
    rng = np.random.default_rng(seed)
    return orc.bf16_from_f32((rng.standard_normal(n, dtype=np.float32) * np.float32(std)))


def prompts_for(name, seed=1):
    rng = np.random.default_rng(seed)
    if name == "config1":
        return [rng.integers(0, 100, 8).astype(np.int32)]
    if name == "config2":
        return [rng.integers(0, 1024, 32).astype(np.int32) for _ in range(4)]
    raise KeyError(name)


def layer_weight_offsets(cfg):
    """Element offsets of W_UK / W_UV of every layer inside the flat weight buffer (order documented in
    oracle/relux_oracle.cpp): used to hand the MLA up-projections to the GPU."""
    D, H, F, V = cfg.dModel, cfg.numHeads, cfg.dFF, cfg.vocab
    hd = D // H
    off = V * D
    out = []
    for _ in range(cfg.numLayers):
        if cfg.mla:
            o_wq = off
            o_dkv = o_wq + D * H * hd
            o_uk = o_dkv + D * cfg.dC
            o_uv = o_uk + cfg.dC * H * hd
            o_kr = o_uv + cfg.dC * H * hd
            o_qr = o_kr + D * cfg.dHR
            o_o = o_qr + D * H * cfg.dHR
            off = o_o + H * hd * D
            out.append((o_uk, o_uv))
        else:
            off += D * H * hd + 2 * D * cfg.numKVHeads * hd + H * hd * D
            out.append(None)
        off += D * F * (2 if cfg.swiglu else 1) + F * D
    return out


class GpuAttention:
    """Plugs the CUDA library into the oracle's decoder forward at the reference's seam: the cache object
    (Append / TotalLen) plus the attention loops of forwardCached.  Everything else of the forward
    (projections, RoPE, norms, MLP, lm head, greedy pick) stays the CPU restatement."""

    def __init__(self, dev, cfg, weights, mode):
        import ctypes as C
        import relux_b200 as rb
        from relux_b200 import lib as L
        self.C, self.cfg, self.mode, self.dev = C, cfg, mode, dev
        self.hd = cfg.dModel // cfg.numHeads
        compat = mode == L.ATTN_REFERENCE_FAITHFUL
        if cfg.mla:
            self.cache = rb.MLACache(dev, cfg.numLayers, cfg.maxSeqLen, cfg.dC, cfg.dHR, reference_compat=compat)
            self.w = [(dev.upload(weights[a:a + cfg.dC * cfg.numHeads * self.hd]), dev.upload(weights[b:b + cfg.dC * cfg.numHeads * self.hd]))
                      for a, b in layer_weight_offsets(cfg)]
            self.scale = float(np.float32(1.0 / np.sqrt(np.float64(self.hd + cfg.dHR))))
        else:
            self.cache = rb.KVCache(dev, cfg.numLayers, cfg.maxSeqLen, cfg.numKVHeads, self.hd, reference_compat=compat)
            self.scale = float(np.float32(1.0 / np.sqrt(np.float64(self.hd))))

    def reset(self):
        self.cache.Reset()

    def _arr(self, ptr, shape):
        return np.ctypeslib.as_array(ptr, shape=shape)

    def mha_hook(self, user, layer, S, start_pos, q, k, v, out):
        cfg, hd = self.cfg, self.hd
        try:
            assert self.cache.TotalLen(layer) == start_pos
            self.cache.Append(layer, self._arr(k, (1, cfg.numKVHeads, S, hd)), self._arr(v, (1, cfg.numKVHeads, S, hd)))
            o = self.cache.attend(layer, self._arr(q, (1, cfg.numHeads, S, hd)), self.scale, causal=bool(cfg.causal), mode=self.mode)
            self._arr(out, (1, cfg.numHeads, S, hd))[...] = o
            return 0
        except Exception as e:  # noqa: BLE001 - must not propagate through the C callback
            self.error = e
            return -100

    def mla_hook(self, user, layer, S, start_pos, qc, qr, ckv, kr, out):
        cfg, hd = self.cfg, self.hd
        try:
            assert self.cache.TotalLen(layer) == start_pos
            self.cache.Append(layer, self._arr(ckv, (1, S, cfg.dC)), self._arr(kr, (1, S, cfg.dHR)))
            wuk, wuv = self.w[layer]
            o = self.cache.attend(layer, self._arr(qc, (1, cfg.numHeads, S, hd)), self._arr(qr, (1, cfg.numHeads, S, cfg.dHR)), wuk, wuv,
                                  self.scale, causal=bool(cfg.causal), mode=self.mode)
            self._arr(out, (1, cfg.numHeads, S, hd))[...] = o
            return 0
        except Exception as e:  # noqa: BLE001
            self.error = e
            return -100

    def close(self):
        self.cache.close()
        if self.cfg.mla:
            for a, b in self.w:
                a.free(); b.free()


def layer_weight_arrays(cfg, weights):
    """Per layer, the attention weight matrices as slices of the flat buffer (order documented in
    oracle/relux_oracle.cpp, ro_model_new), keyed like the arguments of Pool.forward_cached."""
    D, H, F, V = cfg.dModel, cfg.numHeads, cfg.dFF, cfg.vocab
    hd = D // H
    off = V * D
    out = []

    def take(n):
        nonlocal off
        a = weights[off:off + n]
        off += n
        return a

    for _ in range(cfg.numLayers):
        if cfg.mla:
            d = {"w_q": take(D * H * hd), "w_dkv": take(D * cfg.dC), "w_uk": take(cfg.dC * H * hd), "w_uv": take(cfg.dC * H * hd),
                 "w_kr": take(D * cfg.dHR), "w_qr": take(D * H * cfg.dHR), "w_o": take(H * hd * D)}
        else:
            d = {"w_q": take(D * H * hd), "w_k": take(D * cfg.numKVHeads * hd), "w_v": take(D * cfg.numKVHeads * hd), "w_o": take(H * hd * D)}
        out.append(d)
        off += D * F * (2 if cfg.swiglu else 1) + F * D
    return out


class GpuLayer:
    """Plugs the CUDA library into the oracle's decoder forward one level higher than GpuAttention: the whole
    MHA.forwardCached / MLA.forwardCached (projections, RoPE, cache append, attention, output projection) is one
    relux_*_forward_cached call; norms, MLP, lm head and the greedy pick stay the CPU restatement."""

    def __init__(self, dev, cfg, weights, mode, page_tokens=64):
        import relux_b200 as rb
        from relux_b200 import lib as L
        self.cfg, self.mode, self.dev, self.error = cfg, mode, dev, None
        pages = (cfg.maxSeqLen + page_tokens - 1) // page_tokens
        hd = cfg.dModel // cfg.numHeads
        compat = mode == L.ATTN_REFERENCE_FAITHFUL
        if cfg.mla:
            self.pool = rb.Pool(dev, L.POOL_MLA, cfg.numLayers, pages, page_tokens, 1, pages, dC=cfg.dC, dHR=cfg.dHR, reference_compat=compat)
        else:
            self.pool = rb.Pool(dev, L.POOL_GQA, cfg.numLayers, pages, page_tokens, 1, pages, num_kv_heads=cfg.numKVHeads, head_dim=hd,
                                reference_compat=compat)
        self.pool.set_tables(np.arange(pages, dtype=np.int32)[::-1].copy().reshape(1, pages))
        self.w = [{k: dev.upload(np.ascontiguousarray(v)) for k, v in d.items()} for d in layer_weight_arrays(cfg, weights)]

    def hook(self, user, layer, S, x, out):
        cfg = self.cfg
        try:
            xa = np.ctypeslib.as_array(x, shape=(1, S, cfg.dModel))
            oa = np.ctypeslib.as_array(out, shape=(1, S, cfg.dModel))
            res = np.empty((1, S, cfg.dModel), np.float32)
            # the model's MLA rotary embedding has base 10000 (transformer_block.go:70-75); MHA uses the configured base
            base = 10000.0 if cfg.mla else float(cfg.ropeBase)
            self.pool.forward_cached(layer, 1, np.ascontiguousarray(xa), res, self.w[layer], cfg.dModel, cfg.numHeads, q_tokens=S,
                                     causal=bool(cfg.causal), rope_base=base, mode=self.mode)
            oa[...] = res
            return 0
        except Exception as e:  # noqa: BLE001 - must not propagate through the C callback
            self.error = e
            return -100

    def close(self):
        self.pool.destroy()
        for d in self.w:
            for b in d.values():
                b.free()
