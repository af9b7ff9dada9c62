"""MLA layer step on the GPU (relux_mla_forward_cached) against the oracle's restatement of MLA.forwardCached
(mla.go:272-397) composed from its pinned pieces: matmul, RoPE tables and rotation, bf16 cache rows, attention.

RELUX_ATTN_REFERENCE must match BIT FOR BIT (outputs and the rows that land in the cache); RELUX_ATTN_FAST
(activations rounded to bf16 for the tensor cores, exact exp2 softmax) within tolerance."""
import numpy as np
import pytest

from tests.helpers import permuted_tables

pytestmark = pytest.mark.gpu

WEIGHTS = ("w_q", "w_qr", "w_dkv", "w_kr", "w_uk", "w_uv", "w_o")


@pytest.fixture(scope="module")
def dev():
    import relux_b200 as rb
    d = rb.Device(0)
    yield d
    d.close()


def make_weights(oracle, rng, D, H, dC, dHR):
    Dh = D // H
    shapes = {"w_q": (D, H * Dh), "w_qr": (D, H * dHR), "w_dkv": (D, dC), "w_kr": (D, dHR), "w_uk": (dC, H * Dh),
              "w_uv": (dC, H * Dh), "w_o": (H * Dh, D)}
    out = {}
    for k in WEIGHTS:
        r, c = shapes[k]
        w = rng.standard_normal((r, c), dtype=np.float32)
        w *= np.float32(1.0 / np.sqrt(r))      # the spread of NewMLA's initialiser (mla.go:86-95)
        out[k] = oracle.bf16_from_f32(w)
    return out


class OracleLayer:
    """Batch of independent sequences, one MLA layer, INTENDED semantics, bf16 cache rows."""

    def __init__(self, oracle, W, D, H, dC, dHR, rope_base, max_pos, causal):
        self.o, self.W, self.D, self.H, self.dC, self.dHR, self.causal = oracle, W, D, H, dC, dHR, causal
        self.Wf = {k: oracle.f32_from_bf16(v) for k, v in W.items() if k not in ("w_uk", "w_uv")}
        self.rope = oracle.Rope(dHR, rope_base, max_pos)
        self.c, self.kr = [], []   # per sequence: bf16 bits [T, dC], [T, dHR]

    def add_sequences(self, n):
        for _ in range(n):
            self.c.append(np.zeros((0, self.dC), np.uint16))
            self.kr.append(np.zeros((0, self.dHR), np.uint16))

    def step(self, x):
        o, H, dC, dHR = self.o, self.H, self.dC, self.dHR
        B, S, D = x.shape
        Dh = D // H
        x2 = np.ascontiguousarray(x.reshape(B * S, D))
        qc = o.matmul(x2, self.Wf["w_q"]).reshape(B, S, H, Dh)
        qr = o.matmul(x2, self.Wf["w_qr"]).reshape(B, S, H, dHR)
        c = o.matmul(x2, self.Wf["w_dkv"]).reshape(B, S, dC)
        kr = o.matmul(x2, self.Wf["w_kr"]).reshape(B, S, dHR)
        qr_rot = np.empty_like(qr)
        for b in range(B):
            start = self.c[b].shape[0]
            qh = np.ascontiguousarray(qr[b].transpose(1, 0, 2))            # [H, S, dHR] like rearrangeBSNH
            qr_rot[b] = self.rope.apply(qh, start, intended_positions=True).transpose(1, 0, 2)
            kb = self.rope.apply(np.ascontiguousarray(kr[b]), start, intended_positions=True)
            self.c[b] = np.concatenate([self.c[b], o.bf16_from_f32(c[b])])
            self.kr[b] = np.concatenate([self.kr[b], o.bf16_from_f32(kb)])
        lens = [a.shape[0] for a in self.c]
        Tm = max(lens)
        ck = np.zeros((B, Tm, dC), np.uint16)
        kk = np.zeros((B, Tm, dHR), np.uint16)
        for b in range(B):
            ck[b, :lens[b]] = self.c[b]
            kk[b, :lens[b]] = self.kr[b]
        scale = float(np.float32(1.0 / np.sqrt(float(Dh + dHR))))
        attn = o.mla_attend(ck, kk, lens, qc, qr_rot, self.W["w_uk"], self.W["w_uv"], scale, causal=self.causal)
        return o.matmul(np.ascontiguousarray(attn.reshape(B * S, H * Dh)), self.Wf["w_o"]).reshape(B, S, D)


def build_pool(dev, rng, B, capacity, dC, dHR, P=64):
    import relux_b200 as rb
    from relux_b200 import lib as L
    pages_per = (capacity + P - 1) // P
    pool = rb.Pool(dev, L.POOL_MLA, 1, B * pages_per, P, B, pages_per, dC=dC, dHR=dHR)
    pool.set_tables(permuted_tables(rng, B, pages_per))
    return pool


def prefill(rng, oracle, pool, ol, lens, dC, dHR):
    """Seeds caches of different lengths with random rows (the same bf16 rows on both sides)."""
    B = len(lens)
    c = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(lens)), dC), dtype=np.float32))
    r = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(lens)), dHR), dtype=np.float32))
    if int(np.sum(lens)) > 0:
        pool.append(0, c, r, B, n_new=np.asarray(lens, np.int32))
    o = 0
    for b, n in enumerate(lens):
        ol.c[b] = c[o:o + n].copy()
        ol.kr[b] = r[o:o + n].copy()
        o += n


def run_steps(dev, oracle, seed, D, H, dC, dHR, lens, steps, mode, causal=True, rope_base=10000.0, capacity=256):
    from relux_b200 import lib as L
    rng = np.random.default_rng(seed)
    B = len(lens)
    W = make_weights(oracle, rng, D, H, dC, dHR)
    dW = {k: dev.upload(v) for k, v in W.items()}
    pool = build_pool(dev, rng, B, capacity, dC, dHR)
    ol = OracleLayer(oracle, W, D, H, dC, dHR, rope_base, capacity, causal)
    ol.add_sequences(B)
    prefill(rng, oracle, pool, ol, lens, dC, dHR)
    results = []
    for S in steps:
        x = rng.standard_normal((B, S, D), dtype=np.float32)
        got = np.empty((B, S, D), np.float32)
        pool.forward_cached(0, B, x, got, dW, D, H, q_tokens=S, causal=causal, rope_base=rope_base, mode=mode)
        ref = ol.step(x)
        results.append((got, ref))
    assert pool.status() == 0
    caches = []
    for b in range(B):
        n = ol.c[b].shape[0]
        assert pool.seq_len(0, b) == n
        gc, gr = pool.read_rows(0, b, 0, n)
        caches.append((gc, gr, ol.c[b], ol.kr[b]))
    pool.destroy()
    for v in dW.values():
        v.free()
    return results, caches


def test_layer_reference_mode_is_bit_exact_small(dev, oracle):
    """config-2 layer shapes (dModel 256, 8 heads, latent 64, rope 16); ragged caches, decode and multi-token steps."""
    from relux_b200 import lib as L
    results, caches = run_steps(dev, oracle, 11, 256, 8, 64, 16, [0, 5, 70], [1, 3, 1], L.ATTN_REFERENCE)
    for got, ref in results:
        assert np.array_equal(got, ref)
    for gc, gr, rc, rr in caches:
        assert np.array_equal(gc, rc) and np.array_equal(gr, rr)


def _close(oracle, got, ref, what):
    rel = np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref)
    err = np.abs(got - ref)
    assert np.isfinite(got).all()
    assert rel <= 2e-2, "%s: relative error %g" % (what, rel)
    assert err.max() <= 2e-2 * max(1.0, float(np.abs(ref).max())), "%s: max-abs %g" % (what, err.max())
    return rel


def test_layer_fast_mode_small(dev, oracle):
    """Same shapes through the tensor-core projections (K = 256: four pipeline steps, column tiles narrower than a box)."""
    from relux_b200 import lib as L
    with oracle.exact_exp():
        results, caches = run_steps(dev, oracle, 12, 256, 8, 64, 16, [1, 64, 129], [1, 2, 1], L.ATTN_FAST)
    for i, (got, ref) in enumerate(results):
        _close(oracle, got, ref, "step %d" % i)
    for gc, gr, rc, rr in caches:   # rows computed from bf16-rounded activations: close, not identical
        d = np.abs(oracle.f32_from_bf16(gc) - oracle.f32_from_bf16(rc))
        assert d.max() <= 0.05 and d.mean() <= 5e-3
        d = np.abs(oracle.f32_from_bf16(gr) - oracle.f32_from_bf16(rr))
        assert d.max() <= 0.05 and d.mean() <= 5e-3


def test_layer_fast_mode_matches_reference_mode_on_device(dev, oracle):
    """FAST and REFERENCE on the same inputs agree within the bf16 tolerance (no oracle involved: the two device paths)."""
    from relux_b200 import lib as L
    a, _ = run_steps(dev, oracle, 13, 256, 8, 64, 16, [17, 40], [1, 1], L.ATTN_FAST)
    b, _ = run_steps(dev, oracle, 13, 256, 8, 64, 16, [17, 40], [1, 1], L.ATTN_REFERENCE)
    for (ga, _), (gb, _) in zip(a, b):
        assert np.linalg.norm(ga - gb) / np.linalg.norm(gb) <= 3e-2


def test_layer_fast_mode_tcgen05_shapes(dev, oracle):
    """128 heads x 128, latent 512, rope 64 (dModel 16384): split-K tensor-core projections feeding the tcgen05 decode."""
    from relux_b200 import lib as L
    with oracle.exact_exp():
        results, _ = run_steps(dev, oracle, 14, 16384, 128, 512, 64, [130, 300], [1], L.ATTN_FAST, capacity=512)
    for i, (got, ref) in enumerate(results):
        _close(oracle, got, ref, "step %d" % i)


def test_layer_fast_mode_prompt_on_the_prefill_kernels(dev, oracle):
    """128 heads x 128, latent 512, rope 64 over dModel 1024, a 150-token prompt after 70 and 0 cached rows: inside relux_mla_forward_cached the attention
    of a prompt expands the cached latents and runs the tcgen05 prefill kernel; a decode step follows on the rows the
    prompt appended."""
    from relux_b200 import lib as L
    with oracle.exact_exp():
        results, _ = run_steps(dev, oracle, 15, 1024, 128, 512, 64, [70, 0], [150, 1], L.ATTN_FAST, capacity=512)
    for i, (got, ref) in enumerate(results):
        _close(oracle, got, ref, "step %d" % i)


def test_layer_errors(dev, oracle):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(1)
    W = make_weights(oracle, rng, 256, 8, 64, 16)
    dW = {k: dev.upload(v) for k, v in W.items()}
    pool = build_pool(dev, rng, 2, 64, 64, 16)
    x = rng.standard_normal((2, 1, 256), dtype=np.float32)
    out = np.empty_like(x)
    with pytest.raises(L.ReluxCudaError) as e:      # dModel not divisible by numHeads (NewMLA panics, mla.go:72-74)
        pool.forward_cached(0, 2, x, out, dW, 256, 7)
    assert e.value.code == L.ERR_INVALID_ARG
    with pytest.raises(L.ReluxCudaError) as e:      # layer out of range
        pool.forward_cached(3, 2, x, out, dW, 256, 8)
    assert e.value.code == L.ERR_INVALID_ARG
    pool.append(0, oracle.bf16_from_f32(rng.standard_normal((128, 64), dtype=np.float32)),
                oracle.bf16_from_f32(rng.standard_normal((128, 16), dtype=np.float32)), 2, n_new=np.asarray([64, 64], np.int32))
    with pytest.raises(L.ReluxCudaError) as e:      # capacity 64 is full (MLACache.Append panics, mla_cache.go:160-164)
        pool.forward_cached(0, 2, x, out, dW, 256, 8)
    assert e.value.code == L.ERR_OVERFLOW
    pool.destroy()
    for v in dW.values():
        v.free()


# ------------------------------------------------------------------------------------------------ GQA layer step
class OracleGqaLayer:
    """MHA.forwardCached (mha.go:245-369) for a batch of independent sequences, INTENDED semantics, bf16 cache rows."""

    def __init__(self, oracle, W, D, H, Hkv, rope_base, max_pos, causal, rope=True):
        self.o, self.W, self.D, self.H, self.Hkv, self.causal = oracle, W, D, H, Hkv, causal
        self.hd = D // H
        self.Wf = {k: oracle.f32_from_bf16(v) for k, v in W.items()}
        self.rope = oracle.Rope(self.hd, rope_base, max_pos) if rope else None
        self.k, self.v = [], []

    def add_sequences(self, n):
        for _ in range(n):
            self.k.append(np.zeros((0, self.Hkv, self.hd), np.uint16))
            self.v.append(np.zeros((0, self.Hkv, self.hd), np.uint16))

    def step(self, x, keep=None):
        """keep[b] = rows of this step that stay in the cache (None: all; speculative verify commits a prefix)."""
        o, H, Hkv, hd = self.o, self.H, self.Hkv, self.hd
        B, S, D = x.shape
        x2 = np.ascontiguousarray(x.reshape(B * S, D))
        q = o.matmul(x2, self.Wf["w_q"]).reshape(B, S, H, hd)
        k = o.matmul(x2, self.Wf["w_k"]).reshape(B, S, Hkv, hd)
        v = o.matmul(x2, self.Wf["w_v"]).reshape(B, S, Hkv, hd)
        if self.rope is not None:
            for b in range(B):
                start = self.k[b].shape[0]
                q[b] = self.rope.apply(np.ascontiguousarray(q[b].transpose(1, 0, 2)), start, intended_positions=True).transpose(1, 0, 2)
                k[b] = self.rope.apply(np.ascontiguousarray(k[b].transpose(1, 0, 2)), start, intended_positions=True).transpose(1, 0, 2)
        full_k = [np.concatenate([self.k[b], o.bf16_from_f32(k[b])]) for b in range(B)]
        full_v = [np.concatenate([self.v[b], o.bf16_from_f32(v[b])]) for b in range(B)]
        lens = [a.shape[0] for a in full_k]
        Tm = max(lens)
        Kp = np.zeros((B, Tm, Hkv, hd), np.uint16)
        Vp = np.zeros_like(Kp)
        for b in range(B):
            Kp[b, :lens[b]] = full_k[b]
            Vp[b, :lens[b]] = full_v[b]
        scale = float(np.float32(1.0 / np.sqrt(float(hd))))
        attn = o.gqa_attend(Kp, Vp, lens, q, scale, causal=self.causal)
        for b in range(B):
            n = S if keep is None else int(keep[b])
            self.k[b] = full_k[b][:lens[b] - S + n]
            self.v[b] = full_v[b][:lens[b] - S + n]
        return o.matmul(np.ascontiguousarray(attn.reshape(B * S, H * hd)), self.Wf["w_o"]).reshape(B, S, D)


def make_gqa_weights(oracle, rng, D, H, Hkv):
    hd = D // H
    shapes = {"w_q": (D, H * hd), "w_k": (D, Hkv * hd), "w_v": (D, Hkv * hd), "w_o": (H * hd, D)}
    return {k: oracle.bf16_from_f32(rng.standard_normal(sh, dtype=np.float32) * np.float32(1.0 / np.sqrt(sh[0]))) for k, sh in shapes.items()}


def build_gqa_pool(dev, rng, B, capacity, Hkv, hd, P=64):
    import relux_b200 as rb
    from relux_b200 import lib as L
    pages_per = (capacity + P - 1) // P
    pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages_per, P, B, pages_per, num_kv_heads=Hkv, head_dim=hd)
    pool.set_tables(permuted_tables(rng, B, pages_per))
    return pool


def gqa_prefill(rng, oracle, pool, ol, lens):
    B = len(lens)
    K = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(lens)), ol.Hkv, ol.hd), dtype=np.float32))
    V = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(lens)), ol.Hkv, ol.hd), dtype=np.float32))
    if int(np.sum(lens)) > 0:
        pool.append(0, K, V, B, n_new=np.asarray(lens, np.int32))
    o = 0
    for b, n in enumerate(lens):
        ol.k[b], ol.v[b] = K[o:o + n].copy(), V[o:o + n].copy()
        o += n


@pytest.mark.parametrize("rope", [True, False])
def test_gqa_layer_reference_mode_is_bit_exact_small(dev, oracle, rope):
    """config-1 layer shapes (dModel 64, 4 heads, 2 kv heads, head_dim 16): outputs and cache rows, bit for bit."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(31)
    D, H, Hkv, B = 64, 4, 2, 3
    W = make_gqa_weights(oracle, rng, D, H, Hkv)
    dW = {k: dev.upload(v) for k, v in W.items()}
    pool = build_gqa_pool(dev, rng, B, 128, Hkv, D // H)
    ol = OracleGqaLayer(oracle, W, D, H, Hkv, 10000.0, 128, True, rope=rope)
    ol.add_sequences(B)
    gqa_prefill(rng, oracle, pool, ol, [0, 7, 66])
    for S in (1, 3, 1):
        x = rng.standard_normal((B, S, D), dtype=np.float32)
        got = np.empty_like(x)
        pool.forward_cached(0, B, x, got, dW, D, H, q_tokens=S, mode=L.ATTN_REFERENCE, rope=rope)
        assert np.array_equal(got, ol.step(x))
    for b in range(B):
        n = ol.k[b].shape[0]
        assert pool.seq_len(0, b) == n
        gk, gv = pool.read_rows(0, b, 0, n)
        assert np.array_equal(gk, ol.k[b]) and np.array_equal(gv, ol.v[b])
    assert pool.status() == 0
    with pytest.raises(L.ReluxCudaError) as e:     # the tensor-core kernels do not cover head_dim 16: refused before any write
        pool.forward_cached(0, B, x, got, dW, D, H, q_tokens=1, mode=L.ATTN_FAST, rope=rope)
    assert e.value.code == L.ERR_UNSUPPORTED and pool.seq_len(0, 0) == ol.k[0].shape[0]
    pool.destroy()
    for v in dW.values():
        v.free()


def test_gqa_layer_fast_decode_and_verify(dev, oracle):
    """config-5 layer shapes (dModel 4096, 32 heads, 8 kv heads, head_dim 128): a decode step, then speculative verify
    steps of 4 draft tokens (rows left past the cursor) with an accepted prefix committed afterwards."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(32)
    D, H, Hkv, B, S = 4096, 32, 8, 3, 4
    W = make_gqa_weights(oracle, rng, D, H, Hkv)
    dW = {k: dev.upload(v) for k, v in W.items()}
    pool = build_gqa_pool(dev, rng, B, 320, Hkv, D // H)
    ol = OracleGqaLayer(oracle, W, D, H, Hkv, 10000.0, 320, True)
    ol.add_sequences(B)
    gqa_prefill(rng, oracle, pool, ol, [100, 64, 190])
    x = rng.standard_normal((B, 1, D), dtype=np.float32)
    got = np.empty_like(x)
    pool.forward_cached(0, B, x, got, dW, D, H, q_tokens=1)
    with oracle.exact_exp():
        ref = ol.step(x)
    _close(oracle, got, ref, "gqa layer decode")
    for step in range(2):
        x = rng.standard_normal((B, S, D), dtype=np.float32)
        got = np.empty_like(x)
        lens = np.array([pool.seq_len(0, b) for b in range(B)], np.int32)
        pool.forward_cached(0, B, x, got, dW, D, H, q_tokens=S, advance=False)
        accepted = rng.integers(1, S + 1, B).astype(np.int32)
        with oracle.exact_exp():
            ref = ol.step(x, keep=accepted)
        _close(oracle, got, ref, "gqa layer verify %d" % step)
        assert all(pool.seq_len(0, b) == lens[b] for b in range(B))     # verify leaves the cursors alone
        pool.set_len(0, lens + accepted)
        for b in range(B):
            assert pool.seq_len(0, b) == ol.k[b].shape[0]
    assert pool.status() == 0
    pool.destroy()
    for v in dW.values():
        v.free()


def test_gqa_layer_fast_more_rows_than_one_mma_tile(dev, oracle):
    """40 sequences x 4 new tokens = 160 activation rows: the projection GEMM runs two 128-row blocks (the second one
    partly out of range), with two heads of 128 on one kv head."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(33)
    D, H, Hkv, B, S = 256, 2, 1, 40, 4
    W = make_gqa_weights(oracle, rng, D, H, Hkv)
    dW = {k: dev.upload(v) for k, v in W.items()}
    pool = build_gqa_pool(dev, rng, B, 192, Hkv, D // H)
    ol = OracleGqaLayer(oracle, W, D, H, Hkv, 10000.0, 192, True)
    ol.add_sequences(B)
    gqa_prefill(rng, oracle, pool, ol, [int(x) for x in rng.integers(0, 150, B)])
    x = rng.standard_normal((B, S, D), dtype=np.float32)
    got = np.empty_like(x)
    pool.forward_cached(0, B, x, got, dW, D, H, q_tokens=S)
    with oracle.exact_exp():
        ref = ol.step(x)
    _close(oracle, got, ref, "gqa layer 160 rows")
    assert pool.status() == 0
    pool.destroy()
    for v in dW.values():
        v.free()
