"""Randomised differential tests on the device: the FAST kernels against the REFERENCE-arithmetic kernels (which are
themselves bit-exact against the oracle, tests/test_gpu_attention.py) over random batch sizes, ragged lengths, page
placements, query-token counts and head counts.  Aimed at the scheduling arithmetic: item boundaries inside tiles, odd
page counts, ranges that hold several sequences, sequences cut over many ranges."""
import numpy as np
import pytest

from tests.helpers import permuted_tables

pytestmark = pytest.mark.gpu

# The REFERENCE kernels carry the reference's fastexp32 (-3.3 % .. +2.7 % per softmax weight); at a few dozen cached
# tokens that alone moves an output by about 2 % of its size (measured: up to 4.4e-2 absolute on unit-variance values),
# so the bounds here are relative-first and sit above the stated 2e-2 / 2e-3, which tests/test_gpu_attention.py checks
# against the exact-exp oracle.  A scheduling mistake shows as an error of the order of the values themselves.
MAX_ABS, MEAN_ABS, REL = 8e-2, 8e-3, 5e-2


def _check(fast, ref, what):
    err = np.abs(fast - ref)
    rel = np.linalg.norm(fast.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30)
    assert np.isfinite(fast).all(), what
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS and rel <= REL, "%s: max %g mean %g rel %g" % (what, err.max(), err.mean(), rel)


@pytest.fixture(scope="module")
def dev():
    import relux_b200 as rb
    d = rb.Device(0)
    yield d
    d.close()


def _lengths(rng, B, S, hi):
    kind = rng.integers(0, 4)
    if kind == 0:
        lens = rng.integers(S, max(S + 1, hi), B)
    elif kind == 1:                                   # around page and tile boundaries
        lens = rng.choice([63, 64, 65, 127, 128, 129, 191, 192, 193, 256, 257], B) + rng.integers(0, 2, B) * 128
    elif kind == 2:                                   # one long sequence among short ones
        lens = rng.integers(S, max(S + 1, 80), B)
        lens[rng.integers(0, B)] = hi
    else:
        lens = np.full(B, rng.integers(S, max(S + 1, hi)))
    return np.maximum(lens, S).astype(np.int32)


@pytest.mark.parametrize("trial", range(12))
def test_mla_fast_against_reference_kernels(dev, oracle, trial):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(1000 + trial)
    H = int(rng.choice([16, 48, 128]))
    Dh, dC, dHR, P = 128, 512, 64, 64
    B = int(rng.integers(1, 40))
    S = int(rng.choice([1, 1, 2, 4, 9]))
    lens = _lengths(rng, B, S, int(rng.choice([300, 1500, 5000])))
    pages_per = (int(lens.max()) + P - 1) // P + 1
    pool = rb.Pool(dev, L.POOL_MLA, 1, B * pages_per, P, B, pages_per, dC=dC, dHR=dHR)
    pool.set_tables(permuted_tables(rng, B, pages_per))
    n = int(lens.sum())
    pool.append(0, oracle.bf16_from_f32(rng.standard_normal((n, dC), dtype=np.float32)),
                oracle.bf16_from_f32(rng.standard_normal((n, dHR), dtype=np.float32)), B, n_new=lens)
    wuk = dev.upload(oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02))
    wuv = dev.upload(oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02))
    qc = rng.standard_normal((B, S, H, Dh), dtype=np.float32)
    qr = rng.standard_normal((B, S, H, dHR), dtype=np.float32)
    scale = float(1.0 / np.sqrt(Dh + dHR))
    causal = bool(rng.integers(0, 2)) or S == 1
    fast, ref = np.empty_like(qc), np.empty_like(qc)
    pool.decode(0, B, qc, fast, H, Dh, scale, q_rope=qr, w_uk=wuk, w_uv=wuv, q_tokens=S, causal=causal)
    pool.decode(0, B, qc, ref, H, Dh, scale, q_rope=qr, w_uk=wuk, w_uv=wuv, q_tokens=S, causal=causal, mode=L.ATTN_REFERENCE)
    assert pool.status() == 0
    _check(fast, ref, "trial %d: B=%d S=%d H=%d causal=%s lens=%s" % (trial, B, S, H, causal, lens.tolist()[:8]))
    pool.destroy(); wuk.free(); wuv.free()


@pytest.mark.parametrize("trial", range(8))
def test_gqa_fast_against_reference_kernels(dev, oracle, trial):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(2000 + trial)
    Hkv, D, P = int(rng.choice([1, 2, 8])), 128, 64
    H = Hkv * int(rng.choice([1, 4, 8]))
    B = int(rng.integers(1, 24))
    S = int(rng.choice([1, 2, 4, 11]))
    lens = _lengths(rng, B, S, int(rng.choice([300, 2000])))
    pages_per = (int(lens.max()) + P - 1) // P + 1
    pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages_per, P, B, pages_per, num_kv_heads=Hkv, head_dim=D)
    pool.set_tables(permuted_tables(rng, B, pages_per))
    n = int(lens.sum())
    pool.append(0, oracle.bf16_from_f32(rng.standard_normal((n, Hkv, D), dtype=np.float32)),
                oracle.bf16_from_f32(rng.standard_normal((n, Hkv, D), dtype=np.float32)), B, n_new=lens)
    q = rng.standard_normal((B, S, H, D), dtype=np.float32)
    scale = float(1.0 / np.sqrt(D))
    causal = bool(rng.integers(0, 2)) or S == 1
    fast, ref = np.empty_like(q), np.empty_like(q)
    pool.decode(0, B, q, fast, H, D, scale, q_tokens=S, causal=causal)
    pool.decode(0, B, q, ref, H, D, scale, q_tokens=S, causal=causal, mode=L.ATTN_REFERENCE)
    assert pool.status() == 0
    _check(fast, ref, "trial %d: B=%d S=%d H=%d Hkv=%d causal=%s lens=%s" % (trial, B, S, H, Hkv, causal, lens.tolist()[:8]))
    pool.destroy()


@pytest.mark.parametrize("trial", range(5))
def test_gqa_prompt_fast_against_reference_kernels(dev, oracle, trial):
    """Multi-token calls longer than one group of query tokens (prompts): the groups run as slices of one grid over
    chunks of random cached lengths; causal and not."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(2500 + trial)
    Hkv, D, P = int(rng.choice([1, 2, 8])), 128, 64
    H = Hkv * int(rng.choice([1, 4, 8]))
    B = int(rng.integers(1, 7))
    S = int(rng.choice([17, 40, 97, 130]))
    lens = _lengths(rng, B, S, int(rng.choice([300, 700])))
    pages_per = (int(lens.max()) + P - 1) // P + 1
    pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages_per, P, B, pages_per, num_kv_heads=Hkv, head_dim=D)
    pool.set_tables(permuted_tables(rng, B, pages_per))
    n = int(lens.sum())
    pool.append(0, oracle.bf16_from_f32(rng.standard_normal((n, Hkv, D), dtype=np.float32)),
                oracle.bf16_from_f32(rng.standard_normal((n, Hkv, D), dtype=np.float32)), B, n_new=lens)
    q = rng.standard_normal((B, S, H, D), dtype=np.float32)
    scale = float(1.0 / np.sqrt(D))
    causal = bool(rng.integers(0, 4))
    fast, ref = np.empty_like(q), np.empty_like(q)
    pool.decode(0, B, q, fast, H, D, scale, q_tokens=S, causal=causal)
    pool.decode(0, B, q, ref, H, D, scale, q_tokens=S, causal=causal, mode=L.ATTN_REFERENCE)
    assert pool.status() == 0
    _check(fast, ref, "prompt trial %d: B=%d S=%d H=%d Hkv=%d causal=%s lens=%s" % (trial, B, S, H, Hkv, causal, lens.tolist()[:8]))
    pool.destroy()


@pytest.mark.parametrize("trial", range(4))
def test_mla_prompt_fast_against_reference_kernels(dev, oracle, trial):
    """The same for MLA: more than eight query tokens run as rows of workers, few workers per row."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(1500 + trial)
    H = int(rng.choice([16, 128]))
    Dh, dC, dHR, P = 128, 512, 64, 64
    B = int(rng.integers(1, 5))
    S = int(rng.choice([12, 33, 70]))
    lens = _lengths(rng, B, S, int(rng.choice([200, 600])))
    pages_per = (int(lens.max()) + P - 1) // P + 1
    pool = rb.Pool(dev, L.POOL_MLA, 1, B * pages_per, P, B, pages_per, dC=dC, dHR=dHR)
    pool.set_tables(permuted_tables(rng, B, pages_per))
    n = int(lens.sum())
    pool.append(0, oracle.bf16_from_f32(rng.standard_normal((n, dC), dtype=np.float32)),
                oracle.bf16_from_f32(rng.standard_normal((n, dHR), dtype=np.float32)), B, n_new=lens)
    wuk = dev.upload(oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02))
    wuv = dev.upload(oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02))
    qc = rng.standard_normal((B, S, H, Dh), dtype=np.float32)
    qr = rng.standard_normal((B, S, H, dHR), dtype=np.float32)
    scale = float(1.0 / np.sqrt(Dh + dHR))
    causal = bool(rng.integers(0, 4))
    fast, ref = np.empty_like(qc), np.empty_like(qc)
    pool.decode(0, B, qc, fast, H, Dh, scale, q_rope=qr, w_uk=wuk, w_uv=wuv, q_tokens=S, causal=causal)
    pool.decode(0, B, qc, ref, H, Dh, scale, q_rope=qr, w_uk=wuk, w_uv=wuv, q_tokens=S, causal=causal, mode=L.ATTN_REFERENCE)
    assert pool.status() == 0
    _check(fast, ref, "prompt trial %d: B=%d S=%d H=%d causal=%s lens=%s" % (trial, B, S, H, causal, lens.tolist()[:8]))
    pool.destroy(); wuk.free(); wuv.free()


@pytest.mark.parametrize("trial", range(8))
def test_mla_layer_fast_against_reference_mode(dev, oracle, trial):
    """Whole-layer step: tensor-core projections (odd K / N sizes: partial pipeline steps, column tiles narrower than a
    TMA box, several row blocks) + RoPE + append + decode against the reference-order kernels on the same inputs."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(3000 + trial)
    H = int(rng.choice([2, 4, 8]))
    Dh = int(rng.choice([16, 24, 32, 40]))
    D, dC, dHR, P = H * Dh, int(rng.choice([64, 128])), int(rng.choice([8, 16])), 64
    B = int(rng.integers(1, 48))
    S = int(rng.choice([1, 1, 2, 5]))
    lens = rng.integers(0, 200, B).astype(np.int32)
    shapes = {"w_q": (D, H * Dh), "w_qr": (D, H * dHR), "w_dkv": (D, dC), "w_kr": (D, dHR), "w_uk": (dC, H * Dh),
              "w_uv": (dC, H * Dh), "w_o": (H * Dh, D)}
    W = {k: oracle.bf16_from_f32(rng.standard_normal(sh, dtype=np.float32) * np.float32(1.0 / np.sqrt(sh[0]))) for k, sh in shapes.items()}
    dW = {k: dev.upload(v) for k, v in W.items()}
    pages_per = (int(lens.max()) + 2 * S + P - 1) // P + 1
    outs = []
    x1 = rng.standard_normal((B, S, D), dtype=np.float32)
    x2 = rng.standard_normal((B, S, D), dtype=np.float32)
    n = int(lens.sum())
    c0 = oracle.bf16_from_f32(rng.standard_normal((n, dC), dtype=np.float32))
    r0 = oracle.bf16_from_f32(rng.standard_normal((n, dHR), dtype=np.float32))
    tables = permuted_tables(rng, B, pages_per)
    for mode in (L.ATTN_FAST, L.ATTN_REFERENCE):
        pool = rb.Pool(dev, L.POOL_MLA, 1, B * pages_per, P, B, pages_per, dC=dC, dHR=dHR)
        pool.set_tables(tables)
        if n:
            pool.append(0, c0, r0, B, n_new=lens)
        res = []
        for x in (x1, x2):      # the second step attends over rows the first one wrote
            y = np.empty_like(x)
            pool.forward_cached(0, B, x, y, dW, D, H, q_tokens=S, mode=mode)
            res.append(y)
        assert pool.status() == 0
        outs.append(res)
        pool.destroy()
    for v in dW.values():
        v.free()
    for step in range(2):
        fast, ref = outs[0][step], outs[1][step]
        rel = np.linalg.norm(fast.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30)
        assert np.isfinite(fast).all() and rel <= 5e-2, "trial %d step %d: D=%d H=%d dC=%d dHR=%d B=%d S=%d rel %g" % (
            trial, step, D, H, dC, dHR, B, S, rel)
