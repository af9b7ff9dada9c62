"""Cache files in the reference's layouts (NewKVCacheFile kvcache.go:104-166, NewMLACacheFile mla_cache.go:63-113):
file size and bytes as the reference would lay them out, and a save -> load round trip that leaves rows and attention
outputs unchanged bit for bit."""
import os

import numpy as np
import pytest

from tests.helpers import permuted_tables

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import relux_b200 as rb
    d = rb.Device(0)
    yield d
    d.close()


def test_mla_cache_file_round_trip(dev, oracle, tmp_path):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(61)
    layers, dC, dHR, max_len, P = 2, 64, 16, 192, 64
    lens = [100, 37]
    pool = rb.Pool(dev, L.POOL_MLA, layers, 8, P, 2, 3, dC=dC, dHR=dHR)
    pool.set_tables(permuted_tables(rng, 2, 3, 8))
    rows = []
    for l in range(layers):
        c = rng.standard_normal((lens[l], dC), dtype=np.float32)
        r = rng.standard_normal((lens[l], dHR), dtype=np.float32)
        pool.append(l, c, r, 1, seq_ids=[1], n_new=np.asarray([lens[l]], np.int32))
        rows.append((oracle.bf16_from_f32(c), oracle.bf16_from_f32(r)))
    path = str(tmp_path / "mla.cache")
    pool.save_file(1, path, max_len)
    # the reference's file: per layer C_KV [maxLen, dC] then K_R [maxLen, dHR], float32, zeros past the cursor
    assert os.path.getsize(path) == layers * max_len * (dC + dHR) * 4
    raw = np.fromfile(path, np.float32)
    o = 0
    for l in range(layers):
        c = raw[o:o + max_len * dC].reshape(max_len, dC); o += max_len * dC
        r = raw[o:o + max_len * dHR].reshape(max_len, dHR); o += max_len * dHR
        assert np.array_equal(c[:lens[l]], oracle.f32_from_bf16(rows[l][0])) and not c[lens[l]:].any()
        assert np.array_equal(r[:lens[l]], oracle.f32_from_bf16(rows[l][1])) and not r[lens[l]:].any()
    # load into another sequence of another pool with another page placement
    pool2 = rb.Pool(dev, L.POOL_MLA, layers, 8, P, 2, 3, dC=dC, dHR=dHR)
    pool2.set_tables(permuted_tables(np.random.default_rng(5), 2, 3, 8))
    pool2.append(0, rows[0][0][:5], rows[0][1][:5], 1, seq_ids=[0], n_new=np.asarray([5], np.int32))   # stale rows to be replaced
    pool2.load_file(0, path, max_len, lens)
    for l in range(layers):
        assert pool2.seq_len(l, 0) == lens[l]
        gc, gr = pool2.read_rows(l, 0, 0, lens[l])
        assert np.array_equal(gc, rows[l][0]) and np.array_equal(gr, rows[l][1])
    with pytest.raises(L.ReluxCudaError):     # a layer longer than maxLen cannot be written
        pool.save_file(1, path, 64)
    pool.destroy(); pool2.destroy()


def test_kv_cache_file_round_trip(dev, oracle, tmp_path):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(62)
    Hkv, D, H, max_len, n = 8, 128, 32, 256, 150
    pool = rb.Pool(dev, L.POOL_GQA, 1, 4, 64, 1, 4, num_kv_heads=Hkv, head_dim=D)
    pool.set_tables(permuted_tables(rng, 1, 4))
    K = rng.standard_normal((n, Hkv, D), dtype=np.float32)
    V = rng.standard_normal((n, Hkv, D), dtype=np.float32)
    pool.append(0, K, V, 1, n_new=np.asarray([n], np.int32))
    q = rng.standard_normal((1, 1, H, D), dtype=np.float32)
    out1 = np.empty_like(q)
    pool.decode(0, 1, q, out1, H, D, 0.0884)
    path = str(tmp_path / "kv.cache")
    pool.save_file(0, path, max_len)
    # the reference's file: K [numKVHeads, maxLen, headDim] then V, bf16
    assert os.path.getsize(path) == 2 * Hkv * max_len * D * 2
    raw = np.fromfile(path, np.uint16).reshape(2, Hkv, max_len, D)
    assert np.array_equal(raw[0][:, :n], oracle.bf16_from_f32(K).transpose(1, 0, 2)) and not raw[0][:, n:].any()
    assert np.array_equal(raw[1][:, :n], oracle.bf16_from_f32(V).transpose(1, 0, 2)) and not raw[1][:, n:].any()
    pool2 = rb.Pool(dev, L.POOL_GQA, 1, 4, 64, 1, 4, num_kv_heads=Hkv, head_dim=D)
    pool2.set_tables(permuted_tables(np.random.default_rng(9), 1, 4))
    pool2.load_file(0, path, max_len, [n])
    out2 = np.empty_like(q)
    pool2.decode(0, 1, q, out2, H, D, 0.0884)
    assert np.array_equal(out1, out2)     # same rows, other pages: not a bit changes
    pool.destroy(); pool2.destroy()
