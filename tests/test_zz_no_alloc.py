"""relux_gqa_decode_noalloc: the decode entry point for callers that may not allocate device memory while they
decode (its split-KV scratch is a fixed 16 MiB array inside the library instead of cudaMalloc'ed buffers).
Called through the C ABI, twice in a row, and compared with relux_gqa_decode on the same pool and inputs.
The file name keeps it last in collection order."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _setup(dev, oracle, S):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(21)
    ctx = np.array([S, 64, 65, 1000, 2047, 130], np.int32)
    B, H, Hkv, D, P = len(ctx), 32, 8, 128, 64
    pages_per = (int(ctx.max()) + P - 1) // P + 1
    pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages_per, P, B, pages_per, num_kv_heads=Hkv, head_dim=D)
    pool.set_tables(rng.permutation(B * pages_per).astype(np.int32).reshape(B, pages_per))
    K = rng.standard_normal((int(ctx.sum()), Hkv, D)).astype(np.float32)
    V = rng.standard_normal((int(ctx.sum()), Hkv, D)).astype(np.float32)
    pool.append(0, K, V, B, n_new=ctx)
    return pool, rng, B, H, D


@pytest.mark.parametrize("S", [1, 4])
def test_noalloc_matches_the_allocating_entry_point(oracle, S):
    import relux_b200 as rb
    from relux_b200 import lib as L
    dev = rb.Device(0)
    pool, rng, B, H, D = _setup(dev, oracle, S)
    scale = float(1.0 / np.sqrt(D))
    for call in range(2):   # two calls in a row: the second one finds the scratch as the first one left it
        q = rng.standard_normal((B, S, H, D)).astype(np.float32)
        d_q = dev.upload(q)
        d_ref = dev.alloc(q.nbytes, L.DTYPE_F32)
        d_out = dev.alloc(q.nbytes, L.DTYPE_F32)
        d_out.zero()
        pool.decode(0, B, d_q, d_ref, H, D, scale, q_tokens=S, causal=True)
        pool.decode_noalloc(0, B, d_q, d_out, H, D, scale, q_tokens=S, causal=True)
        ref = d_ref.download(q.shape, np.float32)
        out = d_out.download(q.shape, np.float32)
        assert np.isfinite(out).all()
        err = np.abs(out - ref)
        # same kernels, possibly a different chunking of the context: differences are float32 re-association only
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, "call %d: max %g mean %g" % (call, err.max(), err.mean())
        assert err.max() <= 1e-3   # far inside the tolerance: only the bf16 rounding of P relative to another running max differs
        for b in (d_q, d_ref, d_out):
            b.free()
    assert pool.status() == 0
    pool.destroy()
    dev.close()


def test_noalloc_rejects_what_it_cannot_hold(oracle):
    import relux_b200 as rb
    from relux_b200 import lib as L
    dev = rb.Device(0)
    pool, rng, B, H, D = _setup(dev, oracle, 1)
    q = rng.standard_normal((B, 1, H, D)).astype(np.float32)
    out = np.empty_like(q)
    with pytest.raises(L.ReluxCudaError) as e:   # host-resident q would need a staging allocation
        pool.decode_noalloc(0, B, q, out, H, D, 0.088)
    assert e.value.code == L.ERR_UNSUPPORTED
    pool.destroy()
    dev.close()
