"""relux_gqa_decode_noalloc: the decode entry point for callers that may not allocate device memory while they
decode (its split-KV scratch is a fixed 16 MiB array inside the library instead of cudaMalloc'ed buffers).
Called through the C ABI, twice in a row, and compared with relux_gqa_decode on the same pool and inputs and with the
CPU restatement; the limits of the fixed scratch (host arithmetic before any launch) are exercised as well.
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
    # logical caches for the CPU restatement
    Tm = int(ctx.max())
    Kl = np.zeros((B, Tm, Hkv, D), np.uint16)
    Vl = np.zeros((B, Tm, Hkv, D), np.uint16)
    o = 0
    for b in range(B):
        Kl[b, :ctx[b]] = oracle.bf16_from_f32(K[o:o + ctx[b]])
        Vl[b, :ctx[b]] = oracle.bf16_from_f32(V[o:o + ctx[b]])
        o += ctx[b]
    pool.logical = (Kl, Vl, ctx)
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
        # and against the CPU restatement (libm exp: at these short contexts the reference's own exp approximation would dominate)
        Kl, Vl, ctx = pool.logical
        with oracle.exact_exp():
            cpu = oracle.gqa_attend(Kl, Vl, ctx, q, scale, causal=True)
        e2 = np.abs(out - cpu)
        assert e2.max() <= 2e-2 and e2.mean() <= 2e-3, "call %d vs the restatement: max %g mean %g" % (call, e2.max(), e2.mean())
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


def test_noalloc_lengthens_chunks_to_fit_and_names_its_limits(oracle):
    """The partials of a call must fit the fixed 16 MiB array.  With 8 query tokens x 32 heads one work item needs
    256 x 520 bytes, so 125 items fit.  120 sequences of two pages and one of 64 pages start at 133 items (chunks of 5
    pages) and fit only after the chunks have been lengthened; the result must still match relux_gqa_decode.  One more
    page-long sequence per item than the array holds, or more sequences than its work list, is refused by name."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    dev = rb.Device(0)
    rng = np.random.default_rng(22)
    H, Hkv, D, P, S = 32, 8, 128, 64, 8
    lens = [128] * 120 + [4096]
    B = len(lens)
    pool = rb.Pool(dev, L.POOL_GQA, 1, 2 * 120 + 64 + 200, P, 400, 64, num_kv_heads=Hkv, head_dim=D)
    ids = [pool.seq_alloc(n) for n in lens]
    blk = 128
    src = dev.upload(oracle.bf16_from_f32(rng.standard_normal((B * blk, Hkv, D)).astype(np.float32)))
    pool.append(0, src, src, B, seq_ids=ids, n_new=np.full(B, blk, np.int32))
    for _ in range(4096 // blk - 1):
        pool.append(0, src, src, 1, seq_ids=[ids[-1]], n_new=[blk])
    q = rng.standard_normal((B, S, H, D)).astype(np.float32)
    d_q, d_ref, d_out = dev.upload(q), dev.alloc(q.nbytes, L.DTYPE_F32), dev.alloc(q.nbytes, L.DTYPE_F32)
    scale = float(1.0 / np.sqrt(D))
    pool.decode(0, B, d_q, d_ref, H, D, scale, q_tokens=S, causal=True, seq_ids=ids)
    pool.decode_noalloc(0, B, d_q, d_out, H, D, scale, q_tokens=S, causal=True, seq_ids=ids)
    ref, out = d_ref.download(q.shape, np.float32), d_out.download(q.shape, np.float32)
    assert np.isfinite(out).all() and np.abs(out - ref).max() <= 1e-3
    # 126 one-page sequences more: every sequence is at least one item, 247 items cannot fit whatever the chunk length
    more = [pool.seq_alloc(64) for _ in range(126)]
    pool.append(0, src, src, len(more), seq_ids=more, n_new=np.full(len(more), 64, np.int32))
    all_ids = ids + more
    q2 = dev.upload(rng.standard_normal((len(all_ids), S, H, D)).astype(np.float32))
    o2 = dev.alloc(len(all_ids) * S * H * D * 4, L.DTYPE_F32)
    with pytest.raises(L.ReluxCudaError) as e:
        pool.decode_noalloc(0, len(all_ids), q2, o2, H, D, scale, q_tokens=S, causal=True, seq_ids=all_ids)
    assert e.value.code == L.ERR_UNSUPPORTED and "work items" in str(e.value)
    # the allocating entry point takes the same call
    pool.decode(0, len(all_ids), q2, o2, H, D, scale, q_tokens=S, causal=True, seq_ids=all_ids)
    assert pool.status() == 0
    for b in (src, d_q, d_ref, d_out, q2, o2):
        b.free()
    pool.destroy()
    # more sequences than the work list names: refused before anything else is looked at
    big = rb.Pool(dev, L.POOL_GQA, 1, 4, P, 5000, 2, num_kv_heads=Hkv, head_dim=D)
    dq = dev.alloc(4097 * H * D * 2, L.DTYPE_BF16)
    do = dev.alloc(4097 * H * D * 4, L.DTYPE_F32)
    with pytest.raises(L.ReluxCudaError) as e:
        big.decode_noalloc(0, 4097, dq, do, H, D, scale)
    assert e.value.code == L.ERR_UNSUPPORTED and "4096 sequences" in str(e.value)
    dq.free(); do.free()
    big.destroy()
    dev.close()
