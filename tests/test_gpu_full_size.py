"""Parity at the benchmark configurations' full sizes, through properties that do not need a full CPU run:
bit-exact cache round trips, page-permutation invariance, split-KV invariance, exact scaling, plus an oracle check on a
sample of sequences of the full batch."""
import os

import numpy as np
import pytest

from tests.helpers import check_attention

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import relux_b200 as rb
    d = rb.Device(0)
    yield d
    d.close()


def _mla_full(dev, oracle, rng, B, ctx, perm_seed, pages_extra=1):
    import relux_b200 as rb
    from relux_b200 import lib as L
    dC, dHR, P = 512, 64, 64
    pages_per = (int(max(ctx)) + P - 1) // P + pages_extra
    pool = rb.Pool(dev, L.POOL_MLA, 1, B * pages_per, P, B, pages_per, dC=dC, dHR=dHR)
    pool.set_tables(np.random.default_rng(perm_seed).permutation(B * pages_per).astype(np.int32).reshape(B, pages_per))
    return pool


def test_config3_full_batch_properties(dev, oracle):
    """config 3: batch 64, 128 heads, latent 512 + rope 64, context 4096 + 1 appended token, page 64."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(7)
    B, T0, H, Dh, dC, dHR = 64, 4096, 128, 128, 512, 64
    c = oracle.bf16_from_f32(rng.standard_normal((B * T0, dC), dtype=np.float32))
    r = oracle.bf16_from_f32(rng.standard_normal((B * T0, dHR), dtype=np.float32))
    nc = rng.standard_normal((B, dC), dtype=np.float32)
    nr = rng.standard_normal((B, dHR), dtype=np.float32)
    wuk = oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02)
    wuv = oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02)
    wuv2 = oracle.bf16_from_f32(oracle.f32_from_bf16(wuv) * 2.0)
    qc = rng.standard_normal((B, 1, H, Dh), dtype=np.float32)
    qr = rng.standard_normal((B, 1, H, dHR), dtype=np.float32)
    scale = float(1.0 / np.sqrt(Dh + dHR))
    d_wuk, d_wuv, d_wuv2 = dev.upload(wuk), dev.upload(wuv), dev.upload(wuv2)
    outs = []
    for perm_seed in (1, 2):
        pool = _mla_full(dev, oracle, rng, B, [T0 + 1] * B, perm_seed)
        pool.append(0, c, r, B, n_new=np.full(B, T0, np.int32))
        pool.append(0, nc, nr, B)                      # the step's new token, float32 -> bf16 on the device
        # cache round trip at full size: every row of two sequences, bit for bit
        for b in (0, B - 1):
            gc, gr = pool.read_rows(0, b, 0, T0 + 1)
            assert np.array_equal(gc[:T0], c[b * T0:(b + 1) * T0]) and np.array_equal(gr[:T0], r[b * T0:(b + 1) * T0])
            assert np.array_equal(gc[T0], oracle.bf16_from_f32(nc[b])) and np.array_equal(gr[T0], oracle.bf16_from_f32(nr[b]))
        out = np.empty((B, 1, H, Dh), np.float32)
        pool.decode(0, B, qc, out, H, Dh, scale, q_rope=qr, w_uk=d_wuk, w_uv=d_wuv)
        outs.append(out.copy())
        if perm_seed == 1:
            # exact scaling: doubling W_UV (a power of two) doubles every output bit for bit
            out2 = np.empty_like(out)
            pool.decode(0, B, qc, out2, H, Dh, scale, q_rope=qr, w_uk=d_wuk, w_uv=d_wuv2)
            assert np.array_equal(out2, out * 2.0)
            # split-KV invariance: another chunk length changes only float32 association
            pool.tune(L.TUNE_CHUNK_PAGES, 6)
            out3 = np.empty_like(out)
            pool.decode(0, B, qc, out3, H, Dh, scale, q_rope=qr, w_uk=d_wuk, w_uv=d_wuv)
            pool.tune(L.TUNE_CHUNK_PAGES, -1)
            assert np.abs(out3 - out).max() <= 1e-3
        assert pool.status() == 0
        pool.destroy()
    # page-permutation invariance: the physical placement of pages must not change a single bit
    assert np.array_equal(outs[0], outs[1])
    # oracle (reference arithmetic) on a sample of the batch
    sample = [0, 17, 63]
    cl = np.stack([np.concatenate([c[b * T0:(b + 1) * T0], oracle.bf16_from_f32(nc[b])[None]]) for b in sample])
    rl = np.stack([np.concatenate([r[b * T0:(b + 1) * T0], oracle.bf16_from_f32(nr[b])[None]]) for b in sample])
    ref = oracle.mla_attend(cl, rl, [T0 + 1] * len(sample), qc[sample], qr[sample], wuk, wuv, scale, absorbed=True)
    check_attention(outs[0][sample], ref, "config 3 sample")
    for b in (d_wuk, d_wuv, d_wuv2):
        b.free()


def test_config4_ragged_long_context_sample(dev, oracle):
    """config 4 shapes on one GPU's share: 16 sequences with lengths uniform in [1024, 32768] (seed 11), random page
    permutation, 70 append + decode steps, so that EVERY sequence crosses a page boundary (64-token pages) inside the run;
    the shortest and the longest sequence are checked against the oracle on the first steps, around step 64 and at the
    end, and the rows appended during the run are read back bit for bit for every sequence."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(11)
    all_len = rng.integers(1024, 32769, 128)
    B = 16
    ctx = all_len[:B].astype(np.int32).copy()
    H, Dh, dC, dHR = 128, 128, 512, 64
    pool = _mla_full(dev, oracle, rng, B, ctx, perm_seed=3, pages_extra=2)
    c = oracle.bf16_from_f32(rng.standard_normal((int(ctx.sum()), dC), dtype=np.float32))
    r = oracle.bf16_from_f32(rng.standard_normal((int(ctx.sum()), dHR), dtype=np.float32))
    pool.append(0, c, r, B, n_new=ctx)
    wuk = oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02)
    wuv = oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02)
    d_wuk, d_wuv = dev.upload(wuk), dev.upload(wuv)
    scale = float(1.0 / np.sqrt(Dh + dHR))
    off = np.concatenate([[0], np.cumsum(ctx)])
    shortest, longest = int(np.argmin(ctx)), int(np.argmax(ctx))
    rows_c = {b: [c[off[b]:off[b + 1]]] for b in (shortest, longest)}
    rows_r = {b: [r[off[b]:off[b + 1]]] for b in (shortest, longest)}
    n_steps, checked = 70, (0, 1, 63, 64, 69)
    new_c, new_r = [], []
    for step in range(n_steps):
        nc = rng.standard_normal((B, dC), dtype=np.float32)
        nr = rng.standard_normal((B, dHR), dtype=np.float32)
        qc = rng.standard_normal((B, 1, H, Dh), dtype=np.float32)
        qr = rng.standard_normal((B, 1, H, dHR), dtype=np.float32)
        pool.append(0, nc, nr, B)
        out = np.empty((B, 1, H, Dh), np.float32)
        pool.decode(0, B, qc, out, H, Dh, scale, q_rope=qr, w_uk=d_wuk, w_uv=d_wuv)
        assert np.isfinite(out).all()
        new_c.append(oracle.bf16_from_f32(nc)); new_r.append(oracle.bf16_from_f32(nr))
        for b in (shortest, longest):
            rows_c[b].append(oracle.bf16_from_f32(nc[b])[None]); rows_r[b].append(oracle.bf16_from_f32(nr[b])[None])
            if step not in checked:
                continue
            cl, rl = np.concatenate(rows_c[b])[None], np.concatenate(rows_r[b])[None]
            assert pool.seq_len(0, b) == cl.shape[1]
            ref = oracle.mla_attend(cl, rl, [cl.shape[1]], qc[b:b + 1], qr[b:b + 1], wuk, wuv, scale, absorbed=True)
            check_attention(out[b:b + 1], ref, "config 4 step %d seq %d (ctx %d)" % (step, b, cl.shape[1]))
    new_c, new_r = np.stack(new_c, 1), np.stack(new_r, 1)   # [B, steps, ...]
    for b in range(B):   # every sequence crossed a page boundary: the appended rows are where a reader expects them
        assert (int(ctx[b]) // 64) != ((int(ctx[b]) + n_steps) // 64)
        gc, gr = pool.read_rows(0, b, int(ctx[b]), n_steps)
        assert np.array_equal(gc, new_c[b]) and np.array_equal(gr, new_r[b])
    assert pool.status() == 0
    pool.destroy(); d_wuk.free(); d_wuv.free()


def test_config5_full_batch_properties(dev, oracle):
    """config 5: 32 heads / 8 kv heads, head dim 128, batch 128, context 8192, 4 draft tokens, accepted prefix 1..4."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(3)
    B, T0, H, Hkv, D, S, P = 128, 8192, 32, 8, 128, 4, 64
    blk = 1024
    Kb = oracle.bf16_from_f32(rng.standard_normal((B * blk, Hkv, D), dtype=np.float32))
    Vb = oracle.bf16_from_f32(rng.standard_normal((B * blk, Hkv, D), dtype=np.float32))
    dK = rng.standard_normal((B * S, Hkv, D), dtype=np.float32)
    dV = rng.standard_normal((B * S, Hkv, D), dtype=np.float32)
    q = rng.standard_normal((B, S, H, D), dtype=np.float32)
    scale = float(1.0 / np.sqrt(D))
    outs = []
    pages_per = (T0 + 2 * S + P - 1) // P + 1
    for perm_seed in (5, 6):
        pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages_per, P, B, pages_per, num_kv_heads=Hkv, head_dim=D)
        pool.set_tables(np.random.default_rng(perm_seed).permutation(B * pages_per).astype(np.int32).reshape(B, pages_per))
        dKb, dVb = dev.upload(Kb), dev.upload(Vb)
        for _ in range(T0 // blk):   # the context is 8 repetitions of one seeded 1024-token block per sequence
            pool.append(0, dKb, dVb, B, n_new=np.full(B, blk, np.int32))
        dev.sync(); dKb.free(); dVb.free()
        out = np.empty_like(q)
        pool.verify(0, B, q, out, dK, dV, H, D, scale, S)
        outs.append(out.copy())
        if perm_seed == 5:
            accepted = np.random.default_rng(9).integers(1, S + 1, B).astype(np.int32)
            pool.set_len(0, T0 + accepted)
            for b in (0, 77, B - 1):   # accepted prefix is in the cache bit for bit, nothing beyond it is visible
                assert pool.seq_len(0, b) == T0 + accepted[b]
                gk, gv = pool.read_rows(0, b, T0 - 2, 2 + int(accepted[b]))
                assert np.array_equal(gk[:2], Kb[b * blk + blk - 2:(b + 1) * blk]) and np.array_equal(gv[:2], Vb[b * blk + blk - 2:(b + 1) * blk])
                assert np.array_equal(gk[2:], oracle.bf16_from_f32(dK[b * S:b * S + accepted[b]]))
                assert np.array_equal(gv[2:], oracle.bf16_from_f32(dV[b * S:b * S + accepted[b]]))
        assert pool.status() == 0
        pool.destroy()
    assert np.array_equal(outs[0], outs[1])
    sample = [0, 64, 127]
    Kl = np.stack([np.concatenate([np.tile(Kb[b * blk:(b + 1) * blk], (T0 // blk, 1, 1)), oracle.bf16_from_f32(dK[b * S:(b + 1) * S])]) for b in sample])
    Vl = np.stack([np.concatenate([np.tile(Vb[b * blk:(b + 1) * blk], (T0 // blk, 1, 1)), oracle.bf16_from_f32(dV[b * S:(b + 1) * S])]) for b in sample])
    ref = oracle.gqa_attend(Kl, Vl, [T0 + S] * len(sample), q[sample], scale, causal=True)
    check_attention(outs[0][sample], ref, "config 5 sample")


def test_mla_prompt_full_size_properties(dev, oracle):
    """An MLA prompt at the benchmark's widths (128 heads, 2 sequences x 2048 tokens, the second after 300 cached rows)
    on the expansion + prefill kernels, through properties that need no full CPU run: the result does not depend on the
    page permutation (bit for bit), agrees with the absorbed decode kernels on the same inputs (two different
    algorithms: expanded 192-wide scores against 576-wide latent scores), and the last query token of every sequence,
    which sees the whole cache like a decode step, agrees with the restatement's one-token call."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(31)
    H, Dh, dC, dHR, S = 128, 128, 512, 64, 2048
    ctx = [S, 300 + S]
    B = len(ctx)
    c = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(ctx)), dC), dtype=np.float32))
    r = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(ctx)), dHR), dtype=np.float32))
    wuk = oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02)
    wuv = oracle.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02)
    d_wuk, d_wuv = dev.upload(wuk), dev.upload(wuv)
    qc = oracle.bf16_from_f32(rng.standard_normal((B, S, H, Dh), dtype=np.float32))
    qr = oracle.bf16_from_f32(rng.standard_normal((B, S, H, dHR), dtype=np.float32))
    scale = float(1.0 / np.sqrt(Dh + dHR))
    outs = []
    for perm_seed in (1, 2):
        pool = _mla_full(dev, oracle, rng, B, ctx, perm_seed)
        pool.append(0, c, r, B, n_new=np.asarray(ctx, np.int32))
        out = np.full((B, S, H, Dh), np.nan, np.float32)
        n0 = dev.launch_count()
        pool.decode(0, B, qc, out, H, Dh, scale, q_rope=qr, w_uk=d_wuk, w_uv=d_wuv, q_tokens=S, causal=True)
        assert dev.launch_count() - n0 == 3
        assert pool.status() == 0
        outs.append(out)
        if perm_seed == 2:
            pool.tune(L.TUNE_MLA_PROMPT_MIN_TOKENS, 1 << 30)   # the same call on the absorbed decode kernels
            out_abs = np.full((B, S, H, Dh), np.nan, np.float32)
            pool.decode(0, B, qc, out_abs, H, Dh, scale, q_rope=qr, w_uk=d_wuk, w_uv=d_wuv, q_tokens=S, causal=True)
            assert pool.status() == 0
        pool.destroy()
    assert np.array_equal(outs[0], outs[1]), "the result depends on the page permutation"
    check_attention(outs[0], out_abs, "mla prompt: prefill kernels against the absorbed decode kernels")
    # the last query token of every sequence against the restatement (one token over the whole cache)
    Tm = max(ctx)
    cl = np.zeros((B, Tm, dC), np.uint16)
    rl = np.zeros((B, Tm, dHR), np.uint16)
    o = 0
    for b in range(B):
        cl[b, :ctx[b]] = c[o:o + ctx[b]]
        rl[b, :ctx[b]] = r[o:o + ctx[b]]
        o += ctx[b]
    with oracle.exact_exp():
        ref = oracle.mla_attend(cl, rl, ctx, oracle.f32_from_bf16(qc[:, -1:]), oracle.f32_from_bf16(qr[:, -1:]), wuk, wuv, scale, causal=True,
                                absorbed=False)
    check_attention(outs[0][:, -1:], ref, "mla prompt: last token against the restatement")
    d_wuk.free(); d_wuv.free()


def test_gqa_prompt_full_size_properties(dev, oracle):
    """A GQA prompt at the benchmark's widths (32 heads / 8 kv heads, 2 sequences x 4096 tokens, the second after 500
    cached rows) on the prefill kernel: independent of the page permutation bit for bit, equal within tolerance to the
    grid slices of the decode kernel (another algorithm: split-KV partials and a merge), last token against the
    restatement."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(32)
    H, Hkv, D, S, P = 32, 8, 128, 4096, 64
    ctx = [S, 500 + S]
    B = len(ctx)
    K = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(ctx)), Hkv, D), dtype=np.float32))
    V = oracle.bf16_from_f32(rng.standard_normal((int(np.sum(ctx)), Hkv, D), dtype=np.float32))
    q = oracle.bf16_from_f32(rng.standard_normal((B, S, H, D), dtype=np.float32))
    scale = float(1.0 / np.sqrt(D))
    pages_per = (max(ctx) + P - 1) // P + 1
    outs = []
    for perm_seed in (1, 2):
        pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages_per, P, B, pages_per, num_kv_heads=Hkv, head_dim=D)
        pool.set_tables(np.random.default_rng(perm_seed).permutation(B * pages_per).astype(np.int32).reshape(B, pages_per))
        pool.append(0, K, V, B, n_new=np.asarray(ctx, np.int32))
        out = np.full((B, S, H, D), np.nan, np.float32)
        pool.decode(0, B, q, out, H, D, scale, q_tokens=S, causal=True)
        assert pool.status() == 0
        outs.append(out)
        if perm_seed == 2:
            pool.tune(L.TUNE_GQA_PROMPT_SLICES, 1)
            out_sl = np.full((B, S, H, D), np.nan, np.float32)
            pool.decode(0, B, q, out_sl, H, D, scale, q_tokens=S, causal=True)
            assert pool.status() == 0
        pool.destroy()
    assert np.array_equal(outs[0], outs[1]), "the result depends on the page permutation"
    check_attention(outs[0], out_sl, "gqa prompt: prefill kernel against the decode kernel's grid slices")
    Tm = max(ctx)
    Kl = np.zeros((B, Tm, Hkv, D), np.uint16)
    Vl = np.zeros((B, Tm, Hkv, D), np.uint16)
    o = 0
    for b in range(B):
        Kl[b, :ctx[b]] = K[o:o + ctx[b]]
        Vl[b, :ctx[b]] = V[o:o + ctx[b]]
        o += ctx[b]
    with oracle.exact_exp():
        ref = oracle.gqa_attend(Kl, Vl, ctx, oracle.f32_from_bf16(q[:, -1:]), scale, causal=True)
    check_attention(outs[0][:, -1:], ref, "gqa prompt: last token against the restatement")
