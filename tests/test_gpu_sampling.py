"""Token selection after a verify pass on the device against the CPU restatement of acceptPhase / resampleRejected
(speculative.go:211-295) and Sampler.Sample (sampler.go:73-218), with the uniform draws supplied to both sides.

REFERENCE mode walks the reference's float32 order and must agree bit for bit: same number of accepted tokens, same
token.  FAST mode sums in parallel, so it must agree except where a draw lies within SUM_TOL of a decision boundary of
the reference's own distribution: for an accept decision |draw - acceptProb| < SUM_TOL, for a categorical draw the
chosen token's interval of the reference's cumulative distribution, widened by SUM_TOL, must contain the draw."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SUM_TOL = 2e-4   # float32 sums over up to 131072 terms in a different order


@pytest.fixture(scope="module")
def dev():
    import relux_b200 as rb
    d = rb.Device(0)
    yield d
    d.close()


@pytest.fixture(scope="module")
def pool(dev):
    import relux_b200 as rb
    from relux_b200 import lib as L
    p = rb.Pool(dev, L.POOL_MLA, 2, 16, 64, 8, 2, dC=64, dHR=16)
    yield p
    p.destroy()


def make_case(rng, n, k, V, noise=0.6, scale=2.5, identical=False):
    dl = (rng.standard_normal((n, k, V)) * scale).astype(np.float32)
    tl = np.empty((n, k + 1, V), np.float32)
    tl[:, :k] = dl if identical else dl + (rng.standard_normal((n, k, V)) * noise).astype(np.float32)
    tl[:, k] = (rng.standard_normal((n, V)) * scale).astype(np.float32)
    # draft tokens drawn from the draft distribution, like draftPhase does
    toks = np.empty((n, k), np.int32)
    for b in range(n):
        for i in range(k):
            p = np.exp(dl[b, i].astype(np.float64) - dl[b, i].max())
            toks[b, i] = rng.choice(V, p=p / p.sum())
    draws = rng.random((n, k + 1)).astype(np.float32)
    return toks, dl, tl, draws


def reference_run(oracle, cfg, toks, dl, tl, draws):
    out = []
    for b in range(toks.shape[0]):
        out.append(oracle.spec_accept(cfg, toks[b], dl[b], tl[b], draws[b]))
    return out


def final_distribution(oracle, cfg, n_ref, dl_b, tl_b):
    """The distribution the reference draws the last token from, in float64."""
    k = dl_b.shape[0]
    if n_ref == k:
        _, probs = oracle.sampler_sample(cfg, tl_b[k], 0.5, return_probs=True)
        return probs.astype(np.float64), tl_b.shape[1] - 1
    d = oracle.softmax_alloc(dl_b[n_ref]).astype(np.float64)
    t = oracle.softmax_alloc(tl_b[n_ref]).astype(np.float64)
    adj = np.maximum(t - d, 0.0)
    return (adj / adj.sum() if adj.sum() > 0 else t), 0


def check_fast(oracle, cfg, toks, dl, tl, draws, n_acc, nxt):
    ref = reference_run(oracle, cfg, toks, dl, tl, draws)
    exact = 0
    for b, (n_ref, tok_ref, used, ap) in enumerate(ref):
        if n_acc[b] != n_ref:
            j = min(int(n_acc[b]), n_ref)
            assert abs(float(draws[b, j]) - float(ap[j])) < SUM_TOL, \
                "seq %d: accepted %d, reference %d, draw %.7f against acceptProb %.7f" % (b, n_acc[b], n_ref, draws[b, j], ap[j])
            continue
        if nxt[b] == tok_ref:
            exact += 1
            continue
        probs, _ = final_distribution(oracle, cfg, n_ref, dl[b], tl[b])
        cum = np.cumsum(probs)
        g = int(nxt[b])
        r = float(draws[b, used - 1])
        lo = cum[g - 1] if g > 0 else 0.0
        assert lo - SUM_TOL <= r < cum[g] + SUM_TOL, \
            "seq %d: token %d (reference %d) holds [%.7f, %.7f) of the reference's CDF, draw %.7f" % (b, g, tok_ref, lo, cum[g], r)
    return exact / len(ref)


SAMPLERS = [
    dict(),
    dict(temperature=0.7),
    dict(top_k=40),
    dict(top_p=0.9),
    dict(min_p=0.05),
    dict(temperature=1.3, top_k=100, top_p=0.85, min_p=0.02),
    dict(top_k=300, top_p=0.9),                 # above the list path's limit: top-k by the full radix walk
]


@pytest.mark.parametrize("sampler", SAMPLERS)
def test_reference_mode_is_bit_exact(pool, oracle, sampler):
    from relux_b200 import lib as L
    rng = np.random.default_rng(101)
    n, k, V = 8, 4, 1000
    toks, dl, tl, draws = make_case(rng, n, k, V)
    # two sequences whose draft equals the target: every token passes and the sampler runs
    tl[6:8, :k] = dl[6:8]
    cfg = oracle.sampler_cfg(**sampler)
    ref = reference_run(oracle, cfg, toks, dl, tl, draws)
    n_acc, nxt = pool.spec_accept(n, k, V, toks, dl, tl, draws, mode=L.ATTN_REFERENCE, **sampler)
    assert [r[0] for r in ref] == n_acc.tolist()
    assert [r[1] for r in ref] == nxt.tolist()
    assert {r[0] for r in ref} >= {k} and len({r[0] for r in ref}) > 1   # both outcomes were exercised


@pytest.mark.parametrize("sampler", SAMPLERS)
@pytest.mark.parametrize("V", [777, 4096, 32000, 50257])
def test_fast_mode_matches_within_summation_order(pool, oracle, sampler, V):
    rng = np.random.default_rng(7 + V)
    n, k = 6, 3
    toks, dl, tl, draws = make_case(rng, n, k, V)
    tl[4:6, :k] = dl[4:6]
    cfg = oracle.sampler_cfg(**sampler)
    n_acc, nxt = pool.spec_accept(n, k, V, toks, dl, tl, draws, **sampler)
    exact = check_fast(oracle, cfg, toks, dl, tl, draws, n_acc, nxt)
    assert exact >= 0.8, "only %.0f %% of the tokens equal the reference's" % (100 * exact)


def test_plain_sampling_rows(pool, oracle):
    from relux_b200 import lib as L
    rng = np.random.default_rng(5)
    n, V = 16, 5000
    logits = (rng.standard_normal((n, V)) * 3).astype(np.float32)
    draws = rng.random(n).astype(np.float32)
    for sampler in (dict(), dict(temperature=0.8, top_k=50), dict(top_p=0.7)):
        cfg = oracle.sampler_cfg(**sampler)
        want = [oracle.sampler_sample(cfg, logits[i], float(draws[i])) for i in range(n)]
        got = pool.sample(logits, draws, mode=L.ATTN_REFERENCE, **sampler)
        assert got.tolist() == want
        fast = pool.sample(logits, draws, **sampler)
        for i in range(n):
            if fast[i] != want[i]:
                _, probs = oracle.sampler_sample(cfg, logits[i], float(draws[i]), return_probs=True)
                cum = np.cumsum(probs.astype(np.float64))
                g = int(fast[i])
                assert (cum[g - 1] if g else 0.0) - SUM_TOL <= draws[i] < cum[g] + SUM_TOL


@pytest.mark.parametrize("V", [1000, 32000, 131072])
def test_small_top_k_is_bit_exact_in_fast_mode(pool, oracle, V):
    """With top-k <= 128 the fast path finishes the sampler on the list of kept logits in the reference's own order
    of float32 operations: tokens equal the reference's exactly, whatever the other filters."""
    rng = np.random.default_rng(V)
    n = 24
    logits = (rng.standard_normal((n, V)) * 3).astype(np.float32)
    logits[3, :200] = logits[3, 0]          # a plateau of ties around the threshold
    logits[4] = np.round(logits[4])          # many exact ties everywhere
    draws = rng.random(n).astype(np.float32)
    for sampler in (dict(top_k=1), dict(top_k=50), dict(top_k=128, temperature=0.6), dict(top_k=40, top_p=0.9),
                    dict(top_k=64, top_p=0.5, min_p=0.1, temperature=1.4)):
        cfg = oracle.sampler_cfg(**sampler)
        want = [oracle.sampler_sample(cfg, logits[i], float(draws[i])) for i in range(n)]
        got = pool.sample(logits, draws, **sampler)
        assert got.tolist() == want, sampler


def test_repetition_penalties_match_the_reference(pool, oracle):
    """applyRepetitionPenalties (sampler.go:221-266) before the sampler: REFERENCE mode and the small-top-k fast path give
    the reference's token exactly; the input logits stay untouched."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(77)
    n, V = 12, 4000
    logits = (rng.standard_normal((n, V)) * 3).astype(np.float32)
    keep = logits.copy()
    draws = rng.random(n).astype(np.float32)
    prev = []
    for i in range(n):
        top = np.argsort(-logits[i])[:20]                      # likely tokens, so the penalties change the outcome
        hist = rng.choice(top, size=rng.integers(0, 90)).tolist()
        if i == 5:
            hist += [-3, V + 7]                                  # out-of-range ids are ignored like in the reference
        prev.append(hist)
    for pen in (dict(repeat_penalty=1.3), dict(frequency_penalty=0.4, presence_penalty=0.7),
                dict(repeat_penalty=1.2, frequency_penalty=0.2, presence_penalty=0.3, repeat_window=16)):
        for sampler in (dict(), dict(top_k=40, top_p=0.9), dict(temperature=0.7, min_p=0.03)):
            cfg = oracle.sampler_cfg(**sampler, **pen)
            want = [oracle.sampler_sample(cfg, logits[i], float(draws[i]), prev=prev[i]) for i in range(n)]
            plain = [oracle.sampler_sample(oracle.sampler_cfg(**sampler), logits[i], float(draws[i])) for i in range(n)]
            got = pool.sample(logits, draws, mode=L.ATTN_REFERENCE, prev_tokens=prev, **sampler, **pen)
            assert got.tolist() == want, (pen, sampler)
            fast = pool.sample(logits, draws, prev_tokens=prev, **sampler, **pen)
            if sampler.get("top_k"):
                assert fast.tolist() == want, (pen, sampler)
            else:
                for i in range(n):
                    if fast[i] != want[i]:
                        _, probs = oracle.sampler_sample(cfg, logits[i], float(draws[i]), prev=prev[i], return_probs=True)
                        cum = np.cumsum(probs.astype(np.float64))
                        g = int(fast[i])
                        assert (cum[g - 1] if g else 0.0) - SUM_TOL <= draws[i] < cum[g] + SUM_TOL
            assert want != plain                                 # the penalties did change some tokens
    assert np.array_equal(logits, keep)


def _within_cdf(oracle, cfg, logits_row, draw, got, prev=None):
    _, probs = oracle.sampler_sample(cfg, logits_row, float(draw), prev=prev, return_probs=True)
    cum = np.cumsum(probs.astype(np.float64))
    g = int(got)
    return (cum[g - 1] if g else 0.0) - SUM_TOL <= draw < cum[g] + SUM_TOL


def test_more_ties_than_the_list_holds(pool, oracle):
    """A plateau of 1500 equal logits at the top with top-k 50: the reference keeps every tie (it masks only what is
    strictly below the k-th largest), the list path cannot hold them and hands over to the pass-per-step path."""
    rng = np.random.default_rng(21)
    n, V = 8, 20000
    logits = (rng.standard_normal((n, V)) * 2).astype(np.float32)
    for i in range(n):
        logits[i, rng.choice(V, 1500, replace=False)] = 9.5
    draws = rng.random(n).astype(np.float32)
    cfg = oracle.sampler_cfg(top_k=50)
    got = pool.sample(logits, draws, top_k=50)
    for i in range(n):
        assert logits[i, got[i]] == np.float32(9.5)
        assert _within_cdf(oracle, cfg, logits[i], draws[i], got[i])


def test_randomised_shapes_and_settings(pool, oracle):
    """Seeded random vocabularies (aligned and not), batch sizes, draft lengths and sampler settings against the
    restatement, with the summation-order criterion of this file."""
    rng = np.random.default_rng(2024)
    exact = []
    for trial in range(10):
        V = int(rng.choice([257, 1000, 3001, 8192, 20011, 65536]))
        n = int(rng.integers(1, 40))
        k = int(rng.integers(1, 7))
        sampler = {}
        if rng.random() < 0.5:
            sampler["temperature"] = float(rng.choice([0.5, 0.9, 1.5]))
        if rng.random() < 0.6:
            sampler["top_k"] = int(rng.choice([1, 8, 64, 128, 129, 500]))
        if rng.random() < 0.5:
            sampler["top_p"] = float(rng.choice([0.3, 0.8, 0.97]))
        if rng.random() < 0.3:
            sampler["min_p"] = float(rng.choice([0.01, 0.2]))
        toks, dl, tl, draws = make_case(rng, n, k, V, noise=float(rng.choice([0.0, 0.3, 1.0])))
        cfg = oracle.sampler_cfg(**sampler)
        n_acc, nxt = pool.spec_accept(n, k, V, toks, dl, tl, draws, **sampler)
        exact.append(check_fast(oracle, cfg, toks, dl, tl, draws, n_acc, nxt))
    assert np.mean(exact) > 0.9


def test_reference_sampler_properties(pool):
    """The two properties sampler_test.go checks: temperature -> 0 always yields the argmax, top-k 2 only the two
    largest logits."""
    from relux_b200 import lib as L
    draws = np.linspace(0.0, 0.9999, 64).astype(np.float32)
    for mode in (L.ATTN_FAST, L.ATTN_REFERENCE):
        logits = np.tile(np.asarray([1, 5, 3], np.float32), (64, 1))
        assert set(pool.sample(logits, draws, temperature=1e-10, mode=mode).tolist()) == {1}
        logits = np.tile(np.asarray([1, 5, 3, 2, 4], np.float32), (64, 1))
        assert set(pool.sample(logits, draws, top_k=2, mode=mode).tolist()) == {1, 4}


def test_device_resident_inputs_and_commit(dev, pool, oracle):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(9)
    n, k, V = 4, 4, 2048
    toks, dl, tl, draws = make_case(rng, n, k, V)
    host = pool.spec_accept(n, k, V, toks, dl, tl, draws)
    bufs = []
    for a in (toks, dl, tl, draws):
        b = rb.DeviceBuffer(dev, a.nbytes, L.DTYPE_F32)
        b.upload(a)
        bufs.append(b)
    pool.reset()
    pool.set_tables(np.arange(16, dtype=np.int32).reshape(8, 2))
    base = np.asarray([10, 0, 64, 100], np.int32)
    ids = np.asarray([3, 1, 0, 6], np.int32)
    pool.set_len(-1, base, seq_ids=ids)
    n_acc, nxt = pool.spec_accept(n, k, V, *bufs, commit=True, seq_ids=ids)
    assert n_acc.tolist() == host[0].tolist() and nxt.tolist() == host[1].tolist()
    for layer in range(2):
        for i in range(n):
            assert pool.seq_len(layer, int(ids[i])) == base[i] + n_acc[i] + 1
    for b in bufs:
        b.free()


def test_draft_token_outside_vocabulary_is_an_error(dev, pool):
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(3)
    toks, dl, tl, draws = make_case(rng, 2, 2, 300)
    toks[1, 0] = 300
    with pytest.raises(L.ReluxCudaError):
        pool.spec_accept(2, 2, 300, toks, dl, tl, draws)
    # the same from device memory, where only the kernel can see the token: it skips the sequence and reports it
    for mode in (L.ATTN_FAST, L.ATTN_REFERENCE):
        bufs = []
        for a in (toks, dl, tl, draws):
            b = rb.DeviceBuffer(dev, a.nbytes, L.DTYPE_F32)
            b.upload(a)
            bufs.append(b)
        with pytest.raises(L.ReluxCudaError):
            pool.spec_accept(2, 2, 300, *bufs, mode=mode)
        assert pool.status() != 0     # reading the status word clears it
        assert pool.status() == 0
        for b in bufs:
            b.free()


def test_reference_mode_refuses_sizes_it_is_not_meant_for(pool, oracle):
    from relux_b200 import lib as L
    logits = np.zeros((1, 40000), np.float32)
    draws = np.asarray([0.5], np.float32)
    with pytest.raises(L.ReluxCudaError) as e:
        pool.sample(logits, draws, top_p=0.9, mode=L.ATTN_REFERENCE)
    assert e.value.code == L.ERR_UNSUPPORTED
    # without the quadratic filters the same vocabulary is fine
    want = oracle.sampler_sample(oracle.sampler_cfg(), logits[0], 0.5)
    assert pool.sample(logits, draws, mode=L.ATTN_REFERENCE).tolist() == [want]


def test_full_size_properties(dev, pool):
    """Vocabulary of 131072 (a cluster of eight CTAs per sequence), 64 sequences, four draft tokens: a draft equal to the
    target is accepted whole, and a near-zero temperature turns the bonus token into the argmax of the last row."""
    rng = np.random.default_rng(11)
    n, k, V = 64, 4, 131072
    dl = (rng.standard_normal((n, k, V)) * 2).astype(np.float32)
    tl = np.concatenate([dl, (rng.standard_normal((n, 1, V)) * 2).astype(np.float32)], axis=1)
    toks = rng.integers(0, V, (n, k)).astype(np.int32)
    draws = rng.random((n, k + 1)).astype(np.float32)
    n_acc, nxt = pool.spec_accept(n, k, V, toks, dl, tl, draws, temperature=1e-10)
    assert n_acc.tolist() == [k] * n
    assert nxt.tolist() == tl[:, k].argmax(axis=1).tolist()
    # a target that puts no mass on the draft tokens rejects the first one; the resampled token is never the draft's
    tl2 = tl.copy()
    tl2[np.arange(n), 0, toks[:, 0]] = -80.0
    n_acc, nxt = pool.spec_accept(n, k, V, toks, dl, tl2, np.full((n, k + 1), 0.5, np.float32))
    assert n_acc.tolist() == [0] * n
    assert not np.any(nxt == toks[:, 0])
