"""Pins the CPU oracle against every known-answer test the reference ships for this path.

Each test names the reference test it restates (paths inside the relux repository).
"""
import math

import numpy as np
import pytest


# ---- internal/transformer/kvcache_test.go ----------------------------------
def test_kvcache_new_empty(oracle):  # kvcache_test.go:9-14
    c = oracle.KVCache(4, oracle.KVCache.F32)
    assert c.total_len(0) == 0


def test_kvcache_append_first(oracle):  # kvcache_test.go:16-40
    c = oracle.KVCache(2, oracle.KVCache.F32)
    k = np.array([1, 2, 3, 4, 5, 6], np.float32).reshape(1, 2, 1, 3)
    v = np.array([7, 8, 9, 10, 11, 12], np.float32).reshape(1, 2, 1, 3)
    c.append(0, k, v)
    assert c.total_len(0) == 1
    ck, cv = c.view(0)
    assert ck.shape == (1, 2, 1, 3)
    assert ck.ravel().tolist() == [1, 2, 3, 4, 5, 6]
    assert cv.ravel().tolist() == [7, 8, 9, 10, 11, 12]


def test_kvcache_append_grows(oracle):  # kvcache_test.go:42-66
    c = oracle.KVCache(1, oracle.KVCache.F32)
    c.append(0, np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 1, 4), np.array([5, 6, 7, 8], np.float32).reshape(1, 1, 1, 4))
    assert c.total_len(0) == 1
    c.append(0, np.arange(9, 17, dtype=np.float32).reshape(1, 1, 2, 4), np.arange(17, 25, dtype=np.float32).reshape(1, 1, 2, 4))
    assert c.total_len(0) == 3
    ck, cv = c.view(0)
    assert ck.ravel().tolist() == [1, 2, 3, 4, 9, 10, 11, 12, 13, 14, 15, 16]
    assert cv.ravel().tolist() == [5, 6, 7, 8, 17, 18, 19, 20, 21, 22, 23, 24]


def test_kvcache_reset(oracle):  # kvcache_test.go:68-85
    c = oracle.KVCache(1, oracle.KVCache.F32)
    c.append(0, np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 1, 4), np.array([5, 6, 7, 8], np.float32).reshape(1, 1, 1, 4))
    assert c.total_len(0) == 1
    c.reset()
    assert c.total_len(0) == 0
    assert c.view(0) == (None, None)


def test_kvcache_bfloat16(oracle):  # kvcache_test.go:87-107
    c = oracle.KVCache(1, oracle.KVCache.BF16)
    c.append(0, np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 1, 4), np.array([5, 6, 7, 8], np.float32).reshape(1, 1, 1, 4))
    assert c.total_len(0) == 1
    kb, _ = c.view(0, raw_bf16=True)
    assert kb.dtype == np.uint16
    got = oracle.f32_from_bf16(kb.ravel())
    for i, g in enumerate(got):
        assert abs(g - (i + 1)) <= 0.01


def test_kvcache_sized_overflow_panics(oracle):  # kvcache.go:282-285
    c = oracle.KVCache(1, oracle.KVCache.BF16, max_len=2, num_kv_heads=1, head_dim=4)
    one = np.ones((1, 1, 1, 4), np.float32)
    c.append(0, one, one)
    c.append(0, one, one)
    with pytest.raises(RuntimeError):
        c.append(0, one, one)


def test_kvcache_sized_chunk_linear_stream(oracle):
    """kvcache.go:407-438 writes chunks linearly; mha.go:299-312 reads [Hkv,T,D].  With 2 KV heads a
    2-token prefill followed by a 1-token decode leaves the stream
    [h0t0 h0t1 h1t0 h1t1 | h0t2 h1t2] and the head-major view of head 1 starts at row 3."""
    c = oracle.KVCache(1, oracle.KVCache.F32, max_len=8, num_kv_heads=2, head_dim=1)
    pre = np.array([[10, 11], [20, 21]], np.float32).reshape(1, 2, 2, 1)   # [h][t]
    c.append(0, pre, pre)
    dec = np.array([12, 22], np.float32).reshape(1, 2, 1, 1)
    c.append(0, dec, dec)
    k, _ = c.view(0)
    assert k.shape == (1, 2, 3, 1)
    assert k.ravel().tolist() == [10, 11, 20, 21, 12, 22]


# ---- internal/transformer/dtype_test.go ------------------------------------
def test_bf16_round_trip_relative_error(oracle):  # dtype_test.go:10-35
    xs = np.array([0.1, 0.5, 1.0, 1.5, 3.14159, 100.0, 12345.678, -0.1, -100.0], np.float32)
    got = oracle.f32_from_bf16(oracle.bf16_from_f32(xs))
    assert np.all(np.abs(got - xs) / np.abs(xs) <= 0.01)


def test_bf16_powers_of_two_exact(oracle):  # dtype_test.go:37-49
    for p in range(-20, 21):
        x = np.float32(2.0 ** p)
        assert oracle.f32_from_bf16(oracle.bf16_from_f32([x]))[0] == x


def test_bf16_special_values(oracle):  # dtype_test.go:51-67
    r = oracle.f32_from_bf16(oracle.bf16_from_f32(np.array([np.inf, -np.inf, 0.0, -0.0], np.float32)))
    assert r[0] == np.inf and r[1] == -np.inf
    assert r[2] == 0 and not np.signbit(r[2])
    assert r[3] == 0 and np.signbit(r[3])


def test_bf16_slice_round_trip(oracle):  # dtype_test.go:69-81
    src = np.array([0.1, 0.2, 0.3, 1.5, -2.5, 100.25], np.float32)
    got = oracle.f32_from_bf16(oracle.bf16_from_f32(src))
    assert np.all(np.abs(got - src) <= 0.01 * np.abs(src))


def test_bf16_from_f64(oracle):  # dtype_test.go:83-99
    src = np.array([1.0, -1.0, 0.5, 100.5])
    got = oracle.f32_from_bf16(oracle.bf16_from_f64(src))
    assert got.tolist() == [1.0, -1.0, 0.5, 100.5]


def test_bf16_rne_rule(oracle):  # dtype_convert.go:15-24: u += 0x7FFF + lsb
    def enc(bits):
        return int(oracle.bf16_from_f32(np.array([bits], np.uint32).view(np.float32))[0])
    assert enc(0x3F808000) == 0x3F80   # tie, even mantissa stays
    assert enc(0x3F818000) == 0x3F82   # tie, odd mantissa rounds up
    assert enc(0x3F808001) == 0x3F81   # above tie
    assert enc(0x7F800001) == 0x7F80   # NaN with low payload collapses to +Inf (no special case)


# ---- internal/transformer/rope_test.go -------------------------------------
def test_rope_precompute_base(oracle):  # rope_test.go:10-20
    r = oracle.Rope(4, 10000, 4)
    assert r.cos()[0] == 1.0 and r.sin()[0] == 0.0


def test_rope_identity_at_zero(oracle):  # rope_test.go:22-34
    r = oracle.Rope(4, 10000, 4)
    x = np.array([1, 2, 3, 4], np.float32)
    assert np.all(np.abs(r.apply(x, 0) - x) <= 1e-5)


def test_rope_apply_at_position_one(oracle):  # rope_test.go:36-63
    r = oracle.Rope(4, 10000, 4)
    y = r.apply(np.array([1, 0, 0, 1], np.float32), 1)
    c0, s0 = np.float32(math.cos(1)), np.float32(math.sin(1))
    c1, s1 = np.float32(math.cos(0.01)), np.float32(math.sin(0.01))
    want = [c0, s0, -s1, c1]
    assert np.all(np.abs(y - np.array(want, np.float32)) <= 1e-5)


def test_rope_overflow_panics(oracle):  # rope_test.go:84-95
    r = oracle.Rope(4, 10000, 4)
    with pytest.raises(IndexError):
        r.apply(np.array([1, 2, 3, 4], np.float32), 4)


def test_rope_extend_preserves_old_entries(oracle):  # rope_test.go:97-146
    r = oracle.Rope(4, 10000, 4)
    c_old, s_old = r.cos(), r.sin()
    r.extend(8)
    assert r.max_seq_len == 8
    assert np.array_equal(r.cos()[:c_old.size], c_old) and np.array_equal(r.sin()[:s_old.size], s_old)
    r.apply(np.array([1, 2, 3, 4], np.float32), 7)
    with pytest.raises(ValueError):
        r.extend(8)


def test_rope_same_position_for_every_row_when_startpos_positive(oracle):  # rope.go:151-158
    r = oracle.Rope(4, 10000, 16)
    x = np.tile(np.array([1, 0, 0, 1], np.float32), (3, 1))
    y = r.apply(x, 5)
    assert np.array_equal(y[0], y[1]) and np.array_equal(y[1], y[2])
    y2 = r.apply(x, 5, intended_positions=True)
    assert not np.array_equal(y2[0], y2[1])
    assert np.array_equal(y2[0], y[0])


# ---- rmsnorm_test.go, sampler_test.go, mlp_test.go -------------------------
def test_rmsnorm_hand_computed(oracle):  # rmsnorm_test.go:14-25
    y = oracle.rmsnorm(np.array([1, 2, 3, 4], np.float32), 0.0)
    assert np.all(np.abs(y - np.array([0.3651, 0.7303, 1.0954, 1.4606], np.float32)) <= 1e-3)


def test_rmsnorm_identity(oracle):  # rmsnorm_test.go:27-40
    y = oracle.rmsnorm(np.array([2, 2, 2, 2], np.float32), 0.0)
    assert np.all(np.abs(y - 1.0) <= 1e-5)


def test_sampler_greedy(oracle):  # sampler_test.go:11-26
    assert oracle.greedy([1, 5, 3, 2, 4]) == 1
    assert oracle.greedy([5, 5, 3]) == 0


def test_gelu_at_one(oracle):  # mlp_test.go:30-52
    assert abs(oracle.lib().ro_gelu(1.0) - 0.8413) < 1e-3


# ---- softmaxRows / fastexp32 (mha.go:823-861): arithmetic restated, no reference test ----
def test_fastexp32_properties(oracle):
    assert abs(oracle.fastexp32(0.0) - 0.97586) < 1e-4
    assert oracle.fastexp32(-88.0) == 0.0
    xs = np.linspace(-20, 0, 2001)
    rel = np.array([oracle.fastexp32(float(x)) / math.exp(float(np.float32(x))) - 1 for x in xs])
    assert rel.min() > -0.04 and rel.max() < 0.035


def test_softmax_rows_sums_to_one_and_cuts_off(oracle):
    m = np.array([[0.0, -1.0, -30.0, -2.0]], np.float32)
    p = oracle.softmax_rows(m)
    assert abs(p.sum() - 1.0) < 1e-6
    assert p[0, 2] == 0.0
    assert p[0, 0] > p[0, 1] > p[0, 3] > 0


# ---- Sampler.Sample (sampler.go:73-218): the two property tests of sampler_test.go, over many draws ----
def test_sampler_temperature_zero_is_argmax(oracle):  # sampler_test.go:28-40
    cfg = oracle.sampler_cfg(temperature=1e-10)
    for r in np.linspace(0.0, 0.9999, 100):
        assert oracle.sampler_sample(cfg, [1, 5, 3], float(r)) == 1


def test_sampler_top_k_two(oracle):  # sampler_test.go:42-56
    cfg = oracle.sampler_cfg(top_k=2)
    got = {oracle.sampler_sample(cfg, [1, 5, 3, 2, 4], float(r)) for r in np.linspace(0.0, 0.9999, 100)}
    assert got == {1, 4}


def test_sampler_filters_compose(oracle):
    """penalties -> temperature -> top-k -> softmax -> top-p -> min-p -> draw (sampler.go:31-33): each filter only ever
    removes tokens, the result sums to one, and the repetition penalty lowers a seen token's probability."""
    rng = np.random.default_rng(4)
    logits = (rng.standard_normal(500) * 2).astype(np.float32)
    _, base = oracle.sampler_sample(oracle.sampler_cfg(), logits, 0.5, return_probs=True)
    for kw in (dict(top_k=20), dict(top_p=0.8), dict(min_p=0.1), dict(top_k=50, top_p=0.9, min_p=0.05, temperature=0.7)):
        _, p = oracle.sampler_sample(oracle.sampler_cfg(**kw), logits, 0.5, return_probs=True)
        assert abs(float(p.sum()) - 1.0) < 1e-4
        assert np.all((p > 0) <= (base > 0)) and (p > 0).sum() < (base > 0).sum()
    _, p20 = oracle.sampler_sample(oracle.sampler_cfg(top_k=20), logits, 0.5, return_probs=True)
    assert (p20 > 0).sum() == 20 and set(np.argsort(-logits)[:20]) == set(np.nonzero(p20)[0])
    tok = int(np.argmax(logits))
    _, pen = oracle.sampler_sample(oracle.sampler_cfg(repeat_penalty=1.5, presence_penalty=0.5), logits, 0.5, prev=[tok, tok],
                                   return_probs=True)
    assert pen[tok] < base[tok]


# ---- acceptPhase / resampleRejected (speculative.go:211-295): no reference test; properties of the algorithm ----
def test_spec_accept_properties(oracle):
    rng = np.random.default_rng(8)
    k, V = 4, 300
    dl = (rng.standard_normal((k, V)) * 2).astype(np.float32)
    last = (rng.standard_normal((1, V)) * 2).astype(np.float32)
    toks = rng.integers(0, V, k)
    cfg = oracle.sampler_cfg(temperature=1e-10)
    # a draft equal to the target is accepted whole (acceptProb = 1 > every draw) and uses k + 1 draws
    n, nxt, used, ap = oracle.spec_accept(cfg, toks, dl, np.vstack([dl, last]), rng.random(k + 1))
    assert (n, used) == (k, k + 1) and nxt == int(np.argmax(last)) and np.all(ap == 1.0)
    # a target without mass on the second draft token rejects there; the resampled token never is that token
    tl = np.vstack([dl, last])
    tl[1, toks[1]] = -90.0
    n, nxt, used, ap = oracle.spec_accept(cfg, toks, dl, tl, np.asarray([0.0, 0.5, 0.5, 0.5, 0.5], np.float32))
    assert (n, used) == (1, 3) and ap[1] == 0.0 and nxt != toks[1]
    # acceptProb is min(1, p_target / p_draft) of the drafted token
    tl = np.vstack([dl + (rng.standard_normal((k, V)) * 0.5).astype(np.float32), last])
    _, _, _, ap = oracle.spec_accept(cfg, toks, dl, tl, np.zeros(k + 1, np.float32))
    for i in range(k):
        want = min(1.0, float(oracle.softmax_alloc(tl[i])[toks[i]]) / float(oracle.softmax_alloc(dl[i])[toks[i]]))
        assert abs(float(ap[i]) - want) < 1e-6
