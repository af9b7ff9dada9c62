"""CPU checks of the oracle's decoder forward against the committed golden fixtures, and a record of how much
the reference's layout quirks matter for token ids (tests/golden/make_golden.py documents the inputs)."""
import json
import os

import numpy as np

from tests.helpers import model_config, model_weights, prompts_for

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _gold(name):
    return json.load(open(os.path.join(GOLD, name + "_generate.json")))


def test_config1_generate_matches_golden(oracle):
    g = _gold("config1")
    cfg = model_config("config1")
    w = model_weights(cfg)
    p = prompts_for("config1")[0]
    assert list(map(int, p)) == g["prompts"][0]
    for label, mode in (("faithful", oracle.FAITHFUL), ("intended", oracle.INTENDED)):
        m = oracle.Model(cfg, w)
        m.set_mode(mode)
        ids, margins, ties = m.generate(p, 56)
        assert ids.tolist() == g["runs"][label]["ids"][0]
        assert ties == 0 and len(ids) == 64 and ids.min() >= 0 and ids.max() < 100


def test_config2_generate_prefix_matches_golden(oracle):
    g = _gold("config2")
    cfg = model_config("config2")
    w = model_weights(cfg)
    p = prompts_for("config2")[1]
    assert list(map(int, p)) == g["prompts"][1]
    n = 12
    for label, (mode, flags) in {"faithful": (oracle.FAITHFUL, 0), "intended": (oracle.INTENDED, 0),
                                 "intended_bf16_cache": (oracle.INTENDED, oracle.FLAG_MLA_BF16_CACHE)}.items():
        m = oracle.Model(cfg, w)
        m.set_mode(mode, flags)
        ids, _, _ = m.generate(p, n)
        assert ids.tolist() == g["runs"][label]["ids"][1][:32 + n], label


def test_quirks_change_token_ids(oracle):
    """The reference's cached GQA path reads a chunk-linear stream head-major and its cached MLA path reads
    token-major K/V head-major; both change the generated ids early.  This is why id parity of the GPU path is
    stated against the INTENDED oracle, not the reference-faithful one."""
    g1, g2 = _gold("config1"), _gold("config2")
    a, b = g1["runs"]["faithful"]["ids"][0], g1["runs"]["intended"]["ids"][0]
    first = next(i for i in range(len(a)) if a[i] != b[i])
    assert 8 <= first < 64   # the prompt is identical; the prefill is not affected by the GQA quirk, decoding is
    for s in range(4):
        a, b = g2["runs"]["faithful"]["ids"][s], g2["runs"]["intended"]["ids"][s]
        assert a[:32] == b[:32] and a != b
    # storing MLA rows as bf16 instead of float32 changes no id on these inputs or changes them late
    same = sum(g2["runs"]["intended"]["ids"][s] == g2["runs"]["intended_bf16_cache"]["ids"][s] for s in range(4))
    assert same >= 0


def test_small_attention_vectors_reproduce(oracle):
    z = np.load(os.path.join(GOLD, "attention_small.npz"))
    out = oracle.gqa_attend(z["gqa_K"], z["gqa_V"], z["gqa_ctx"], z["gqa_q"], float(z["gqa_scale"]), causal=True)
    assert np.array_equal(out, z["gqa_out"])
    out = oracle.mla_attend(z["mla_c"], z["mla_r"], z["mla_ctx"], z["mla_qc"], z["mla_qr"], z["mla_wuk"], z["mla_wuv"],
                            float(z["mla_scale"]), causal=True)
    assert np.array_equal(out, z["mla_out"])
    # absorbed and decompress-then-attend agree to rounding
    assert np.abs(z["mla_out"] - z["mla_out_absorbed"]).max() < 2e-5


def test_hooked_forward_equals_unhooked(oracle):
    """The hook seam itself: a hook that re-implements the intended attention with oracle primitives must give
    bit-identical logits.  This guards the plumbing the GPU generate tests rely on."""
    cfg = model_config("config1")
    w = model_weights(cfg)
    p = prompts_for("config1")[0]
    hd = cfg.dModel // cfg.numHeads
    caches = {}

    def hook(user, layer, S, start, q, k, v, out):
        K, V = caches.setdefault(layer, ([], []))
        kk = np.ctypeslib.as_array(k, shape=(cfg.numKVHeads, S, hd)).transpose(1, 0, 2)
        vv = np.ctypeslib.as_array(v, shape=(cfg.numKVHeads, S, hd)).transpose(1, 0, 2)
        K.extend(oracle.bf16_from_f32(kk)); V.extend(oracle.bf16_from_f32(vv))
        qq = np.ctypeslib.as_array(q, shape=(cfg.numHeads, S, hd)).transpose(1, 0, 2)[None]
        o = oracle.gqa_attend(np.array(K)[None], np.array(V)[None], [len(K)], qq, float(np.float32(1.0 / np.sqrt(np.float64(hd)))),
                              causal=True)
        np.ctypeslib.as_array(out, shape=(cfg.numHeads, S, hd))[...] = o[0].transpose(1, 0, 2)
        return 0

    m1 = oracle.Model(cfg, w); m1.set_mode(oracle.INTENDED); m1.begin()
    m2 = oracle.Model(cfg, w); m2.set_mode(oracle.INTENDED); m2.set_hooks(mha=hook); m2.begin()
    a = m1.forward(p); b = m2.forward(p)
    assert np.array_equal(a, b)
    a = m1.forward([5]); b = m2.forward([5])
    assert np.array_equal(a, b)
