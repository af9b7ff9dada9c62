"""Pins the oracle against a real relux run, when one is available.

tests/golden/relux_golden_dump_test.go is a Go test for a maintainer with relux and a Go toolchain: it runs
MHA.forwardCached and MLA.forwardCached (a prompt of 8 tokens, then 4 single-token steps) on LCG-generated weights and
inputs and writes the outputs' float32 bit patterns to a JSON file.  With that file at tests/golden/relux_go_golden.json
the test below requires the oracle (FAITHFUL mode) to reproduce every bit.  Without it the comparison is skipped; the
harness itself (LCG, weight order, oracle layer call) still runs so that it cannot rot."""
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "relux_go_golden.json")
MASK = (1 << 64) - 1


class LCG:
    def __init__(self, seed):
        self.s = seed

    def take(self, n):
        out = np.empty(n, np.float32)
        s = self.s
        for i in range(n):
            s = (s * 6364136223846793005 + 1442695040888963407) & MASK
            v = (s >> 32) & 0xFFFFFFFF
            if v >= 1 << 31:
                v -= 1 << 32
            out[i] = np.float32(v) / np.float32(2147483648.0)
        self.s = s
        return out


def _run(oracle, mla):
    D, H, F, V = 64, 4, 4, 2
    hd = D // H
    if mla:
        cfg = oracle.ModelCfg(vocab=V, dModel=D, numHeads=H, numKVHeads=H, numLayers=1, dFF=F, maxSeqLen=64, ropeBase=10000.0, causal=1,
                              swiglu=0, mla=1, dC=32, dHR=8)
        # flat order of the oracle model: W_Q, W_DKV, W_UK, W_UV, W_KR, W_QR, W_O (the dumper draws in the same order)
        sizes = [D * H * hd, D * 32, 32 * H * hd, 32 * H * hd, D * 8, D * H * 8, H * hd * D]
        g = LCG(54321)
    else:
        cfg = oracle.ModelCfg(vocab=V, dModel=D, numHeads=H, numKVHeads=2, numLayers=1, dFF=F, maxSeqLen=64, ropeBase=10000.0, causal=1,
                              swiglu=0, mla=0, dC=0, dHR=0)
        sizes = [D * H * hd, D * 2 * hd, D * 2 * hd, H * hd * D]
        g = LCG(12345)
    attn = np.concatenate([oracle.bf16_from_f32(g.take(n) * np.float32(0.25)) for n in sizes])
    flat = np.concatenate([np.zeros(V * D, np.uint16), attn, np.zeros(D * F + F * D + D * V, np.uint16)])
    assert flat.size == oracle.Model.weight_count(cfg)
    m = oracle.Model(cfg, flat)
    m.set_mode(oracle.FAITHFUL)
    m.begin()
    outs = [m.attention_forward(0, g.take(8 * D).reshape(8, D))]
    for _ in range(4):
        outs.append(m.attention_forward(0, g.take(D).reshape(1, D)))
    return outs


@pytest.mark.parametrize("mla", [False, True])
def test_harness_runs_and_is_deterministic(oracle, mla):
    a, b = _run(oracle, mla), _run(oracle, mla)
    assert [x.shape for x in a] == [(8, 64)] + [(1, 64)] * 4
    assert all(np.isfinite(x).all() and np.abs(x).max() > 0 for x in a)
    assert all(np.array_equal(x, y) for x, y in zip(a, b))


@pytest.mark.parametrize("mla", [False, True])
def test_oracle_matches_a_real_relux_run(oracle, mla):
    if not os.path.exists(GOLD):
        pytest.skip("no tests/golden/relux_go_golden.json (produced by relux_golden_dump_test.go on a machine with Go)")
    gold = json.load(open(GOLD))["mla" if mla else "mha"]["outputs_f32_bits"]
    outs = _run(oracle, mla)
    for step, (o, gbits) in enumerate(zip(outs, gold)):
        want = np.asarray(gbits, np.uint32).view(np.float32).reshape(o.shape)
        assert np.array_equal(o.view(np.uint32), want.view(np.uint32)), "step %d differs from the relux run" % step


SAMPLER_SETTINGS = [
    dict(), dict(temperature=0.7), dict(top_k=40), dict(top_p=0.9), dict(min_p=0.05),
    dict(temperature=1.3, top_k=100, top_p=0.85, min_p=0.02, repeat_penalty=1.2, frequency_penalty=0.2, presence_penalty=0.3,
         repeat_window=16),
]


def _sampler_inputs():
    """Logits and token histories of the dumper's sampler section, in its order of draws."""
    g = LCG(777)
    rows = []
    for si in range(len(SAMPLER_SETTINGS)):
        for _ in range(8):
            logits = g.take(500) * np.float32(6)
            prev = ((g.take(24) + np.float32(1)) * np.float32(250)).astype(np.int64)
            rows.append((si, logits, prev))
    return rows


def test_sampler_harness_runs(oracle):
    rows = _sampler_inputs()
    assert len(rows) == 48
    for si, logits, prev in rows[::7]:
        tok = oracle.sampler_sample(oracle.sampler_cfg(**SAMPLER_SETTINGS[si]), logits, 0.5, prev=prev)
        assert 0 <= tok < 500 and prev.min() >= 0 and prev.max() < 500


def test_oracle_sampler_matches_a_real_relux_run(oracle):
    if not os.path.exists(GOLD) or "sampler" not in json.load(open(GOLD)):
        pytest.skip("no sampler section in tests/golden/relux_go_golden.json (produced by relux_golden_dump_test.go with Go)")
    cases = json.load(open(GOLD))["sampler"]["cases"]
    for (si, logits, prev), case in zip(_sampler_inputs(), cases):
        assert case["setting"] == si
        draw = float(np.asarray([case["draw_bits"]], np.uint32).view(np.float32)[0])
        tok = oracle.sampler_sample(oracle.sampler_cfg(**SAMPLER_SETTINGS[si]), logits, draw, prev=prev)
        assert tok == case["token"], "setting %d: oracle %d, relux %d" % (si, tok, case["token"])
