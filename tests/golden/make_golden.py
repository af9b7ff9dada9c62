"""Generates the golden fixtures of this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Go) cannot be executed where this repository is built, so these vectors come from the
C++ restatement in oracle/ -- they pin the oracle against regressions and give the GPU tests fixed
targets; they are NOT outputs of a real relux run (parity of cached attention stays unpinned).

Inputs follow the benchmark configurations:
  config 1: vocab 100, dModel 64, 4 heads / 2 KV heads, 2 layers, SwiGLU dFF 128, maxSeqLen 64, causal, RoPE;
            weights N(0, 0.02) from numpy PCG64 seed 0 rounded to bf16; prompt = 8 ids uniform in [0,100) from seed 1;
            56 greedy tokens.
  config 2: vocab 1024, dModel 256, 8 heads (content 32 + rope 16, value 32), latent 64, 4 layers, GELU dFF 512
            (the reference's default FFN), maxSeqLen 512; 4 prompts of 32 ids from seed 1; greedy decode to 512.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import binding as orc  # noqa: E402
from tests.helpers import model_config, model_weights, prompts_for  # noqa: E402


def run(cfg_name, modes, max_new=None):
    cfg = model_config(cfg_name)
    w = model_weights(cfg)
    out = {"config": cfg_name, "weights_seed": 0, "prompts_seed": 1, "runs": {}}
    prompts = prompts_for(cfg_name)
    for label, (mode, flags) in modes.items():
        ids_all, margins_all, ties_all = [], [], 0
        for p in prompts:
            m = orc.Model(cfg, w)
            m.set_mode(mode, flags)
            n_new = (cfg.maxSeqLen - len(p)) if max_new is None else max_new
            ids, margins, ties = m.generate(p, n_new)
            ids_all.append(ids.tolist())
            margins_all.append(float(margins.min()))
            ties_all += ties
        out["runs"][label] = {"ids": ids_all, "min_top1_top2_margin": margins_all, "exact_ties": ties_all}
        print(cfg_name, label, "min margin", min(margins_all), "ties", ties_all, flush=True)
    out["prompts"] = [list(map(int, p)) for p in prompts]
    return out


def attention_vectors():
    """Small standalone attention cases (oracle outputs with the reference arithmetic)."""
    rng = np.random.default_rng(42)
    out = {}
    # GQA: 2 sequences, 4 heads / 2 kv heads, head dim 16, 3 query tokens, causal
    K = orc.bf16_from_f32(rng.standard_normal((2, 40, 2, 16)).astype(np.float32))
    V = orc.bf16_from_f32(rng.standard_normal((2, 40, 2, 16)).astype(np.float32))
    q = rng.standard_normal((2, 3, 4, 16)).astype(np.float32)
    ctx = np.array([40, 23], np.int32)
    out["gqa"] = dict(K=K, V=V, q=q, ctx=ctx, scale=np.float32(0.25), out=orc.gqa_attend(K, V, ctx, q, 0.25, causal=True))
    # MLA: 2 sequences, 8 heads, content 32, rope 16, latent 64, 2 query tokens
    c = orc.bf16_from_f32(rng.standard_normal((2, 50, 64)).astype(np.float32))
    r = orc.bf16_from_f32(rng.standard_normal((2, 50, 16)).astype(np.float32))
    wuk = orc.bf16_from_f32(rng.standard_normal((64, 8 * 32)).astype(np.float32) * 0.1)
    wuv = orc.bf16_from_f32(rng.standard_normal((64, 8 * 32)).astype(np.float32) * 0.1)
    qc = rng.standard_normal((2, 2, 8, 32)).astype(np.float32)
    qr = rng.standard_normal((2, 2, 8, 16)).astype(np.float32)
    ctx = np.array([50, 17], np.int32)
    sc = np.float32(1.0 / np.sqrt(48.0))
    out["mla"] = dict(c=c, r=r, wuk=wuk, wuv=wuv, qc=qc, qr=qr, ctx=ctx, scale=sc,
                      out=orc.mla_attend(c, r, ctx, qc, qr, wuk, wuv, float(sc), causal=True),
                      out_absorbed=orc.mla_attend(c, r, ctx, qc, qr, wuk, wuv, float(sc), causal=True, absorbed=True))
    return out


if __name__ == "__main__":
    modes1 = {"faithful": (orc.FAITHFUL, 0), "intended": (orc.INTENDED, 0)}
    modes2 = {"faithful": (orc.FAITHFUL, 0), "intended": (orc.INTENDED, 0),
              "intended_bf16_cache": (orc.INTENDED, orc.FLAG_MLA_BF16_CACHE)}
    g1 = run("config1", modes1)
    json.dump(g1, open(os.path.join(HERE, "config1_generate.json"), "w"))
    g2 = run("config2", modes2)
    json.dump(g2, open(os.path.join(HERE, "config2_generate.json"), "w"))
    av = attention_vectors()
    flat = {}
    for k, d in av.items():
        for n, a in d.items():
            flat["%s_%s" % (k, n)] = np.asarray(a)
    np.savez_compressed(os.path.join(HERE, "attention_small.npz"), **flat)
    print("written")
