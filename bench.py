#!/usr/bin/env python
"""Benchmark of the hot path: per-step append + absorbed MLA flash-decode over a paged latent cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload `mla_decode_b64_ctx32k` (default): DeepSeek-V2-like MLA shapes (128 heads, latent 512, rope key 64,
nope/v 128), batch 64 per GPU, 32768 cached tokens per sequence, 64-token pages in a randomly permuted
page table; one step = append one new token per sequence, then decode.  Synthetic seeded data.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank owns its own batch of 64
sequences and its own pool: sequences are independent, so there is no data-path collective (weak scaling).

One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, batch per GPU, context, heads, head_dim, dC, dHR)
    "mla_decode_b64_ctx32k": dict(kind="mla", B=64, ctx=32768, H=128, Dh=128, dC=512, dHR=64),
    "mla_decode_b64_ctx4k": dict(kind="mla", B=64, ctx=4096, H=128, Dh=128, dC=512, dHR=64),
    # the reference's own MLA example shape (mla_test.go:96-101: d_model 4096, 32 heads of 128, latent 512, rope 64)
    "mla_decode_h32_b64_ctx32k": dict(kind="mla", B=64, ctx=32768, H=32, Dh=128, dC=512, dHR=64),
    # MLA speculative verify: 4 draft tokens per step (the tensor work is 4x a decode step, the cache is read from HBM once)
    "mla_verify_b64_ctx32k": dict(kind="mla", B=64, ctx=32768, H=128, Dh=128, dC=512, dHR=64, S=4),
    # config 4 per GPU: 16 sequences with context lengths uniform in [1024, 32768] (one global seeded draw of 16 x world
    # lengths, dealt to the ranks longest-first so that every GPU holds about the same number of cached tokens)
    "mla_decode_ragged_b16": dict(kind="mla", B=16, ctx=32768, H=128, Dh=128, dC=512, dHR=64, ragged=True),
    # the whole attention layer step on the device (projections + RoPE + append + decode + output projection)
    "mla_layer_b64_ctx32k": dict(kind="mla", B=64, ctx=32768, H=128, Dh=128, dC=512, dHR=64, layer=True),
    "mla_layer_b16_ctx4k": dict(kind="mla", B=16, ctx=4096, H=128, Dh=128, dC=512, dHR=64, layer=True),
    # small enough for an ncu --set full capture (302 MB of cache rows, still larger than the 126 MB L2)
    "mla_decode_b16_ctx16k": dict(kind="mla", B=16, ctx=16384, H=128, Dh=128, dC=512, dHR=64),
    # GQA flash-decode + speculative verify: 4 draft tokens per step, accepted prefix uniform in 1..4
    "gqa_verify_b128_ctx8k": dict(kind="gqa", B=128, ctx=8192, H=32, Hkv=8, D=128, S=4),
    "gqa_verify_b16_ctx8k": dict(kind="gqa", B=16, ctx=8192, H=32, Hkv=8, D=128, S=4),
    # the whole GQA layer step of a verify: x [B, 4, 4096] -> projections + RoPE + draft rows + attention + Wo
    # token selection after a verify pass (acceptPhase + resampleRejected + Sampler.Sample) for 64 sequences, four draft
    # tokens, a vocabulary of 131072: 302 MB of float32 logits per step
    "spec_accept_b64_k4_v128k": dict(kind="accept", B=64, k=4, V=131072),
    # smaller case for profiler captures (151 MB of logits, still larger than L2)
    "spec_accept_b32_k4_v128k": dict(kind="accept", B=32, k=4, V=131072),
    # prompt processing through the decode kernels (a multi-token cached call on an empty cache): 8 sequences x 2048 tokens
    "gqa_prompt_b8_2k": dict(kind="prompt", pool="gqa", B=8, S=2048, H=32, Hkv=8, D=128),
    "gqa_prompt_b2_2k": dict(kind="prompt", pool="gqa", B=2, S=2048, H=32, Hkv=8, D=128),   # small case for profiler captures
    "gqa_prompt_b2_8k": dict(kind="prompt", pool="gqa", B=2, S=8192, H=32, Hkv=8, D=128),   # a long prompt: 32 tiles per block on average
    "mla_prompt_b4_1k": dict(kind="prompt", pool="mla", B=4, S=1024, H=128, Dh=128, dC=512, dHR=64),
    "mla_prompt_b1_2k": dict(kind="prompt", pool="mla", B=1, S=2048, H=128, Dh=128, dC=512, dHR=64),   # small case for profiler captures
    "mla_prompt_b8_2k": dict(kind="prompt", pool="mla", B=8, S=2048, H=128, Dh=128, dC=512, dHR=64),
    "mla_prompt_b2_8k": dict(kind="prompt", pool="mla", B=2, S=8192, H=128, Dh=128, dC=512, dHR=64),
    "gqa_layer_verify_b128_ctx8k": dict(kind="gqa", B=128, ctx=8192, H=32, Hkv=8, D=128, S=4, layer=True),
}
DEFAULT_WORKLOAD = "mla_decode_b64_ctx32k"
# config 3, config 4 (one GPU's share) and config 5 of the benchmark definition, then the two prompt workloads (the
# prefill kernels): run after the headline workload
ALSO_WORKLOADS = ("mla_decode_b64_ctx4k", "mla_decode_ragged_b16", "gqa_verify_b128_ctx8k", "gqa_prompt_b8_2k", "mla_prompt_b4_1k")
# dram__bytes_read + dram__bytes_write of the dominant kernel divided by its algorithmic bytes, from the ncu captures
# summarised under profiles/ (small case, traffic grows in proportion to the cached tokens read).
TRAFFIC_RATIO = {"mla": 1.04, "gqa": 1.015, "accept": 1.08}
PAGE = 64


def bf16_bits(x):
    """float32 array -> bf16 bit patterns, round to nearest even with the reference's rule (dtype_convert.go:15-24).
    Input preparation of the GPU arm; the oracle is not involved."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def workload_config(name, w, lens0=None):
    """The `config` object of a workload: the same keys in the GPU arm and in the reference arm."""
    kind = w["kind"]
    if kind == "mla":
        ctx0 = w["ctx"]
        rows = float(np.sum(lens0)) if lens0 is not None else float(w["B"]) * ctx0 * (0.515 if w.get("ragged") else 1.0)
        return {"workload": name, "batch_per_gpu": w["B"],
                "context": ("uniform[1024,%d] (seed 11), dealt to the ranks longest-first" % ctx0) if w.get("ragged") else ctx0,
                "heads": w["H"], "latent": w["dC"], "rope": w["dHR"], "query_tokens": int(w.get("S", 1)), "page_tokens": PAGE,
                "page_table": "random permutation",
                "l2": "inputs (about %.1f GB of cache rows per GPU) are larger than L2" % (rows * (w["dC"] + w["dHR"]) * 2 / 1e9)}
    if kind == "gqa":
        return {"workload": name, "batch_per_gpu": w["B"], "context": w["ctx"], "heads": w["H"], "kv_heads": w["Hkv"], "head_dim": w["D"],
                "draft_tokens": w["S"], "page_tokens": PAGE, "page_table": "random permutation",
                "l2": "inputs (%.2f GB of K/V per GPU) are larger than L2" % (w["B"] * w["ctx"] * w["Hkv"] * w["D"] * 4 / 1e9)}
    if kind == "accept":
        return {"workload": name, "batch_per_gpu": w["B"], "draft_tokens": w["k"], "vocab": w["V"],
                "sampler": dict(temperature=0.8, top_k=50, top_p=0.95),
                "l2": "inputs (%.2f GB of logits per GPU) are larger than L2" % (w["B"] * (2 * w["k"] + 1) * w["V"] * 4 / 1e9)}
    mla = w["pool"] == "mla"
    return {"workload": name, "batch_per_gpu": w["B"], "prompt_tokens": w["S"], "heads": w["H"],
            "l2": "every step rewrites and re-reads %.1f MB of cache rows; the flush between steps is the append itself"
                  % ((w["B"] * w["S"] * ((w["dC"] + w["dHR"]) if mla else 2 * w["Hkv"] * w["D"]) * 2) / 1e6)}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with a separate `nvidia-smi -lms 50` process while the timed region runs
    (read-only).  In-process NVML polling was tried and dropped: its queries share driver locks with kernel launches
    and slowed the timed loop by up to 2x."""

    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []   # (arrival time, fields)
        self.t_begin = None
        self.stop_flag = False
        self.proc = None

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw,clocks_event_reasons.active")
        vis = [x for x in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if x.strip()]
        dev_id = vis[self.index] if self.index < len(vis) else str(self.index)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", dev_id, "--query-gpu=" + q, "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                if self.stop_flag:
                    break
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 6:
                    self.samples.append((time.time(), parts))
        except Exception:
            pass

    def begin(self):
        """Marks the start of the timed region; earlier samples (warm-up) are used only if the region saw none."""
        self.t_begin = time.time()

    def finish(self):
        t_end = time.time()
        time.sleep(0.06)   # let the sample that covers the end of the region arrive
        self.stop_flag = True
        if self.proc:
            self.proc.terminate()
        inside = [s for t, s in self.samples if self.t_begin is not None and self.t_begin <= t <= t_end + 0.06]
        used = inside if inside else [s for _, s in self.samples]
        sm = [int(s[0]) for s in used if s[0].isdigit()]
        mx = [int(s[1]) for s in used if s[1].isdigit()]
        reasons = sorted({self.NAMES[i] for s in used for i in range(4) if s[2 + i].lower().startswith("active")})
        power = []
        masks = set()
        for s in used:
            if len(s) >= 8:
                try:
                    power.append(float(s[6]))
                except ValueError:
                    pass
                masks.add(s[7])
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm),
                "samples_inside_timed_region": len(inside), "power_w_max": max(power) if power else None,
                "reason_masks": sorted(masks), "source": "nvidia-smi -lms 50"}


def bind_rank_to_cores(local, world):
    """Gives every rank of a node its own slice of the host cores this process may use (affinity only; nothing of the
    GPU is touched): eight single-threaded ranks that share one affinity mask otherwise migrate over each other while
    they feed their copy streams.  Returns the cores chosen (for the JSON line)."""
    if not hasattr(os, "sched_getaffinity") or world <= 1:
        return None
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = max(1, len(cores) // world)
        mine = cores[local * per:(local + 1) * per] or cores
        os.sched_setaffinity(0, mine)
        return [mine[0], mine[-1]]
    except OSError:
        return None


HOST_CORES = None


def dist_setup(n_gpus):
    global HOST_CORES
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    HOST_CORES = bind_rank_to_cores(local, world)
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return world, rank, local, dist
    return 1, 0, 0, None


def barrier(dist):
    if dist is not None:
        dist.barrier()


def max_over_ranks(dist, x):
    if dist is None:
        return x
    import torch
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())



MIN_SECONDS = 3.0      # the timed region of --steps steps is repeated back to back until this much device time has passed
SETTLE_SECONDS = 1.0   # repeats that end within the first second (boost clocks, power-cap transient) do not enter the headline


def timed_repeats(dev, dist, step, steps, warmup, reset=None, min_seconds=MIN_SECONDS, sampler=None):
    """W warm-up steps, then the K-step region again and again, back to back with no host synchronisation in between,
    until `min_seconds` have passed; every repeat is bracketed by its own CUDA events on the launching stream.  `reset`
    runs between two repeats, outside their event pairs (it puts the sequence lengths back, so that every repeat is the
    same workload).  Returns the per-repeat device times (ms, max over ranks at the same repeat index is taken by the
    caller through `summarise`), the launches counted, and the host time of the loop."""
    for _ in range(warmup):
        step()
    if reset is not None:
        reset()
    dev.sync()
    barrier(dist)
    n0 = dev.launch_count()
    if sampler is not None:
        sampler.begin()
    events = []
    t0 = time.perf_counter()
    while True:
        a, b = dev.event(), dev.event()
        a.record()
        for _ in range(steps):
            step()
        b.record()
        events.append((a, b))
        if reset is not None:
            reset()
        if time.perf_counter() - t0 >= min_seconds or len(events) >= 4000:
            break
    dev.sync()
    host_s = time.perf_counter() - t0
    launches = dev.launch_count() - n0
    ms = [a.elapsed_ms(b) for a, b in events]
    for a, b in events:
        a.close(); b.close()
    barrier(dist)
    return ms, launches, host_s


def summarise(dist, ms, settle_seconds=SETTLE_SECONDS):
    """(headline ms of one K-step region, burst ms = the first repeat, repeats used, index of the first repeat used).
    Headline = median of the repeats that START after the first `settle_seconds` of device time (all repeats when the
    run is shorter than that); with several ranks, the maximum over ranks of each rank's median."""
    t, first = 0.0, len(ms)
    for i, x in enumerate(ms):
        if t >= settle_seconds * 1e3:
            first = i
            break
        t += x
    used = ms[first:] if first < len(ms) else ms
    if first >= len(ms):
        first = 0
    med = float(np.median(used))
    return max_over_ranks(dist, med), max_over_ranks(dist, float(ms[0])), len(used), first

# --------------------------------------------------------------------------------------------------
def run_mla(args, w, world, rank, local, dist):
    import relux_b200 as rb
    from relux_b200 import lib as L

    B, ctx0, H, Dh, dC, dHR = w["B"], w["ctx"], w["H"], w["Dh"], w["dC"], w["dHR"]
    S = int(w.get("S", 1))
    # the lengths are put back between repeats of the timed region, so a sequence grows by one region (+ warm-up) at most
    pages_per = (ctx0 + (args.steps + args.warmup + 2) * S + S + PAGE - 1) // PAGE + 1
    dev = rb.Device(local)
    rng = np.random.default_rng(7 + rank)
    pool = rb.Pool(dev, L.POOL_MLA, 1, B * pages_per, PAGE, B, pages_per, dC=dC, dHR=dHR)
    pool.set_tables(rng.permutation(B * pages_per).astype(np.int32).reshape(B, pages_per))
    # fill the cache: one seeded N(0,1) block of `blk` tokens per sequence, appended from device memory until every
    # sequence has its context length
    if w.get("ragged"):
        from relux_b200.sharding import balanced_assignment
        all_lens = np.random.default_rng(11).integers(1024, ctx0 + 1, B * world)
        lens0 = all_lens[balanced_assignment(all_lens, world, per_rank=B)[rank]].astype(np.int64)
    else:
        lens0 = np.full(B, ctx0, np.int64)
    blk = min(ctx0, 2048)
    src_c = bf16_bits(rng.standard_normal((B * blk, dC), dtype=np.float32))
    src_r = bf16_bits(rng.standard_normal((B * blk, dHR), dtype=np.float32))
    d_c, d_r = dev.upload(src_c), dev.upload(src_r)
    for off in range(0, int(lens0.max()), blk):
        pool.append(0, d_c, d_r, B, n_new=np.clip(lens0 - off, 0, blk).astype(np.int32))
    dev.sync()
    d_c.free(); d_r.free()
    wuk = bf16_bits((rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02))
    wuv = bf16_bits((rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02))
    d_wuk, d_wuv = dev.upload(wuk), dev.upload(wuv)
    scale = float(1.0 / np.sqrt(Dh + dHR))
    # per-step inputs: new latent row + rope key per sequence, queries; resident copies and pinned host copies
    new_c = rng.standard_normal((B, dC), dtype=np.float32)
    new_r = rng.standard_normal((B, dHR), dtype=np.float32)
    qc = rng.standard_normal((B, 1, H, Dh), dtype=np.float32)
    qr = rng.standard_normal((B, 1, H, dHR), dtype=np.float32)
    d_new_c, d_new_r = dev.upload(bf16_bits(new_c)), dev.upload(bf16_bits(new_r))
    d_qc, d_qr = dev.upload(bf16_bits(qc)), dev.upload(bf16_bits(qr))
    d_out = dev.alloc(B * H * Dh * 4, L.DTYPE_F32)
    # end-to-end arm: the new rows arrive as float32 (the reference appends float32 rows), the queries as bf16 (the
    # benchmark's standalone op is defined on bf16 q), the output leaves as bf16; all in page-locked host memory
    pins = [dev.pinned(a.shape, np.float32) for a in (new_c, new_r)] + [dev.pinned(a.shape, np.uint16) for a in (qc, qr)]
    for p_, a in zip(pins, (new_c, new_r, bf16_bits(qc), bf16_bits(qr))):
        p_.array[...] = a
    pin_outs = [dev.pinned((B, 1, H, Dh), np.uint16) for _ in range(2)]
    pin_out = pin_outs[0]
    e2e_calls = [0]
    e2e_checksum = [0]

    lens0_i32 = lens0.astype(np.int32)
    rows_now = [float(lens0.sum())]   # cached rows of all sequences, as the host tracks them
    rows_log = []                     # rows read by every attention call of the resident arm
    accepted = [0]

    def reset():
        pool.set_len(0, lens0_i32)
        rows_now[0] = float(lens0.sum())

    def step_resident():
        # one call per decode step: append of the new rows + attention over the cache that now holds them
        rows_now[0] += B
        rows_log.append(rows_now[0])
        pool.step(0, B, d_new_c, d_new_r, d_qc, d_out, H, Dh, scale, q_rope=d_qr, w_uk=d_wuk, w_uv=d_wuv)

    def step_e2e():
        # pipelined calls: this step's host -> device copies overlap the previous step's kernels; the previous step's
        # output is read (one value of it) once its copy has landed
        i = e2e_calls[0]
        pool.step(0, B, pins[0].array, pins[1].array, pins[2].array, pin_outs[i % 2].array, H, Dh, scale, q_rope=pins[3].array,
                  w_uk=d_wuk, w_uv=d_wuv, pipelined=True)
        if i >= 1:
            pool.wait_output(1)
            e2e_checksum[0] ^= int(pin_outs[(i - 1) % 2].array[0, 0, 0, 0])
        e2e_calls[0] = i + 1

    if S > 1:
        # verify step: S draft rows per sequence written past the cursor, S query tokens (causal inside the draft), then
        # an accepted prefix of 1..S tokens is committed; tokens/s counts accepted tokens
        dr_c = rng.standard_normal((B * S, dC), dtype=np.float32)
        dr_r = rng.standard_normal((B * S, dHR), dtype=np.float32)
        vq = rng.standard_normal((B, S, H, Dh), dtype=np.float32)
        vqr = rng.standard_normal((B, S, H, dHR), dtype=np.float32)
        d_dr_c, d_dr_r = dev.upload(bf16_bits(dr_c)), dev.upload(bf16_bits(dr_r))
        d_vq, d_vqr = dev.upload(bf16_bits(vq)), dev.upload(bf16_bits(vqr))
        d_vout = dev.alloc(B * S * H * Dh * 4, L.DTYPE_F32)
        vpins = [dev.pinned(a_.shape, np.float32) for a_ in (dr_c, dr_r, vq, vqr)]
        for p_, a_ in zip(vpins, (dr_c, dr_r, vq, vqr)):
            p_.array[...] = a_
        vpin_out = dev.pinned((B, S, H, Dh), np.float32)
        vlens = lens0.copy()

        def reset():
            vlens[:] = lens0
            pool.set_len(0, lens0_i32)

        def commit():
            acc = rng.integers(1, S + 1, B)
            vlens[:] += acc
            accepted[0] += int(acc.sum())
            pool.set_len(0, vlens.astype(np.int32))

        def step_resident():
            rows_log.append(float(vlens.sum()) + B * S)   # committed rows + the S draft rows of every sequence
            pool.verify(0, B, d_vq, d_vout, d_dr_c, d_dr_r, H, Dh, scale, S, q_rope=d_vqr, w_uk=d_wuk, w_uv=d_wuv)
            commit()

        def step_e2e():
            pool.verify(0, B, vpins[2].array, vpin_out.array, vpins[0].array, vpins[1].array, H, Dh, scale, S, q_rope=vpins[3].array,
                        w_uk=d_wuk, w_uv=d_wuv)
            commit()

    layer = bool(w.get("layer"))
    if layer:
        # layer step: x [B, 1, dModel] in, [B, 1, dModel] out; dModel = H * Dh like NewMLA.  Weights N(0, 1/in) -> bf16,
        # generated as one 1024-column block repeated along the output dimension (the values do not matter to the timing)
        D = H * Dh

        def weight(rows, cols):
            blk_cols = min(cols, 1024)
            blk_w = bf16_bits(rng.standard_normal((rows, blk_cols), dtype=np.float32) * np.float32(1.0 / np.sqrt(rows)))
            return dev.upload(np.ascontiguousarray(np.tile(blk_w, (1, cols // blk_cols))))

        dW = {"w_q": weight(D, H * Dh), "w_qr": weight(D, H * dHR), "w_dkv": weight(D, dC), "w_kr": weight(D, dHR),
              "w_uk": d_wuk, "w_uv": d_wuv, "w_o": weight(H * Dh, D)}
        weight_bytes = 2 * (D * (H * Dh + H * dHR + dC + dHR) + H * Dh * D)
        x_host = rng.standard_normal((B, 1, D), dtype=np.float32)
        d_x = dev.upload(x_host)
        d_y = dev.alloc(B * D * 4, L.DTYPE_F32)
        pin_x = dev.pinned(x_host.shape, np.float32)
        pin_x.array[...] = x_host
        pin_y = dev.pinned(x_host.shape, np.float32)

        def step_resident():
            rows_now[0] += B
            rows_log.append(rows_now[0])
            pool.forward_cached(0, B, d_x, d_y, dW, D, H)

        def step_e2e():
            pool.forward_cached(0, B, pin_x.array, pin_y.array, dW, D, H)

    K = args.steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_list, launches, host_s = timed_repeats(dev, dist, step_resident, K, args.warmup, reset, args.min_seconds, sampler if rank == 0 else None)
    clocks = sampler.finish() if rank == 0 else None
    ms_res, ms_burst, used, first_used = summarise(dist, ms_list)
    acc_per_step = accepted[0] / float(len(ms_list) * K + args.warmup) if S > 1 else 0.0
    # dominant kernel: the decode kernel; every call records a CUDA event pair around that launch on the launching
    # stream; read here for the calls of the repeats that make the headline (the library keeps the last 8192)
    kms = pool.kernel_ms_list(min(used * K, 8192))
    counted = len(kms)
    kernel_ms = float(np.mean(kms))
    rows_mean = float(np.mean(rows_log[-counted:]))            # cached rows read per launch, mean over those calls
    kernel_ms_burst = float(np.mean(pool.kernel_ms_list(len(ms_list) * K)[:K])) if len(ms_list) * K <= 8192 else None
    accepted[0] = 0
    # the end-to-end arm reads no kernel times: the decode kernel's event pairs (a measuring aid of the resident arm, two
    # records per call between the launches) are left out, as in a caller that does not profile
    pool.tune(L.TUNE_KERNEL_TIMING_STRIDE, 1 << 30)
    ms_e2e_list, _, _ = timed_repeats(dev, dist, step_e2e, K, args.warmup, reset, args.min_seconds)
    pool.tune(L.TUNE_KERNEL_TIMING_STRIDE, 1)
    ms_e2e, ms_e2e_burst, _, _ = summarise(dist, ms_e2e_list)
    acc_per_step_e2e = accepted[0] / float(len(ms_e2e_list) * K + args.warmup) if S > 1 else 0.0
    assert pool.status() == 0, "device status word is set"
    alg_bytes = rows_mean * (dC + dHR) * 2
    alg_flops = 2.0 * H * S * rows_mean * ((dC + dHR) + dC)
    peak, peak_src = read_peaks()
    pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if peak_src == "measured" else {}
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    tflops = alg_flops / (kernel_ms * 1e-3) / 1e12
    tokens = B * world
    value = tokens * K / (ms_res * 1e-3)
    e2e = tokens * K / (ms_e2e * 1e-3)
    value_burst = tokens * K / (ms_burst * 1e-3)
    h2d = sum(p_.array.nbytes for p_ in pins)
    d2h = pin_out.array.nbytes
    if layer:
        h2d, d2h = x_host.nbytes, x_host.nbytes
    if S > 1:   # accepted tokens; every rank draws from its own seeded stream with the same law
        value = acc_per_step * K * world / (ms_res * 1e-3)
        e2e = acc_per_step_e2e * K * world / (ms_e2e * 1e-3)
        value_burst = acc_per_step * K * world / (ms_burst * 1e-3)
        h2d, d2h = sum(a_.nbytes for a_ in (dr_c, dr_r, vq, vqr)), vpin_out.array.nbytes
    sm_mhz = (clocks or {}).get("sm_mhz")
    line = {
        "metric": "mla_layer_decode_tokens_per_s" if layer else ("mla_verify_accepted_tokens_per_s" if S > 1 else "mla_decode_tokens_per_s"), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": args.warmup, "ms_per_step": ms_res / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, w), "cached_tokens_rank0": int(lens0.sum()),
        "timing": {"repeats": len(ms_list), "repeats_in_headline": used, "first_repeat_in_headline": first_used,
                   "rule": "the %d-step region is repeated back to back for >= %.1f s; value = median of the repeats that start after the "
                           "first %.1f s of device time; lengths are put back between repeats" % (K, args.min_seconds, SETTLE_SECONDS),
                   "device_seconds": sum(ms_list) / 1e3, "host_seconds": host_s},
        "burst": {"value": value_burst, "ms_per_step": ms_burst / K, "kernel_ms": kernel_ms_burst,
                  "roofline_frac": (alg_bytes / (kernel_ms_burst * 1e-3) / 1e9 / peak) if kernel_ms_burst else None,
                  "what": "the first repeat of the timed region (boost clocks, before the power cap settles)"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (alg_bytes * TRAFFIC_RATIO["mla"]) if TRAFFIC_RATIO["mla"] else None,
                     "peak_source": peak_src, "kernel": "mla_decode_sm100_kernel", "kernel_ms": kernel_ms, "launches_timed": counted,
                     "algorithmic_bytes_per_launch": alg_bytes, "frac_of_nominal_8TBs": achieved / 8000.0,
                     "kernel_ms_x_sm_mhz": (kernel_ms * sm_mhz) if sm_mhz else None,
                     # the same kernel against the tensor roofline (128 heads put it at the ridge point)
                     "tensor": {"achieved": tflops, "unit": "TFLOP/s", "algorithmic_flops_per_launch": alg_flops,
                                "peak_burst": pk.get("bf16_tflops", 1590.0), "peak_sustained": pk.get("bf16_tflops_sustained", 1400.0),
                                "frac_of_burst": tflops / pk.get("bf16_tflops", 1590.0),
                                "frac_of_sustained": tflops / pk.get("bf16_tflops_sustained", 1400.0)}},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / K, "burst_value": (e2e * ms_e2e / ms_e2e_burst),
                "h2d_d2h_gbs_per_rank": (h2d + d2h) / (ms_e2e / K * 1e-3) / 1e9, "host_cores_rank0": HOST_CORES,
                "how": "pipelined calls (copies on their own streams, two steps in flight), page-locked host buffers; q and out "
                       "travel as bf16, the new rows as float32"},
        "gpu_launches": int(round(launches / float(len(ms_list)))), "clocks": clocks,
        "kv_read_gbs_whole_step": alg_bytes * world / (ms_res / K * 1e-3) / 1e9,
    }
    if layer:
        proj_ms, proj_n = pool.mean_projection_ms(args.steps)
        in_bytes = 2 * H * Dh * (H * Dh + H * dHR + dC + dHR)
        line["projections"] = {"kernel": "skinny_gemm_sm100_kernel (x . [W_Q | W_QR | W_DKV | W_KR])", "kernel_ms": proj_ms,
                               "launches_timed": proj_n, "weight_bytes_per_launch": in_bytes,
                               "achieved_gbs": in_bytes / (proj_ms * 1e-3) / 1e9, "frac_of_measured_hbm": in_bytes / (proj_ms * 1e-3) / 1e9 / peak,
                               "weight_bytes_per_step_all_projections": weight_bytes}
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_bounded(w)
        if layer:
            line["cpu_baseline"]["sample"] += "; attention part of the layer only (the projections are not included)"
    for b in (d_new_c, d_new_r, d_qc, d_qr, d_out, d_wuk, d_wuv):
        b.free()
    pool.destroy()
    dev.close()
    return line


def run_gqa(args, w, world, rank, local, dist):
    """GQA verify step: write 4 draft K/V rows per sequence past the cursor, attend causally inside the draft,
    commit an accepted prefix of 1..4 tokens.  tokens/s counts accepted tokens."""
    import relux_b200 as rb
    from relux_b200 import lib as L

    B, ctx0, H, Hkv, D, S = w["B"], w["ctx"], w["H"], w["Hkv"], w["D"], w["S"]
    # the lengths are put back between repeats of the timed region, so a sequence grows by one region (+ warm-up) at most
    pages_per = (ctx0 + (args.steps + args.warmup + 2) * S + S + PAGE - 1) // PAGE + 1
    dev = rb.Device(local)
    rng = np.random.default_rng(3 + rank)
    pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages_per, PAGE, B, pages_per, num_kv_heads=Hkv, head_dim=D)
    pool.set_tables(rng.permutation(B * pages_per).astype(np.int32).reshape(B, pages_per))
    blk = min(ctx0, 1024)
    srcK = bf16_bits(rng.standard_normal((B * blk, Hkv, D), dtype=np.float32))
    srcV = bf16_bits(rng.standard_normal((B * blk, Hkv, D), dtype=np.float32))
    dK, dV = dev.upload(srcK), dev.upload(srcV)
    for _ in range(ctx0 // blk):
        pool.append(0, dK, dV, B, n_new=np.full(B, blk, np.int32))
    dev.sync()
    dK.free(); dV.free()
    scale = float(1.0 / np.sqrt(D))
    q = rng.standard_normal((B, S, H, D), dtype=np.float32)
    nk = rng.standard_normal((B * S, Hkv, D), dtype=np.float32)
    nv = rng.standard_normal((B * S, Hkv, D), dtype=np.float32)
    d_q, d_nk, d_nv = dev.upload(bf16_bits(q)), dev.upload(bf16_bits(nk)), dev.upload(bf16_bits(nv))
    d_out = dev.alloc(q.size * 4, L.DTYPE_F32)
    # end to end: q and out travel as bf16 (the kernels' own input type; out is rounded on the device), the draft rows
    # as float32 like the rows of an append
    pins = [dev.pinned(q.shape, np.uint16), dev.pinned(nk.shape, np.float32), dev.pinned(nv.shape, np.float32)]
    for p_, a in zip(pins, (bf16_bits(q), nk, nv)):
        p_.array[...] = a
    pin_outs = [dev.pinned(q.shape, np.uint16) for _ in range(2)]
    pin_out = pin_outs[0]
    e2e_calls = [0]
    e2e_checksum = [0.0]
    lens = np.full(B, ctx0, np.int64)
    lens0_i32 = np.full(B, ctx0, np.int32)
    accepted_total = [0]

    def reset():
        lens[:] = ctx0
        pool.set_len(0, lens0_i32)

    def commit():
        acc = rng.integers(1, S + 1, B)
        lens[:] += acc
        accepted_total[0] += int(acc.sum())
        pool.set_len(0, lens.astype(np.int32))

    rows_read = []

    def step_resident():
        rows_read.append(float(lens.sum()) + B * S)   # committed rows + the S draft rows of every sequence
        pool.verify(0, B, d_q, d_out, d_nk, d_nv, H, D, scale, S)
        commit()

    def step_e2e():
        # pipelined calls (two independent batches in flight): this step's copies overlap the previous step's kernels; the
        # previous step's output is read once its copy has landed
        i = e2e_calls[0]
        pool.verify(0, B, pins[0].array, pin_outs[i % 2].array, pins[1].array, pins[2].array, H, D, scale, S, pipelined=True)
        commit()
        if i >= 1:
            pool.wait_output(1)
            e2e_checksum[0] += float(pin_outs[(i - 1) % 2].array[0, 0, 0, 0])
        e2e_calls[0] = i + 1

    layer = bool(w.get("layer"))
    if layer:
        dm = H * D   # dModel = numHeads * headDim like NewMHA

        def weight(rows, cols):
            return dev.upload(bf16_bits(rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(1.0 / np.sqrt(rows))))

        dW = {"w_q": weight(dm, H * D), "w_k": weight(dm, Hkv * D), "w_v": weight(dm, Hkv * D), "w_o": weight(H * D, dm)}
        x_host = rng.standard_normal((B, S, dm), dtype=np.float32)
        d_x = dev.upload(x_host)
        d_y = dev.alloc(x_host.size * 4, L.DTYPE_F32)
        pin_x = dev.pinned(x_host.shape, np.float32)
        pin_x.array[...] = x_host
        pin_y = dev.pinned(x_host.shape, np.float32)

        def step_resident():
            rows_read.append(float(lens.sum()) + B * S)
            pool.forward_cached(0, B, d_x, d_y, dW, dm, H, q_tokens=S, advance=False)
            commit()

        def step_e2e():
            pool.forward_cached(0, B, pin_x.array, pin_y.array, dW, dm, H, q_tokens=S, advance=False)
            commit()

    K = args.steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_list, launches, host_s = timed_repeats(dev, dist, step_resident, K, args.warmup, reset, args.min_seconds, sampler if rank == 0 else None)
    clocks = sampler.finish() if rank == 0 else None
    ms_res, ms_burst, used, first_used = summarise(dist, ms_list)
    # accepted tokens per step: the acceptance law is uniform on 1..S, every rank draws from its own seeded stream
    acc_per_step = accepted_total[0] / float((len(ms_list) * K + args.warmup))
    # dominant kernel: event pairs recorded by the calls of the repeats that make the headline (the library keeps the last 8192)
    kms = pool.kernel_ms_list(min(used * K, 8192))
    counted = len(kms)
    kernel_ms = float(np.mean(kms))
    alg_bytes = float(np.mean(rows_read[-counted:])) * Hkv * D * 2 * 2
    ms_e2e_list, _, _ = timed_repeats(dev, dist, step_e2e, K, args.warmup, reset, args.min_seconds)
    ms_e2e, ms_e2e_burst, _, _ = summarise(dist, ms_e2e_list)
    assert pool.status() == 0, "device status word is set"
    peak, peak_src = read_peaks()
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    sm_mhz = (clocks or {}).get("sm_mhz")
    line = {
        "metric": "gqa_layer_verify_accepted_tokens_per_s" if layer else "gqa_verify_accepted_tokens_per_s",
        "value": acc_per_step * K * world / (ms_res * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": K, "warmup": args.warmup, "ms_per_step": ms_res / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, w),
        "timing": {"repeats": len(ms_list), "repeats_in_headline": used, "first_repeat_in_headline": first_used,
                   "rule": "the %d-step region is repeated back to back for >= %.1f s; value = median of the repeats that start after the "
                           "first %.1f s of device time; lengths are put back between repeats" % (K, args.min_seconds, SETTLE_SECONDS),
                   "device_seconds": sum(ms_list) / 1e3, "host_seconds": host_s, "accepted_per_step": acc_per_step},
        "burst": {"value": acc_per_step * K * world / (ms_burst * 1e-3), "ms_per_step": ms_burst / K,
                  "what": "the first repeat of the timed region (boost clocks, before the power cap settles)"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": alg_bytes * TRAFFIC_RATIO["gqa"],
                     "peak_source": peak_src, "kernel": "gqa_decode_kernel", "kernel_ms": kernel_ms, "launches_timed": counted,
                     "algorithmic_bytes_per_launch": alg_bytes, "frac_of_nominal_8TBs": achieved / 8000.0,
                     "kernel_ms_x_sm_mhz": (kernel_ms * sm_mhz) if sm_mhz else None},
        "e2e": {"value": acc_per_step * K * world / (ms_e2e * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": int(x_host.nbytes) if layer else int(sum(p_.array.nbytes for p_ in pins)),
                "d2h_bytes_per_step": int(x_host.nbytes) if layer else int(pin_out.array.nbytes), "ms_per_step": ms_e2e / K,
                "how": "pipelined calls (copies on their own streams, two steps in flight), page-locked host buffers; q and out "
                       "travel as bf16, the draft rows as float32"},
        "gpu_launches": int(round(launches / float(len(ms_list)))), "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_bounded(w)
    for b in (d_q, d_nk, d_nv, d_out):
        b.free()
    pool.destroy()
    dev.close()
    return line


_CPU_INPUTS = {}   # inputs of the CPU legs, kept between steps of the reference arm


def run_prompt(args, w, world, rank, local, dist):
    """Prompt processing: every step empties the sequences, appends the S prompt rows and runs one causal multi-token
    attention call over them (device-resident inputs).  GQA prompts run on the tcgen05 prefill kernel (128 query rows per
    CTA); MLA prompts expand the cached latents into per-head keys / values (one tcgen05 GEMM) and run the same kernel
    with 192-wide scores.  The bound reported is the tensor pipe, for the attention kernel alone: 2 * S^2 / 2 * H * (Dqk +
    Dv) flop per sequence (GQA 128 + 128, MLA 192 + 128); the MLA line also carries the expansion's flops
    (2 * S * dC * 2 * H * 128 per sequence) and the time of the step outside the attention kernel."""
    import relux_b200 as rb
    from relux_b200 import lib as L

    B, S, H = w["B"], w["S"], w["H"]
    mla = w["pool"] == "mla"
    dev = rb.Device(local)
    rng = np.random.default_rng(7 + rank)
    pages = (S + PAGE - 1) // PAGE + 1
    if mla:
        dC, dHR, Dh = w["dC"], w["dHR"], w["Dh"]
        pool = rb.Pool(dev, L.POOL_MLA, 1, B * pages, PAGE, B, pages, dC=dC, dHR=dHR)
        rows_a = dev.upload(bf16_bits(rng.standard_normal((B * S, dC), dtype=np.float32)))
        rows_b = dev.upload(bf16_bits(rng.standard_normal((B * S, dHR), dtype=np.float32)))
        q = dev.upload(bf16_bits(rng.standard_normal((B, S, H, Dh), dtype=np.float32)))
        qr = dev.upload(bf16_bits(rng.standard_normal((B, S, H, dHR), dtype=np.float32)))
        wuk = dev.upload(bf16_bits(rng.standard_normal((dC, H * Dh), dtype=np.float32) * np.float32(0.02)))
        wuv = dev.upload(bf16_bits(rng.standard_normal((dC, H * Dh), dtype=np.float32) * np.float32(0.02)))
        out = dev.alloc(B * S * H * Dh * 4, L.DTYPE_F32)
        scale = float(1.0 / np.sqrt(Dh + dHR))
        flops = B * (S * (S + 1) / 2) * H * 2 * (Dh + dHR + Dh)
        expand_flops = B * S * 2.0 * dC * 2 * H * Dh
        kw = dict(q_rope=qr, w_uk=wuk, w_uv=wuv)
        head_dim = Dh
    else:
        Hkv, D = w["Hkv"], w["D"]
        pool = rb.Pool(dev, L.POOL_GQA, 1, B * pages, PAGE, B, pages, num_kv_heads=Hkv, head_dim=D)
        rows_a = dev.upload(bf16_bits(rng.standard_normal((B * S, Hkv, D), dtype=np.float32)))
        rows_b = dev.upload(bf16_bits(rng.standard_normal((B * S, Hkv, D), dtype=np.float32)))
        q = dev.upload(bf16_bits(rng.standard_normal((B, S, H, D), dtype=np.float32)))
        out = dev.alloc(B * S * H * D * 4, L.DTYPE_F32)
        scale = float(1.0 / np.sqrt(D))
        flops = B * (S * (S + 1) / 2) * H * 2 * 2 * D
        kw = {}
        head_dim = D
    pool.set_tables(rng.permutation(B * pages).astype(np.int32).reshape(B, pages))
    zeros, n_new = np.zeros(B, np.int32), np.full(B, S, np.int32)

    def step():
        pool.set_len(-1, zeros)
        pool.append(0, rows_a, rows_b, B, n_new=n_new)
        pool.decode(0, B, q, out, H, head_dim, scale, q_tokens=S, causal=True, **kw)

    steps, warmup = min(args.steps, 200), args.warmup
    for _ in range(warmup):
        step()
    dev.sync()
    barrier(dist)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
        sampler.begin()
    n0 = dev.launch_count()
    e0, e1 = dev.event(), dev.event()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    dev.sync()
    ms = max_over_ranks(dist, e0.elapsed_ms(e1))
    launches = dev.launch_count() - n0
    clocks = sampler.finish() if rank == 0 else None
    kernel_ms, counted = pool.mean_kernel_ms(steps)
    assert pool.status() == 0, "device status word is set"
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = json.load(open(pk)) if os.path.exists(pk) else {}
    peak = float(peaks.get("bf16_tflops", 1590.0))
    achieved = flops / (kernel_ms * 1e-3) / 1e12
    line = {
        "metric": "prompt_tokens_per_s", "value": B * S * world * steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args.workload, w),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": "measured" if peaks else "fallback", "kernel": "prefill_sm100_kernel<mla>" if mla else "prefill_sm100_kernel<gqa>",
                     "kernel_ms": kernel_ms, "launches_timed": counted, "algorithmic_flops_per_launch": flops},
        "e2e": None, "gpu_launches": launches, "clocks": clocks,
    }
    if mla:
        # everything of the step that is not the attention kernel: set_len, append, the expansion GEMM and its plan
        rest_ms = ms / steps - kernel_ms
        line["roofline"]["expansion"] = {"kernel": "mla_expand_sm100_kernel", "flops_per_launch": expand_flops,
                                         "step_ms_outside_attention": rest_ms,
                                         "whole_step_tflops": (flops + expand_flops) / (ms / steps * 1e-3) / 1e12}
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_prompt(w)
    pool.destroy()
    dev.close()
    return line


def cpu_baseline_prompt(w, threads=1, sample_S=None):
    """The CPU restatement on ONE sequence with a prompt of sample_S tokens (the cost grows with the square of the
    prompt length, so the figure belongs to that length)."""
    from oracle import binding as ob
    rng = np.random.default_rng(7)
    H = w["H"]
    if sample_S is None:
        sample_S = 96 if w["pool"] == "mla" else 512     # a few seconds each
    if w["pool"] == "mla":
        dC, dHR, Dh = w["dC"], w["dHR"], w["Dh"]
        c = bf16_bits(rng.standard_normal((1, sample_S, dC), dtype=np.float32))
        r = bf16_bits(rng.standard_normal((1, sample_S, dHR), dtype=np.float32))
        qc = rng.standard_normal((1, sample_S, H, Dh), dtype=np.float32)
        qr = rng.standard_normal((1, sample_S, H, dHR), dtype=np.float32)
        wuk = bf16_bits(rng.standard_normal((dC, H * Dh), dtype=np.float32) * np.float32(0.02))
        wuv = bf16_bits(rng.standard_normal((dC, H * Dh), dtype=np.float32) * np.float32(0.02))
        t0 = time.perf_counter()
        ob.mla_attend(c, r, np.asarray([sample_S], np.int32), qc, qr, wuk, wuv, float(1.0 / np.sqrt(Dh + dHR)), causal=True, threads=threads)
    else:
        Hkv, D = w["Hkv"], w["D"]
        K = bf16_bits(rng.standard_normal((1, sample_S, Hkv, D), dtype=np.float32))
        V = bf16_bits(rng.standard_normal((1, sample_S, Hkv, D), dtype=np.float32))
        q = rng.standard_normal((1, sample_S, H, D), dtype=np.float32)
        t0 = time.perf_counter()
        ob.gqa_attend(K, V, np.asarray([sample_S], np.int32), q, float(1.0 / np.sqrt(D)), causal=True, threads=threads)
    dt = time.perf_counter() - t0
    return {"value": sample_S / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": "one sequence, prompt of %d tokens instead of %d (%.1f s); cost grows with the square of the length" % (sample_S, w["S"], dt)}


def accept_inputs(w, seed):
    """Seeded logits with the shape of a verify pass: draft rows N(0, 2.5), target rows = draft + N(0, 0.6) noise, the
    drafted token is the draft row's argmax."""
    B, k, V = w["B"], w["k"], w["V"]
    rng = np.random.default_rng(seed)
    dl = rng.standard_normal((B, k, V), dtype=np.float32) * np.float32(2.5)
    tl = np.empty((B, k + 1, V), np.float32)
    tl[:, :k] = dl + rng.standard_normal((B, k, V), dtype=np.float32) * np.float32(0.6)
    tl[:, k] = rng.standard_normal((B, V), dtype=np.float32) * np.float32(2.5)
    toks = dl.argmax(axis=2).astype(np.int32)
    return toks, dl, tl, rng


def run_accept(args, w, world, rank, local, dist):
    import relux_b200 as rb
    from relux_b200 import lib as L

    B, k, V = w["B"], w["k"], w["V"]
    dev = rb.Device(local)
    pool = rb.Pool(dev, L.POOL_MLA, 1, 2, PAGE, 1, 2, dC=64, dHR=16)   # the call needs a pool for its stream and scratch
    toks, dl, tl, rng = accept_inputs(w, 7 + rank)
    n_draws = 32
    draws = [rng.random((B, k + 1), dtype=np.float32) for _ in range(n_draws)]
    d_toks, d_dl, d_tl = dev.upload(toks), dev.upload(dl), dev.upload(tl)
    d_draws = [dev.upload(d) for d in draws]
    pins = [dev.pinned(a.shape, a.dtype) for a in (toks, dl, tl)]
    for pin, a in zip(pins, (toks, dl, tl)):
        pin.array[...] = a
    sampler_kw = dict(temperature=0.8, top_k=50, top_p=0.95)
    step_no = [0]
    accepted_total = [0]
    rows_needed = []

    def account(n_acc):
        accepted_total[0] += int(n_acc.sum()) + B          # accepted draft tokens plus the resampled / bonus token
        rows_needed.append(float(np.where(n_acc < k, 2 * (n_acc + 1), 2 * k + 1).sum()))

    def step_resident():
        i = step_no[0] % n_draws
        step_no[0] += 1
        n_acc, _ = pool.spec_accept(B, k, V, d_toks, d_dl, d_tl, d_draws[i], **sampler_kw)
        account(n_acc)

    def step_e2e():
        i = step_no[0] % n_draws
        step_no[0] += 1
        n_acc, _ = pool.spec_accept(B, k, V, pins[0].array, pins[1].array, pins[2].array, draws[i], **sampler_kw)
        account(n_acc)

    e0, e1 = dev.event(), dev.event()

    def timed(fn, steps, warmup, sampler=None):
        for _ in range(warmup):
            fn()
        dev.sync()
        barrier(dist)
        n0 = dev.launch_count()
        accepted_total[0] = 0
        del rows_needed[:]
        if sampler is not None:
            sampler.begin()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        dev.sync()
        ms = e0.elapsed_ms(e1)
        barrier(dist)
        return max_over_ranks(dist, ms), dev.launch_count() - n0, accepted_total[0]

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_res, launches, acc_res = timed(step_resident, args.steps, args.warmup, sampler if rank == 0 else None)
    clocks = sampler.finish() if rank == 0 else None
    kernel_ms, counted = pool.mean_kernel_ms(args.steps)
    # algorithmic bytes: the logit rows the reference's loop touches (two per examined draft token, the last row when all
    # pass), each read once, float32
    alg_bytes = float(np.mean(rows_needed[-counted:])) * V * 4
    e2e_steps = max(3, min(args.steps, 50))
    ms_e2e, _, acc_e2e = timed(step_e2e, e2e_steps, 3)
    assert pool.status() == 0, "device status word is set"
    peak, peak_src = read_peaks()
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "spec_accept_tokens_per_s", "value": acc_res * world / (ms_res * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_res / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, w),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": alg_bytes * TRAFFIC_RATIO["accept"],
                     "peak_source": peak_src, "kernel": "spec_accept_kernel", "kernel_ms": kernel_ms, "launches_timed": counted,
                     "algorithmic_bytes_per_launch": alg_bytes},
        "e2e": {"value": acc_e2e * world / (ms_e2e * 1e-3), "unit": "tokens/s", "steps": e2e_steps,
                "h2d_bytes_per_step": int(toks.nbytes + dl.nbytes + tl.nbytes + draws[0].nbytes), "d2h_bytes_per_step": 8 * B},
        "gpu_launches": launches, "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_accept(w)
    pool.destroy()
    dev.close()
    return line


def cpu_baseline_accept(w, seqs=16, seconds=10.0):
    """The CPU restatement on `seqs` sequences of the same workload, one core, repeated with fresh draws for `seconds`."""
    from oracle import binding as ob
    key = ("accept", seqs)
    if key not in _CPU_INPUTS:
        _CPU_INPUTS[key] = accept_inputs(dict(w, B=seqs), 7)
    toks, dl, tl, rng = _CPU_INPUTS[key]
    cfg = ob.sampler_cfg(temperature=0.8, top_k=50, top_p=0.95)
    t0 = time.perf_counter()
    tokens = passes = 0
    while passes == 0 or time.perf_counter() - t0 < seconds:
        draws = rng.random((seqs, w["k"] + 1), dtype=np.float32)
        for b in range(seqs):
            tokens += ob.spec_accept(cfg, toks[b], dl[b], tl[b], draws[b])[0] + 1
        passes += 1
    dt = time.perf_counter() - t0
    return {"value": tokens / dt, "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": "%d of the %d sequences, %d passes with fresh draws, %.1f s" % (seqs, w["B"], passes, dt)}


def cpu_baseline_mla(w, sample_T, threads, seqs=None):
    """Times the oracle's restatement of the reference's own path (decompress every latent, then attend;
    mla.go:323-377) on `threads` host threads, one sequence per thread, at a reduced context, and scales the time
    linearly in context length to the workload's (the work is linear in T)."""
    from oracle import binding as orc
    H, Dh, dC, dHR, ctx = w["H"], w["Dh"], w["dC"], w["dHR"], w["ctx"]
    nb = seqs or threads
    key = ("mla", nb, sample_T, H, Dh, dC, dHR)
    if key not in _CPU_INPUTS:   # inputs are generated once per shape; only the oracle call is timed
        rng = np.random.default_rng(0)
        _CPU_INPUTS.clear()
        _CPU_INPUTS[key] = (orc.bf16_from_f32(rng.standard_normal((nb, sample_T, dC), dtype=np.float32)),
                            orc.bf16_from_f32(rng.standard_normal((nb, sample_T, dHR), dtype=np.float32)),
                            rng.standard_normal((nb, 1, H, Dh), dtype=np.float32), rng.standard_normal((nb, 1, H, dHR), dtype=np.float32),
                            orc.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02),
                            orc.bf16_from_f32(rng.standard_normal((dC, H * Dh), dtype=np.float32) * 0.02))
    ckv, kr, qc, qr, wuk, wuv = _CPU_INPUTS[key]
    t0 = time.time()
    orc.mla_attend(ckv, kr, [sample_T] * nb, qc, qr, wuk, wuv, 0.0722, threads=threads)
    dt = time.time() - t0
    return {"value": nb / (dt * (ctx / sample_T)), "unit": "tokens/s",
            "cores": threads, "kind": "port",
            "sample": "%d sequence(s) x 1 decode step at context %d (%.1f s), time scaled x%d to context %d; reference-style "
                      "decompress-then-attend in float32" % (nb, sample_T, dt, ctx // sample_T, ctx)}


def cpu_baseline_gqa(w, sample_T, threads, seqs=None):
    """Times the oracle's restatement of the reference's GQA verify step (widen the cached bf16 rows to float32,
    expand the KV heads by copy, attend S draft rows causally; mha.go:292-348) on `threads` host threads, one
    sequence per thread, at a reduced context, scaled linearly in context length.  tokens/s counts accepted tokens
    with the bench's acceptance law (uniform on 1..S, mean (S + 1) / 2 per sequence and step)."""
    from oracle import binding as orc
    H, Hkv, D, S, ctx = w["H"], w["Hkv"], w["D"], w["S"], w["ctx"]
    nb = seqs or threads
    key = ("gqa", nb, sample_T, H, Hkv, D, S)
    if key not in _CPU_INPUTS:
        rng = np.random.default_rng(0)
        _CPU_INPUTS.clear()
        _CPU_INPUTS[key] = (orc.bf16_from_f32(rng.standard_normal((nb, sample_T + S, Hkv, D), dtype=np.float32)),
                            orc.bf16_from_f32(rng.standard_normal((nb, sample_T + S, Hkv, D), dtype=np.float32)),
                            rng.standard_normal((nb, S, H, D), dtype=np.float32))
    K, V, q = _CPU_INPUTS[key]
    t0 = time.time()
    orc.gqa_attend(K, V, [sample_T + S] * nb, q, float(1.0 / np.sqrt(D)), causal=True, threads=threads, reference_cost=True)
    dt = time.time() - t0
    return {"value": nb * (S + 1) / 2.0 / (dt * (ctx / sample_T)), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": "%d sequence(s) x 1 verify step of %d draft tokens at context %d (%.2f s), time scaled x%d to context %d; "
                      "reference-style widen + head expansion + attend in float32" % (nb, S, sample_T, dt, ctx // sample_T, ctx)}


def cpu_baseline(w, threads, sample_T, seqs=None):
    if w["kind"] == "mla":
        return cpu_baseline_mla(w, sample_T=sample_T, threads=threads, seqs=seqs)
    return cpu_baseline_gqa(w, sample_T=sample_T, threads=threads, seqs=seqs)


def cpu_baseline_bounded(w):
    """The cpu_baseline leg of the default run: one host core, a sample of about 10 s."""
    if w["kind"] == "mla":
        return cpu_baseline(w, 1, sample_T=512)
    return cpu_baseline(w, 1, sample_T=w["ctx"], seqs=32)


def run_reference(args, w, world, rank):
    """--impl reference: the reference's own CPU algorithm (oracle restatement; the Go sources cannot be built
    here) on all host threads, on the same workload definition.  One step = one sequence per thread at a sample
    context chosen from a short calibration run so that warm-up + steps take about 100 s in total."""
    from oracle import binding as orc
    if rank != 0:
        return None
    if w["kind"] == "prompt":
        vals = [cpu_baseline_prompt(w) for _ in range(args.warmup + args.steps)][args.warmup:]
        v = float(np.mean([x["value"] for x in vals]))
        cb = dict(vals[-1], value=v)
        return {"impl": "reference", "metric": "prompt_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": w["B"] * w["S"] * world / v * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(args.workload, w),
                "cpu_baseline": cb, "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
    if w["kind"] == "accept":
        # the reference's accept loop is scalar Go: one core, sixteen sequences of the workload per pass
        vals = [cpu_baseline_accept(w, seconds=min(2.0, 100.0 / max(1, args.warmup + args.steps))) for _ in range(args.warmup + args.steps)][args.warmup:]
        v = float(np.mean([x["value"] for x in vals]))
        cb = dict(vals[-1], value=v)
        return {"impl": "reference", "metric": "spec_accept_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": w["B"] * world * (w["k"] + 2) / 2.0 / v * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(args.workload, w),
                "cpu_baseline": cb, "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
    # every host core this process may run on (a launcher's OMP_NUM_THREADS=1 default is not a property of the box)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or orc.num_threads())
    cpu_baseline(w, threads, sample_T=16)            # builds the inputs, warms the threads
    t0 = time.time()
    cpu_baseline(w, threads, sample_T=16)
    per_token = max(1e-6, (time.time() - t0) / 16)
    budget = 100.0 / max(1, args.warmup + args.steps)
    cap = 512 if w["kind"] == "mla" else w["ctx"]
    sample_T = int(max(2, min(w["ctx"], cap, budget / per_token)))
    if sample_T >= 16:
        sample_T = sample_T // 8 * 8
    vals = []
    for _ in range(args.warmup + args.steps):
        vals.append(cpu_baseline(w, threads, sample_T=sample_T))
    vals = vals[args.warmup:]
    v = float(np.mean([x["value"] for x in vals]))
    cb = dict(vals[-1])
    cb["value"] = v
    B = w["B"]
    metric = "mla_decode_tokens_per_s" if w["kind"] == "mla" else "gqa_verify_accepted_tokens_per_s"
    per_step = B * world if w["kind"] == "mla" else B * world * (w["S"] + 1) / 2.0
    return {"impl": "reference", "metric": metric, "value": v, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step / v * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.workload, w),
            "cpu_baseline": cb, "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="profiling runs: leave out the 10-30 s CPU baseline leg")
    ap.add_argument("--min-seconds", type=float, default=MIN_SECONDS,
                    help="the timed region of --steps steps is repeated back to back until this much time has passed (0: run it once)")
    ap.add_argument("--only", action="store_true", help="run the named workload alone (the default run appends short passes of the other "
                                                        "benchmark configurations under `also`)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        line = run_reference(args, w, world, rank)
        if line is not None:
            print(json.dumps(line))
        return
    world, rank, local, dist = dist_setup(args.gpus)
    runners = {"mla": run_mla, "gqa": run_gqa, "accept": run_accept, "prompt": run_prompt}
    line = runners[w["kind"]](args, w, world, rank, local, dist)
    if args.workload == DEFAULT_WORKLOAD and not args.only:
        # the other benchmark configurations, as shorter passes of the same measurement (every rank runs them, in this order)
        also = []
        for name in ALSO_WORKLOADS:
            sub = argparse.Namespace(**vars(args))
            sub.workload, sub.skip_cpu_baseline, sub.min_seconds = name, True, min(args.min_seconds, 2.0)
            wl = WORKLOADS[name]
            also.append(runners[wl["kind"]](sub, wl, world, rank, local, dist))
        line["also"] = also
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
