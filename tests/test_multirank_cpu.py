"""The N>1 path of the benchmark on CPU: two gloo ranks shard a batch with no data-path collective, time their own
share, and agree on max-over-ranks timing -- the same calls bench.py makes under NCCL."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_cover_the_batch():
    from relux_b200.sharding import shard_range
    for n in (1, 7, 64, 128, 129):
        for world in (1, 2, 4, 8):
            got = []
            for r in range(world):
                b, e = shard_range(n, world, r)
                got.extend(range(b, e))
            assert got == list(range(n))
            sizes = [shard_range(n, world, r)[1] - shard_range(n, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def test_balanced_assignment_of_ragged_lengths():
    from relux_b200.sharding import balanced_assignment
    rng = np.random.default_rng(11)
    lens = rng.integers(1024, 32769, 128)   # the ragged long-context configuration
    parts = balanced_assignment(lens, 8)
    assert sorted(i for p in parts for i in p) == list(range(128))
    loads = [int(lens[p].sum()) for p in parts]
    assert (max(loads) - min(loads)) / max(loads) < 0.02
    # with a fixed number of sequence slots per rank (the benchmark's pools hold 16 sequences each)
    parts = balanced_assignment(lens, 8, per_rank=16)
    assert sorted(i for p in parts for i in p) == list(range(128)) and all(len(p) == 16 for p in parts)
    loads = [int(lens[p].sum()) for p in parts]
    assert (max(loads) - min(loads)) / max(loads) < 0.05
    with pytest.raises(ValueError):
        balanced_assignment(lens, 4, per_rank=16)


def test_two_gloo_ranks_shard_and_reduce_timings():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    prog = textwrap.dedent("""
        import os, sys, json
        sys.path.insert(0, %r)
        import torch, torch.distributed as dist
        from relux_b200.sharding import shard_range, aggregate_throughput
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        b, e = shard_range(129, world, rank)
        dist.barrier()
        my_ms = 10.0 + 5.0 * rank          # pretend device times
        t = torch.tensor([my_ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n = torch.tensor([e - b], dtype=torch.int64)
        dist.all_reduce(n)                 # only the bookkeeping is reduced; no cache data ever moves
        if rank == 0:
            print(json.dumps({"max_ms": float(t.item()), "units": int(n.item()),
                              "tps": aggregate_throughput([int(n.item())], [float(t.item())])}))
        dist.destroy_process_group()
    """ % ROOT)
    import json
    import tempfile
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    with tempfile.TemporaryDirectory() as d:
        script = os.path.join(d, "ranks.py")
        open(script, "w").write(prog)
        out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                              "127.0.0.1", "--master-port", str(port), script], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    d = json.loads(line)
    assert d["max_ms"] == 15.0 and d["units"] == 129 and abs(d["tps"] - 129 / 0.015) < 1e-6


def test_stream_partition_properties():
    """The partition the persistent MLA decode kernel walks (host statement of the same arithmetic): every page of every
    sequence is in exactly one item, items of a sequence and of a worker are contiguous, no worker holds more than one
    range, ranges are whole tiles."""
    import __graft_entry__ as g
    g.build()     # the partition arithmetic is the library's own host code (no GPU needed to call it)
    from relux_b200.sharding import stream_partition
    rng = np.random.default_rng(4)
    cases = [[512] * 64, [1], [0, 3, 0, 9], list(rng.integers(1, 200, 300)), [9000], list(rng.integers(16, 513, 16))]
    for pages in cases:
        for workers in (1, 7, 74):
            G, W, items, wf, co = stream_partition(pages, workers, 2)
            total = int(np.sum(pages))
            assert G % 2 == 0 and G >= 4
            assert W == max(1, -(-total // G)) and W <= max(workers, 1)
            covered = {}
            start = np.concatenate([[0], np.cumsum(pages)])
            for k, (i, b, e, w) in enumerate(items):
                assert 0 <= b < e <= pages[i]
                lo, hi = start[i] + b, start[i] + e
                assert lo // G == w == (hi - 1) // G                      # an item lies inside its worker's range
                for pg in range(b, e):
                    assert (i, pg) not in covered
                    covered[(i, pg)] = k
            assert len(covered) == total
            assert list(items[:, 0]) == sorted(items[:, 0]) and list(items[:, 3]) == sorted(items[:, 3])
            for i in range(len(pages)):
                assert list(items[co[i]:co[i + 1], 0]) == [i] * (co[i + 1] - co[i])
            for w in range(W):
                assert all(items[k, 3] == w for k in range(wf[w], wf[w + 1]))
            assert wf[W] == len(items)
            loads = np.bincount(items[:, 3], weights=items[:, 2] - items[:, 1], minlength=W)
            assert loads.max() <= G
