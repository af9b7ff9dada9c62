"""Batch sharding across GPUs: sequences are independent, so a rank owns a contiguous slice of the batch and its
own pool; there is no data-path collective.  Used by the benchmark's multi-rank mode."""


def shard_range(n_items, world, rank):
    """Contiguous, balanced slice [begin, end) of n_items owned by `rank` (earlier ranks get the remainder)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank %d/%d" % (world, rank))
    base, rem = divmod(n_items, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def balanced_assignment(lengths, world, per_rank=None):
    """Greedy longest-first assignment of sequences to ranks by context length (for ragged batches):
    returns a list of index lists, one per rank.  With `per_rank` every rank receives at most that many
    sequences (a rank whose pool has a fixed number of sequence slots)."""
    if per_rank is not None and per_rank * world < len(lengths):
        raise ValueError("%d sequences do not fit %d ranks of %d slots" % (len(lengths), world, per_rank))
    order = sorted(range(len(lengths)), key=lambda i: -int(lengths[i]))
    loads = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        open_ranks = [r for r in range(world) if per_rank is None or len(out[r]) < per_rank]
        r = min(open_ranks, key=lambda k: loads[k])
        out[r].append(i)
        loads[r] += int(lengths[i])
    return out


def aggregate_throughput(units_per_rank, ms_per_rank):
    """Whole-job throughput: all units of all ranks over the slowest rank's device time."""
    return float(sum(units_per_rank)) / (max(ms_per_rank) * 1e-3)


def stream_partition(pages, workers, page_multiple=2):
    """The stream partition of the persistent MLA decode kernel for sequences of pages[i] pages (computed by the
    library on the host; no GPU needed).  Returns (range_pages, n_workers, items, worker_first, chunk_off) with items an
    int32 array [n, 4] of {seq_index, page_begin, page_end, worker}."""
    import ctypes as C

    import numpy as np

    from . import lib as L
    lib = L.load()
    pg = np.ascontiguousarray(pages, dtype=np.int32)
    cap = int(len(pg) + max(1, workers) + int(pg.sum()) // 2 + 8)
    items = np.empty((cap, 4), np.int32)
    wf = np.empty(cap + 2, np.int32)
    co = np.empty(len(pg) + 1, np.int32)
    G, W = C.c_int32(), C.c_int32()
    args = L.StreamPartitionArgs(pages=pg.ctypes.data, n_seqs=len(pg), workers=int(workers), page_multiple=int(page_multiple), cap=cap,
                                 range_pages_out=C.addressof(G), workers_out=C.addressof(W), items_out=items.ctypes.data,
                                 worker_first=wf.ctypes.data, chunk_off=co.ctypes.data)
    n = lib.relux_stream_partition(C.byref(args))
    if n < 0:
        raise ValueError("stream_partition: bad arguments")
    return G.value, W.value, items[:n].copy(), wf[:W.value + 1].copy(), co
