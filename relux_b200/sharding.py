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
