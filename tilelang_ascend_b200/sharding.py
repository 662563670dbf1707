"""Work partition for 1/2/4/8 GPUs: every (batch, query) row of the path is independent, so ranks take
contiguous blocks of queries (prefill, indexer, backward dQ) or of sequences (decode) and no
collective is needed inside the hot path; the small KV / index-key tensors are replicated."""
from __future__ import annotations

from typing import Tuple


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, end) of ``n`` items for ``rank`` of ``world``: contiguous, sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


# Cost of one query of the causal prefill forward in key tiles: the tiles of 64 keys it gathers plus a fixed part (loading
# its 128 x 576 Q block, draining and storing its 128 x 512 output, the hand-over between two queries) worth about three
# tiles -- fitted to the per-rank times of a 4-GPU run, where the rank with the many short queries was 4 % slower than
# the others under a fixed part of two.
KEYS_PER_TILE = 64
FIXED_TILES_PER_QUERY = 3


def causal_query_costs(S: int, s_kv: int, topk: int):
    """Relative cost of each of the S queries of a causal prefill call: query t sees min(s_kv - S + t + 1, topk) keys."""
    import numpy as np
    keys = np.minimum(np.arange(S, dtype=np.int64) + (s_kv - S) + 1, topk)
    return (keys + KEYS_PER_TILE - 1) // KEYS_PER_TILE + FIXED_TILES_PER_QUERY


def shard_range_balanced(costs, rank: int, world: int) -> Tuple[int, int]:
    """[start, end) of ``len(costs)`` items for ``rank`` of ``world``: contiguous, cut where the running sum of ``costs``
    crosses rank / world of the total, so that every rank gets about the same cost instead of the same count.  With equal
    counts the causal prefill shape is unbalanced -- the early queries see few keys -- and the slowest rank, which sets the
    time, would carry 1 / 0.75 of the average work at 8 ranks."""
    import numpy as np
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    c = np.asarray(costs, dtype=np.float64)
    n = int(c.shape[0])
    if n == 0:
        return 0, 0
    cum = np.cumsum(c)
    total = float(cum[-1])
    # item i belongs to the rank whose share contains the midpoint of the item's cost interval
    mid = cum - 0.5 * c
    bounds = [int(np.searchsorted(mid, total * r / world, side="left")) for r in range(world + 1)]
    bounds[0], bounds[-1] = 0, n
    return bounds[rank], bounds[rank + 1]


MAX_TAIL_SHARES = 4          # into how many shares the queries of a partly filled last round are split at most
SPLIT_EXTRA_TILES = 1        # what a split query costs beside its tiles: fp32 partial results written and combined


def tail_split_plan(costs, start: int, end: int, units_per_round: int):
    """(m, n, time) for the LAST round of a block -- its first m = (end - start) % units_per_round items, the ones a persistent
    kernel reaches last: split into n shares each so that they fill the round (m * n <= units_per_round), if that is faster
    than leaving them whole; (0, 1, time) otherwise.  ``costs`` are tiles + FIXED_TILES_PER_QUERY; only the tiles shrink."""
    import numpy as np
    m = (end - start) % units_per_round
    if m == 0:
        return 0, 1, 0
    worst = int(np.asarray(costs)[start:start + m].max())
    best = (0, 1, worst)
    for n in range(2, MAX_TAIL_SHARES + 1):
        if m * n > units_per_round:
            break
        tiles = max(worst - FIXED_TILES_PER_QUERY, 0)
        t = -(-tiles // n) + FIXED_TILES_PER_QUERY + SPLIT_EXTRA_TILES
        if t < best[2]:
            best = (m, n, t)
    return best


def block_time_in_rounds(costs, start: int, end: int, units_per_round: int, tail_split: bool = False) -> int:
    """Time (in the unit of ``costs``) a persistent kernel needs for items [start, end) when it walks them from the last
    item backwards in rounds of ``units_per_round`` (one item per SM pair and round; every round lasts as long as its most
    expensive item): the sum over rounds of the largest cost in the round.  ``tail_split``: the last, partly filled round
    may be run with its items split into shares (:func:`tail_split_plan`)."""
    import numpy as np
    c = np.asarray(costs)
    t = 0
    full = (end - start) // units_per_round
    for r in range(full):
        hi = end - r * units_per_round
        t += int(c[hi - units_per_round:hi].max())
    m = (end - start) - full * units_per_round
    if m > 0:
        t += tail_split_plan(c, start, end, units_per_round)[2] if tail_split else int(c[start:start + m].max())
    return t


def shard_ranges_by_rounds(costs, world: int, units_per_round: int, tail_split: bool = False):
    """Contiguous [start, end) blocks of ``len(costs)`` items for all ``world`` ranks that minimise the slowest rank's
    :func:`block_time_in_rounds`.  Cutting by the plain sum of costs ignores that a GPU works in rounds of
    ``units_per_round`` items: a block of 5.4 rounds takes as long as one of 6, which at 8 GPUs (about 400 long queries per
    rank on 74 SM pairs) is a tenth of the step.  Found by bisection on the time limit, each rank taking as many items as
    fit (the time of a block is non-decreasing in its end).  ``tail_split``: blocks may end in a round whose queries are split
    into shares (:func:`tail_split_plan`; the caller then launches its block with that plan), which makes half and third
    rounds available to the partition."""
    import numpy as np
    c = np.asarray(costs, dtype=np.int64)
    n = int(c.shape[0])
    if world <= 0:
        raise ValueError(f"bad world {world}")
    if n == 0:
        return [(0, 0)] * world

    def cut(limit: int):
        spans, s = [], 0
        for _ in range(world):
            # largest e with time(s, e) <= limit: grow in whole rounds first, then item by item
            e = s
            while e < n and block_time_in_rounds(c, s, min(n, e + units_per_round), units_per_round, tail_split) <= limit:
                e = min(n, e + units_per_round)
            lo, hi = e, min(n, e + units_per_round)
            while lo < hi:  # binary search inside the last partial round
                mid = (lo + hi + 1) // 2
                if block_time_in_rounds(c, s, mid, units_per_round, tail_split) <= limit:
                    lo = mid
                else:
                    hi = mid - 1
            spans.append((s, lo))
            s = lo
        return spans if s == n else None

    lo_t, hi_t = 1, block_time_in_rounds(c, 0, n, units_per_round, tail_split)
    while lo_t < hi_t:
        mid = (lo_t + hi_t) // 2
        if cut(mid) is not None:
            hi_t = mid
        else:
            lo_t = mid + 1
    return cut(lo_t)


def shard_queries(q, indices, rank: int, world: int, s_kv: int, balance: bool = False, units_per_round: int = 0):
    """Query block of this rank for a BSND prefill call: (q_shard, indices_shard, q_start_index_s).

    The causal position of local query t is ``q_start_index_s + t`` with ``q_start_index_s = (s_kv - S) + start``.
    ``balance``: cut by the cost model of :func:`causal_query_costs` instead of by query count; with ``units_per_round``
    (the GPU's SM pairs: one (query, 128 heads) unit per pair and round) by :func:`shard_ranges_by_rounds`."""
    S = q.shape[1]
    if balance and units_per_round > 0:
        s, e = shard_ranges_by_rounds(causal_query_costs(S, s_kv, indices.shape[-1]), world, units_per_round)[rank]
    elif balance:
        s, e = shard_range_balanced(causal_query_costs(S, s_kv, indices.shape[-1]), rank, world)
    else:
        s, e = shard_range(S, rank, world)
    return q[:, s:e].contiguous(), indices[:, s:e].contiguous(), (s_kv - S) + s


def shard_batch(tensors, rank: int, world: int):
    """Sequence block of this rank for a decode call (first dimension = batch)."""
    s, e = shard_range(tensors[0].shape[0], rank, world)
    return [t[s:e].contiguous() for t in tensors]


def all_reduce_key_gradient(d_kv, group=None):
    """Sum the fp32 key gradient over the ranks of ``group`` in place and return it.

    The backward is the one step of the path with an exchange: dQ shards by query like the forward, but dKV of a key
    sums the contributions of every query that selected it, and those queries live on different ranks.  One all-reduce
    (NCCL for CUDA tensors) of the fp32 buffer after the local kernel -- 9.4 MB at the prefill shape -- completes it.
    Without an initialised process group (single process) the tensor is returned unchanged."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(d_kv, op=dist.ReduceOp.SUM, group=group)
    return d_kv


def sparse_mla_bwd_sharded(q_shard, kv, indices_shard, out_shard, lse_shard, d_out_shard, *, sm_scale: float, q_start_index_s: int,
                           group=None, bwd=None):
    """Backward of one rank's query block: (dQ of the block, dKV summed over all ranks).

    ``q_start_index_s`` is the value returned by :func:`shard_queries` for this rank.  ``bwd`` replaces the device kernel
    (the CPU tests pass the oracle); by default it is :func:`sparse_mla_bwd_raw`."""
    if bwd is None:
        from .sparse_flash_attention import sparse_mla_bwd_raw as bwd
    d_q, d_kv = bwd(q_shard, kv, indices_shard, out_shard, lse_shard, d_out_shard, sm_scale=sm_scale, q_start=q_start_index_s,
                    causal=True)
    return d_q, all_reduce_key_gradient(d_kv, group)
