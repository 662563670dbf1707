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


def shard_queries(q, indices, rank: int, world: int, s_kv: int):
    """Query block of this rank for a BSND prefill call: (q_shard, indices_shard, q_start_index_s).

    The causal position of local query t is ``q_start_index_s + t`` with
    ``q_start_index_s = (s_kv - S) + start``."""
    S = q.shape[1]
    s, e = shard_range(S, rank, world)
    return q[:, s:e].contiguous(), indices[:, s:e].contiguous(), (s_kv - S) + s


def shard_batch(tensors, rank: int, world: int):
    """Sequence block of this rank for a decode call (first dimension = batch)."""
    s, e = shard_range(tensors[0].shape[0], rank, world)
    return [t[s:e].contiguous() for t in tensors]
