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
