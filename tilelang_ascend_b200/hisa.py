"""HISA block-sparse indexer logits behind the factory signature of the reference
(examples/HISA/block_sparse_mqa_attn_expert_test.py:24-45): the step before the token-level top-k at very long context --
the lightning-indexer score of every key of a query's selected KV blocks."""
from __future__ import annotations

import torch

from . import _lib
from .adapter import check_inputs, current_stream, dtype_code, ptr

_W_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def block_sparse_logits_raw(q, k, topk_block_indices, weights, cu_seqlen_ks, cu_seqlen_ke, kv_block_size: int, impl: int = _lib.IMPL_AUTO,
                            block_table=None, tokens_per_seq: int = 0):
    """One launch through the C ABI.  q [S,H,D], k [S_kv,D], topk_block_indices [S,topk] int32, weights [S,H] (q's dtype or
    fp32), cu_seqlen_ks / cu_seqlen_ke [S] int32 -> logits [S, topk, kv_block_size] fp32.  impl: _lib.IMPL_AUTO (tcgen05 kernel
    for blocks of 128 keys, index_dim 128, at most 64 heads), IMPL_GENERIC (CUDA cores) or IMPL_TENSOR_CORE.
    Paged keys: block_table [B, max_blocks] int32, k = the cache viewed as [num_phys_blocks * kv_block_size, D], the indices
    name logical blocks of sequence s // tokens_per_seq."""
    dev = check_inputs([q, k, topk_block_indices, weights, cu_seqlen_ks, cu_seqlen_ke], [None, q.dtype, torch.int32, None, torch.int32, torch.int32],
                       ["q", "k", "topk_block_indices", "weights", "cu_seqlen_ks", "cu_seqlen_ke"])
    if block_table is not None:
        check_inputs([q, block_table], [None, torch.int32], ["q", "block_table"])
        if block_table.dim() != 2 or tokens_per_seq <= 0 or q.shape[0] != block_table.shape[0] * tokens_per_seq:
            raise ValueError("block_table must be [B, max_blocks] with B * tokens_per_seq queries")
    if q.dim() != 3 or k.dim() != 2 or k.shape[1] != q.shape[2]:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}")
    S, H, D = q.shape
    if topk_block_indices.shape[0] != S or tuple(weights.shape) != (S, H) or cu_seqlen_ks.shape != (S,) or cu_seqlen_ke.shape != (S,):
        raise ValueError("topk_block_indices / weights / cu_seqlen_ks / cu_seqlen_ke do not match q")
    if weights.dtype not in _W_DTYPES:
        raise ValueError(f"weights must be bfloat16, float16 or float32, got {weights.dtype}")
    topk = topk_block_indices.shape[1]
    logits = torch.empty((S, topk, kv_block_size), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().dsa_block_sparse_logits(ptr(q), ptr(k), ptr(topk_block_indices), ptr(weights), ptr(cu_seqlen_ks), ptr(cu_seqlen_ke),
                                                       ptr(logits), S, k.shape[0], H, D, int(kv_block_size), topk, dtype_code(q.dtype),
                                                       _W_DTYPES[weights.dtype], int(impl), ptr(block_table),
                                                       0 if block_table is None else block_table.shape[1], int(tokens_per_seq), current_stream(dev)))
    return logits


class BlockSparseLogitsKernel:
    """Callable returned by :func:`block_sparse_mqa_attn_return_logits`:
    ``kernel(q, k, topk_block_indices, weights, cu_seqlen_ks, cu_seqlen_ke) -> logits``; only inputs are passed, the output
    is allocated on the device of ``q`` and the launch goes to the current stream without synchronising."""

    def __init__(self, seq_len, seq_len_kv, kv_block_size, topk, heads, index_dim):
        self.shape = (seq_len, seq_len_kv, kv_block_size, topk, heads, index_dim)

    def __call__(self, q, k, topk_block_indices, weights, cu_seqlen_ks, cu_seqlen_ke):
        seq_len, seq_len_kv, kv_block_size, topk, heads, index_dim = self.shape
        if tuple(q.shape) != (seq_len, heads, index_dim) or tuple(k.shape) != (seq_len_kv, index_dim) or \
                tuple(topk_block_indices.shape) != (seq_len, topk):
            raise ValueError("tensor shapes differ from the factory's static parameters")
        return block_sparse_logits_raw(q, k, topk_block_indices, weights, cu_seqlen_ks, cu_seqlen_ke, kv_block_size)


def block_sparse_mqa_attn_return_logits(seq_len: int, seq_len_kv: int, kv_block_size: int, topk: int, heads: int, index_dim: int,
                                        block_N: int = 8, num_stages: int = 2, threads: int = 2, grid_size: int = 24):
    """Factory with the reference's signature; ``block_N``, ``num_stages``, ``threads`` and ``grid_size`` (tile / core-count
    knobs of the Ascend kernel) are accepted and ignored, its argument checks are kept (:54-55)."""
    assert kv_block_size % block_N == 0, "block_N must divide kv_block_size"
    assert topk % 4 == 0, "topk must be divisible by 4 for 4x unrolled loop"
    return BlockSparseLogitsKernel(seq_len, seq_len_kv, kv_block_size, topk, heads, index_dim)


class PagedBlockSparseLogitsKernel:
    """Callable returned by :func:`paged_block_sparse_mqa_attn_return_logits`:
    ``kernel(q, kv_cache, topk_block_indices, weights, context_lens, block_tables) -> logits [B * S, topk, kv_block_size]``."""

    def __init__(self, batch, seq_len, num_phys_blocks, kv_block_size, topk, heads, index_dim, max_blocks):
        self.shape = (batch, seq_len, num_phys_blocks, kv_block_size, topk, heads, index_dim, max_blocks)

    def __call__(self, q, kv_cache, topk_block_indices, weights, context_lens, block_tables):
        batch, seq_len, num_phys_blocks, kv_block_size, topk, heads, index_dim, max_blocks = self.shape
        T = batch * seq_len
        if tuple(q.shape) != (T, heads, index_dim) or tuple(kv_cache.shape) != (num_phys_blocks, kv_block_size, 1, index_dim) or \
                tuple(topk_block_indices.shape) != (T, topk) or tuple(block_tables.shape) != (batch, max_blocks) or \
                tuple(context_lens.shape) != (batch,):
            raise ValueError("tensor shapes differ from the factory's static parameters")
        # per-token key range [0, context length of the token's sequence)
        ke = context_lens.to(torch.int32).repeat_interleave(seq_len).contiguous()
        ks = torch.zeros_like(ke)
        return block_sparse_logits_raw(q, kv_cache.view(num_phys_blocks * kv_block_size, index_dim), topk_block_indices, weights, ks, ke,
                                       kv_block_size, block_table=block_tables, tokens_per_seq=seq_len)


def paged_block_sparse_mqa_attn_return_logits(batch: int, seq_len: int, num_phys_blocks: int, kv_block_size: int, topk: int, heads: int,
                                              index_dim: int, max_blocks: int, num_stages: int = 2, threads: int = 2):
    """Factory with the signature of the reference's paged variant
    (examples/HISA/paged_block_sparse_mqa_attn_expert.py:54-66); ``num_stages`` and ``threads`` are accepted and ignored."""
    assert topk % 4 == 0, "topk must be divisible by 4"
    return PagedBlockSparseLogitsKernel(batch, seq_len, num_phys_blocks, kv_block_size, topk, heads, index_dim, max_blocks)
