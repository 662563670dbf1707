"""Lightning indexer behind the reference's entry points.

* ``lightning_indexer(query, key, weights, *, ...)`` -- the production ("li_v2") function-style API of
  examples/deepseek_v4/lightning_indexer.py:1202-1370 (BSND / TND queries, BSND / TND / paged keys).
* ``indexer(B, N2, G, S1, S2, D, TOP_K, ...)`` -- the factory of the simple example,
  examples/lightning_indexer/example_lightning_indexer.py:19-125 (no causal mask).
"""
from __future__ import annotations

import functools
from typing import Optional, Tuple

import torch

from . import _lib
from .adapter import check_inputs, current_stream, dtype_code, ptr, torch_dtype

_INT64_MAX = (1 << 63) - 1


def indexer_scores_raw(query, key, weights, *, sparse_mode: int = 3, q_len_b=None, k_len_b=None, fill_masked: bool = True,
                       return_limits: bool = False):
    """fp32 score matrix [B, S1, S2] of BSND inputs (query [B,S1,N1,D], key [B,S2,1,D], weights [B,S1,N1])."""
    opt = [t for t in (q_len_b, k_len_b) if t is not None]
    dev = check_inputs([query, key, weights] + opt, [None, query.dtype, torch.float32] + [torch.int32] * len(opt),
                       ["query", "key", "weights"] + ["actual lengths"] * len(opt))
    B, S1, N1, D = query.shape
    S2 = key.shape[1]
    if key.shape != (B, S2, 1, D) or weights.shape != (B, S1, N1):
        raise ValueError(f"shape mismatch: query {tuple(query.shape)}, key {tuple(key.shape)}, weights {tuple(weights.shape)}")
    scores = torch.empty((B, S1, S2), dtype=torch.float32, device=dev)
    limits = torch.empty((B, S1), dtype=torch.int32, device=dev) if return_limits else None
    with torch.cuda.device(dev):
        _lib.check(_lib.load().dsa_indexer_scores(ptr(query), ptr(key), ptr(weights), ptr(scores), B, S1, S2, N1, D,
                                                  dtype_code(query.dtype), int(sparse_mode), ptr(q_len_b), ptr(k_len_b),
                                                  ptr(limits), 1 if fill_masked else 0, current_stream(dev)))
    return (scores, limits) if return_limits else scores


# Largest score workspace (B * S1 * S2 fp32) a fused call allocates at once; calls that need more are run over blocks of
# queries (4096 queries against 131072 keys would otherwise materialise 2 GB of scores).
MAX_WORKSPACE_BYTES = 1 << 30


def lightning_indexer_raw(query, key, weights, *, sparse_count: int, sparse_mode: int, q_len_b=None, k_len_b=None,
                          return_value: bool = False, workspace: Optional[torch.Tensor] = None, block_table=None,
                          max_keys: Optional[int] = None, ordered: bool = True, max_workspace_bytes: Optional[int] = None):
    """Fused scores + top-k of BSND inputs: indices int32 [B,S1,1,K] (+ fp32 values).

    A call whose score matrix would exceed ``max_workspace_bytes`` (default MAX_WORKSPACE_BYTES) runs over blocks of
    queries, each with the per-sequence lengths that give its queries the causal limits they have in the whole call
    (dense keys, no caller-owned workspace or lengths, at least as many keys as queries); results are identical.

    ``ordered=False`` leaves the selector's final sort out: the same index SETS, in ascending index order (enough for the
    sparse attention that consumes them, which does not depend on the order of a query's list).

    With ``block_table`` [B, max_blocks] int32, ``key`` is a paged cache [num_blocks, block_size, 1, D] that the kernel
    addresses through the table (no dense copy); ``max_keys`` (default max_blocks * block_size) is the largest logical
    key count, i.e. the width of the score rows."""
    opt = [t for t in (q_len_b, k_len_b, block_table) if t is not None]
    dev = check_inputs([query, key, weights] + opt, [None, query.dtype, torch.float32] + [torch.int32] * len(opt),
                       ["query", "key", "weights"] + ["int32 side input"] * len(opt))
    B, S1, N1, D = query.shape
    if block_table is not None:
        if key.dim() != 4 or key.shape[2] != 1 or key.shape[3] != D or block_table.dim() != 2 or block_table.shape[0] != B:
            raise ValueError(f"paged keys: cache {tuple(key.shape)} / block table {tuple(block_table.shape)} do not fit query {tuple(query.shape)}")
        num_blocks, block_size, max_blocks = key.shape[0], key.shape[1], block_table.shape[1]
        S2 = max_blocks * block_size if max_keys is None else int(max_keys)
        if not 1 <= S2 <= max_blocks * block_size:
            raise ValueError(f"max_keys must be in [1, {max_blocks * block_size}]")
    else:
        S2 = key.shape[1]
        if key.shape != (B, S2, 1, D):
            raise ValueError(f"shape mismatch: query {tuple(query.shape)}, key {tuple(key.shape)}")
    if weights.shape != (B, S1, N1):
        raise ValueError(f"shape mismatch: query {tuple(query.shape)}, weights {tuple(weights.shape)}")
    lib = _lib.load()
    need = lib.dsa_lightning_indexer_workspace_bytes(B, S1, S2)
    limit = MAX_WORKSPACE_BYTES if max_workspace_bytes is None else int(max_workspace_bytes)
    if (need > limit and S1 > 1 and workspace is None and block_table is None and q_len_b is None and k_len_b is None and S2 >= S1):
        rows = max(1, min(S1 - 1, limit // max(1, B * S2 * 4)))
        idx = torch.empty((B, S1, 1, sparse_count), dtype=torch.int32, device=dev)
        val = torch.empty((B, S1, 1, sparse_count), dtype=torch.float32, device=dev) if return_value else None
        for s0 in range(0, S1, rows):
            e0 = min(S1, s0 + rows)
            # queries [s0, e0) of S1 against S2 keys have the limits of e0 - s0 queries against S2 - (S1 - e0) keys
            ql = torch.full((B,), e0 - s0, dtype=torch.int32, device=dev)
            kl = torch.full((B,), S2 - (S1 - e0) if sparse_mode == 3 else S2, dtype=torch.int32, device=dev)
            i_c, v_c = lightning_indexer_raw(query[:, s0:e0].contiguous(), key, weights[:, s0:e0].contiguous(), sparse_count=sparse_count,
                                             sparse_mode=sparse_mode, q_len_b=ql, k_len_b=kl, return_value=return_value, ordered=ordered,
                                             max_workspace_bytes=1 << 62)
            idx[:, s0:e0] = i_c
            if return_value:
                val[:, s0:e0] = v_c
        return idx, val
    if workspace is None:
        workspace = torch.empty((need,), dtype=torch.uint8, device=dev)
    elif workspace.numel() * workspace.element_size() < need or workspace.device != dev:
        raise ValueError(f"workspace must hold {need} bytes on {dev}")
    idx = torch.empty((B, S1, 1, sparse_count), dtype=torch.int32, device=dev)
    val = torch.empty((B, S1, 1, sparse_count), dtype=torch.float32, device=dev) if return_value else None
    with torch.cuda.device(dev):
        if block_table is not None:
            if not ordered:
                raise ValueError("ordered=False is not available with paged keys")
            _lib.check(lib.dsa_lightning_indexer_paged(ptr(query), ptr(key), ptr(weights), B, S1, S2, N1, D, dtype_code(query.dtype),
                                                       int(sparse_mode), ptr(q_len_b), ptr(k_len_b), ptr(block_table), block_size, max_blocks,
                                                       num_blocks, int(sparse_count), ptr(idx), ptr(val), ptr(workspace), need,
                                                       current_stream(dev)))
        else:
            if block_table is None and not ordered:
                entry = lib.dsa_lightning_indexer_unordered
            else:
                entry = lib.dsa_lightning_indexer
            _lib.check(entry(ptr(query), ptr(key), ptr(weights), B, S1, S2, N1, D, dtype_code(query.dtype),
                                                 int(sparse_mode), ptr(q_len_b), ptr(k_len_b), int(sparse_count), ptr(idx), ptr(val),
                                                 ptr(workspace), need, current_stream(dev)))
    return idx, val


def _per_batch(lengths, B: int, default: int, dev) -> torch.Tensor:
    if lengths is None:
        return torch.full((B,), default, dtype=torch.int32, device=dev)
    return torch.as_tensor(lengths).to(device=dev, dtype=torch.int32).contiguous()


def _prefix_to_lengths(prefix) -> list:
    p = [int(x) for x in torch.as_tensor(prefix).tolist()]
    return [p[0]] + [p[i] - p[i - 1] for i in range(1, len(p))]


def _packed_positions(lengths: list, dev):
    """(sequence number, position inside the sequence) of every token of a packed (TND) tensor, on ``dev``."""
    lens = torch.tensor(lengths, dtype=torch.int64, device=dev)
    seq = torch.repeat_interleave(torch.arange(len(lengths), device=dev), lens)
    starts = torch.cumsum(lens, 0) - lens
    return seq, torch.arange(int(lens.sum().item()), device=dev) - starts[seq]


def lightning_indexer(
    query: torch.Tensor,
    key: torch.Tensor,
    weights: torch.Tensor,
    *,
    actual_seq_lengths_query: Optional[torch.Tensor] = None,
    actual_seq_lengths_key: Optional[torch.Tensor] = None,
    block_table: Optional[torch.Tensor] = None,
    layout_query: str = "BSND",
    layout_key: str = "BSND",
    sparse_count: int = 2048,
    sparse_mode: int = 3,
    pre_tokens: int = _INT64_MAX,
    next_tokens: int = _INT64_MAX,
    return_value: bool = False,
    block_n: Optional[int] = None,
    pp_slots: int = 2,
    max_cores: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same arguments, checks and return convention as the reference wrapper
    (examples/deepseek_v4/lightning_indexer.py:1202-1370): returns ``(indices, values)`` where
    ``values`` is an empty tensor unless ``return_value``; TND lengths are prefix sums; ``block_n``,
    ``pp_slots`` and ``max_cores`` are tuning knobs of the reference kernel and are ignored."""
    assert layout_query in ("BSND", "TND"), f"Unsupported query layout: {layout_query}"
    assert layout_key in ("BSND", "PA_BSND", "TND"), f"Unsupported key layout: {layout_key}"
    is_pa, is_tnd, is_tnd_key = layout_key == "PA_BSND", layout_query == "TND", layout_key == "TND"
    if is_pa and return_value:
        raise ValueError("PA_BSND layout does not support return_value")
    if not is_pa and layout_query != layout_key:
        raise ValueError(f"layout_query({layout_query}) must equal layout_key({layout_key}) when key is non-PA_BSND")
    if not (1 <= sparse_count <= 2048 or (sparse_count % 1024 == 0 and sparse_count <= 8192)):
        raise ValueError(f"sparse_count must be in [1,2048] or a multiple of 1024 up to 8192, got {sparse_count}")
    if sparse_mode not in (0, 3):
        raise ValueError(f"sparse_mode must be 0 (defaultMask) or 3 (rightDownCausal), got {sparse_mode}")
    if pre_tokens != _INT64_MAX:
        raise ValueError(f"pre_tokens must be INT64_MAX, got {pre_tokens}")
    if next_tokens != _INT64_MAX:
        raise ValueError(f"next_tokens must be INT64_MAX, got {next_tokens}")
    if query.dtype != key.dtype:
        raise ValueError(f"query dtype {query.dtype} must equal key dtype {key.dtype}")
    if query.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"query/key dtype must be float16 or bfloat16, got {query.dtype}")
    if weights.dtype != torch.float32 and weights.dtype != query.dtype:
        raise ValueError(f"weights dtype {weights.dtype} must be float32 or same as query {query.dtype}")
    dev = query.device
    weights = weights.float()

    # ---- queries: BSND as is, TND padded to BSND on the host side (as the reference does) ----------
    if is_tnd:
        q_lens = _prefix_to_lengths(actual_seq_lengths_query)
        q_tot, N1, D = query.shape
        B, S1 = len(q_lens), max(q_lens) if q_lens else 0
        q_pad = query.new_zeros((B, max(S1, 1), N1, D))
        w_pad = weights.new_zeros((B, max(S1, 1), N1))
        q_seq, q_pos = _packed_positions(q_lens, dev)   # one scatter per tensor, whatever the number of sequences
        q_pad[q_seq, q_pos] = query[:q_seq.numel()]
        w_pad[q_seq, q_pos] = weights[:q_seq.numel()]
        query, weights = q_pad, w_pad
        q_len_b = torch.tensor(q_lens, dtype=torch.int32, device=dev)
    else:
        B, S1, N1, D = query.shape
        q_tot = B * S1
        q_len_b = _per_batch(actual_seq_lengths_query, B, S1, dev)

    # ---- keys: BSND as is; TND padded; a paged cache is passed on with its block table -------------------
    if is_tnd_key:
        k_lens = _prefix_to_lengths(actual_seq_lengths_key)
        S2 = max(k_lens) if k_lens else 0
        k_pad = key.new_zeros((B, max(S2, 1), key.shape[1], key.shape[2]))
        k_seq, k_pos = _packed_positions(k_lens, dev)
        k_pad[k_seq, k_pos] = key[:k_seq.numel()]
        key = k_pad
        k_len_b = torch.tensor(k_lens, dtype=torch.int32, device=dev)
    elif is_pa:
        if block_table is None:
            raise ValueError("block_table required for PA_BSND layout")
        _, bs, n2k, _ = key.shape
        if bs % 16 != 0 or bs > 1024 or bs <= 0:
            raise ValueError(f"PA block_size must be a positive multiple of 16 and <= 1024, got {bs}")
        k_len_b = _per_batch(actual_seq_lengths_key, B, 0, dev)
        S2 = int(k_len_b.max().item()) if B else 0
        # the cache stays where it is: the kernel walks it through the block table
        paged_table = block_table.to(device=dev, dtype=torch.int32).contiguous()
        if S2 > paged_table.shape[1] * bs:
            raise ValueError(f"block_table covers {paged_table.shape[1] * bs} keys, actual_seq_lengths_key asks for {S2}")
    else:
        S2 = key.shape[1]
        k_len_b = _per_batch(actual_seq_lengths_key, B, S2, dev)
    assert D == 128, f"head dim must be 128, got {D}"
    assert key.shape[2] == 1, f"N2 must be 1, got N2={key.shape[2]}"
    assert key.shape[-1] == D, f"key head dim {key.shape[-1]} differs from query head dim {D}"
    if N1 > 64:
        raise ValueError(f"query head_num (N1) must be <= 64, got {N1}")
    assert query.device == key.device == weights.device, "tensors must be on same device"

    empty_vals = torch.empty((0,), dtype=query.dtype, device=dev)
    out_rows = q_tot if is_tnd else B * S1
    if B == 0 or int(q_len_b.max().item()) == 0 or int(k_len_b.max().item()) == 0:  # early exit of the reference
        indices = torch.full((out_rows, 1, sparse_count), -1, dtype=torch.int32, device=dev)
        values = torch.full((out_rows, 1, sparse_count), float("-inf"), dtype=query.dtype, device=dev) if return_value else empty_vals
        return indices, values

    idx, val = lightning_indexer_raw(query.contiguous(), key.contiguous(), weights.contiguous(), sparse_count=sparse_count,
                                     sparse_mode=sparse_mode, q_len_b=q_len_b, k_len_b=k_len_b, return_value=return_value,
                                     block_table=paged_table if is_pa else None, max_keys=max(S2, 1) if is_pa else None)
    if is_tnd:
        idx = idx[q_seq, q_pos]
        if return_value:
            val = val[q_seq, q_pos]
    values = val.to(query.dtype) if return_value else empty_vals
    return idx, values


class SimpleIndexerKernel:
    """``kernel(Query, KEY, WEIGHTS) -> OUT`` of the simple example: Query [B,S1,N2,G*D], KEY [B,S2,N2,D],
    WEIGHTS [B,S1,N2,G] fp32 -> OUT [B,N2,S1,TOP_K] int32 (no causal mask)."""

    def __init__(self, B, N2, G, S1, S2, D, TOP_K, dtype):
        self.B, self.N2, self.G, self.S1, self.S2, self.D, self.TOP_K, self.dtype = B, N2, G, S1, S2, D, TOP_K, dtype

    def __call__(self, Query, KEY, WEIGHTS):
        B, N2, G, S1, S2, D = self.B, self.N2, self.G, self.S1, self.S2, self.D
        check_inputs([Query, KEY, WEIGHTS], [self.dtype, self.dtype, torch.float32], ["Query", "KEY", "WEIGHTS"])
        if tuple(Query.shape) != (B, S1, N2, G * D) or tuple(KEY.shape) != (B, S2, N2, D) or WEIGHTS.numel() != B * S1 * N2 * G:
            raise ValueError("input shapes differ from the factory arguments")
        out = torch.empty((B, N2, S1, self.TOP_K), dtype=torch.int32, device=Query.device)
        q5 = Query.view(B, S1, N2, G, D)
        w4 = WEIGHTS.view(B, S1, N2, G)
        for n2 in range(N2):
            idx, _ = lightning_indexer_raw(q5[:, :, n2].contiguous(), KEY[:, :, n2:n2 + 1].contiguous(), w4[:, :, n2].contiguous(),
                                           sparse_count=self.TOP_K, sparse_mode=0)
            out[:, n2] = idx[:, :, 0]
        return out


@functools.lru_cache(maxsize=None)
def _indexer_cached(B, N2, G, S1, S2, D, TOP_K, input_dtype):
    return SimpleIndexerKernel(B, N2, G, S1, S2, D, TOP_K, torch_dtype(input_dtype))


def indexer(B, N2, G, S1, S2, D, TOP_K, VECTOR_BASEN, VECTOR_BASEG, BLOCK_M, BLOCK_N, BLOCK_K, input_dtype="float16",
            calc_dtype="float"):
    """Factory with the reference's signature; the VECTOR_* / BLOCK_* tile sizes are ignored."""
    if torch_dtype(calc_dtype) != torch.float32:
        raise ValueError("calc_dtype must be float (fp32 accumulation)")
    return _indexer_cached(int(B), int(N2), int(G), int(S1), int(S2), int(D), int(TOP_K), str(input_dtype))
