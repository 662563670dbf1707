"""DeepSeek-V4 ``sparse_flash_mla``: sliding window over the original KV cache + selected (or all) compressed KV tokens,
with a per-head attention sink, behind the signature of the reference's front door
(examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_api.py:94-253; golden sparse_flash_mla_golden.py:56-153).

What runs where: the index lists of both key sets are built on the device from the lengths, block tables and the
caller's compressed-token indices (integer tensor ops, a few KB per token); the attention itself is two calls of the
sparse forward kernel (one per key set, physical row numbers into the paged pools) and one call of the sink-combine
kernel that merges the two partial results and the sink.  K and V are the same 512-d rows (MLA latent), one KV head.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from . import _lib
from .adapter import check_inputs, current_stream, dtype_code, ptr
from .sparse_flash_attention import sparse_mla_fwd_raw

DEFAULT_CORE_NUM = 24  # accepted and ignored (a tile-scheduling knob of the reference kernel)


def _physical_rows(block_table: torch.Tensor, bid: torch.Tensor, pos: torch.Tensor, valid: torch.Tensor, block_size: int) -> torch.Tensor:
    """Row numbers inside a paged pool [blocks * block_size] of logical positions ``pos`` [T, n] of sequences ``bid`` [T];
    -1 where ``valid`` is False."""
    safe = torch.where(valid, pos, torch.zeros_like(pos))
    blk = torch.gather(block_table[bid.long()], 1, (safe // block_size).clamp_(max=block_table.shape[1] - 1).long())
    rows = blk.long() * block_size + safe % block_size
    return torch.where(valid, rows, torch.full_like(rows, -1)).to(torch.int32)


def sink_combine_raw(out_a, lse_a, out_b, lse_b, sinks, H: int):
    """``dsa_sink_combine`` on [T, H, DV] partial outputs and [T, H] log-sum-exps; returns (out, lse)."""
    dev = out_a.device
    out = torch.empty_like(out_a)
    lse = torch.empty_like(lse_a)
    rows, DV = out_a.shape[0] * out_a.shape[1], out_a.shape[-1]
    with torch.cuda.device(dev):
        _lib.check(_lib.load().dsa_sink_combine(ptr(out_a), ptr(lse_a), ptr(out_b), ptr(lse_b), ptr(sinks), ptr(out), ptr(lse), rows, H, DV,
                                                dtype_code(out_a.dtype), current_stream(dev)))
    return out, lse


def sparse_flash_mla(
    q: torch.Tensor,
    *,
    ori_kv: torch.Tensor,
    cmp_kv: Optional[torch.Tensor] = None,
    cmp_sparse_indices: Optional[torch.Tensor] = None,
    ori_block_table: torch.Tensor,
    cmp_block_table: Optional[torch.Tensor] = None,
    cu_seqlens_q: Optional[torch.Tensor] = None,
    seqused_q: Optional[torch.Tensor] = None,
    seqused_kv: torch.Tensor,
    sinks: torch.Tensor,
    softmax_scale: float,
    cmp_ratio: Optional[int] = None,
    ori_mask_mode: int = 4,
    cmp_mask_mode: int = 3,
    ori_win_left: int = 127,
    ori_win_right: int = 0,
    layout_q: str = "TND",
    layout_kv: str = "PA_ND",
    return_softmax_lse: bool = False,
    core_num: int = DEFAULT_CORE_NUM,
    topk_cmp: Optional[int] = None,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Same arguments, checks and return convention as the reference's ``sparse_flash_mla``.

    q: [T, N1, D] ("TND", with ``cu_seqlens_q`` [B + 1]) or [B, S, N1, D] ("BSND"); ori_kv / cmp_kv: paged pools
    [blocks, block_size, 1, D] with block tables [B, n]; cmp_sparse_indices: [T, 1, K] / [B, S, 1, K] int32 token numbers
    into the compressed cache (-1 ends a list) or None (= every compressed token below the causal threshold);
    seqused_kv [B]; sinks [N1] fp32.  Token s of sequence b sits at position p = seqused_kv[b] - len_q[b] + s and attends to
    original tokens [max(p - ori_win_left, 0), p] and to compressed tokens below floor((p + 1) / cmp_ratio)."""
    del seqused_q, core_num
    assert ori_mask_mode == 4, "only ori_mask_mode=4 supported"
    assert cmp_mask_mode == 3 or cmp_kv is None, "only cmp_mask_mode=3 supported"
    assert ori_win_right == 0, "only ori_win_right=0 supported"
    assert layout_kv == "PA_ND", "only layout_kv=PA_ND supported"
    assert layout_q in ("TND", "BSND"), f"unsupported layout_q={layout_q!r}"
    dev = check_inputs([q, ori_kv], [None, q.dtype], ["q", "ori_kv"])
    scenario = 1 if cmp_kv is None else (2 if cmp_sparse_indices is None else 3)

    if layout_q == "TND":
        assert cu_seqlens_q is not None, "cu_seqlens_q is required for TND"
        T, N1, D = q.shape
        cu = cu_seqlens_q.to(device=dev, dtype=torch.int64)
        B = cu.numel() - 1
        len_q = cu[1:] - cu[:-1]
        tok = torch.arange(T, device=dev)
        bid = torch.searchsorted(cu[1:].contiguous(), tok, right=True).clamp_(max=B - 1)
        s_local = tok - cu[bid]
        exists = torch.ones(T, dtype=torch.bool, device=dev)
        q_flat = q
        ci = cmp_sparse_indices
    else:
        B, S, N1, D = q.shape
        T = B * S
        len_q = torch.full((B,), S, dtype=torch.int64, device=dev)
        if cu_seqlens_q is not None:
            cu = cu_seqlens_q.to(device=dev, dtype=torch.int64)
            len_q = cu[1:] - cu[:-1]
        tok = torch.arange(T, device=dev)
        bid, s_local = tok // S, tok % S
        exists = s_local < len_q[bid]
        q_flat = q.reshape(T, N1, D)
        ci = None if cmp_sparse_indices is None else cmp_sparse_indices.reshape(T, cmp_sparse_indices.shape[2], cmp_sparse_indices.shape[3])
    if ori_kv.shape[2] != 1 or ori_kv.shape[3] != D:
        raise ValueError(f"ori_kv must be [blocks, block_size, 1, {D}], got {tuple(ori_kv.shape)}")
    if D % 8 != 0 or D > 512:
        raise ValueError(f"head dim must be a multiple of 8, at most 512 (got {D})")
    if scenario == 3:
        if ci.shape[1] != 1:
            raise ValueError("only one KV head is supported (cmp_sparse_indices.shape[-2] must be 1)")
        if topk_cmp is not None:
            assert ci.shape[2] == topk_cmp, "topk_cmp does not match cmp_sparse_indices last dim"
    if scenario != 1 and (cmp_ratio is None or cmp_ratio <= 0):
        raise ValueError("cmp_ratio must be a positive integer when cmp_kv is given")

    act_kv = seqused_kv.to(device=dev, dtype=torch.int64)
    pos = act_kv[bid] - len_q[bid] + s_local                      # absolute position of every token
    sinks_dev = sinks.to(device=dev, dtype=torch.float32).contiguous()

    # ---- key set 1: the sliding window of the original cache ------------------------------------------------------
    W = ori_win_left + 1
    w = pos[:, None] - ori_win_left + torch.arange(W, device=dev)[None, :]
    w_valid = (w >= 0) & exists[:, None] & (pos[:, None] >= 0)
    ori_bs = ori_kv.shape[1]
    ori_rows = _physical_rows(ori_block_table.to(device=dev, dtype=torch.int64), bid, w, w_valid, ori_bs)
    q4 = q_flat.reshape(1, T, N1, D)
    pool = ori_kv.reshape(1, ori_kv.shape[0] * ori_bs, 1, D)
    out_a, lse_a = sparse_mla_fwd_raw(q4, pool, ori_rows.reshape(1, T, 1, W).contiguous(), sm_scale=softmax_scale, q_start=0, causal=False, dv=D)

    # ---- key set 2: compressed tokens ------------------------------------------------------------------------------
    out_b = lse_b = None
    if scenario != 1:
        check_inputs([cmp_kv], [q.dtype], ["cmp_kv"])
        threshold = torch.div(pos + 1, cmp_ratio, rounding_mode="floor").clamp_(min=0)
        cmp_len = torch.div(act_kv[bid], cmp_ratio, rounding_mode="floor")
        if scenario == 3:
            ci = ci[:, 0, :].to(device=dev, dtype=torch.int64)
            K = ci.shape[1]
            slot = torch.arange(K, device=dev)[None, :]
            ended = torch.cumsum((ci == -1).to(torch.int32), dim=1) > 0          # a -1 ends the list
            c_valid = (slot < threshold[:, None]) & ~ended & (ci >= 0) & (ci < torch.minimum(threshold, cmp_len)[:, None])
            c_pos = ci
        else:
            K = max(int(threshold.max().item()) if T > 0 else 0, 1)
            c_pos = torch.arange(K, device=dev)[None, :].expand(T, K)
            c_valid = c_pos < threshold[:, None]
        c_valid = c_valid & exists[:, None]
        cmp_bs = cmp_kv.shape[1]
        cmp_rows = _physical_rows(cmp_block_table.to(device=dev, dtype=torch.int64), bid, c_pos, c_valid, cmp_bs)
        cpool = cmp_kv.reshape(1, cmp_kv.shape[0] * cmp_bs, 1, D)
        out_b, lse_b = sparse_mla_fwd_raw(q4, cpool, cmp_rows.reshape(1, T, 1, K).contiguous(), sm_scale=softmax_scale, q_start=0, causal=False, dv=D)
        out_b, lse_b = out_b.reshape(T, N1, D), lse_b.reshape(T, N1)

    out, lse = sink_combine_raw(out_a.reshape(T, N1, D), lse_a.reshape(T, N1), out_b, lse_b, sinks_dev, N1)
    if layout_q == "BSND":
        if not bool(exists.all()):  # padded tokens of short sequences: the reference leaves them at zero
            out = out * exists[:, None, None].to(out.dtype)
            lse = lse * exists[:, None].to(lse.dtype)
        out, lse = out.reshape(B, S, N1, D), lse.reshape(B, S, N1)
    return (out, lse) if return_softmax_lse else out
