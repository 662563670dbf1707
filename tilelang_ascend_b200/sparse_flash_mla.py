"""DeepSeek-V4 ``sparse_flash_mla``: sliding window over the original KV cache + selected (or all) compressed KV tokens,
with a per-head attention sink, behind the signature of the reference's front door
(examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_api.py:94-253; golden sparse_flash_mla_golden.py:56-153).

What runs where: one kernel builds the index lists of both key sets (physical row numbers into the paged pools) from the
lengths, block tables and the caller's compressed-token indices; the attention itself is two calls of the sparse forward
kernel (one per key set; the tcgen05 kernel for D = 512) and one call of the sink-combine kernel that merges the two
partial results and the sink.  K and V are the same 512-d rows (MLA latent), one KV head.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from . import _lib
from .adapter import check_inputs, current_stream, dtype_code, ptr
from .sparse_flash_attention import sparse_mla_fwd_raw

DEFAULT_CORE_NUM = 24  # accepted and ignored (a tile-scheduling knob of the reference kernel)


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


_CONCURRENT_MAX_TOKENS = 64     # calls of at most this many query tokens run their two attention parts side by side
_SIDE_STREAMS = {}


def _side_stream(dev):
    key = (dev.type, dev.index)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=dev)
    return _SIDE_STREAMS[key]


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

    lib = _lib.load()
    if layout_q == "TND":
        assert cu_seqlens_q is not None, "cu_seqlens_q is required for TND"
        T, N1, D = q.shape
        B, S = cu_seqlens_q.numel() - 1, 0
        q_flat = q
        ci = cmp_sparse_indices
    else:
        B, S, N1, D = q.shape
        T = B * S
        q_flat = q.reshape(T, N1, D)
        ci = None if cmp_sparse_indices is None else cmp_sparse_indices.reshape(T, cmp_sparse_indices.shape[2], cmp_sparse_indices.shape[3])
    if ori_kv.shape[2] != 1 or ori_kv.shape[3] != D:
        raise ValueError(f"ori_kv must be [blocks, block_size, 1, {D}], got {tuple(ori_kv.shape)}")
    if D % 8 != 0 or D > 512:
        raise ValueError(f"head dim must be a multiple of 8, at most 512 (got {D})")
    K = 0
    if scenario == 3:
        if ci.shape[1] != 1:
            raise ValueError("only one KV head is supported (cmp_sparse_indices.shape[-2] must be 1)")
        K = ci.shape[2]
        if topk_cmp is not None:
            assert K == topk_cmp, "topk_cmp does not match cmp_sparse_indices last dim"
        ci = ci.reshape(T, K).to(device=dev, dtype=torch.int32).contiguous()
    if scenario != 1:
        if cmp_ratio is None or cmp_ratio <= 0:
            raise ValueError("cmp_ratio must be a positive integer when cmp_kv is given")
        check_inputs([cmp_kv], [q.dtype], ["cmp_kv"])
    if scenario == 2:
        # every compressed token below the threshold: the list is as wide as the longest sequence needs (the reference's
        # front door reads seqused_kv on the host for the same purpose, sparse_flash_mla_api.py:176-180)
        # A caller that knows an upper bound of the compressed tokens per sequence passes it as topk_cmp: no host read, and
        # the call can then be captured in a CUDA graph (tokens beyond a sequence's own threshold are masked on the device).
        longest = int(topk_cmp) if topk_cmp is not None else int(seqused_kv.max().item()) // cmp_ratio
        K = max(-(-longest // 64) * 64, 64)

    def i32(t):
        return None if t is None else t.to(device=dev, dtype=torch.int32).contiguous()

    cu, used, ori_bt, cmp_bt = i32(cu_seqlens_q), i32(seqused_kv), i32(ori_block_table), i32(cmp_block_table)
    sinks_dev = sinks.to(device=dev, dtype=torch.float32).contiguous()
    W = ori_win_left + 1
    ori_rows = torch.empty((1, T, 1, W), dtype=torch.int32, device=dev)
    cmp_rows = torch.empty((1, T, 1, K), dtype=torch.int32, device=dev) if scenario != 1 else None
    ori_bs = ori_kv.shape[1]
    cmp_bs = cmp_kv.shape[1] if scenario != 1 else 0
    with torch.cuda.device(dev):
        _lib.check(lib.dsa_v4_build_indices(ptr(cu), ptr(used), ptr(ori_bt), ptr(cmp_bt), ptr(ci) if scenario == 3 else None, ptr(ori_rows),
                                            ptr(cmp_rows), B, T, S, 1 if layout_q == "TND" else 0, ori_bt.shape[1], ori_bs, int(ori_win_left),
                                            cmp_bt.shape[1] if scenario != 1 else 0, cmp_bs, int(cmp_ratio or 0), scenario, K,
                                            current_stream(dev)))
    q4 = q_flat.reshape(1, T, N1, D)
    pool = ori_kv.reshape(1, ori_kv.shape[0] * ori_bs, 1, D)
    out_b = lse_b = None
    side = None
    if scenario != 1:
        cpool = cmp_kv.reshape(1, cmp_kv.shape[0] * cmp_bs, 1, D)
        if T <= _CONCURRENT_MAX_TOKENS:
            # a decode-sized call: each of the two attention launches occupies a few SM pairs only, so the compressed-token
            # part runs beside the window part on a second stream (forked from and joined to the caller's stream; inside a
            # CUDA graph capture this becomes two parallel branches)
            cur = torch.cuda.current_stream(dev)
            side = _side_stream(dev)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                out_b, lse_b = sparse_mla_fwd_raw(q4, cpool, cmp_rows, sm_scale=softmax_scale, q_start=0, causal=False, dv=D)
    out_a, lse_a = sparse_mla_fwd_raw(q4, pool, ori_rows, sm_scale=softmax_scale, q_start=0, causal=False, dv=D)
    if scenario != 1:
        if side is not None:
            torch.cuda.current_stream(dev).wait_stream(side)
        else:
            out_b, lse_b = sparse_mla_fwd_raw(q4, cpool, cmp_rows, sm_scale=softmax_scale, q_start=0, causal=False, dv=D)
        out_b, lse_b = out_b.reshape(T, N1, D), lse_b.reshape(T, N1)

    out, lse = sink_combine_raw(out_a.reshape(T, N1, D), lse_a.reshape(T, N1), out_b, lse_b, sinks_dev, N1)
    if layout_q == "BSND":
        if cu is not None:  # padded tokens of short sequences: the reference leaves them at zero
            exists = (torch.arange(S, device=dev)[None, :] < (cu[1:] - cu[:-1])[:, None]).reshape(T)
            out = out * exists[:, None, None].to(out.dtype)
            lse = lse * exists[:, None].to(lse.dtype)
        out, lse = out.reshape(B, S, N1, D), lse.reshape(B, S, N1)
    return (out, lse) if return_softmax_lse else out
