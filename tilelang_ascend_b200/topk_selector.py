"""Stand-alone top-k selector behind the reference's factory signature
(examples/topk_selector/example_topk_selector.py:10-54)."""
from __future__ import annotations

import functools
from typing import Optional

import torch

from . import _lib
from .adapter import current_stream, ptr, torch_dtype


def topk_select_raw(scores: torch.Tensor, top_k: int, limits: Optional[torch.Tensor] = None, return_values: bool = False,
                    ordered: bool = True):
    """scores fp32 [rows, n] (row stride may exceed n) -> int32 [rows, top_k] (+ fp32 values).

    Descending score, equal scores by ascending index; -1 / -inf in unused slots.  ``ordered=False``: the same set of
    indices per row (same tie rule at the threshold) in ascending index order, without the final sort."""
    if scores.dim() != 2 or scores.stride(1) != 1:
        raise ValueError("scores must be 2-dimensional with unit inner stride")
    dev = _check(scores, limits)
    rows, n = scores.shape
    idx = torch.empty((rows, top_k), dtype=torch.int32, device=dev)
    val = torch.empty((rows, top_k), dtype=torch.float32, device=dev) if return_values else None
    with torch.cuda.device(dev):
        entry = _lib.load().dsa_topk_select if ordered else _lib.load().dsa_topk_select_unordered
        _lib.check(entry(ptr(scores), rows, n, scores.stride(0), ptr(limits), int(top_k), ptr(idx),
                         ptr(val), current_stream(dev)))
    return (idx, val) if return_values else idx


def _check(scores, limits):
    if scores.dtype != torch.float32:
        raise ValueError(f"Input tensor scores has dtype {scores.dtype}, expected torch.float32")
    if scores.device.type != "cuda":
        raise ValueError(f"kernels run on CUDA tensors only (got device {scores.device}); there is no CPU path")
    if limits is not None:
        if limits.dtype != torch.int32:
            raise ValueError(f"Input tensor limits has dtype {limits.dtype}, expected torch.int32")
        if limits.device != scores.device:
            raise ValueError(f"Input tensor limits is on {limits.device}, expected {scores.device}")
        if limits.numel() != scores.shape[0]:
            raise ValueError("limits must hold one entry per row")
    return scores.device


class TopkSelectorKernel:
    """``kernel(x) -> indices`` with x fp32 [B, N] and indices int32 [B, top_k]."""

    def __init__(self, B, N, top_k):
        self.B, self.N, self.top_k = B, N, top_k

    def __call__(self, x):
        if tuple(x.shape) != (self.B, self.N):
            raise ValueError(f"x must be [{self.B}, {self.N}], got {tuple(x.shape)}")
        if not x.is_contiguous():
            raise ValueError("Input tensor x must be contiguous")
        return topk_select_raw(x, self.top_k)


@functools.lru_cache(maxsize=None)
def _cached(B, N, top_k, block_N, dtype):
    if torch_dtype(dtype) != torch.float32:
        raise ValueError("simple_topk_selector supports float32 scores")
    if not 0 < top_k <= N:
        raise ValueError("top_k must be in [1, N]")
    return TopkSelectorKernel(B, N, top_k)


def simple_topk_selector(B: int, N: int, top_k: int, block_N: int, dtype="float32"):
    """Factory with the reference's signature; ``block_N`` is a tiling hint and is ignored."""
    return _cached(int(B), int(N), int(top_k), int(block_N), str(dtype))
