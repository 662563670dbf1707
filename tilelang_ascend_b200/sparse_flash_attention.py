"""Sparse MLA forward / backward behind the reference's entry signatures.

``sparse_attention_fwd(...)`` keeps the factory signature of
examples/sparse_flash_attention/example_sparse_flash_attn.py:18-28 and returns a kernel called as
``kernel(q, kv, indices)``; ``sparse_attn_tilelang(...)`` keeps the paged / decode wrapper signature of
examples/sparse_flash_attention/bench_sfa/sparse_flash_attn_pa_no_cv_pipeline.py:384-400.  The LSE
output follows the reference's own keyword ``return_softmax_lse``
(examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_api.py:114,251-253).
"""
from __future__ import annotations

import functools
import os
from typing import Optional

import torch

from . import _lib
from .adapter import check_inputs, current_stream, dtype_code, ptr, torch_dtype


def _check_distinct_indices(indices: torch.Tensor, S_kv: int) -> None:
    """Debug check (DSA_DEBUG_BOUNDS=1; synchronises): every query's list must name each key at most once.  The kernels
    count a repeated index once per occurrence, the reference's torch golden counts it once
    (example_sparse_flash_attn.py:277-280 builds a mask): results differ silently unless the lists are distinct."""
    srt, _ = torch.sort(indices.reshape(-1, indices.shape[-1]), dim=1)
    dup = (srt[:, 1:] == srt[:, :-1]) & (srt[:, 1:] >= 0) & (srt[:, 1:] < S_kv)
    if bool(dup.any()):
        row = int(torch.nonzero(dup.any(dim=1))[0])
        raise ValueError(f"indices of query row {row} name a key more than once; the kernels would count it once per occurrence")


# fp32 scratch of split-KV calls, kept per (device, stream) and grown on demand: a decode step runs every few tens of
# microseconds and an allocation per call costs about as much as the kernel's host side.  Calls on one stream are ordered,
# so they can share a buffer; calls on different streams get different buffers.
_SPLIT_WORKSPACES = {}


def _split_workspace(dev, nbytes: int) -> torch.Tensor:
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    buf = _SPLIT_WORKSPACES.get(key)
    if buf is None or buf.numel() * 4 < nbytes:
        buf = torch.empty(((nbytes + 3) // 4,), dtype=torch.float32, device=dev)
        _SPLIT_WORKSPACES[key] = buf
    return buf


def _next_pow2(x: int) -> int:
    return 1 << (max(int(x), 1) - 1).bit_length()


def sparse_mla_fwd_raw(q, kv, indices, *, sm_scale: float, q_start: int, causal: bool, dv: int, out=None,
                       return_lse: bool = True, q_start_b=None, kv_len_b=None, q_len_b=None, block_table=None,
                       block_size: int = 0, impl: int = _lib.IMPL_AUTO, nsplit=None, kv_rope=None, split_queries: int = 0):
    """One launch of the forward through the C ABI.  q [B,S,H,D], kv [B,S_kv,1,D] (or paged blocks),
    indices [B,S,1,topk] int32.  Returns (out, lse-or-None).

    nsplit: None = let the library decide whether the keys of every query are split over several work units (it does for
    D=576 / dv=512 calls with fewer queries than SM pairs, e.g. decode of a few sequences); 1 = never; n > 1 = n shares.
    The fp32 workspace of a split call is owned here (one per device and stream, reused between calls), as the reference's
    adapter owns its kernels' workspaces (tilelang/jit/adapter/cython/cython_wrapper.pyx:98-137).

    ``split_queries`` = m with ``nsplit`` = n > 1: only the first m of the B * S queries (memory order) are split; a persistent
    kernel reaches them last, and their shares fill its last round of work units when the other queries leave it partly
    empty (one GPU's block of a sharded prefill).  Their results are combined from fp32 partial results; all other rows are
    bit-equal to an unsplit call.

    ``kv_rope``: key rows in two parts -- ``kv`` then holds the dv latent values of every row ([B,S_kv,1,dv] or paged blocks)
    and ``kv_rope`` the D - dv rope values with the same leading shape (the KV / K_pe tensors of the dense MLA decode
    kernels, used in place); D = 576, dv = 512, topk <= 8192 only."""
    if kv_rope is not None:
        return _fwd_two_part(q, kv, kv_rope, indices, sm_scale=sm_scale, q_start=q_start, causal=causal, dv=dv, return_lse=return_lse,
                             q_start_b=q_start_b, kv_len_b=kv_len_b, q_len_b=q_len_b, block_table=block_table, block_size=block_size,
                             nsplit=nsplit)
    opt = [t for t in (q_start_b, kv_len_b, q_len_b, block_table) if t is not None]
    dev = check_inputs([q, kv, indices] + opt, [None, q.dtype, torch.int32] + [torch.int32] * len(opt),
                       ["q", "kv", "indices"] + ["int32 side input"] * len(opt))
    code = dtype_code(q.dtype)
    if q.dim() != 4 or kv.dim() != 4 or indices.dim() != 4:
        raise ValueError("q, kv and indices must be 4-dimensional ([B,S,H,D], [B,S_kv,1,D], [B,S,1,topk])")
    B, S, H, D = q.shape
    if kv.shape[2] != 1 or kv.shape[3] != D or indices.shape[:3] != (B, S, 1):
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, kv {tuple(kv.shape)}, indices {tuple(indices.shape)}")
    if block_table is None:
        if kv.shape[0] != B:
            raise ValueError("kv batch size differs from q")
        S_kv, max_blocks = kv.shape[1], 0
    else:
        block_size = int(block_size) if block_size else kv.shape[1]
        max_blocks = block_table.shape[1]
        S_kv = max_blocks * block_size
    topk = indices.shape[3]
    if os.environ.get("DSA_DEBUG_BOUNDS") == "1":
        _check_distinct_indices(indices, S_kv)
    if out is None:
        out = torch.empty((B, S, H, dv), dtype=q.dtype, device=dev)
    lse = torch.empty((B, S, H), dtype=torch.float32, device=dev) if return_lse else None
    lib = _lib.load()
    with torch.cuda.device(dev):
        tc_shape = D in (576, 512) and dv == 512 and topk <= 8192 and impl != _lib.IMPL_GENERIC
        if nsplit is None:
            nsplit = int(lib.dsa_sparse_mla_fwd_splitkv_nsplit(B, S, H, topk)) if tc_shape else 1
        nsplit = int(nsplit)
        if nsplit > 1 and 0 < int(split_queries) < B * S:
            if not tc_shape:
                raise ValueError("a split tail needs D = 576 or 512, dv = 512, topk <= 8192 and the tensor-core kernel")
            nbytes = int(lib.dsa_sparse_mla_fwd_splitkv_workspace_bytes(1, int(split_queries), H, dv, nsplit))
            workspace = _split_workspace(dev, nbytes)
            _lib.check(lib.dsa_sparse_mla_fwd_split_tail(
                ptr(q), ptr(kv), ptr(indices), ptr(out), ptr(lse), B, S, S_kv, H, D, dv, topk, float(sm_scale), int(q_start),
                1 if causal else 0, code, ptr(q_start_b), ptr(kv_len_b), ptr(q_len_b), ptr(block_table), int(block_size),
                int(max_blocks), int(split_queries), nsplit, ptr(workspace), nbytes, current_stream(dev)))
        elif nsplit > 1:
            if not tc_shape:
                raise ValueError("nsplit > 1 needs D = 576, dv = 512, topk <= 8192 and the tensor-core kernel")
            nbytes = int(lib.dsa_sparse_mla_fwd_splitkv_workspace_bytes(B, S, H, dv, nsplit))
            workspace = _split_workspace(dev, nbytes)
            _lib.check(lib.dsa_sparse_mla_fwd_splitkv(
                ptr(q), ptr(kv), ptr(indices), ptr(out), ptr(lse), B, S, S_kv, H, D, dv, topk, float(sm_scale), int(q_start),
                1 if causal else 0, code, ptr(q_start_b), ptr(kv_len_b), ptr(q_len_b), ptr(block_table), int(block_size),
                int(max_blocks), nsplit, ptr(workspace), nbytes, current_stream(dev)))
        else:
            _lib.check(lib.dsa_sparse_mla_fwd(
                ptr(q), ptr(kv), ptr(indices), ptr(out), ptr(lse), B, S, S_kv, H, D, dv, topk, float(sm_scale), int(q_start),
                1 if causal else 0, code, ptr(q_start_b), ptr(kv_len_b), ptr(q_len_b), ptr(block_table), int(block_size),
                int(max_blocks), int(impl), current_stream(dev)))
    return out, lse


def _fwd_two_part(q, kv, kv_rope, indices, *, sm_scale, q_start, causal, dv, return_lse, q_start_b, kv_len_b, q_len_b, block_table,
                  block_size, nsplit):
    opt = [t for t in (q_start_b, kv_len_b, q_len_b, block_table) if t is not None]
    dev = check_inputs([q, kv, kv_rope, indices] + opt, [None, q.dtype, q.dtype, torch.int32] + [torch.int32] * len(opt),
                       ["q", "kv", "kv_rope", "indices"] + ["int32 side input"] * len(opt))
    code = dtype_code(q.dtype)
    B, S, H, D = q.shape
    if D != 576 or dv != 512 or kv.dim() != 4 or kv_rope.dim() != 4 or kv.shape[2:] != (1, dv) or kv_rope.shape[2:] != (1, D - dv) \
            or kv.shape[:2] != kv_rope.shape[:2] or indices.shape[:3] != (B, S, 1):
        raise ValueError(f"key rows in two parts need D = 576, dv = 512, kv [...,1,512] and kv_rope [...,1,64] of equal leading shape "
                         f"(got q {tuple(q.shape)}, kv {tuple(kv.shape)}, kv_rope {tuple(kv_rope.shape)})")
    if block_table is None:
        if kv.shape[0] != B:
            raise ValueError("kv batch size differs from q")
        S_kv, max_blocks = kv.shape[1], 0
    else:
        block_size = int(block_size) if block_size else kv.shape[1]
        max_blocks = block_table.shape[1]
        S_kv = max_blocks * block_size
    topk = indices.shape[3]
    if topk > 8192:
        raise ValueError("key rows in two parts need topk <= 8192")
    out = torch.empty((B, S, H, dv), dtype=q.dtype, device=dev)
    lse = torch.empty((B, S, H), dtype=torch.float32, device=dev) if return_lse else None
    lib = _lib.load()
    with torch.cuda.device(dev):
        nsplit = int(lib.dsa_sparse_mla_fwd_splitkv_nsplit(B, S, H, topk)) if nsplit is None else int(nsplit)
        nbytes = int(lib.dsa_sparse_mla_fwd_splitkv_workspace_bytes(B, S, H, dv, nsplit)) if nsplit > 1 else 0
        workspace = _split_workspace(dev, nbytes) if nsplit > 1 else None
        _lib.check(lib.dsa_sparse_mla_fwd_two_part(
            ptr(q), ptr(kv), ptr(kv_rope), ptr(indices), ptr(out), ptr(lse), B, S, S_kv, H, D, dv, topk, float(sm_scale), int(q_start),
            1 if causal else 0, code, ptr(q_start_b), ptr(kv_len_b), ptr(q_len_b), ptr(block_table), int(block_size), int(max_blocks),
            nsplit, ptr(workspace), nbytes, current_stream(dev)))
    return out, lse


# queries whose P / dS tiles one pass of the tensor-core backward keeps in its workspace (1 MiB each at H = 128, topk = 2048):
# eight per SM of a B200.  Larger passes mean fewer launches and fewer partly filled waves (8.9 ms with 296, 8.6 ms with 1184
# on the prefill shape); whether a pass fits the L2 makes no measurable difference.
BWD_TC_QUERIES_PER_PASS = 1184


def sparse_mla_bwd_raw(q, kv, indices, out, lse, d_out, *, sm_scale: float, q_start: int, causal: bool, impl: str = "auto",
                       queries_per_pass: int | None = None):
    """dQ (input dtype) and dKV (fp32) of the forward; no reference counterpart (see the C header).

    ``impl``: "auto" = the tensor-core kernels when D = 576 / DV = 512 / topk <= 8192, else the CUDA-core kernel;
    "tensor_core" / "cuda_core" force one.  The tensor-core path works in passes of ``queries_per_pass`` queries and
    allocates its workspace (P and dS of one pass) here, as the reference's adapter does for its kernels' workspaces."""
    dev = check_inputs([q, kv, indices, out, lse, d_out], [None, q.dtype, torch.int32, q.dtype, torch.float32, q.dtype],
                       ["q", "kv", "indices", "out", "lse", "d_out"])
    B, S, H, D = q.shape
    S_kv, dv, topk = kv.shape[1], out.shape[3], indices.shape[3]
    if impl not in ("auto", "tensor_core", "cuda_core"):
        raise ValueError(f"unknown impl {impl!r}")
    tc_ok = D == 576 and dv == 512 and topk <= 8192
    if impl == "tensor_core" and not tc_ok:
        raise ValueError("the tensor-core backward needs D = 576, DV = 512 and topk <= 8192")
    use_tc = tc_ok and impl != "cuda_core"
    d_q = torch.empty_like(q)
    d_kv = torch.zeros(kv.shape, dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        if use_tc:
            qpp = min(B * S, int(queries_per_pass) if queries_per_pass else BWD_TC_QUERIES_PER_PASS)
            nbytes = int(lib.dsa_sparse_mla_bwd_tc_workspace_bytes(B, S, H, topk, qpp))
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            _lib.check(lib.dsa_sparse_mla_bwd_tc(
                ptr(q), ptr(kv), ptr(indices), ptr(out), ptr(lse), ptr(d_out), ptr(d_q), ptr(d_kv), B, S, S_kv, H, D, dv, topk,
                float(sm_scale), int(q_start), 1 if causal else 0, dtype_code(q.dtype), None, None, None, None, 0, 0,
                ptr(workspace), nbytes, qpp, current_stream(dev)))
        else:
            _lib.check(lib.dsa_sparse_mla_bwd(
                ptr(q), ptr(kv), ptr(indices), ptr(out), ptr(lse), ptr(d_out), ptr(d_q), ptr(d_kv), B, S, S_kv, H, D, dv, topk,
                float(sm_scale), int(q_start), 1 if causal else 0, dtype_code(q.dtype), None, None, None, None, 0, 0,
                current_stream(dev)))
    return d_q, d_kv


class SparseAttentionFwdKernel:
    """Callable returned by :func:`sparse_attention_fwd`; ``kernel(q, kv, indices) -> out`` (or
    ``(out, lse)`` with ``return_softmax_lse=True``).  Only inputs are passed; outputs are allocated
    on the device of ``q`` and the launch goes to the current stream without synchronising."""

    def __init__(self, heads, dim, tail_dim, topk, sm_scale, dtype, return_softmax_lse, impl):
        self.heads, self.dim, self.tail_dim, self.topk = heads, dim, tail_dim, topk
        self.sm_scale, self.dtype, self.return_softmax_lse, self.impl = sm_scale, dtype, return_softmax_lse, impl

    def __call__(self, q, kv, indices, q_start_index_s: Optional[int] = None, split_tail: Optional[tuple] = None):
        """``split_tail=(m, n)`` (not in the reference): the first m queries are split into n shares of their keys each, so that
        they fill the launch's last, partly filled round of work units (see :func:`sparse_mla_fwd_raw`)."""
        if q.dtype != self.dtype:
            raise ValueError(f"Input tensor q has dtype {q.dtype}, expected {self.dtype}")
        if q.dim() != 4 or q.shape[2] != self.heads or q.shape[3] != self.dim + self.tail_dim:
            raise ValueError(f"q must be [B, S, {self.heads}, {self.dim + self.tail_dim}], got {tuple(q.shape)}")
        if indices.dim() != 4 or indices.shape[3] != self.topk:
            raise ValueError(f"indices must be [B, S, 1, {self.topk}], got {tuple(indices.shape)}")
        S, S_kv = q.shape[1], kv.shape[1]
        q_start = S_kv - S if q_start_index_s is None else int(q_start_index_s)
        extra = {} if not split_tail or split_tail[0] <= 0 or split_tail[1] <= 1 else {"split_queries": int(split_tail[0]), "nsplit": int(split_tail[1])}
        out, lse = sparse_mla_fwd_raw(q, kv, indices, sm_scale=self.sm_scale, q_start=q_start, causal=True, dv=self.dim,
                                      return_lse=self.return_softmax_lse, impl=self.impl, **extra)
        return (out, lse) if self.return_softmax_lse else out


@functools.lru_cache(maxsize=None)
def _sparse_attention_fwd_cached(heads, dim, tail_dim, topk, kv_stride, kv_group, sm_scale, is_causal, block_I, dtype,
                                 return_softmax_lse, impl):
    # argument rules of the reference factory (example_sparse_flash_attn.py:30-36)
    assert dim == _next_pow2(dim), f"haven't check padding correctness yet, dim={dim}"
    assert tail_dim == _next_pow2(tail_dim), f"haven't check padding correctness yet, dim={tail_dim}"
    assert is_causal, "non-casual is not supported"
    assert topk % block_I == 0, "otherwise will load some index=0 thus causing wrong kv to be loaded"
    if kv_group != 1:
        raise ValueError("kv_group must be 1 (one latent KV head shared by all query heads)")
    if kv_stride != 1:
        raise ValueError("kv_stride must be 1")
    scale = (1.0 / (dim + tail_dim)) ** 0.5 if sm_scale is None else float(sm_scale)
    return SparseAttentionFwdKernel(heads, dim, tail_dim, topk, scale, torch_dtype(dtype), return_softmax_lse, impl)


def sparse_attention_fwd(heads, dim, tail_dim, topk, kv_stride, kv_group=1, sm_scale=None, is_causal=True, block_I=64,
                         dtype="bfloat16", return_softmax_lse=False, impl=_lib.IMPL_AUTO):
    """Factory with the reference's signature; cached per argument tuple like the reference's
    ``@tilelang.jit`` (tilelang/jit/__init__.py:216-255).  ``block_I`` is a tiling hint of the
    reference kernel: it is validated and otherwise ignored."""
    return _sparse_attention_fwd_cached(heads, dim, tail_dim, topk, kv_stride, kv_group, sm_scale, is_causal, block_I,
                                        str(dtype).replace("torch.", ""), bool(return_softmax_lse), int(impl))


def sparse_attn_tilelang(query, key, value, sparse_indices, scale_value, sparse_block_size, actual_seq_lengths_query,
                         actual_seq_lengths_kv, query_rope=None, key_rope=None, layout_query="BSND", layout_kv="BSND",
                         sparse_mode=3, block_table=None, attention_mode=None, return_softmax_lse=False):
    """Paged / variable-length front end (decode and chunked prefill).

    query [B,S,H,512] + query_rope [B,S,H,64]; key / key_rope either BSND ([B,S_kv,1,*]) or paged
    PA_BSND ([num_blocks, block_size, 1, *]) with ``block_table`` [B, max_blocks]; ``value`` is the
    latent itself and is not read; sparse_indices [B,S,1,topk] int32, -1 terminated; per-batch actual
    lengths give the causal rule idx <= act_kv - act_q + s.  Mirrors sparse_attn_tilelang
    (bench_sfa/sparse_flash_attn_pa_no_cv_pipeline.py:384-419) and the NumPy golden
    cpu_sparse_flash_attention (examples/sparse_flash_attention/sfa_golden.py:117-199).  The reference
    wrapper takes a single un-batched [S,H,*] query as well; that form is accepted too.
    """
    if layout_query != "BSND":
        raise ValueError("only layout_query='BSND' is supported")
    if layout_kv not in ("BSND", "PA_BSND"):
        raise ValueError(f"unsupported layout_kv {layout_kv}")
    if sparse_block_size != 1:
        raise ValueError("sparse_block_size must be 1 (token-level indices)")
    if sparse_mode not in (0, 3):
        raise ValueError("sparse_mode must be 0 or 3")
    squeeze = query.dim() == 3
    if squeeze:
        query, query_rope, sparse_indices = query.unsqueeze(0), query_rope.unsqueeze(0), sparse_indices.unsqueeze(0)
    q = torch.cat((query, query_rope), dim=-1).contiguous()
    # the key cache and its rope part are read in place as the two parts of a key row where the kernel can do that
    # (512 + 64 values, lists of at most 8192 keys); otherwise they are concatenated into rows of D values first
    two_part = (key.shape[-1] == 512 and key_rope.shape[-1] == 64 and sparse_indices.shape[-1] <= 8192 and key.is_contiguous()
                and key_rope.is_contiguous())
    kv = key if two_part else torch.cat((key, key_rope), dim=-1).contiguous()
    dev = q.device
    B, S = q.shape[0], q.shape[1]
    act_q = torch.as_tensor(actual_seq_lengths_query, dtype=torch.int32).to(dev).contiguous()
    act_kv = torch.as_tensor(actual_seq_lengths_kv, dtype=torch.int32).to(dev).contiguous()
    q_start_b = (act_kv - act_q).contiguous()
    bt = None
    if layout_kv == "PA_BSND":
        if block_table is None:
            raise ValueError("block_table is required for PA_BSND")
        bt = block_table.to(device=dev, dtype=torch.int32).contiguous()
    out, lse = sparse_mla_fwd_raw(q, kv, sparse_indices.to(torch.int32).contiguous(), sm_scale=float(scale_value), q_start=0,
                                  causal=(sparse_mode == 3), dv=query.shape[-1], return_lse=return_softmax_lse,
                                  q_start_b=q_start_b, kv_len_b=act_kv, q_len_b=act_q, block_table=bt,
                                  block_size=kv.shape[1] if bt is not None else 0, kv_rope=key_rope if two_part else None)
    if squeeze:
        out = out.squeeze(0)
        lse = lse.squeeze(0) if lse is not None else None
    return (out, lse) if return_softmax_lse else out


class SparseMLAFunction(torch.autograd.Function):
    """Autograd node over the forward / backward kernels (causal, BSND)."""

    @staticmethod
    def forward(ctx, q, kv, indices, sm_scale, q_start, dv):
        out, lse = sparse_mla_fwd_raw(q, kv, indices, sm_scale=sm_scale, q_start=q_start, causal=True, dv=dv)
        ctx.save_for_backward(q, kv, indices, out, lse)
        ctx.sm_scale, ctx.q_start = sm_scale, q_start
        return out, lse

    @staticmethod
    def backward(ctx, d_out, _d_lse):
        q, kv, indices, out, lse = ctx.saved_tensors
        d_q, d_kv = sparse_mla_bwd_raw(q, kv, indices, out, lse, d_out.contiguous(), sm_scale=ctx.sm_scale,
                                       q_start=ctx.q_start, causal=True)
        return d_q, d_kv.to(kv.dtype), None, None, None, None


def sparse_mla(q, kv, indices, sm_scale=None, q_start_index_s=None, dv=512):
    """Differentiable sparse MLA: returns (out, lse)."""
    scale = q.shape[-1] ** -0.5 if sm_scale is None else float(sm_scale)
    q_start = kv.shape[1] - q.shape[1] if q_start_index_s is None else int(q_start_index_s)
    return SparseMLAFunction.apply(q, kv, indices, scale, q_start, dv)
