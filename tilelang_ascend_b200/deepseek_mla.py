"""Dense MLA decode behind the reference's three factory signatures
(examples_experiment/deepseek_mla/): every key of a sequence's latent cache takes part, so each call is the
sparse forward with the identity index list -- one query token per sequence, non-causal, split over the
keys when there are fewer sequences than SM pairs.

* ``mla_decode``            example_mla_decode/example_mla_decode.py:46-92 (dense cache, optional actual length)
* ``mla_decode_tilelang``   example_mla_decode_paged/example_mla_decode_paged.py:41-131 (paged cache + block table)
* ``flashattn_mla_decode``  example_mla_decode_persistent/example_mla_decode_persistent.py:57-101 (dense cache, 3-D KV)
* ``run_mla_decode``        the persistent example's checked host entry (:322-440)
"""
from __future__ import annotations

import functools

import torch

from .adapter import check_inputs
from .sparse_flash_attention import sparse_mla_fwd_raw

# the tensor-core forward walks index lists of up to this many keys; the dense decode has no other kernel to fall to
MAX_KEYS = 8192


def _identity_indices(cache: dict, dev, batch: int, n: int) -> torch.Tensor:
    key = (dev, batch, n)
    if key not in cache:
        cache[key] = torch.arange(n, dtype=torch.int32, device=dev).view(1, 1, 1, n).expand(batch, 1, 1, n).contiguous()
    return cache[key]


def _check_keys(n: int) -> None:
    if n > MAX_KEYS:
        raise ValueError(f"dense MLA decode handles at most {MAX_KEYS} keys per sequence, got {n}")
    if n < 1:
        raise ValueError("at least one key per sequence is needed")


class MlaDecodeKernel:
    """``kernel(q, q_pe, kv, k_pe, col_indices) -> out``: q [B,H,dim], q_pe [B,H,pe], kv [B,N,1,dim],
    k_pe [B,N,1,pe] -> [B,H,dim].  ``col_indices`` (a 0..127 ramp the reference kernel needs for its
    tail mask) is accepted and not read."""

    def __init__(self, batch, heads, seqlen_kv, dim, pe_dim, actual_seqlen_kv):
        self.batch, self.heads, self.seqlen_kv, self.dim, self.pe_dim = batch, heads, seqlen_kv, dim, pe_dim
        self.actual = seqlen_kv if actual_seqlen_kv in (-1, None) else int(actual_seqlen_kv)
        if not 1 <= self.actual <= seqlen_kv:
            raise ValueError(f"actual_seqlen_kv must be in [1, {seqlen_kv}], got {self.actual}")
        _check_keys(self.actual)
        self._idx = {}

    def __call__(self, q, q_pe, kv, k_pe, col_indices=None):
        dev = check_inputs([q, q_pe, kv, k_pe], [None, q.dtype, q.dtype, q.dtype], ["q", "q_pe", "kv", "k_pe"])
        B, H, N = self.batch, self.heads, self.seqlen_kv
        if tuple(q.shape) != (B, H, self.dim) or tuple(q_pe.shape) != (B, H, self.pe_dim) \
                or tuple(kv.shape) != (B, N, 1, self.dim) or tuple(k_pe.shape) != (B, N, 1, self.pe_dim):
            raise ValueError("input shapes differ from the factory arguments")
        qq = torch.cat((q, q_pe), dim=-1).unsqueeze(1).contiguous()
        idx = _identity_indices(self._idx, dev, B, self.actual)
        scale = (self.dim + self.pe_dim) ** -0.5
        if self.dim == 512 and self.pe_dim == 64:
            # kv and k_pe are read in place (rows in two parts): no concatenated copy of the cache per call
            out, _ = sparse_mla_fwd_raw(qq, kv, idx, sm_scale=scale, q_start=0, causal=False, dv=self.dim, return_lse=False, kv_rope=k_pe)
        else:
            kk = torch.cat((kv, k_pe), dim=-1).contiguous()
            out, _ = sparse_mla_fwd_raw(qq, kk, idx, sm_scale=scale, q_start=0, causal=False, dv=self.dim, return_lse=False)
        return out.squeeze(1)


@functools.lru_cache(maxsize=None)
def _cached(batch, heads, kv_head_num, seqlen_kv, dim, pe_dim, actual_seqlen_kv):
    if kv_head_num != 1:
        raise ValueError("kv_head_num must be 1")
    return MlaDecodeKernel(batch, heads, seqlen_kv, dim, pe_dim, actual_seqlen_kv)


def mla_decode(batch, heads, kv_head_num, seqlen_kv, dim, pe_dim, actual_seqlen_kv=-1, core_num=20):
    """Factory with the reference's signature; ``core_num`` is ignored."""
    return _cached(int(batch), int(heads), int(kv_head_num), int(seqlen_kv), int(dim), int(pe_dim), int(actual_seqlen_kv))


class MlaDecodePagedKernel:
    """``kernel(Q, Q_pe, KV, K_pe, block_table) -> Output``: Q [batch,h_q,dv], Q_pe [batch,h_q,dpe],
    KV [batch*max_seqlen_pad, 1, dv], K_pe [batch*max_seqlen_pad, 1, dpe] (pools of blocks of ``block_size`` rows),
    block_table [batch, max_seqlen_pad // block_size] int32 -> [batch,h_q,dv].  The first ``cache_seqlen`` logical
    positions of every sequence take part.  As in the reference kernel the scores are NOT scaled here: the caller
    pre-multiplies Q and Q_pe by the softmax scale (example_mla_decode_paged.py:284,403-406)."""

    def __init__(self, batch, h_q, max_seqlen_pad, dv, dpe, block_size, cache_seqlen):
        self.batch, self.h_q, self.max_seqlen_pad, self.dv, self.dpe = batch, h_q, max_seqlen_pad, dv, dpe
        self.block_size, self.cache_seqlen = block_size, cache_seqlen
        self._idx, self._len = {}, {}

    def __call__(self, Q, Q_pe, KV, K_pe, block_table):
        dev = check_inputs([Q, Q_pe, KV, K_pe, block_table], [None, Q.dtype, Q.dtype, Q.dtype, torch.int32],
                           ["Q", "Q_pe", "KV", "K_pe", "block_table"])
        B, H, rows, nb = self.batch, self.h_q, self.batch * self.max_seqlen_pad, self.max_seqlen_pad // self.block_size
        if tuple(Q.shape) != (B, H, self.dv) or tuple(Q_pe.shape) != (B, H, self.dpe) or tuple(KV.shape) != (rows, 1, self.dv) \
                or tuple(K_pe.shape) != (rows, 1, self.dpe) or tuple(block_table.shape) != (B, nb):
            raise ValueError("input shapes differ from the factory arguments")
        qq = torch.cat((Q, Q_pe), dim=-1).unsqueeze(1).contiguous()
        if dev not in self._len:
            self._len[dev] = torch.full((B,), self.cache_seqlen, dtype=torch.int32, device=dev)
        idx = _identity_indices(self._idx, dev, B, self.cache_seqlen)
        common = dict(sm_scale=1.0, q_start=0, causal=False, dv=self.dv, return_lse=False, kv_len_b=self._len[dev], block_table=block_table,
                      block_size=self.block_size)
        nblk = rows // self.block_size
        if self.dv == 512 and self.dpe == 64:
            # the two pools are read in place through the same block table (rows in two parts)
            out, _ = sparse_mla_fwd_raw(qq, KV.view(nblk, self.block_size, 1, self.dv), idx, kv_rope=K_pe.view(nblk, self.block_size, 1, self.dpe),
                                        **common)
        else:
            pool = torch.cat((KV, K_pe), dim=-1).view(nblk, self.block_size, 1, self.dv + self.dpe)
            out, _ = sparse_mla_fwd_raw(qq, pool, idx, **common)
        return out.squeeze(1)


@functools.lru_cache(maxsize=None)
def _paged_cached(batch, h_q, max_seqlen_pad, dv, dpe, block_size, cache_seqlen):
    return MlaDecodePagedKernel(batch, h_q, max_seqlen_pad, dv, dpe, block_size, cache_seqlen)


def mla_decode_tilelang(batch, h_q, h_kv, max_seqlen_pad, dv, dpe, block_N, block_H, block_size, cache_seqlen, core_num,
                        softmax_scale=None):
    """Factory with the reference's signature and argument rules (example_mla_decode_paged.py:96-101).  ``block_N``,
    ``block_H`` and ``core_num`` only enter those rules; ``softmax_scale`` is accepted and -- as in the reference
    kernel -- not applied (the caller pre-scales Q)."""
    assert h_kv == 1, "h_kv must be 1"
    assert block_size >= block_N and block_size % block_N == 0
    assert max_seqlen_pad % block_N == 0
    assert cache_seqlen >= 1, "cache_seqlen must be >= 1"
    assert cache_seqlen <= max_seqlen_pad, f"cache_seqlen ({cache_seqlen}) must <= max_seqlen_pad ({max_seqlen_pad})"
    _check_keys(int(cache_seqlen))
    return _paged_cached(int(batch), int(h_q), int(max_seqlen_pad), int(dv), int(dpe), int(block_size), int(cache_seqlen))


class MlaDecodePersistentKernel:
    """``kernel(Q, Q_pe, KV, K_pe) -> Output``: Q [batch,heads,dim], Q_pe [batch,heads,pe_dim], KV [batch,seqlen_kv,dim],
    K_pe [batch,seqlen_kv,pe_dim] -> [batch,heads,dim]; scores scaled by (dim + pe_dim)^-0.5 inside."""

    def __init__(self, batch, heads, seqlen_kv, dim, pe_dim):
        self.batch, self.heads, self.seqlen_kv, self.dim, self.pe_dim = batch, heads, seqlen_kv, dim, pe_dim
        self._idx = {}

    def __call__(self, Q, Q_pe, KV, K_pe):
        dev = check_inputs([Q, Q_pe, KV, K_pe], [None, Q.dtype, Q.dtype, Q.dtype], ["Q", "Q_pe", "KV", "K_pe"])
        B, H, N = self.batch, self.heads, self.seqlen_kv
        if tuple(Q.shape) != (B, H, self.dim) or tuple(Q_pe.shape) != (B, H, self.pe_dim) or tuple(KV.shape) != (B, N, self.dim) \
                or tuple(K_pe.shape) != (B, N, self.pe_dim):
            raise ValueError("input shapes differ from the factory arguments")
        qq = torch.cat((Q, Q_pe), dim=-1).unsqueeze(1).contiguous()
        idx = _identity_indices(self._idx, dev, B, N)
        scale = (self.dim + self.pe_dim) ** -0.5
        if self.dim == 512 and self.pe_dim == 64:   # KV and K_pe read in place (rows in two parts)
            out, _ = sparse_mla_fwd_raw(qq, KV.unsqueeze(2), idx, sm_scale=scale, q_start=0, causal=False, dv=self.dim, return_lse=False,
                                        kv_rope=K_pe.unsqueeze(2))
        else:
            kk = torch.cat((KV, K_pe), dim=-1).unsqueeze(2).contiguous()
            out, _ = sparse_mla_fwd_raw(qq, kk, idx, sm_scale=scale, q_start=0, causal=False, dv=self.dim, return_lse=False)
        return out.squeeze(1)


@functools.lru_cache(maxsize=None)
def _persistent_cached(batch, heads, seqlen_kv, dim, pe_dim):
    return MlaDecodePersistentKernel(batch, heads, seqlen_kv, dim, pe_dim)


def flashattn_mla_decode(batch, heads, seqlen_kv, dim, pe_dim, block_N, block_H, core_num):
    """Factory with the reference's signature; ``block_N``, ``block_H`` and ``core_num`` are tiling knobs of the
    reference kernel and are ignored (any ``seqlen_kv`` is accepted, not only multiples of ``block_N``)."""
    _check_keys(int(seqlen_kv))
    return _persistent_cached(int(batch), int(heads), int(seqlen_kv), int(dim), int(pe_dim))


def run_mla_decode(q, q_pe, kv, k_pe, block_N, block_H, core_num):
    """Checked host entry of the persistent example: q [B,H,dim], q_pe [B,H,pe], kv [B,N,1,dim], k_pe [B,N,1,pe];
    same dtype / rank / shape-consistency assertions (example_mla_decode_persistent.py:339-390), then the kernel on
    the 3-D views of the caches."""
    assert q.dtype == q_pe.dtype == kv.dtype == k_pe.dtype, "q, q_pe, kv and k_pe must have one dtype"
    assert q.ndim == 3, f"q.ndim must be 3 [batch, heads, dim], got {q.ndim}"
    assert q_pe.ndim == 3, f"q_pe.ndim must be 3 [batch, heads, pe_dim], got {q_pe.ndim}"
    assert kv.ndim == 4, f"kv.ndim must be 4 [batch, seqlen_kv, 1, dim], got {kv.ndim}"
    assert k_pe.ndim == 4, f"k_pe.ndim must be 4 [batch, seqlen_kv, 1, pe_dim], got {k_pe.ndim}"
    assert q.shape[0] == q_pe.shape[0] == kv.shape[0] == k_pe.shape[0], "batch mismatch"
    assert q.shape[1] == q_pe.shape[1], f"heads mismatch: q={q.shape[1]}, q_pe={q_pe.shape[1]}"
    assert kv.shape[1] == k_pe.shape[1], f"seqlen_kv mismatch: kv={kv.shape[1]}, k_pe={k_pe.shape[1]}"
    assert kv.shape[3] == q.shape[2], f"dim mismatch: kv.shape[3]={kv.shape[3]}, q.shape[2]={q.shape[2]}"
    assert k_pe.shape[3] == q_pe.shape[2], f"pe_dim mismatch: k_pe.shape[3]={k_pe.shape[3]}, q_pe.shape[2]={q_pe.shape[2]}"
    assert kv.shape[2] == 1, "kv_head_num must be 1"
    batch, heads, seqlen_kv, dim, pe_dim = q.shape[0], q.shape[1], kv.shape[1], q.shape[2], q_pe.shape[2]
    assert min(batch, heads, seqlen_kv, dim, pe_dim, block_N, block_H, core_num) > 0, "sizes must be positive"
    kernel = flashattn_mla_decode(batch, heads, seqlen_kv, dim, pe_dim, block_N, block_H, core_num)
    return kernel(q, q_pe, kv.view(batch, seqlen_kv, dim), k_pe.view(batch, seqlen_kv, pe_dim))
