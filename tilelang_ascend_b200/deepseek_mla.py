"""Dense MLA decode behind the reference's factory signature
(examples_experiment/deepseek_mla/example_mla_decode/example_mla_decode.py:46-92): every key of the
latent cache takes part, so the call is the sparse forward with the identity index list."""
from __future__ import annotations

import functools

import torch

from .adapter import check_inputs
from .sparse_flash_attention import sparse_mla_fwd_raw


class MlaDecodeKernel:
    """``kernel(q, q_pe, kv, k_pe, col_indices) -> out``: q [B,H,dim], q_pe [B,H,pe], kv [B,N,1,dim],
    k_pe [B,N,1,pe] -> [B,H,dim].  ``col_indices`` (a 0..127 ramp the reference kernel needs for its
    tail mask) is accepted and not read."""

    def __init__(self, batch, heads, seqlen_kv, dim, pe_dim, actual_seqlen_kv):
        self.batch, self.heads, self.seqlen_kv, self.dim, self.pe_dim = batch, heads, seqlen_kv, dim, pe_dim
        self.actual = seqlen_kv if actual_seqlen_kv in (-1, None) else int(actual_seqlen_kv)
        self._idx = {}

    def __call__(self, q, q_pe, kv, k_pe, col_indices=None):
        dev = check_inputs([q, q_pe, kv, k_pe], [None, q.dtype, q.dtype, q.dtype], ["q", "q_pe", "kv", "k_pe"])
        B, H, N = self.batch, self.heads, self.seqlen_kv
        if tuple(q.shape) != (B, H, self.dim) or tuple(q_pe.shape) != (B, H, self.pe_dim) \
                or tuple(kv.shape) != (B, N, 1, self.dim) or tuple(k_pe.shape) != (B, N, 1, self.pe_dim):
            raise ValueError("input shapes differ from the factory arguments")
        if dev not in self._idx:
            self._idx[dev] = torch.arange(self.actual, dtype=torch.int32, device=dev).view(1, 1, 1, -1).expand(B, 1, 1, -1).contiguous()
        qq = torch.cat((q, q_pe), dim=-1).unsqueeze(1).contiguous()
        kk = torch.cat((kv, k_pe), dim=-1).contiguous()
        out, _ = sparse_mla_fwd_raw(qq, kk, self._idx[dev], sm_scale=(self.dim + self.pe_dim) ** -0.5, q_start=0, causal=False,
                                    dv=self.dim, return_lse=False)
        return out.squeeze(1)


@functools.lru_cache(maxsize=None)
def _cached(batch, heads, kv_head_num, seqlen_kv, dim, pe_dim, actual_seqlen_kv):
    if kv_head_num != 1:
        raise ValueError("kv_head_num must be 1")
    return MlaDecodeKernel(batch, heads, seqlen_kv, dim, pe_dim, actual_seqlen_kv)


def mla_decode(batch, heads, kv_head_num, seqlen_kv, dim, pe_dim, actual_seqlen_kv=-1, core_num=20):
    """Factory with the reference's signature; ``core_num`` is ignored."""
    return _cached(int(batch), int(heads), int(kv_head_num), int(seqlen_kv), int(dim), int(pe_dim), int(actual_seqlen_kv))
