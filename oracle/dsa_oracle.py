"""CPU oracle for the DeepSeek-sparse-attention hot path.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared
with; it is never the thing that is shipped or measured as the product.  Only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark may import it.

Parity status: PINNED.  Every function below is checked in ``tests/test_oracle.py``
against fixtures under ``tests/golden/`` that were produced by running the reference's
own PyTorch / NumPy golden functions (``tests/golden/make_golden.py`` is the
generating script; it needs the reference checkout and is not run on the GPU box).

Each function restates, in fp32 on the CPU, the arithmetic of one reference golden and
cites the file:line (paths relative to the reference project root) it follows.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

NEG_INF = float("-inf")


# ---------------------------------------------------------------------------
# lightning indexer
# ---------------------------------------------------------------------------
def indexer_scores(
    query: torch.Tensor,
    key: torch.Tensor,
    weights: torch.Tensor,
    *,
    sparse_mode: int = 3,
    actual_q: Optional[int] = None,
    actual_k: Optional[int] = None,
    q_chunk: int = 256,
) -> torch.Tensor:
    """score[b, s1, s2] = sum_h w[b,s1,h] * relu(q[b,s1,h,:] . k[b,s2,0,:]) in fp32.

    query [B,S1,N1,D], key [B,S2,1,D], weights [B,S1,N1].  Keys at or beyond the causal
    limit ``s2 >= actual_k - actual_q + s1 + 1`` are set to -inf when ``sparse_mode == 3``;
    a non-positive limit means "all keys valid".
    Follows examples/deepseek_v4/lightning_indexer.py:303-314 (score, mask).
    """
    B, S1, N1, D = query.shape
    S2 = key.shape[1]
    aq = S1 if actual_q is None else int(actual_q)
    ak = S2 if actual_k is None else int(actual_k)
    out = torch.full((B, S1, S2), NEG_INF, dtype=torch.float32)
    kf = key[:, :ak, 0, :].float()
    cols = torch.arange(ak)
    for b in range(B):
        for s in range(0, aq, q_chunk):
            e = min(aq, s + q_chunk)
            qb = query[b, s:e].float()  # [c, N1, D]
            wb = weights[b, s:e].float()  # [c, N1]
            qk = torch.relu(torch.einsum("qgd,kd->qgk", qb, kf[b]))
            sc = (qk * wb.unsqueeze(2)).sum(dim=1)  # [c, ak]
            if sparse_mode == 3:
                lim = ak - aq + torch.arange(s, e) + 1
                lim = torch.where(lim > 0, lim, torch.full_like(lim, ak))
            else:
                lim = torch.full((e - s,), ak)
            sc = sc.masked_fill(~(cols[None, :] < lim[:, None]), NEG_INF)
            out[b, s:e, :ak] = sc
    return out


def causal_limits(S1: int, S2: int, sparse_mode: int = 3, actual_q: Optional[int] = None,
                  actual_k: Optional[int] = None) -> np.ndarray:
    """Number of leading keys that are valid for each query row (int32 [S1]).

    Follows examples/deepseek_v4/lightning_indexer.py:308-314.
    """
    aq = S1 if actual_q is None else int(actual_q)
    ak = S2 if actual_k is None else int(actual_k)
    if sparse_mode == 3:
        lim = ak - aq + np.arange(S1, dtype=np.int64) + 1
        lim = np.where(lim > 0, lim, ak)
    else:
        lim = np.full((S1,), ak, dtype=np.int64)
    lim[aq:] = 0
    return np.minimum(lim, ak).astype(np.int32)


def topk_select(scores: np.ndarray, top_k: int, limits: Optional[np.ndarray] = None,
                return_values: bool = False):
    """Row-wise top-k: descending score, ties resolved towards the lower index.

    scores fp32 [rows, n]; ``limits[r]`` (optional) is the number of leading entries of row r
    that are candidates.  Slots without a candidate, and selected slots whose score is
    <= -1e30, hold -1 (value -inf).  The output order is the sorted order, so the whole
    index array -- not only the index set -- is determined.
    Follows examples/deepseek_v4/lightning_indexer.py:316-325 (stable argsort of -score,
    -1 fill) and examples/topk_selector/example_topk_selector.py:57-58 (set of the
    ``top_k`` largest).
    """
    scores = np.asarray(scores, dtype=np.float32)
    rows, n = scores.shape
    idx = np.full((rows, top_k), -1, dtype=np.int32)
    val = np.full((rows, top_k), -np.inf, dtype=np.float32)
    for r in range(rows):
        lim = n if limits is None else int(limits[r])
        lim = max(0, min(lim, n))
        if lim == 0:
            continue
        row = scores[r, :lim]
        order = np.argsort(-row, kind="stable")
        kk = min(top_k, lim)
        sel = order[:kk]
        v = row[sel]
        bad = v <= -1e30
        idx[r, :kk] = np.where(bad, -1, sel).astype(np.int32)
        val[r, :kk] = np.where(bad, -np.inf, v)
    if return_values:
        return idx, val
    return idx


def lightning_indexer(
    query: torch.Tensor,
    key: torch.Tensor,
    weights: torch.Tensor,
    *,
    sparse_count: int = 2048,
    sparse_mode: int = 3,
    actual_seq_lengths_query=None,
    actual_seq_lengths_key=None,
    return_value: bool = False,
):
    """BSND lightning indexer: indices int32 [B,S1,1,K] (and values in the input dtype).

    Follows cpu_lightning_indexer, examples/deepseek_v4/lightning_indexer.py:199-335
    (BSND layout, N2 == 1).  Per-batch actual lengths may shorten the query / key ranges.
    """
    B, S1, N1, D = query.shape
    S2 = key.shape[1]
    K = sparse_count
    asq = [S1] * B if actual_seq_lengths_query is None else [int(x) for x in actual_seq_lengths_query]
    ask = [S2] * B if actual_seq_lengths_key is None else [int(x) for x in actual_seq_lengths_key]
    idx = torch.full((B, S1, 1, K), -1, dtype=torch.int32)
    val = torch.full((B, S1, 1, K), NEG_INF, dtype=query.dtype)
    for b in range(B):
        aq, ak = asq[b], ask[b]
        if aq == 0 or ak == 0:
            continue
        sc = indexer_scores(query[b:b + 1], key[b:b + 1], weights[b:b + 1], sparse_mode=sparse_mode,
                            actual_q=aq, actual_k=ak)[0]
        # every key column < ak is a candidate; masked ones carry -inf and turn into -1
        lim = np.zeros((S1,), dtype=np.int32)
        lim[:aq] = ak
        i, v = topk_select(sc.numpy(), K, lim, return_values=True)
        idx[b, :, 0, :] = torch.from_numpy(i)
        val[b, :, 0, :] = torch.from_numpy(v).to(query.dtype)
    if return_value:
        return idx, val
    return idx


# ---------------------------------------------------------------------------
# sparse MLA forward / backward
# ---------------------------------------------------------------------------
def _valid_mask(indices: torch.Tensor, S_kv: int, pos: torch.Tensor) -> torch.Tensor:
    """valid[q, j]: index j of query q names a key that takes part.

    A slot takes part when 0 <= idx < S_kv and idx <= pos[q]; a repeated index counts once
    (mask semantics of examples/sparse_flash_attention/example_sparse_flash_attn.py:277-280).
    """
    idx = indices.long()
    ok = (idx >= 0) & (idx < S_kv) & (idx <= pos[:, None])
    # drop repeats: keep the first occurrence in sorted order
    key = torch.where(ok, idx, torch.full_like(idx, S_kv + 1))
    srt, perm = torch.sort(key, dim=1, stable=True)
    dup_sorted = torch.zeros_like(srt, dtype=torch.bool)
    dup_sorted[:, 1:] = srt[:, 1:] == srt[:, :-1]
    dup = torch.zeros_like(dup_sorted)
    dup.scatter_(1, perm, dup_sorted)
    return ok & ~dup


def sparse_mla_fwd(
    q: torch.Tensor,
    kv: torch.Tensor,
    indices: torch.Tensor,
    *,
    q_start_index_s: Optional[int] = None,
    sm_scale: Optional[float] = None,
    dv: int = 512,
    q_chunk: int = 32,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse MLA forward in fp32: (out [B,S,H,dv] fp32, lse [B,S,H] fp32).

    q [B,S,H,D], kv [B,S_kv,1,D], indices [B,S,1,topk] int32 (-1 or S_kv = padding).
    For query t (absolute position p = q_start + t, q_start defaulting to S_kv - S) the key
    set is {idx : 0 <= idx < S_kv, idx <= p}; s = sm_scale * q.kv[idx] over all D dims,
    p = softmax(s), out = sum p * kv[idx][:dv]; lse = m + ln(sum exp(s - m)), natural log.
    Follows ref_sparse_attention_fwd_interface,
    examples/sparse_flash_attention/example_sparse_flash_attn.py:255-292 (kv_stride = 1), and
    the LSE definition of examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_golden.py:149.
    A query whose key set is empty gets out = 0 and lse = -inf.
    """
    B, S, H, D = q.shape
    S_kv = kv.shape[1]
    if q_start_index_s is None:
        q_start_index_s = S_kv - S
    if sm_scale is None:
        sm_scale = D ** -0.5
    out = torch.zeros((B, S, H, dv), dtype=torch.float32)
    lse = torch.full((B, S, H), NEG_INF, dtype=torch.float32)
    for b in range(B):
        kvf = kv[b, :, 0, :].float()
        for s in range(0, S, q_chunk):
            e = min(S, s + q_chunk)
            idx = indices[b, s:e, 0, :]
            pos = torch.arange(s, e) + q_start_index_s
            valid = _valid_mask(idx, S_kv, pos)  # [c, topk]
            g = kvf[idx.long().clamp(0, S_kv - 1)]  # [c, topk, D]
            sc = torch.einsum("chd,ckd->chk", q[b, s:e].float(), g) * sm_scale
            sc = sc.masked_fill(~valid[:, None, :], NEG_INF)
            m = sc.max(dim=-1, keepdim=True).values
            m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
            p = torch.exp(sc - m_safe)
            l = p.sum(dim=-1, keepdim=True)
            o = torch.einsum("chk,ckd->chd", p, g[..., :dv])
            has = l > 0
            out[b, s:e] = torch.where(has, o / torch.where(has, l, torch.ones_like(l)), torch.zeros_like(o))
            lse[b, s:e] = torch.where(has, m_safe + torch.log(torch.where(has, l, torch.ones_like(l))),
                                      torch.full_like(l, NEG_INF)).squeeze(-1)
    return out, lse


def sparse_mla_bwd(
    q: torch.Tensor,
    kv: torch.Tensor,
    indices: torch.Tensor,
    d_out: torch.Tensor,
    *,
    q_start_index_s: Optional[int] = None,
    sm_scale: Optional[float] = None,
    dv: int = 512,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dQ [B,S,H,D] fp32, dKV [B,S_kv,1,D] fp32) by autograd through :func:`sparse_mla_fwd`.

    The reference has no sparse-MLA backward; this follows the way its dense backward golden is
    built (autograd of the forward golden,
    examples_experiment/example_gqa_bwd/example_gqa_bwd.py:623-658).
    """
    qf = q.float().detach().requires_grad_(True)
    kvf = kv.float().detach().requires_grad_(True)
    o, _ = sparse_mla_fwd(qf, kvf, indices, q_start_index_s=q_start_index_s, sm_scale=sm_scale, dv=dv)
    o.backward(d_out.float())
    return qf.grad.detach(), kvf.grad.detach()


def mla_decode(q: torch.Tensor, q_pe: torch.Tensor, kv: torch.Tensor, k_pe: torch.Tensor) -> torch.Tensor:
    """Dense MLA decode in fp32: softmax((q.kv^T + q_pe.k_pe^T)/sqrt(D+pe)) . kv -> [B,H,D] fp32.

    Follows ref_mla_decode,
    examples_experiment/deepseek_mla/example_mla_decode/test_mla_decode.py:59-84.
    """
    D, pe = q.shape[-1], q_pe.shape[-1]
    k2 = kv[:, :, 0, :].float()
    p2 = k_pe[:, :, 0, :].float()
    s = torch.matmul(q.float(), k2.transpose(1, 2)) + torch.matmul(q_pe.float(), p2.transpose(1, 2))
    s = s / math.sqrt(D + pe)
    return torch.matmul(torch.softmax(s, dim=-1), k2)


def mla_decode_paged(q: torch.Tensor, q_pe: torch.Tensor, kv_pool: torch.Tensor, k_pe_pool: torch.Tensor, block_table: torch.Tensor,
                     cache_seqlens, block_size: int, softmax_scale: float = 1.0) -> torch.Tensor:
    """Dense MLA decode over a paged cache in fp32 -> [B,H,dv] fp32.  kv_pool [rows,1,dv], k_pe_pool [rows,1,dpe]; logical
    position p of sequence b is pool row block_table[b, p // block_size] * block_size + p % block_size; the first
    cache_seqlens[b] positions take part.  ``softmax_scale`` multiplies the scores (the reference test passes 1.0 because
    its Q is pre-scaled).

    Follows golden_mla_decode_paged,
    examples_experiment/deepseek_mla/example_mla_decode_paged/test_mla_decode_paged.py:35-87.
    """
    B, H, dv = q.shape
    out = torch.zeros((B, H, dv), dtype=torch.float32)
    bt = block_table.long()
    for b in range(B):
        n = int(cache_seqlens[b])
        pos = torch.arange(n)
        rows = bt[b, pos // block_size] * block_size + pos % block_size
        k2 = kv_pool[rows, 0, :].float()
        p2 = k_pe_pool[rows, 0, :].float()
        s = (q[b].float() @ k2.T + q_pe[b].float() @ p2.T) * float(softmax_scale)
        out[b] = torch.softmax(s, dim=-1) @ k2
    return out


# ---------------------------------------------------------------------------
# DeepSeek-V4 sparse_flash_mla: sliding window + compressed tokens + sink
# ---------------------------------------------------------------------------
def sparse_flash_mla_v4(
    q: torch.Tensor,                      # [B, S, N1, D]
    ori_k: torch.Tensor,                  # [B, S_kv, D]   original cache (K = V, one KV head)
    sinks: torch.Tensor,                  # [N1]
    *,
    act_q_lens,
    act_kv_lens,
    softmax_scale: float,
    cmp_k: Optional[torch.Tensor] = None,             # [B, S_cmp, D] compressed cache
    cmp_sparse_indices: Optional[torch.Tensor] = None,  # [B, S, K] int, -1 ends a list; None = all tokens below the threshold
    cmp_ratio: Optional[int] = None,
    ori_win_left: int = 127,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """out [B,S,N1,D] (input dtype) and lse [B,S,N1] fp32 (natural log, sink included); rows s >= act_q stay zero.

    Follows sparse_flash_mla_golden_bnsd
    (examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_golden.py:56-153): token s of sequence b sits at
    p = act_kv - act_q + s (:97); window keys [max(p - win, 0), p] (:100-102); compressed keys: the listed tokens, the
    list cut at min(K, threshold) entries and at the first -1, entries >= min(threshold, floor(act_kv / ratio)) skipped,
    threshold = floor((p + 1) / ratio) (_gather_cmp_kv_tokens :16-53; dense variant :116-118); the softmax starts from
    row_max = sink, row_sum = 1 (:121-122), i.e. the sink adds exp(sink) to the denominator and nothing to the
    numerator; lse = max + log(sum) (:149).  The golden rounds P to the input dtype before P.V (:143); this restatement
    keeps fp32 (difference far below the comparison tolerance)."""
    B, S, N1, D = q.shape
    out = torch.zeros((B, S, N1, D), dtype=torch.float32)
    lse = torch.zeros((B, S, N1), dtype=torch.float32)
    sk = sinks.to(torch.float32)
    for b in range(B):
        aq, akv = int(act_q_lens[b]), int(act_kv_lens[b])
        for s in range(aq):
            p = akv - aq + s
            keys = [ori_k[b, max(p - ori_win_left, 0): p + 1].to(torch.float32)]
            if cmp_k is not None:
                threshold = (p + 1) // cmp_ratio
                if cmp_sparse_indices is None:
                    keys.append(cmp_k[b, : max(threshold, 0)].to(torch.float32))
                else:
                    cmp_len = akv // cmp_ratio
                    picked = []
                    for i in range(min(cmp_sparse_indices.shape[-1], max(threshold, 0))):
                        t = int(cmp_sparse_indices[b, s, i])
                        if t == -1:
                            break
                        if 0 <= t < min(threshold, cmp_len):
                            picked.append(t)
                    keys.append(cmp_k[b, picked].to(torch.float32) if picked else cmp_k.new_zeros((0, D), dtype=torch.float32))
            kk = torch.cat(keys, dim=0)                                     # [n, D]
            sc = q[b, s].to(torch.float32) @ kk.T * softmax_scale           # [N1, n]
            m = torch.maximum(sc.amax(dim=1), sk) if kk.shape[0] else sk.clone()
            e = torch.exp(sc - m[:, None])
            den = e.sum(dim=1) + torch.exp(sk - m)
            out[b, s] = (e @ kk) / den[:, None]
            lse[b, s] = m + torch.log(den)
    return out.to(q.dtype), lse


# ---------------------------------------------------------------------------
# HISA block-sparse indexer logits
# ---------------------------------------------------------------------------
def block_sparse_logits(q: torch.Tensor, k: torch.Tensor, topk_block_indices: torch.Tensor, kv_block_size: int,
                        weights: torch.Tensor, cu_seqlen_ks: torch.Tensor, cu_seqlen_ke: torch.Tensor) -> torch.Tensor:
    """logits [S, topk, kv_block_size] fp32: sum_h w[s,h] * relu(q[s,h,:] . k[pos,:]) at pos = block * kv_block_size + b, -inf
    where pos >= S_kv or pos outside [ks[s], ke[s]).  Follows ref_block_sparse_mqa_attn
    (examples/HISA/block_sparse_mqa_attn_expert_test.py:548-587); positions beyond the key tensor are not read here
    (the reference's gather would fail on them)."""
    S, H, D = q.shape
    S_kv = k.shape[0]
    pos = topk_block_indices.long()[:, :, None] * kv_block_size + torch.arange(kv_block_size)[None, None, :]   # [S, topk, bs]
    safe = pos.clamp(0, S_kv - 1)
    kg = k.float()[safe.reshape(-1)].reshape(S, -1, D)                                                         # [S, topk*bs, D]
    sc = torch.einsum("shd,snd->snh", q.float(), kg).relu() * weights.float()[:, None, :]
    logits = sc.sum(-1).reshape(S, -1, kv_block_size)
    bad = (pos >= S_kv) | (pos < 0) | (pos < cu_seqlen_ks.long()[:, None, None]) | (pos >= cu_seqlen_ke.long()[:, None, None])
    return logits.masked_fill(bad, NEG_INF)


def paged_block_sparse_logits(q: torch.Tensor, kv_cache: torch.Tensor, topk_block_indices: torch.Tensor, kv_block_size: int,
                              weights: torch.Tensor, context_lens: torch.Tensor, block_tables: torch.Tensor) -> torch.Tensor:
    """Paged variant: q [B,S,H,D], kv_cache [blocks, bs, 1, D], topk_block_indices [B,S,topk] (logical blocks), weights [B,S,H],
    context_lens [B], block_tables [B, max_blocks] -> logits [B, S, topk * bs] fp32, -inf at logical positions >= the context
    length.  Follows ref_paged_block_sparse_mqa_attn (examples/HISA/paged_block_sparse_mqa_attn_expert.py:425-468)."""
    B, S, H, D = q.shape
    topk = topk_block_indices.shape[2]
    phys = torch.gather(block_tables.long(), 1, topk_block_indices.long().reshape(B, S * topk)).reshape(B, S, topk)
    kb = kv_cache.float()[:, :, 0, :][phys]                                     # [B, S, topk, bs, D]
    sc = torch.einsum("bshd,bstnd->bstnh", q.float(), kb).relu() * weights.float()[:, :, None, None, :]
    logits = sc.sum(-1)                                                         # [B, S, topk, bs]
    pos = topk_block_indices.long()[..., None] * kv_block_size + torch.arange(kv_block_size)
    logits = logits.masked_fill(pos >= context_lens.long()[:, None, None, None], NEG_INF)
    return logits.reshape(B, S, topk * kv_block_size)


# ---------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# ---------------------------------------------------------------------------
def make_sparse_mla_inputs(B: int, S: int, S_kv: int, H: int, topk: int, *, D: int = 576, seed: int = 0,
                           dtype=torch.bfloat16, causal: bool = True, pad: int = -1):
    """q, kv ~ N(0,1) and per-query distinct indices.

    causal: query t (absolute position p = S_kv - S + t) draws min(topk, p+1) distinct positions
    from [0, p]; the remaining slots hold ``pad``.  non-causal: topk distinct positions from
    [0, S_kv).  Mirrors the input construction of
    examples/sparse_flash_attention/example_sparse_flash_attn.py:295-308.
    """
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, S, H, D), generator=g, dtype=torch.float32).to(dtype)
    kv = torch.randn((B, S_kv, 1, D), generator=g, dtype=torch.float32).to(dtype)
    rng = np.random.default_rng(seed + 1)
    idx = np.full((B, S, 1, topk), pad, dtype=np.int32)
    for b in range(B):
        for t in range(S):
            n = (S_kv - S + t + 1) if causal else S_kv
            if n <= topk:
                sel = rng.permutation(n)
            else:
                sel = rng.choice(n, size=topk, replace=False)
            idx[b, t, 0, : len(sel)] = sel
    return q, kv, torch.from_numpy(idx)


def make_indexer_inputs(B: int, S1: int, S2: int, N1: int = 64, D: int = 128, *, seed: int = 0,
                        dtype=torch.bfloat16):
    """q_idx [B,S1,N1,D], k_idx [B,S2,1,D] ~ N(0,1); weights [B,S1,N1] fp32 ~ N(0,1)/8."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, S1, N1, D), generator=g, dtype=torch.float32).to(dtype)
    k = torch.randn((B, S2, 1, D), generator=g, dtype=torch.float32).to(dtype)
    w = torch.randn((B, S1, N1), generator=g, dtype=torch.float32) / 8
    return q, k, w


def valid_pairs_causal(S: int, S_kv: int, topk: int) -> int:
    """Number of (query, key) pairs that take part for causally sampled indices."""
    p = np.arange(S, dtype=np.int64) + (S_kv - S) + 1
    return int(np.minimum(p, topk).sum())
