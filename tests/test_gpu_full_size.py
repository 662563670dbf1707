"""Full-size cases on the GPU (the named benchmark shapes and the reference examples' own shapes): size-independent
properties plus oracle checks on sampled rows.

The oracle is too slow for the full tensors, so each case checks (a) a sample of query rows against the fp32
oracle, and (b) properties that hold for every row: determinism, agreement between the tensor-core and the
generic kernel, sortedness / distinctness / causality of the selected indices, additivity of dKV over queries.
"""
import numpy as np
import pytest
import torch

from gpu_util import assert_close_fp, check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _causal_indices(S, S_kv, topk, gen):
    pos = torch.arange(S, device=DEV) + (S_kv - S)
    r = torch.rand((S, S_kv), generator=gen, device=DEV)
    r = torch.where(torch.arange(S_kv, device=DEV)[None, :] <= pos[:, None], r, torch.full_like(r, -1.0))
    vals, sel = torch.topk(r, topk, dim=1)
    return torch.where(vals >= 0, sel, torch.full_like(sel, -1)).to(torch.int32).view(1, S, 1, topk)


def test_prefill_forward_full_size():
    import tilelang_ascend_b200 as dsa
    S = S_kv = 4096
    H, topk = 128, 2048
    g = torch.Generator(device=DEV).manual_seed(0)
    q = torch.randn((1, S, H, 576), generator=g, device=DEV).to(torch.bfloat16)
    kv = torch.randn((1, S_kv, 1, 576), generator=g, device=DEV).to(torch.bfloat16)
    idx = _causal_indices(S, S_kv, topk, g)
    kernel = dsa.sparse_attention_fwd(H, 512, 64, topk, 1, return_softmax_lse=True)
    out, lse = kernel(q, kv, idx)
    out2, lse2 = kernel(q, kv, idx)
    check_status()
    assert torch.equal(out, out2) and torch.equal(lse, lse2)  # deterministic
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    rows = torch.tensor([0, 1, 63, 64, 65, 1000, 2046, 2047, 2048, 3000, 4095])
    qc, kvc, ic = q.cpu(), kv.cpu(), idx.cpu()
    for r in rows.tolist():
        ro, rl = orc.sparse_mla_fwd(qc[:, r:r + 1], kvc, ic[:, r:r + 1], q_start_index_s=r)
        assert_close_fp(out[:, r:r + 1].cpu(), ro, f"out row {r}")
        assert_close_fp(lse[:, r:r + 1].cpu(), rl, f"lse row {r}")
    # the generic kernel must agree with the tensor-core kernel on a block of rows
    sl = slice(2040, 2056)
    og, lg = dsa.sparse_mla_fwd_raw(q[:, sl].contiguous(), kv, idx[:, sl].contiguous(), sm_scale=576 ** -0.5, q_start=2040, causal=True,
                                    dv=512, impl=1)
    assert_close_fp(out[:, sl].cpu(), og.float().cpu(), "tensor-core vs generic out")
    assert_close_fp(lse[:, sl].cpu(), lg.cpu(), "tensor-core vs generic lse", atol=1e-3, rtol=1e-4)
    # a permutation of a query's index list must not change its result beyond rounding
    perm = torch.randperm(topk, generator=torch.Generator().manual_seed(1)).to(DEV)
    o3, l3 = kernel(q[:, -8:].contiguous(), kv, idx[:, -8:, :, perm].contiguous(), q_start_index_s=S_kv - 8)
    assert_close_fp(o3.cpu(), out[:, -8:].float().cpu(), "permuted index list")
    assert_close_fp(l3.cpu(), lse[:, -8:].cpu(), "permuted index list lse", atol=1e-3, rtol=1e-4)


def test_indexer_topk_full_size():
    import tilelang_ascend_b200 as dsa
    S1, S2, K = 4096, 8192, 2048
    g = torch.Generator(device=DEV).manual_seed(0)
    q = torch.randn((1, S1, 64, 128), generator=g, device=DEV).to(torch.bfloat16)
    k = torch.randn((1, S2, 1, 128), generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn((1, S1, 64), generator=g, device=DEV) / 8).float()
    idx, _ = dsa.lightning_indexer(q, k, w, sparse_count=K, sparse_mode=3)
    idx2, _ = dsa.lightning_indexer(q, k, w, sparse_count=K, sparse_mode=3)
    scores, limits = dsa.indexer_scores_raw(q, k, w, sparse_mode=3, return_limits=True)
    check_status()
    assert torch.equal(idx, idx2)
    ii = idx[0, :, 0].long()
    lim = limits[0].long()
    assert bool((ii >= 0).all())                                  # every row has >= K candidates (limit >= 4097)
    assert bool((ii < lim[:, None]).all())                        # causal: only keys below the row's limit
    assert bool((torch.sort(ii, dim=1).values.diff(dim=1) > 0).all())   # distinct
    sel = torch.gather(scores[0], 1, ii)
    assert bool((sel.diff(dim=1) <= 0).all())                     # descending score order
    # nothing outside the selection beats the K-th selected score
    masked = scores[0].clone()
    masked.scatter_(1, ii, float("-inf"))
    masked = torch.where(torch.arange(S2, device=DEV)[None, :] < lim[:, None], masked, torch.full_like(masked, float("-inf")))
    assert bool((masked.max(dim=1).values <= sel[:, -1]).all())
    # the selector is bit-exact on the kernel's own scores; the scores agree with the CPU oracle on sampled rows
    qc, kc, wc = q.cpu(), k.cpu(), w.cpu()
    sc_cpu = scores[0].cpu().numpy()
    for r in (0, 1, 777, 2048, 4095):
        ref = orc.topk_select(sc_cpu[r:r + 1], K, np.array([int(lim[r])]))[0]
        assert np.array_equal(ref, idx[0, r, 0].cpu().numpy())
        s = orc.indexer_scores(qc[:, r:r + 1], kc, wc[:, r:r + 1], sparse_mode=0)[0, 0].numpy()
        np.testing.assert_allclose(sc_cpu[r, : int(lim[r])], s[: int(lim[r])], rtol=2e-5, atol=2e-4)


def test_decode_full_size():
    import tilelang_ascend_b200 as dsa
    B, S_kv, H, topk = 64, 32768, 128, 2048
    g = torch.Generator(device=DEV).manual_seed(0)
    q = torch.randn((B, 1, H, 576), generator=g, device=DEV).to(torch.bfloat16)
    kv = torch.randn((B, S_kv, 1, 576), generator=g, device=DEV).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(S_kv, generator=g, device=DEV)[:topk] for _ in range(B)]).to(torch.int32).view(B, 1, 1, topk)
    out, lse = dsa.sparse_mla_fwd_raw(q, kv, idx, sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512)
    check_status()
    for b in (0, 17, 63):
        ro, rl = orc.sparse_mla_fwd(q[b:b + 1].cpu(), kv[b:b + 1].cpu(), idx[b:b + 1].cpu(), q_start_index_s=10 ** 9)
        assert_close_fp(out[b:b + 1].cpu(), ro, f"decode out {b}")
        assert_close_fp(lse[b:b + 1].cpu(), rl, f"decode lse {b}")
    # sharded by batch (8 "ranks"): identical to the unsharded call with one work unit per query; with 8 sequences on a
    # GPU the library splits every query's keys over several units, which changes the summation order only
    for rank in (0, 5):
        qs, kvs, ixs = dsa.shard_batch([q, kv, idx], rank, 8)
        s, e = dsa.shard_range(B, rank, 8)
        o, l = dsa.sparse_mla_fwd_raw(qs, kvs, ixs, sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512, nsplit=1)
        assert torch.equal(o, out[s:e]) and torch.equal(l, lse[s:e])
        o, l = dsa.sparse_mla_fwd_raw(qs, kvs, ixs, sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512)
        check_status()
        assert_close_fp(o.cpu(), out[s:e].cpu(), f"split-KV decode out, shard {rank}")
        assert_close_fp(l.cpu(), lse[s:e].cpu(), f"split-KV decode lse, shard {rank}")


def test_backward_prefill_shape_properties():
    import tilelang_ascend_b200 as dsa
    # the prefill shape of the backward configuration (tensor-core kernels)
    S, S_kv, H, topk = 4096, 4096, 128, 2048
    g = torch.Generator(device=DEV).manual_seed(0)
    q = torch.randn((1, S, H, 576), generator=g, device=DEV).to(torch.bfloat16)
    kv = torch.randn((1, S_kv, 1, 576), generator=g, device=DEV).to(torch.bfloat16)
    d_out = torch.randn((1, S, H, 512), generator=g, device=DEV).to(torch.bfloat16)
    idx = _causal_indices(S, S_kv, topk, g)
    scale, qs = 576 ** -0.5, S_kv - S
    out, lse = dsa.sparse_mla_fwd_raw(q, kv, idx, sm_scale=scale, q_start=qs, causal=True, dv=512)
    d_q, d_kv = dsa.sparse_mla_bwd_raw(q, kv, idx, out, lse, d_out, sm_scale=scale, q_start=qs, causal=True)
    check_status()
    # dQ of a query depends on that query only: oracle on two sampled queries
    for r in (0, 1000, S - 1):
        ref_dq, _ = orc.sparse_mla_bwd(q[:, r:r + 1].cpu(), kv.cpu(), idx[:, r:r + 1].cpu(), d_out[:, r:r + 1].cpu(), q_start_index_s=qs + r)
        assert_close_fp(d_q[:, r:r + 1].cpu(), ref_dq, f"dQ row {r}")
    # dKV is additive over queries: the two halves sum to the whole (fp32 atomics: order-dependent rounding only)
    halves = []
    for sl, start in ((slice(0, S // 2), qs), (slice(S // 2, S), qs + S // 2)):
        _, dk = dsa.sparse_mla_bwd_raw(q[:, sl].contiguous(), kv, idx[:, sl].contiguous(), out[:, sl].contiguous(), lse[:, sl].contiguous(),
                                       d_out[:, sl].contiguous(), sm_scale=scale, q_start=start, causal=True)
        halves.append(dk)
    torch.testing.assert_close(halves[0] + halves[1], d_kv, rtol=1e-3, atol=5e-2)
    # and the oracle on a small query block (the last four queries: 2048 keys each) pins its values
    sl = slice(S - 4, S)
    _, ref_dkv = orc.sparse_mla_bwd(q[:, sl].cpu(), kv.cpu(), idx[:, sl].cpu(), d_out[:, sl].cpu(), q_start_index_s=qs + S - 4)
    _, dk4 = dsa.sparse_mla_bwd_raw(q[:, sl].contiguous(), kv, idx[:, sl].contiguous(), out[:, sl].contiguous(), lse[:, sl].contiguous(),
                                    d_out[:, sl].contiguous(), sm_scale=scale, q_start=qs + S - 4, causal=True)
    assert_close_fp(dk4.cpu(), ref_dkv, "dKV of 4 queries", atol=1e-1)
    # the tensor-core and the CUDA-core kernels agree on a block of queries
    sl = slice(2000, 2064)
    args = (q[:, sl].contiguous(), kv, idx[:, sl].contiguous(), out[:, sl].contiguous(), lse[:, sl].contiguous(), d_out[:, sl].contiguous())
    dq_t, dk_t = dsa.sparse_mla_bwd_raw(*args, sm_scale=scale, q_start=qs + 2000, causal=True, impl="tensor_core")
    dq_c, dk_c = dsa.sparse_mla_bwd_raw(*args, sm_scale=scale, q_start=qs + 2000, causal=True, impl="cuda_core")
    check_status()
    assert_close_fp(dq_t.float().cpu(), dq_c.float().cpu(), "dQ tensor-core vs CUDA-core")
    assert_close_fp(dk_t.cpu(), dk_c.cpu(), "dKV tensor-core vs CUDA-core", atol=5e-2)


@pytest.mark.parametrize("name,B,S,S_kv,q_start", [
    ("base_example", 1, 128, 32768, 28672),        # example_sparse_flash_attn.py:295-326
    ("dynamic_shape", 2, 273, 44444, 28672),       # example_sparse_flash_attn_dynamic_shape.py:341-373
    ("mask_from_zero", 1, 1024, 32768, 0),         # example_sparse_flash_attn_mask.py:350-383 (query t sees keys 0..t)
])
def test_reference_example_shapes(name, B, S, S_kv, q_start):
    """The shapes the reference's own example scripts pin (H=128, D=576, topk=2048, bf16, padding sentinel S_kv, index lists
    drawn as randperm(max(1, t + q_start))[:topk]); sampled rows against the oracle with the scripts' rtol = atol = 1e-2."""
    import tilelang_ascend_b200 as dsa
    H, topk = 128, 2048
    g = torch.Generator().manual_seed(0)
    q = torch.randn((B, S, H, 576), generator=g).to(torch.bfloat16)
    kv = torch.randn((B, S_kv, 1, 576), generator=g).to(torch.bfloat16)
    idx = torch.full((B, S, 1, topk), S_kv, dtype=torch.int32)
    for b in range(B):
        for t in range(S):
            sel = torch.randperm(max(1, t + q_start), generator=g)[:topk]
            idx[b, t, 0, :len(sel)] = sel.to(torch.int32)
    kernel = dsa.sparse_attention_fwd(H, 512, 64, topk, 1, return_softmax_lse=True)
    out, lse = kernel(q.to(DEV), kv.to(DEV), idx.to(DEV), q_start_index_s=q_start)
    check_status()
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    rows = sorted(set([0, 1, 2, 63, 64, 65, S // 2, S - 2, S - 1]))
    for b in range(B):
        for r in rows:
            ro, rl = orc.sparse_mla_fwd(q[b:b + 1, r:r + 1], kv[b:b + 1], idx[b:b + 1, r:r + 1], q_start_index_s=q_start + r)
            torch.testing.assert_close(out[b:b + 1, r:r + 1].float().cpu(), ro, rtol=1e-2, atol=1e-2)
            assert_close_fp(lse[b:b + 1, r:r + 1].cpu(), rl, f"{name} lse row {r}")


@pytest.mark.parametrize("world", [2, 8])
def test_cost_balanced_query_shards_reassemble_bit_exactly(world):
    """The multi-GPU partition on one GPU: every rank's block of the prefill workload (cut where the cost model says the
    work is equal) is run in turn with its own q_start, and the concatenation must equal the unsharded call bit for bit --
    per-query results do not depend on which other queries share the launch."""
    import tilelang_ascend_b200 as dsa
    S = S_kv = 4096
    H, topk = 128, 2048
    g = torch.Generator(device=DEV).manual_seed(3)
    q = torch.randn((1, S, H, 576), generator=g, device=DEV).to(torch.bfloat16)
    kv = torch.randn((1, S_kv, 1, 576), generator=g, device=DEV).to(torch.bfloat16)
    idx = _causal_indices(S, S_kv, topk, g)
    kernel = dsa.sparse_attention_fwd(H, 512, 64, topk, 1, return_softmax_lse=True)
    out, lse = kernel(q, kv, idx)
    costs = dsa.causal_query_costs(S, S_kv, topk)
    # the partition by summed cost, and the one the bench uses (equal time in rounds of one query per SM pair)
    for pairs in (0, 74):
        spans = dsa.shard_ranges_by_rounds(costs, world, pairs) if pairs else [dsa.shard_range_balanced(costs, r, world) for r in range(world)]
        outs, lses, loads, prev = [], [], [], 0
        for r in range(world):
            qs, ix, q0 = dsa.shard_queries(q, idx, r, world, s_kv=S_kv, balance=True, units_per_round=pairs)
            s, e = spans[r]
            assert s == prev and q0 == s and qs.shape[1] == e - s
            prev = e
            loads.append(int(costs[s:e].sum()))
            o, l = kernel(qs, kv, ix, q_start_index_s=q0)
            outs.append(o)
            lses.append(l)
        check_status()
        assert prev == S
        if not pairs:
            assert max(loads) <= 1.01 * sum(loads) / world
        assert torch.equal(torch.cat(outs, 1), out) and torch.equal(torch.cat(lses, 1), lse)
    # the partition with split last rounds: rows of a block's split tail within tolerance, all others bit-equal
    spans = dsa.shard_ranges_by_rounds(costs, world, 74, tail_split=True)
    for s, e in spans:
        m, n, _ = dsa.tail_split_plan(costs, s, e, 74)
        o, l = kernel(q[:, s:e].contiguous(), kv, idx[:, s:e].contiguous(), q_start_index_s=s, split_tail=(m, n))
        check_status()
        cut = m if n > 1 else 0
        assert torch.equal(o[:, cut:], out[:, s + cut:e]) and torch.equal(l[:, cut:], lse[:, s + cut:e])
        if cut:
            assert (o[:, :cut].float() - out[:, s:s + cut].float()).abs().max().item() <= 2e-2
            assert (l[:, :cut] - lse[:, s:s + cut]).abs().max().item() <= 1e-3
