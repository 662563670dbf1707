"""DeepSeek-V4 sparse_flash_mla front door (window + compressed tokens + sinks) on the GPU against the oracle."""
import numpy as np
import pytest
import torch

from gpu_util import assert_close_fp, check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu


def _paged(dense: torch.Tensor, block_size: int, rng) -> tuple:
    """[B, S, D] -> (pool [blocks, block_size, 1, D] with the sequences' blocks shuffled, block table [B, n])."""
    B, S, D = dense.shape
    n = (S + block_size - 1) // block_size
    perm = rng.permutation(B * n + 2)[: B * n]          # two blocks of the pool stay unused
    pool = torch.zeros((B * n + 2, block_size, 1, D), dtype=dense.dtype)
    table = torch.from_numpy(perm.reshape(B, n).astype(np.int32))
    for b in range(B):
        for j in range(n):
            chunk = dense[b, j * block_size:(j + 1) * block_size]
            pool[int(table[b, j]), : chunk.shape[0], 0] = chunk
    return pool, table


def _case(seed, B, S, S_kv, N1, D, K, ratio, act_q, act_kv):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, S, N1, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, S_kv, D), generator=g).to(torch.bfloat16)
    c = torch.randn((B, S_kv // ratio, D), generator=g).to(torch.bfloat16)
    sinks = torch.randn((N1,), generator=g)
    rng = np.random.default_rng(seed)
    ci = np.full((B, S, 1, K), -1, dtype=np.int32)
    for b in range(B):
        for s in range(act_q[b]):
            n = int(rng.integers(0, K + 1))
            ci[b, s, 0, :n] = rng.choice(S_kv // ratio, size=n, replace=False) if n <= S_kv // ratio else rng.integers(0, S_kv // ratio, size=n)
    return q, k, c, sinks, torch.from_numpy(ci), rng


@pytest.mark.parametrize("scenario", [1, 2, 3])
@pytest.mark.parametrize("layout", ["TND", "BSND"])
def test_sparse_flash_mla_matches_oracle(scenario, layout):
    import tilelang_ascend_b200 as dsa
    B, S, S_kv, N1, D, K, ratio, win = 2, 9, 300, 64, 512, 32, 4, 127
    act_q, act_kv = [9, 5], [300, 171]
    q, k, c, sinks, ci, rng = _case(scenario, B, S, S_kv, N1, D, K, ratio, act_q, act_kv)
    scale = D ** -0.5
    kw = {}
    if scenario >= 2:
        kw.update(cmp_k=c, cmp_ratio=ratio)
    if scenario == 3:
        kw.update(cmp_sparse_indices=ci[:, :, 0, :])
    ref_out, ref_lse = orc.sparse_flash_mla_v4(q, k, sinks, act_q_lens=act_q, act_kv_lens=act_kv, softmax_scale=scale, ori_win_left=win, **kw)

    ori_pool, ori_bt = _paged(k, 128, rng)
    cmp_pool, cmp_bt = _paged(c, 16, rng)
    cu = torch.tensor([0, act_q[0], act_q[0] + act_q[1]], dtype=torch.int32)
    args = dict(ori_kv=ori_pool.cuda(), ori_block_table=ori_bt.cuda(), seqused_kv=torch.tensor(act_kv, dtype=torch.int32).cuda(), sinks=sinks.cuda(),
                softmax_scale=scale, ori_win_left=win, layout_q=layout, return_softmax_lse=True, cu_seqlens_q=cu.cuda())
    if scenario >= 2:
        args.update(cmp_kv=cmp_pool.cuda(), cmp_block_table=cmp_bt.cuda(), cmp_ratio=ratio)
    if layout == "TND":
        q_in = torch.cat([q[b, : act_q[b]] for b in range(B)]).cuda()
        if scenario == 3:
            args.update(cmp_sparse_indices=torch.cat([ci[b, : act_q[b]] for b in range(B)]).cuda())
        out, lse = dsa.sparse_flash_mla(q_in, **args)
        check_status()
        ref_o = torch.cat([ref_out[b, : act_q[b]] for b in range(B)])
        ref_l = torch.cat([ref_lse[b, : act_q[b]] for b in range(B)])
    else:
        if scenario == 3:
            args.update(cmp_sparse_indices=ci.cuda())
        out, lse = dsa.sparse_flash_mla(q.cuda(), **args)
        check_status()
        ref_o, ref_l = ref_out, ref_lse       # rows beyond a sequence's length are zero on both sides
    assert_close_fp(out.cpu(), ref_o, f"out, scenario {scenario} {layout}")
    assert_close_fp(lse.cpu(), ref_l, f"lse, scenario {scenario} {layout}")


def test_sink_combine_single_partial_without_sink_is_identity():
    import tilelang_ascend_b200 as dsa
    g = torch.Generator().manual_seed(0)
    out = torch.randn((5, 8, 64), generator=g).to(torch.bfloat16).cuda()
    lse = torch.randn((5, 8), generator=g).cuda()
    o2, l2 = dsa.sink_combine_raw(out, lse, None, None, None, 8)
    assert torch.equal(o2, out) and torch.allclose(l2, lse, rtol=1e-6, atol=1e-6)
