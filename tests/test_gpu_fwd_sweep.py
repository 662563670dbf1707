"""Seeded sweep of the sparse MLA forward over shapes the fixed cases do not visit: head counts around the 64 / 128
boundaries of the SM-pair kernel, list lengths that are not multiples of the 64-key tile, short key caches, several
batches, both dtypes, padding sentinels in random places, q_start offsets and split-KV -- each against the fp32 oracle."""
import numpy as np
import pytest
import torch

from gpu_util import assert_close_fp, check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu


def _cases():
    rng = np.random.default_rng(2025)
    cases = []
    for i in range(28):
        H = int(rng.choice([1, 8, 16, 31, 64, 65, 96, 127, 128, 130, 192, 256]))
        topk = int(rng.choice([1, 7, 63, 64, 65, 128, 200, 320, 511, 1024]))
        S_kv = int(rng.choice([topk, topk + 1, 2 * topk + 3, 700, 1500]))
        S_kv = max(S_kv, 2)
        S = int(rng.integers(1, 7))
        B = int(rng.integers(1, 4))
        dtype = torch.bfloat16 if rng.random() < 0.7 else torch.float16
        nsplit = int(rng.choice([0, 0, 1, 2, 3, 7]))
        pad = int(rng.choice([-1, S_kv]))
        cases.append((i, B, S, S_kv, H, topk, dtype, nsplit, pad))
    return cases


@pytest.mark.parametrize("case", _cases(), ids=lambda c: f"{c[0]}-B{c[1]}S{c[2]}kv{c[3]}H{c[4]}k{c[5]}n{c[7]}")
def test_forward_sweep(case):
    import tilelang_ascend_b200 as dsa
    i, B, S, S_kv, H, topk, dtype, nsplit, pad = case
    S = min(S, S_kv)
    q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, min(topk, S_kv), seed=100 + i, dtype=dtype, pad=pad)
    if idx.shape[-1] < topk:  # lists longer than the cache: the tail is padding
        idx = torch.cat([idx, torch.full(idx.shape[:-1] + (topk - idx.shape[-1],), pad, dtype=idx.dtype)], dim=-1)
    rng = np.random.default_rng(i)
    holes = torch.from_numpy(rng.random(tuple(idx.shape)) < 0.1)   # padding in random places, not only at the end
    idx = torch.where(holes, torch.full_like(idx, pad), idx)
    kw = {} if nsplit == 0 else {"nsplit": nsplit}
    out, lse = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=S_kv - S, causal=True, dv=512, **kw)
    check_status()
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(out.cpu(), ref_o, f"out (case {case})")
    assert_close_fp(lse.cpu(), ref_l, f"lse (case {case})")
    # the CUDA-core kernel on the same inputs
    gen_o, gen_l = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=S_kv - S, causal=True, dv=512, impl=1)
    check_status()
    assert_close_fp(gen_o.cpu(), ref_o, "CUDA-core kernel out")
    assert_close_fp(gen_l.cpu(), ref_l, "CUDA-core kernel lse")
