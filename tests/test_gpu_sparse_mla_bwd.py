"""Sparse MLA backward on the GPU against autograd through the fp32 oracle forward."""
import pytest
import torch

from gpu_util import assert_close_fp, check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("impl", ["tensor_core", "cuda_core"])
@pytest.mark.parametrize("B,S,S_kv,H,topk", [(1, 8, 96, 16, 32), (2, 5, 300, 128, 64), (1, 3, 64, 7, 40)])
def test_backward_matches_autograd_oracle(B, S, S_kv, H, topk, impl):
    import tilelang_ascend_b200 as dsa
    q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, seed=S)
    g = torch.Generator().manual_seed(1)
    d_out = torch.randn((B, S, H, 512), generator=g).to(torch.bfloat16)
    scale = 576 ** -0.5
    qc, kvc, ic = q.cuda(), kv.cuda(), idx.cuda()
    out, lse = dsa.sparse_mla_fwd_raw(qc, kvc, ic, sm_scale=scale, q_start=S_kv - S, causal=True, dv=512)
    d_q, d_kv = dsa.sparse_mla_bwd_raw(qc, kvc, ic, out, lse, d_out.cuda(), sm_scale=scale, q_start=S_kv - S, causal=True, impl=impl)
    check_status()
    ref_dq, ref_dkv = orc.sparse_mla_bwd(q, kv, idx, d_out)
    # dKV sums H * (queries that picked the key) terms: scale the absolute tolerance with that count
    assert_close_fp(d_q.cpu(), ref_dq, "dQ")
    assert_close_fp(d_kv.cpu(), ref_dkv, "dKV", atol=2e-2 * max(1.0, (H * S / 16) ** 0.5))


def test_autograd_function():
    import tilelang_ascend_b200 as dsa
    q, kv, idx = orc.make_sparse_mla_inputs(1, 4, 128, 16, 32, seed=3)
    qc = q.cuda().requires_grad_(True)
    kvc = kv.cuda().requires_grad_(True)
    out, lse = dsa.sparse_mla(qc, kvc, idx.cuda())
    d_out = torch.randn_like(out)
    out.backward(d_out)
    check_status()
    ref_dq, ref_dkv = orc.sparse_mla_bwd(q, kv, idx, d_out.cpu())
    assert_close_fp(qc.grad.cpu(), ref_dq, "dQ")
    assert_close_fp(kvc.grad.cpu(), ref_dkv, "dKV", atol=4e-2)


@pytest.mark.parametrize("B,S,S_kv,H,topk,qpp", [
    (1, 6, 700, 128, 448, 4),     # 7 tiles (odd count), two passes, ring buffers wrap
    (1, 5, 40, 128, 192, 2),      # more slots than keys: tiles without any key are skipped, early queries nearly empty
    (2, 3, 520, 200, 320, 0),     # two head blocks, the second partly filled
    (1, 2, 3000, 128, 2112, 0),   # more than 2048 slots: the index list stays in global memory; 33 tiles
])
def test_tensor_core_backward_passes_and_tiles(B, S, S_kv, H, topk, qpp):
    """Tensor-core backward: several passes through a small workspace, many key tiles, skipped tiles, padded head blocks."""
    import tilelang_ascend_b200 as dsa
    q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, seed=topk)
    g = torch.Generator().manual_seed(2)
    d_out = torch.randn((B, S, H, 512), generator=g).to(torch.bfloat16)
    scale = 576 ** -0.5
    qc, kvc, ic = q.cuda(), kv.cuda(), idx.cuda()
    out, lse = dsa.sparse_mla_fwd_raw(qc, kvc, ic, sm_scale=scale, q_start=S_kv - S, causal=True, dv=512)
    d_q, d_kv = dsa.sparse_mla_bwd_raw(qc, kvc, ic, out, lse, d_out.cuda(), sm_scale=scale, q_start=S_kv - S, causal=True,
                                       impl="tensor_core", queries_per_pass=qpp or None)
    check_status()
    ref_dq, ref_dkv = orc.sparse_mla_bwd(q, kv, idx, d_out)
    assert_close_fp(d_q.cpu(), ref_dq, "dQ")
    assert_close_fp(d_kv.cpu(), ref_dkv, "dKV", atol=2e-2 * max(1.0, (H * S / 16) ** 0.5))


def test_tensor_core_backward_rejects_other_shapes():
    import tilelang_ascend_b200 as dsa
    q = torch.zeros((1, 2, 4, 128), dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros((1, 16, 1, 128), dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros((1, 2, 1, 8), dtype=torch.int32, device="cuda")
    out = torch.zeros((1, 2, 4, 128), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((1, 2, 4), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        dsa.sparse_mla_bwd_raw(q, kv, idx, out, lse, out, sm_scale=0.1, q_start=14, causal=True, impl="tensor_core")


def test_tensor_core_backward_fp16():
    import tilelang_ascend_b200 as dsa
    B, S, S_kv, H, topk = 1, 4, 200, 128, 128
    q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, seed=9, dtype=torch.float16)
    g = torch.Generator().manual_seed(4)
    d_out = torch.randn((B, S, H, 512), generator=g).to(torch.float16)
    scale = 576 ** -0.5
    qc, kvc, ic = q.cuda(), kv.cuda(), idx.cuda()
    out, lse = dsa.sparse_mla_fwd_raw(qc, kvc, ic, sm_scale=scale, q_start=S_kv - S, causal=True, dv=512)
    d_q, d_kv = dsa.sparse_mla_bwd_raw(qc, kvc, ic, out, lse, d_out.cuda(), sm_scale=scale, q_start=S_kv - S, causal=True, impl="tensor_core")
    check_status()
    ref_dq, ref_dkv = orc.sparse_mla_bwd(q, kv, idx, d_out)
    assert_close_fp(d_q.cpu(), ref_dq, "dQ fp16")
    assert_close_fp(d_kv.cpu(), ref_dkv, "dKV fp16", atol=2e-2 * max(1.0, (H * S / 16) ** 0.5))
