"""Lightning indexer on the GPU against the reference fixtures and the oracle."""
import numpy as np
import pytest
import torch

from conftest import from_bits
from gpu_util import check_status, topk_three_step
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu


def _scores_close(got: np.ndarray, ref: np.ndarray):
    fin = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), fin), "masked (-inf) pattern differs"
    # bf16 x bf16 products are exact in fp32; only the summation order differs from the CPU einsum
    np.testing.assert_allclose(got[fin], ref[fin], rtol=2e-5, atol=2e-4)


@pytest.mark.parametrize("tag", ["causal", "full", "ties"])
def test_reference_golden_fixture(golden, tag):
    import tilelang_ascend_b200 as dsa
    g = golden("lightning_indexer.npz")
    q, k, w = from_bits(g[f"{tag}_q"]), from_bits(g[f"{tag}_k"]), torch.from_numpy(g[f"{tag}_w"])
    aq, ak, mode, K = g[f"{tag}_aq"], g[f"{tag}_ak"], int(g[f"{tag}_mode"]), int(g[f"{tag}_K"])
    idx, val = dsa.lightning_indexer(q.cuda(), k.cuda(), w.cuda(), actual_seq_lengths_query=torch.from_numpy(aq),
                                     actual_seq_lengths_key=torch.from_numpy(ak), sparse_count=K, sparse_mode=mode,
                                     return_value=True)
    check_status()
    B, S1 = q.shape[0], q.shape[1]
    idx = idx.cpu().numpy().reshape(B, S1, K)
    ref = g[f"{tag}_idx"].reshape(B, S1, K)
    ref_scores = g[f"{tag}_scores"]
    for b in range(B):
        a_q, a_k = int(aq[b]), int(ak[b])
        sc = dsa.indexer_scores_raw(q[b:b + 1, :a_q].cuda().contiguous(), k[b:b + 1, :a_k].cuda().contiguous(),
                                    w[b:b + 1, :a_q].cuda().contiguous(), sparse_mode=mode)
        _scores_close(sc[0].cpu().numpy(), ref_scores[b, 0, :a_q, :a_k])
        assert np.array_equal(idx[b, a_q:], ref[b, a_q:])  # padding rows stay -1
        # -1 pattern (rows with fewer than K candidates) must agree exactly
        assert np.array_equal(idx[b, :a_q] < 0, ref[b, :a_q] < 0)
        same, rows = topk_three_step(idx[b, :a_q], ref[b, :a_q], ref_scores[b, 0, :a_q, :a_k], K)
        if tag != "ties":
            assert same == rows, f"{rows - same} of {rows} rows differ as sets"
    assert val.dtype == q.dtype


def test_selector_on_oracle_scores_is_bit_exact():
    # identical fp32 scores in -> identical index arrays out (the bit-exact claim of the path)
    import tilelang_ascend_b200 as dsa
    q, k, w = orc.make_indexer_inputs(1, 64, 2048, 64, 128, seed=5)
    sc = orc.indexer_scores(q, k, w, sparse_mode=3)[0]
    lim = orc.causal_limits(64, 2048)
    got = dsa.topk_select_raw(sc.cuda().contiguous(), 512, torch.from_numpy(lim).cuda()).cpu().numpy()
    check_status()
    assert np.array_equal(got, orc.topk_select(sc.numpy(), 512, lim))


@pytest.mark.parametrize("N1", [64, 32, 16, 8, 5])
def test_scores_and_topk_match_oracle(N1):
    import tilelang_ascend_b200 as dsa
    B, S1, S2, K = 2, 37, 700, 128
    q, k, w = orc.make_indexer_inputs(B, S1, S2, N1, 128, seed=N1)
    sc = dsa.indexer_scores_raw(q.cuda(), k.cuda(), w.cuda(), sparse_mode=3)
    idx, _ = dsa.lightning_indexer(q.cuda(), k.cuda(), w.cuda(), sparse_count=K, sparse_mode=3)
    check_status()
    ref_sc = orc.indexer_scores(q, k, w, sparse_mode=3)
    _scores_close(sc.cpu().numpy(), ref_sc.numpy())
    ref_idx = orc.lightning_indexer(q, k, w, sparse_count=K, sparse_mode=3).numpy()
    got = idx.cpu().numpy()
    for b in range(B):
        same, rows = topk_three_step(got[b, :, 0], ref_idx[b, :, 0], ref_sc[b].numpy(), K)
        assert same >= rows - 1


def test_simple_indexer_factory(golden):
    import tilelang_ascend_b200 as dsa
    g = golden("simple_indexer.npz")
    q, k = from_bits(g["q"], torch.float16), from_bits(g["k"], torch.float16)
    w = torch.from_numpy(g["w"])
    B, S1, N2, G, D = q.shape
    S2, K = k.shape[1], g["indices"].shape[-1]
    kernel = dsa.indexer(B, N2, G, S1, S2, D, K, 256, 16, 64, 64, 64)
    out = kernel(q.view(B, S1, N2, G * D).cuda(), k.cuda(), w.view(B, S1, N2, G).cuda().contiguous())
    check_status()
    assert tuple(out.shape) == (B, N2, S1, K) and out.dtype == torch.int32
    got, ref = out.cpu().numpy()[0, 0], g["indices"][0, 0]
    same = sum(len(set(got[r]) & set(ref[r])) for r in range(S1)) / ref.size
    assert same > 0.99  # the reference's own bar (its golden accumulates q.k in fp16)


def test_wrapper_validation_and_early_exit():
    import tilelang_ascend_b200 as dsa
    q, k, w = orc.make_indexer_inputs(1, 4, 64, 8, 128, seed=0)
    q, k, w = q.cuda(), k.cuda(), w.cuda()
    with pytest.raises(ValueError):
        dsa.lightning_indexer(q, k, w, sparse_count=3000)
    with pytest.raises(ValueError):
        dsa.lightning_indexer(q, k, w, sparse_mode=1)
    with pytest.raises(ValueError):
        dsa.lightning_indexer(q, k.half(), w)
    with pytest.raises(ValueError):
        dsa.lightning_indexer(q, k, w, layout_query="TND")
    idx, val = dsa.lightning_indexer(q, k, w, sparse_count=16, actual_seq_lengths_query=torch.tensor([0]))
    assert tuple(idx.shape) == (4, 1, 16) and bool((idx == -1).all()) and val.numel() == 0


def test_tnd_layout_matches_bsnd():
    import tilelang_ascend_b200 as dsa
    q, k, w = orc.make_indexer_inputs(2, 6, 150, 16, 128, seed=9)
    ql, kl = [6, 4], [150, 90]
    q_t = torch.cat([q[0, :6], q[1, :4]]).cuda()
    w_t = torch.cat([w[0, :6], w[1, :4]]).cuda()
    k_t = torch.cat([k[0, :150], k[1, :90]]).cuda()
    idx_t, _ = dsa.lightning_indexer(q_t, k_t, w_t, actual_seq_lengths_query=torch.tensor([6, 10]),
                                     actual_seq_lengths_key=torch.tensor([150, 240]), layout_query="TND", layout_key="TND",
                                     sparse_count=32)
    idx_b, _ = dsa.lightning_indexer(q.cuda(), k.cuda(), w.cuda(), actual_seq_lengths_query=torch.tensor(ql),
                                     actual_seq_lengths_key=torch.tensor(kl), sparse_count=32)
    check_status()
    assert torch.equal(idx_t[:6], idx_b[0, :6]) and torch.equal(idx_t[6:], idx_b[1, :4])


def test_tma_and_cp_async_key_tiles_agree(monkeypatch):
    """The tensor-core score kernel fetches key tiles with TMA tile loads; its cp.async producers (used when no tensor
    map can be made for k) must give bit-identical scores.  Two batch entries, so that a key tile of the first entry
    reaches into the rows of the second one, and actual lengths shorter than the tensors."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator().manual_seed(5)
    B, S1, S2, N1 = 2, 96, 1000, 64
    q = torch.randn((B, S1, N1, 128), generator=g).to(torch.bfloat16).cuda()
    k = torch.randn((B, S2, 1, 128), generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn((B, S1, N1), generator=g) / 8).float().cuda()
    a = dsa.indexer_scores_raw(q, k, w, sparse_mode=3)
    check_status()
    monkeypatch.setenv("DSA_INDEXER_NO_TMA", "1")
    b = dsa.indexer_scores_raw(q, k, w, sparse_mode=3)
    check_status()
    assert torch.equal(torch.isfinite(a), torch.isfinite(b))
    fin = torch.isfinite(a)
    assert torch.equal(a[fin], b[fin])
    ref = orc.indexer_scores(q.cpu(), k.cpu(), w.cpu(), sparse_mode=3)
    _scores_close(a.cpu().numpy(), ref.numpy() if hasattr(ref, "numpy") else np.asarray(ref))
