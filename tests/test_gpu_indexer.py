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


def _build_paged(k: torch.Tensor, act_k, block_size: int, block_num: int, seed: int = 42):
    """Scatter BSND keys [B, S2, 1, D] into a paged cache [block_num, block_size, 1, D] with a shuffled block table whose
    unused entries are -1 (the construction of the reference's own examples,
    examples/deepseek_v4/lightning_indexer.py:1505-1533)."""
    B, S2, _, D = k.shape
    cols = -(-S2 // block_size)
    perm = np.random.default_rng(seed).permutation(block_num)
    bt = np.full((B, max(cols, 1)), -1, dtype=np.int32)
    cache = torch.zeros((block_num, block_size, 1, D), dtype=k.dtype)
    c = 0
    for b in range(B):
        for i in range(-(-int(act_k[b]) // block_size)):
            bt[b, i] = perm[c]
            s0, s1 = i * block_size, min((i + 1) * block_size, int(act_k[b]))
            cache[perm[c], : s1 - s0] = k[b, s0:s1]
            c += 1
    return cache, torch.from_numpy(bt)


@pytest.mark.parametrize("block_size,N1,no_tma", [(128, 64, False), (256, 32, False), (48, 16, False), (16, 8, False),
                                                  (128, 64, True), (80, 16, True), (64, 5, False)])
def test_paged_keys_match_dense_keys(block_size, N1, no_tma, monkeypatch):
    """layout_key="PA_BSND": the kernel walks the cache through the block table (TMA boxes inside a block, per-row copies
    when DSA_INDEXER_NO_TMA is set, CUDA cores for a head count the tensor-core kernel does not take); the result must be
    bit-equal to the dense-key call on the same logical keys, and equal to the oracle."""
    import tilelang_ascend_b200 as dsa
    if no_tma:
        monkeypatch.setenv("DSA_INDEXER_NO_TMA", "1")
    B, S1, S2, K = 2, 33, 1000, 256
    act_k = [1000, 517]
    q, k, w = orc.make_indexer_inputs(B, S1, S2, N1, 128, seed=block_size + N1)
    k[1, act_k[1]:] = 0
    nblk = sum(-(-a // block_size) for a in act_k) + 5
    cache, bt = _build_paged(k, act_k, block_size, nblk)
    aq = torch.tensor([S1, 20])
    ak = torch.tensor(act_k)
    dense_idx, _ = dsa.lightning_indexer(q.cuda(), k.cuda(), w.cuda(), actual_seq_lengths_query=aq, actual_seq_lengths_key=ak,
                                         sparse_count=K, sparse_mode=3)
    paged_idx, vals = dsa.lightning_indexer(q.cuda(), cache.cuda(), w.cuda(), actual_seq_lengths_query=aq, actual_seq_lengths_key=ak,
                                            block_table=bt.cuda(), layout_key="PA_BSND", sparse_count=K, sparse_mode=3)
    check_status()
    assert vals.numel() == 0
    assert torch.equal(paged_idx, dense_idx)
    ref = orc.lightning_indexer(q, k, w, sparse_count=K, sparse_mode=3, actual_seq_lengths_query=aq, actual_seq_lengths_key=ak).numpy()
    got = paged_idx.cpu().numpy()
    for b in range(B):
        sc = orc.indexer_scores(q[b:b + 1], k[b:b + 1], w[b:b + 1], sparse_mode=3, actual_q=int(aq[b]), actual_k=act_k[b])[0].numpy()
        n = int(aq[b])
        same, rows = topk_three_step(got[b, :n, 0], ref[b, :n, 0], sc, K)
        assert same >= rows - 1
        assert (got[b, n:] == -1).all()
    with pytest.raises(ValueError, match="return_value"):
        dsa.lightning_indexer(q.cuda(), cache.cuda(), w.cuda(), block_table=bt.cuda(), layout_key="PA_BSND", return_value=True)


def _uniform(shape, g, absolute=False):
    x = (torch.rand(shape, generator=g) * 2 - 1).half()
    return x.abs() if absolute else x


def test_reference_layout_scenarios():
    """The four layout scenarios the reference runs against its CPU golden (examples/deepseek_v4/lightning_indexer.py:1574-1647;
    fp16 uniform(-1, 1) inputs, non-negative weights), checked with the reference's 3-step rule against the oracle."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator().manual_seed(0)

    def check(idx, q, k, w, aq, ak, K, mode):
        ref = orc.lightning_indexer(q, k, w, sparse_count=K, sparse_mode=mode, actual_seq_lengths_query=aq, actual_seq_lengths_key=ak).numpy()
        for b in range(q.shape[0]):
            n = int(aq[b])
            sc = orc.indexer_scores(q[b:b + 1], k[b:b + 1], w[b:b + 1], sparse_mode=mode, actual_q=n, actual_k=int(ak[b]))[0].numpy()
            assert np.array_equal(idx[b, :n] < 0, ref[b, :n, 0] < 0)
            topk_three_step(idx[b, :n], ref[b, :n, 0], sc, K)

    # 1: BSND + BSND, B=2, S1=3, S2=32768, 64 heads, top 2048, causal
    B, S1, S2, N1, K = 2, 3, 32768, 64, 2048
    q, k, w = _uniform((B, S1, N1, 128), g), _uniform((B, S2, 1, 128), g), _uniform((B, S1, N1), g, True)
    idx, val = dsa.lightning_indexer(q.cuda(), k.cuda(), w.cuda(), actual_seq_lengths_query=torch.full((B,), S1), actual_seq_lengths_key=torch.full((B,), S2),
                                     sparse_count=K, sparse_mode=3, return_value=True)
    check(idx.cpu().numpy().reshape(B, S1, K), q, k, w.float(), [S1] * B, [S2] * B, K, 3)
    assert val.dtype == torch.float16 and val.numel() == B * S1 * K

    # 2: BSND + PA_BSND, B=2, S1=1, 8 heads, blocks of 128, 32 blocks, keys 1024 / 2048, all keys candidates
    B, S1, N1, K, bs, nb, act_k = 2, 1, 8, 2048, 128, 32, [1024, 2048]
    q, w, k = _uniform((B, S1, N1, 128), g), _uniform((B, S1, N1), g, True), _uniform((B, max(act_k), 1, 128), g)
    cache, bt = _build_paged(k, act_k, bs, nb)
    bt_full = torch.full((B, nb), -1, dtype=torch.int32)
    bt_full[:, :bt.shape[1]] = bt
    idx, _ = dsa.lightning_indexer(q.cuda(), cache.cuda(), w.cuda(), actual_seq_lengths_query=torch.full((B,), S1), actual_seq_lengths_key=torch.tensor(act_k),
                                   block_table=bt_full.cuda(), layout_key="PA_BSND", sparse_count=K, sparse_mode=0)
    check(idx.cpu().numpy().reshape(B, S1, K), q, k, w.float(), [S1] * B, act_k, K, 0)

    # 3: TND + TND, B=8, S1=64, S2=3072, 24 heads, all keys candidates
    B, S1, S2, N1 = 8, 64, 3072, 24
    q, k, w = _uniform((B * S1, N1, 128), g), _uniform((B * S2, 1, 128), g), _uniform((B * S1, N1), g, True)
    idx, _ = dsa.lightning_indexer(q.cuda(), k.cuda(), w.cuda(), actual_seq_lengths_query=torch.arange(1, B + 1) * S1,
                                   actual_seq_lengths_key=torch.arange(1, B + 1) * S2, layout_query="TND", layout_key="TND", sparse_count=K, sparse_mode=0)
    check(idx.cpu().numpy().reshape(B, S1, K), q.view(B, S1, N1, 128), k.view(B, S2, 1, 128), w.view(B, S1, N1).float(), [S1] * B, [S2] * B, K, 0)

    # 4: TND + PA_BSND, 8 heads, blocks of 128, queries 1024 / 2048 (here 96 / 160: the CPU oracle is the slow part), keys 4096 / 8192
    N1, bs, nb, act_q, act_k = 8, 128, 128, [96, 160], [4096, 8192]
    q, w, k = _uniform((sum(act_q), N1, 128), g), _uniform((sum(act_q), N1), g, True), _uniform((2, max(act_k), 1, 128), g)
    cache, bt = _build_paged(k, act_k, bs, nb)
    idx, _ = dsa.lightning_indexer(q.cuda(), cache.cuda(), w.cuda(), actual_seq_lengths_query=torch.tensor(act_q).cumsum(0),
                                   actual_seq_lengths_key=torch.tensor(act_k), block_table=bt.cuda(), layout_query="TND", layout_key="PA_BSND",
                                   sparse_count=K, sparse_mode=0)
    idx = idx.cpu().numpy().reshape(sum(act_q), K)
    qp, wp = torch.zeros((2, max(act_q), N1, 128), dtype=torch.float16), torch.zeros((2, max(act_q), N1))
    qp[0, :96], qp[1] = q[:96], q[96:]
    wp[0, :96], wp[1] = w[:96].float(), w[96:].float()
    ip = np.full((2, max(act_q), K), -1, dtype=np.int32)
    ip[0, :96], ip[1] = idx[:96], idx[96:]
    check(ip, qp, k, wp, act_q, act_k, K, 0)
    check_status()


@pytest.mark.parametrize("B,S1,S2,K,mode", [(2, 50, 300, 64, 3), (1, 33, 200, 16, 0), (1, 64, 64, 32, 3)])
def test_fused_call_over_query_blocks_gives_the_same_arrays(B, S1, S2, K, mode):
    """A fused scores + top-k call whose score matrix exceeds the workspace limit runs over blocks of queries, each with the
    lengths that keep its queries' causal limits: index and value arrays equal the one-piece call's bit for bit."""
    import tilelang_ascend_b200 as dsa
    q, k, w = orc.make_indexer_inputs(B, S1, S2, seed=S1)
    whole_i, whole_v = dsa.lightning_indexer_raw(q.cuda(), k.cuda(), w.cuda(), sparse_count=K, sparse_mode=mode, return_value=True)
    for limit in (B * S2 * 4 * 7, B * S2 * 4):            # blocks of 7 queries / of a single query
        part_i, part_v = dsa.lightning_indexer_raw(q.cuda(), k.cuda(), w.cuda(), sparse_count=K, sparse_mode=mode, return_value=True,
                                                   max_workspace_bytes=limit)
        check_status()
        assert torch.equal(part_i, whole_i) and torch.equal(part_v, whole_v)


def test_long_key_cache_131072_keys():
    """The token-level indexer at the key count of HISA's default shape: 131072 keys per row do not fit the selector's shared
    memory (rows are streamed) and 256 x 131072 scores are 128 MB; sampled rows against the CPU oracle (index sets; the scores
    of the kept keys to rtol 2e-5)."""
    import tilelang_ascend_b200 as dsa
    B, S1, S2, K = 1, 256, 131072, 2048
    q, k, w = orc.make_indexer_inputs(B, S1, S2, seed=77)
    idx, val = dsa.lightning_indexer_raw(q.cuda(), k.cuda(), w.cuda(), sparse_count=K, sparse_mode=3, return_value=True,
                                         max_workspace_bytes=64 << 20)   # forces two blocks of queries
    check_status()
    idx, val = idx.cpu(), val.cpu()
    for t in (0, 100, 255):
        sc = orc.indexer_scores(q[:, t:t + 1], k, w[:, t:t + 1])[0, 0]               # [S2] fp32 of this query
        lim = S2 - S1 + t + 1
        ref_i, ref_v = orc.topk_select(sc[None, :].numpy(), K, limits=np.array([lim], dtype=np.int32), return_values=True)
        got = idx[0, t, 0].numpy()
        assert set(got.tolist()) == set(ref_i[0].tolist())
        np.testing.assert_allclose(val[0, t, 0].numpy(), ref_v[0], rtol=2e-5, atol=2e-4)
