"""Top-k selector on the GPU against the oracle: bit-exact index arrays."""
import numpy as np
import pytest
import torch

from gpu_util import check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu


def _run(x: np.ndarray, k: int, limits=None, values=False):
    import tilelang_ascend_b200 as dsa
    xs = torch.from_numpy(x).cuda()
    lim = None if limits is None else torch.from_numpy(np.asarray(limits, dtype=np.int32)).cuda()
    out = dsa.topk_select_raw(xs, k, lim, return_values=values)
    check_status()
    return (out[0].cpu().numpy(), out[1].cpu().numpy()) if values else out.cpu().numpy()


def test_fixture_from_reference_topk(golden):
    g = golden("topk_selector.npz")
    assert np.array_equal(_run(g["x"], g["indices"].shape[1]), g["indices"])


@pytest.mark.parametrize("B,N,K", [(64, 4096, 2048), (1024, 1024, 128), (7, 8192, 2048), (3, 1000, 1000), (5, 33, 1),
                                   (2, 32768, 2048), (4, 5000, 4096), (3, 8192, 8192), (3, 500, 64), (3, 500, 65), (2, 3000, 2049)])
def test_random_rows_match_oracle(B, N, K):
    rng = np.random.default_rng(B * 131 + N)
    x = rng.standard_normal((B, N)).astype(np.float32)
    idx, val = _run(x, K, values=True)
    ref_i, ref_v = orc.topk_select(x, K, return_values=True)
    assert np.array_equal(idx, ref_i)
    assert np.array_equal(val, ref_v)


def test_reference_factory_signature():
    import tilelang_ascend_b200 as dsa
    torch.manual_seed(0)
    x = torch.randn(64, 4096).cuda()
    kernel = dsa.simple_topk_selector(64, 4096, 2048, 512)
    idx = kernel(x)
    check_status()
    ref = torch.topk(x.cpu(), 2048, dim=-1)[1]  # the reference's ref_program
    assert idx.dtype == torch.int32 and tuple(idx.shape) == (64, 2048)
    # same index set per row (torch.topk leaves the order of equal values open; the selector puts the lower index first)
    assert torch.equal(torch.sort(idx.cpu().long(), dim=1).values, torch.sort(ref, dim=1).values)
    assert np.array_equal(idx.cpu().numpy(), orc.topk_select(x.cpu().numpy(), 2048))


def test_ties_lower_index_wins_and_heavy_duplicates():
    rng = np.random.default_rng(3)
    x = rng.integers(0, 6, size=(16, 3000)).astype(np.float32)  # only 6 distinct values: ties everywhere
    for K in (1, 100, 2048):
        assert np.array_equal(_run(x, K), orc.topk_select(x, K))
    x = np.zeros((2, 4096), dtype=np.float32)  # all equal
    assert np.array_equal(_run(x, 2048), orc.topk_select(x, 2048))


def test_limits_short_rows_and_masked_scores():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((9, 2500)).astype(np.float32)
    x[:, 1700:] = -np.inf
    x[3, ::2] = -np.inf
    x[4, :] = -np.inf
    lim = np.array([0, 1, 5, 2500, 2500, 1024, 2047, 2048, 2049], dtype=np.int32)
    idx, val = _run(x, 2048, lim, values=True)
    ref_i, ref_v = orc.topk_select(x, 2048, lim, return_values=True)
    assert np.array_equal(idx, ref_i)
    assert np.array_equal(val, ref_v)


def test_negative_zero_denormals_and_extremes():
    x = np.array([[0.0, -0.0, 1e-45, -1e-45, 3.4e38, -3.4e38, 1.0, -1.0, np.inf, -1e30, -0.99e30, 2.0]], dtype=np.float32)
    x = np.repeat(x, 3, axis=0)
    assert np.array_equal(_run(x, 12), orc.topk_select(x, 12))


def test_strided_rows():
    import tilelang_ascend_b200 as dsa
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 4096)).astype(np.float32)
    xs = torch.from_numpy(x).cuda()
    got = dsa.topk_select_raw(xs[:, :3000], 256).cpu().numpy()  # row stride 4096, n = 3000
    check_status()
    assert np.array_equal(got, orc.topk_select(x[:, :3000], 256))


@pytest.mark.parametrize("rows,n,k", [(64, 4096, 2048), (33, 8192, 2048), (16, 1000, 100), (8, 300, 512)])
def test_unordered_mode_returns_the_same_sets_in_index_order(rows, n, k):
    """ordered=False skips the final sort: per row the same index set as the ordered call (ties at the threshold resolved
    towards the lower index in both), ascending, values in step with the indices, -1 / -inf behind the selected ones."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator().manual_seed(rows + n)
    x = torch.randn((rows, n), generator=g)
    cols = torch.arange(7, n, 7)
    x[:, cols] = x[:, cols - 1]                               # plenty of exact ties
    lim = torch.randint(1, n + 1, (rows,), generator=g, dtype=torch.int32)
    xs, ls = x.cuda(), lim.cuda()
    a, av = dsa.topk_select_raw(xs, k, ls, return_values=True)
    b, bv = dsa.topk_select_raw(xs, k, ls, return_values=True, ordered=False)
    check_status()
    a, b, bv = a.cpu().numpy(), b.cpu().numpy(), bv.cpu().numpy()
    ref = orc.topk_select(x.numpy(), k, lim.numpy())
    assert np.array_equal(a, ref)
    for r in range(rows):
        sel = b[r][b[r] >= 0]
        assert np.array_equal(sel, np.sort(ref[r][ref[r] >= 0]))           # same set, ascending
        assert (b[r][len(sel):] == -1).all() and np.isneginf(bv[r][len(sel):]).all()
        assert np.array_equal(bv[r][: len(sel)], x.numpy()[r, sel])


@pytest.mark.parametrize("rows,n,k", [(6, 131072, 2048), (3, 60000, 2048), (2, 131072, 8192), (3, 100003, 100)])
def test_rows_longer_than_shared_memory_are_streamed(rows, n, k):
    """Rows whose keys do not fit in shared memory (more than about 52 k candidates, e.g. the 131072 keys of a long decode
    cache): every pass reads the scores again from global memory.  Same arrays as the oracle, with heavy ties (values
    rounded to 1/8), per-row limits, masked entries, and in the mode without the final sort."""
    import tilelang_ascend_b200 as dsa
    rng = np.random.default_rng(rows * 7 + n)
    x = rng.standard_normal((rows, n)).astype(np.float32)
    x[0] = np.round(x[0] * 8) / 8                      # a few hundred distinct values: the threshold bin is full of ties
    x[1, ::3] = -np.inf
    limits = np.full(rows, n, dtype=np.int32)
    limits[-1] = n - 12345
    idx, val = _run(x, k, limits=limits, values=True)
    ref_i, ref_v = orc.topk_select(x, k, limits=limits, return_values=True)
    assert np.array_equal(idx, ref_i)
    assert np.array_equal(val, ref_v)
    sets = dsa.topk_select_raw(torch.from_numpy(x).cuda(), k, torch.from_numpy(limits).cuda(), ordered=False)
    check_status()
    sets = sets.cpu().numpy()
    for r in range(rows):
        want = np.sort(ref_i[r][ref_i[r] >= 0])
        got = sets[r][sets[r] >= 0]
        assert np.array_equal(got, want)
