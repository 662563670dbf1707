"""Helpers shared by the GPU parity tests (every call goes through the package, i.e. the C ABI)."""
import numpy as np
import torch

ATOL, RTOL = 2e-2, 1e-2  # max-abs 2e-2 / relative 1e-2 against the fp32 oracle


def assert_close_fp(actual: torch.Tensor, expected: torch.Tensor, what: str, atol: float = ATOL, rtol: float = RTOL):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    fin = torch.isfinite(e)
    assert torch.equal(torch.isfinite(a), fin), f"{what}: non-finite pattern differs"
    assert torch.equal(a[~fin], e[~fin]), f"{what}: non-finite values differ"
    err = (a[fin] - e[fin]).abs()
    bound = atol + rtol * e[fin].abs()
    bad = err > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} of {err.numel()} beyond tolerance, max abs err {float(err.max()):.4g}"


def check_status():
    import tilelang_ascend_b200 as dsa
    st = dsa.kernel_status()
    assert st == 0, f"kernel status word = {st} (a bounded in-kernel wait gave up)"


def topk_three_step(idx: np.ndarray, ref_idx: np.ndarray, scores: np.ndarray, K: int):
    """The reference's 3-step check for indexer results (examples/deepseek_v4/lightning_indexer.py:1394-1503):
    per-row index sets equal, else every differing index must score within 1e-4 (relative) of the K-th
    boundary score.  Returns (rows with exactly equal sets, rows checked)."""
    rows = idx.shape[0]
    same = 0
    for r in range(rows):
        a, b = set(idx[r][idx[r] >= 0].tolist()), set(ref_idx[r][ref_idx[r] >= 0].tolist())
        if a == b:
            same += 1
            continue
        assert len(a) == len(b), f"row {r}: {len(a)} vs {len(b)} valid indices"
        kth = scores[r, sorted(b, key=lambda i: -scores[r, i])[-1]]
        for i in a ^ b:
            rel = abs(scores[r, i] - kth) / max(abs(kth), 1e-12)
            assert rel < 1e-4, f"row {r}: index {i} scores {scores[r, i]} vs boundary {kth}"
    return same, rows
