"""The allocation-free indexer entry point, called straight through the C ABI.

`dsa_lightning_indexer_noalloc` exists for callers that cannot allocate device memory (a process whose own pool
owns all free GPU memory, or a loop that cannot take an allocation's device-wide synchronisation): its scratch
is an array inside the library.  Its results must equal those of `dsa_lightning_indexer`, which is handed a
workspace, also when the array still holds the previous call's data -- hence two calls in a row with different
shapes.  This file sorts last so that a run that stops at the first failure has run every other test before it.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu


def _both_entry_points(B, S1, S2, N1, K, mode, seed):
    from tilelang_ascend_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    q, k, w = (t.to(dev) for t in orc.make_indexer_inputs(B, S1, S2, N1, 128, seed=seed))
    stream = torch.cuda.current_stream(dev).cuda_stream
    # existing entry point: caller-provided workspace
    ws = torch.empty(lib.dsa_lightning_indexer_workspace_bytes(B, S1, S2), dtype=torch.uint8, device=dev)
    ref_idx = torch.empty((B, S1, 1, K), dtype=torch.int32, device=dev)
    ref_val = torch.empty((B, S1, 1, K), dtype=torch.float32, device=dev)
    _lib.check(lib.dsa_lightning_indexer(q.data_ptr(), k.data_ptr(), w.data_ptr(), B, S1, S2, N1, 128, 0, mode, None, None, K,
                                         ref_idx.data_ptr(), ref_val.data_ptr(), ws.data_ptr(), ws.numel(), stream))
    # new entry point: no workspace, outputs and the status read-back are the only device buffers passed
    idx = torch.full((B, S1, 1, K), -7, dtype=torch.int32, device=dev)
    val = torch.full((B, S1, 1, K), 123.0, dtype=torch.float32, device=dev)
    status = torch.full((1,), -1, dtype=torch.int32, device=dev)
    _lib.check(lib.dsa_lightning_indexer_noalloc(q.data_ptr(), k.data_ptr(), w.data_ptr(), B, S1, S2, N1, 128, 0, mode, None, None,
                                                 K, idx.data_ptr(), val.data_ptr(), status.data_ptr(), stream))
    torch.cuda.synchronize(dev)
    assert _lib.kernel_status() == 0
    assert int(status.item()) == 0
    # same kernels on the same inputs: the index arrays and the values are identical, not merely close
    assert torch.equal(idx, ref_idx)
    assert torch.equal(val, ref_val)
    return idx


def test_noalloc_entry_point_matches_workspace_entry_point_twice_in_a_row():
    first = _both_entry_points(B=1, S1=96, S2=3000, N1=64, K=512, mode=3, seed=11)
    # second call: smaller problem, other mode -- the array still holds the first call's scores
    second = _both_entry_points(B=2, S1=40, S2=700, N1=16, K=128, mode=0, seed=12)
    assert first.shape != second.shape
    # and the first shape once more, after the array was reused
    again = _both_entry_points(B=1, S1=96, S2=3000, N1=64, K=512, mode=3, seed=11)
    assert torch.equal(first, again)


def test_noalloc_entry_point_refuses_what_does_not_fit():
    from tilelang_ascend_b200 import _lib
    lib = _lib.load()
    cap = lib.dsa_lightning_indexer_noalloc_max_bytes()
    assert cap == 32 << 20
    dev = torch.device("cuda", 0)
    B, S1, S2 = 1, 2048, 8192  # 64 MiB of scores
    q = torch.zeros((B, S1, 64, 128), dtype=torch.bfloat16, device=dev)
    k = torch.zeros((B, S2, 1, 128), dtype=torch.bfloat16, device=dev)
    w = torch.zeros((B, S1, 64), dtype=torch.float32, device=dev)
    idx = torch.empty((B, S1, 1, 16), dtype=torch.int32, device=dev)
    rc = lib.dsa_lightning_indexer_noalloc(q.data_ptr(), k.data_ptr(), w.data_ptr(), B, S1, S2, 64, 128, 0, 3, None, None, 16,
                                           idx.data_ptr(), None, None, None)
    assert rc != 0
    msg = lib.dsa_get_last_error().decode()
    assert "too large for the built-in scratch" in msg and str(cap) in msg
