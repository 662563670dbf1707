"""CPU-side checks: the C-ABI library loads and exports every declared symbol, host logic, sharding."""
import os
import re

import pytest
import torch

import tilelang_ascend_b200 as dsa
from tilelang_ascend_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    with open(os.path.join(ROOT, "include", "dsa_b200.h")) as fh:
        header = fh.read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(dsa_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None


def test_error_reporting_without_compute():
    lib = _lib.load()
    # argument validation happens before any CUDA call
    rc = lib.dsa_topk_select(None, 1, 1, 1, None, 1, None, None, None)
    assert rc != 0 and b"null" in lib.dsa_get_last_error()
    rc = lib.dsa_sparse_mla_fwd(None, None, None, None, None, 1, 1, 1, 1, 576, 512, 1, 1.0, 0, 1, 0, None, None, None, None, 0, 0, 0, None)
    assert rc != 0


def test_cpu_tensors_are_rejected_not_computed():
    x = torch.randn(4, 64)
    with pytest.raises(ValueError, match="no CPU path"):
        dsa.simple_topk_selector(4, 64, 8, 2)(x)
    q = torch.randn(1, 2, 16, 576).bfloat16()
    kv = torch.randn(1, 8, 1, 576).bfloat16()
    idx = torch.zeros(1, 2, 1, 64, dtype=torch.int32)
    with pytest.raises(ValueError, match="no CPU path"):
        dsa.sparse_attention_fwd(16, 512, 64, 64, 1)(q, kv, idx)


def test_factory_argument_rules():
    with pytest.raises(AssertionError):
        dsa.sparse_attention_fwd(16, 500, 64, 64, 1)
    with pytest.raises(ValueError):
        dsa.sparse_attention_fwd(16, 512, 64, 64, 4)
    with pytest.raises(ValueError):
        dsa.simple_topk_selector(4, 64, 128, 2)
    with pytest.raises(ValueError):
        dsa.mla_decode(1, 16, 2, 128, 512, 64)


def test_shard_range_covers_everything_once():
    for n in (0, 1, 7, 64, 4096, 4097):
        for world in (1, 2, 3, 4, 8):
            spans = [dsa.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        dsa.shard_range(4, 2, 2)


def test_shard_queries_keeps_causal_positions():
    q = torch.zeros(1, 10, 2, 8)
    idx = torch.zeros(1, 10, 1, 4, dtype=torch.int32)
    starts = []
    for r in range(4):
        qs, ix, q_start = dsa.shard_queries(q, idx, r, 4, s_kv=32)
        assert qs.shape[1] == ix.shape[1]
        starts.append((q_start, qs.shape[1]))
    assert starts[0][0] == 22
    for (a, n), (b, _) in zip(starts, starts[1:]):
        assert a + n == b


def test_balanced_shards_cover_everything_once_and_equalise_cost():
    costs = dsa.causal_query_costs(4096, 4096, 2048)
    assert int(costs[0]) == 1 + dsa.sharding.FIXED_TILES_PER_QUERY and int(costs[-1]) == 32 + dsa.sharding.FIXED_TILES_PER_QUERY
    for world in (1, 2, 3, 4, 8):
        spans = [dsa.shard_range_balanced(costs, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 4096
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        loads = [int(costs[s:e].sum()) for s, e in spans]
        assert max(loads) <= 1.005 * sum(loads) / world
    # equal counts leave the last rank with 1 / 0.75 of the average number of (query, key) pairs at 8 ranks
    pairs = [sum(min(t + 1, 2048) for t in range(*dsa.shard_range(4096, r, 8))) for r in range(8)]
    assert abs(max(pairs) / (sum(pairs) / 8) - 1 / 0.75) < 0.01
    assert dsa.shard_range_balanced([], 0, 2) == (0, 0)
    assert [dsa.shard_range_balanced([1.0] * 5, r, 5) for r in range(5)] == [(i, i + 1) for i in range(5)]
    with pytest.raises(ValueError):
        dsa.shard_range_balanced(costs, 3, 2)


def test_partition_by_rounds_beats_the_cost_sum_partition_and_covers_everything():
    """Blocks cut for a kernel that walks its items in rounds of one per SM pair: contiguous, complete, never slower (in
    the round model) than the partition by summed cost, and better where the latter leaves a rank with a partial round."""
    import tilelang_ascend_b200 as dsa
    costs = dsa.causal_query_costs(4096, 4096, 2048)
    for world in (1, 2, 3, 4, 8):
        spans = dsa.shard_ranges_by_rounds(costs, world, 74)
        assert spans[0][0] == 0 and spans[-1][1] == 4096 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        t_new = max(dsa.block_time_in_rounds(costs, s, e, 74) for s, e in spans)
        t_sum = max(dsa.block_time_in_rounds(costs, *dsa.shard_range_balanced(costs, r, world), 74) for r in range(world))
        assert t_new <= t_sum
    spans = dsa.shard_ranges_by_rounds(costs, 4, 74)
    assert max(dsa.block_time_in_rounds(costs, s, e, 74) for s, e in spans) < \
        max(dsa.block_time_in_rounds(costs, *dsa.shard_range_balanced(costs, r, 4), 74) for r in range(4))
    assert dsa.shard_ranges_by_rounds([], 2, 74) == [(0, 0), (0, 0)]
    assert dsa.shard_ranges_by_rounds([5, 5, 5], 5, 2) [:2] == [(0, 2), (2, 3)] or sum(e - s for s, e in dsa.shard_ranges_by_rounds([5, 5, 5], 5, 2)) == 3


def test_partition_with_split_tails_reaches_half_rounds():
    """With the queries of a partly filled last round split into shares, the 8-GPU partition of the prefill shape gets blocks
    of 5.5 rounds of long queries instead of 6 (model time 195 against 210; 190.75 would be perfect)."""
    import tilelang_ascend_b200 as dsa
    costs = dsa.causal_query_costs(4096, 4096, 2048)
    plain = dsa.shard_ranges_by_rounds(costs, 8, 74)
    split = dsa.shard_ranges_by_rounds(costs, 8, 74, tail_split=True)
    assert split[0][0] == 0 and split[-1][1] == 4096 and all(a[1] == b[0] for a, b in zip(split, split[1:]))
    t_plain = max(dsa.block_time_in_rounds(costs, s, e, 74) for s, e in plain)
    t_split = max(dsa.block_time_in_rounds(costs, s, e, 74, True) for s, e in split)
    assert t_split < t_plain and t_split <= 1.03 * dsa.block_time_in_rounds(costs, 0, 4096, 74) / 8
    for s, e in split:
        m, n, t = dsa.tail_split_plan(costs, s, e, 74)
        assert (m == 0 and n == 1) or (m == (e - s) % 74 and 2 <= n <= 4 and m * n <= 74)
    assert dsa.tail_split_plan(costs, 0, 74, 74) == (0, 1, 0)                 # whole rounds: nothing to split
    assert dsa.tail_split_plan(costs, 0, 30, 74)[:2] == (0, 1)                # one-tile queries: splitting cannot pay
    assert dsa.tail_split_plan(costs, 4096 - 74 - 20, 4096, 74)[:2] == (20, 3)  # 20 long queries fill the round as 3 shares each
