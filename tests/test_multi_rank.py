"""world_size-2 gloo run of the sharded driver logic on CPU: ranks split the queries with no
data-path collective, a verification all-gather reassembles the result, timing is max over ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dsa_oracle as orc


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import tilelang_ascend_b200 as dsa
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    q, kv, idx = orc.make_sparse_mla_inputs(1, 10, 64, 4, 16, seed=0)
    qs, ix, q_start = dsa.shard_queries(q, idx, rank, world, s_kv=64, balance=True)
    # the oracle stands in for the device kernel here: only the partition and reassembly are under test
    out, _ = orc.sparse_mla_fwd(qs, kv, ix, q_start_index_s=q_start)
    costs = dsa.causal_query_costs(10, 64, 16)
    sizes = [dsa.shard_range_balanced(costs, r, world) for r in range(world)]
    pad = max(e - s for s, e in sizes)
    buf = torch.zeros((1, pad) + tuple(out.shape[2:]))
    buf[:, : out.shape[1]] = out
    gathered = [torch.zeros_like(buf) for _ in range(world)]
    dist.all_gather(gathered, buf)
    full = torch.cat([g[:, : e - s] for g, (s, e) in zip(gathered, sizes)], dim=1)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ref, _ = orc.sparse_mla_fwd(q, kv, idx)
        ret["ok"] = bool(torch.allclose(full, ref, atol=1e-6)) and float(t) == float(world)
    dist.destroy_process_group()


def _rounds_worker(rank: int, world: int, port: int, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import tilelang_ascend_b200 as dsa
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    S, S_kv, topk, pairs = 23, 64, 16, 4          # rounds of 4 queries: blocks end in whole rounds or in a split last round
    q, kv, idx = orc.make_sparse_mla_inputs(1, S, S_kv, 4, topk, seed=3)
    costs = dsa.causal_query_costs(S, S_kv, topk)
    spans = dsa.shard_ranges_by_rounds(costs, world, pairs, tail_split=True)
    s, e = spans[rank]
    qs, ix, q_start = dsa.shard_queries(q, idx, rank, world, s_kv=S_kv, balance=True, units_per_round=pairs)
    plain = dsa.shard_ranges_by_rounds(costs, world, pairs)[rank]
    assert (qs.shape[1], q_start) == (plain[1] - plain[0], (S_kv - S) + plain[0])   # shard_queries cuts whole rounds
    # the oracle stands in for the device kernel: the split-tail partition and the reassembly are under test
    out, _ = orc.sparse_mla_fwd(q[:, s:e], kv, idx[:, s:e], q_start_index_s=(S_kv - S) + s)
    pad = max(b - a for a, b in spans)
    buf = torch.zeros((1, pad) + tuple(out.shape[2:]))
    buf[:, : out.shape[1]] = out
    gathered = [torch.zeros_like(buf) for _ in range(world)]
    dist.all_gather(gathered, buf)
    full = torch.cat([g[:, : b - a] for g, (a, b) in zip(gathered, spans)], dim=1)
    if rank == 0:
        ref, _ = orc.sparse_mla_fwd(q, kv, idx)
        plans = [dsa.tail_split_plan(costs, a, b, pairs)[:2] for a, b in spans]
        ret["ok"] = bool(torch.allclose(full, ref, atol=1e-6)) and spans[0][0] == 0 and spans[-1][1] == S and \
            all((m == 0 and n == 1) or (2 <= n <= 4 and m * n <= pairs) for m, n in plans)
    dist.destroy_process_group()


def test_two_rank_partition_by_rounds_with_split_tails_reassembles():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        ret = m.dict()
        port = _free_port()
        procs = [ctx.Process(target=_rounds_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret.get("ok") is True


def test_two_rank_query_sharding_reassembles():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        ret = m.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret.get("ok") is True


def _bwd_worker(rank: int, world: int, port: int, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import tilelang_ascend_b200 as dsa
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    S, S_kv = 9, 48
    q, kv, idx = orc.make_sparse_mla_inputs(1, S, S_kv, 4, 16, seed=1)
    d_out = torch.randn((1, S, 4, 512), generator=torch.Generator().manual_seed(2))
    qs, ix, q_start = dsa.shard_queries(q, idx, rank, world, s_kv=S_kv)
    s, e = dsa.shard_range(S, rank, world)

    def oracle_bwd(q_, kv_, idx_, out_, lse_, d_out_, *, sm_scale, q_start, causal):  # stands in for the device kernel
        return orc.sparse_mla_bwd(q_, kv_, idx_, d_out_, q_start_index_s=q_start, sm_scale=sm_scale)

    d_q, d_kv = dsa.sparse_mla_bwd_sharded(qs, kv, ix, None, None, d_out[:, s:e].contiguous(), sm_scale=576 ** -0.5,
                                           q_start_index_s=q_start, bwd=oracle_bwd)
    ref_dq, ref_dkv = orc.sparse_mla_bwd(q, kv, idx, d_out)
    ok = bool(torch.allclose(d_q, ref_dq[:, s:e], atol=1e-5)) and bool(torch.allclose(d_kv, ref_dkv, atol=1e-4))
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret["ok"] = float(flag) == 1.0
    dist.destroy_process_group()


def test_two_rank_backward_sums_key_gradient():
    """dQ shards by query; dKV needs the one all-reduce of the path: every rank ends with the full key gradient."""
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        ret = m.dict()
        port = _free_port()
        procs = [ctx.Process(target=_bwd_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
        assert ret.get("ok") is True
