#!/usr/bin/env python
"""Benchmark of the sparse-attention hot path on B200.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --gpus 1 --steps 3 --warmup 1     # CPU arm (reference golden / oracle port on host cores)

One step = one pass of the sparse MLA forward over the DeepSeek-V3.2 prefill workload
(B=1, S_q=S_kv=4096, H=128, D=576, dv=512, topk=2048, bf16, causal index lists, synthetic N(0,1)).
With N GPUs the 4096 queries of that ONE workload are cut into N contiguous blocks that take equal time in rounds of one
query per SM pair (strong scaling: total work fixed; the latent KV is replicated; no collective in the timed region; a
block may end in a round whose queries are split into shares of their keys), `value` is 4096 tokens divided by the slowest
rank's device time -- a step is one replay of a CUDA graph holding the step's launches -- and after the timing an NCCL
all-gather reassembles out / lse, which rank 0 compares with its own unsharded run: bit for bit, except the rows of split
last rounds, which are sums of fp32 partial results and are compared within the tolerance of the parity tests.
Rank 0 prints ONE JSON line on standard output (everything else, also what libraries print from C, goes to standard error).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(B=1, S=4096, S_kv=4096, H=128, D=576, DV=512, topk=2048)
FLOP_PER_PAIR_HEAD = 2 * 576 + 2 * 512  # QK^T over 576 dims + PV over 512 dims
METRIC, UNIT = "dsa_prefill_tokens_per_s", "tokens/s"
# DRAM bytes per query of the forward kernel, from the ncu capture summarised in profiles/ (dram__bytes_read.sum +
# dram__bytes_write.sum of one launch divided by its queries); re-derived whenever the kernel changes
DRAM_CAPTURE = {"read": 96940032, "write": 39233536, "queries": 592,
                "summary": "profiles/sparse_mla_fwd_pair_kernel__prefill_592q.md"}
CPU_SAMPLE_BLOCKS, CPU_SAMPLE_BLOCK = 16, 16   # the CPU arm's step: 16 evenly spaced blocks of 16 queries of the workload


_RESULT_FD = None


def claim_stdout() -> None:
    """Keeps the process's standard output for the one result line: everything else that writes to it -- Python prints, and
    libraries that print from C (NCCL's version banner) -- goes to standard error from here on."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(obj) -> None:
    data = (json.dumps(obj) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def valid_pairs(S: int, S_kv: int, topk: int, lo: int = 0, hi: int | None = None) -> int:
    p = np.arange(S, dtype=np.int64) + (S_kv - S) + 1
    return int(np.minimum(p, topk)[lo:hi].sum())


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0) or 0),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def workload_config(world: int) -> dict:
    """The `config` object: identical for both arms of a run (--impl ours / reference) at the same N."""
    w = WORKLOAD
    return {"workload": f"sparse_mla_fwd prefill B=1 S_q={w['S']} S_kv={w['S_kv']} H=128 D=576 dv=512 topk=2048 (DeepSeek-V3.2), "
                        "causal index lists, bf16 N(0,1), seed 1000",
            "partition": f"the {w['S']} queries cut into {world} contiguous block(s) that take equal time in rounds of one query per SM pair (key tiles + a fixed part per query; the queries of a partly filled last round split into shares of their keys), "
                         "one per GPU; latent KV replicated; no collective in the timed region",
            "l2": "every rank's inputs and outputs of one step (1.18 GB / N, 148 MB at N=8) exceed the 126 MB L2; no extra flush"}


def make_inputs_cuda(seed: int, dev: torch.device):
    """q, kv ~ N(0,1) bf16 and causally sampled distinct indices (-1 padded), generated on the device."""
    w = WORKLOAD
    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn((w["B"], w["S"], w["H"], w["D"]), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    kv = torch.randn((w["B"], w["S_kv"], 1, w["D"]), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    idx = torch.empty((w["B"], w["S"], 1, w["topk"]), dtype=torch.int32, device=dev)
    pos = torch.arange(w["S"], device=dev) + (w["S_kv"] - w["S"])
    cols = torch.arange(w["S_kv"], device=dev)
    for b in range(w["B"]):
        r = torch.rand((w["S"], w["S_kv"]), generator=g, device=dev)
        r = torch.where(cols[None, :] <= pos[:, None], r, torch.full_like(r, -1.0))
        vals, sel = torch.topk(r, w["topk"], dim=1)  # random distinct subset of the causal range
        idx[b, :, 0] = torch.where(vals >= 0, sel, torch.full_like(sel, -1)).to(torch.int32)
    return q, kv, idx


def bind_to_local_cores(local_rank: int, local_world: int) -> list:
    """Give this rank its own slice of the host cores (those the GPU reports as NUMA-local when NVML knows them, else the
    process's current set), so that N ranks do not time-share the same cores while they feed their copies; pinned buffers
    are allocated after this call.  Returns the cores taken."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
            words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
            local = [i * 64 + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1]
            if set(local) & set(cores):
                cores = sorted(set(local) & set(cores))
        except Exception:
            pass
        per = max(1, len(cores) // max(local_world, 1))
        mine = cores[local_rank * per:(local_rank + 1) * per] or cores
        os.sched_setaffinity(0, mine)
        torch.set_num_threads(max(1, len(mine)))
        return mine
    except Exception:
        return []


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only NVML)."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    _NAMES = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
              0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
              0x100: "display_clock_setting"}

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                try:
                    mask = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self._NAMES.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(2)

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def _time_ms(fn, reps: int = 10, warm: int = 3) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _time_graph_ms(fn, calls: int = 10, reps: int = 10, warm: int = 3) -> float:
    """Device time per call of `fn` with `calls` calls captured in one CUDA graph and the graph replayed `reps` times: for
    calls of a few tens of microseconds, which back-to-back eager calls cannot time (the host needs longer to issue one than
    the GPU to run it).  fn must launch on the current stream and must not synchronise."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(calls):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * calls)


def measure_backward(dev, peaks, S_b: int, reps: int = 10, warm: int = 3) -> dict:
    """Sparse MLA backward over the last S_b queries of the prefill shape (dKV accumulated in fp32)."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator(device=dev).manual_seed(13)
    saved = WORKLOAD["S"]
    q, kv, idx = make_inputs_cuda(11, dev)
    q, idx = q[:, saved - S_b:].contiguous(), idx[:, saved - S_b:].contiguous()
    scale, q0 = WORKLOAD["D"] ** -0.5, WORKLOAD["S_kv"] - S_b
    out, lse = dsa.sparse_mla_fwd_raw(q, kv, idx, sm_scale=scale, q_start=q0, causal=True, dv=WORKLOAD["DV"], return_lse=True)
    d_out = torch.randn(out.shape, generator=g, device=dev).to(torch.bfloat16)
    t_bwd = _time_ms(lambda: dsa.sparse_mla_bwd_raw(q, kv, idx, out, lse, d_out, sm_scale=scale, q_start=q0, causal=True), reps=reps, warm=warm)
    bwd_pairs = int((idx >= 0).sum().item())
    bwd_tflops = bwd_pairs * WORKLOAD["H"] * 5504 / (t_bwd * 1e-3) / 1e12
    assert dsa.kernel_status() == 0
    return {"ms": t_bwd, "tokens_per_s": S_b / (t_bwd * 1e-3), "tflops": bwd_tflops, "frac_of_bf16_peak": bwd_tflops / peaks["bf16_tflops"],
            "workload": f"sparse MLA backward, last {S_b} queries of the prefill shape, dQ bf16 + dKV fp32 (tensor-core kernels, workspace "
                        "allocation and dKV zeroing inside the timed call)"}


def measure_v4(dev) -> dict:
    """DeepSeek-V4 sparse_flash_mla on the shapes of the reference's own benchmark table
    (examples/deepseek_v4/sparse_flash_mla/bench_mark.md: B=1, 64 heads, D=512, TND, bf16, block 128, window 127, K=512,
    S=8192 prefill / one token against 8193 keys decode); synthetic tensors, whole front-door call timed (index lists built
    on the device, two sparse-forward calls, sink combine)."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator(device=dev).manual_seed(5)
    N1, D, bs, K = 64, 512, 128, 512
    res = {}
    for mode, S_q, S_kv in (("prefill", 8192, 8192), ("decode", 1, 8193)):
        q = torch.randn((S_q, N1, D), generator=g, device=dev).to(torch.bfloat16)
        nblk = (S_kv + bs - 1) // bs
        ori = torch.randn((nblk, bs, 1, D), generator=g, device=dev).to(torch.bfloat16)
        ori_bt = torch.randperm(nblk, generator=g, device=dev).to(torch.int32).view(1, nblk)
        cu = torch.tensor([0, S_q], dtype=torch.int32, device=dev)
        used = torch.tensor([S_kv], dtype=torch.int32, device=dev)
        sinks = torch.randn((N1,), generator=g, device=dev)
        common = dict(ori_kv=ori, ori_block_table=ori_bt, cu_seqlens_q=cu, seqused_kv=used, sinks=sinks, softmax_scale=D ** -0.5,
                      return_softmax_lse=True)
        for name, ratio in (("swa", 4), ("hca", 128), ("csa", 4)):
            kw = dict(common)
            if name != "swa":
                ncmp = max(S_kv // ratio, 1)
                cblk = (ncmp + bs - 1) // bs
                kw.update(cmp_kv=torch.randn((cblk, bs, 1, D), generator=g, device=dev).to(torch.bfloat16),
                          cmp_block_table=torch.arange(cblk, dtype=torch.int32, device=dev).view(1, cblk), cmp_ratio=ratio)
                if name == "hca":
                    kw.update(topk_cmp=ncmp)   # upper bound of the compressed tokens: spares the front door its host read
            if name == "csa":
                pos = torch.arange(S_q, device=dev) + (S_kv - S_q)
                thr = ((pos + 1) // ratio).clamp(min=1)
                ci = (torch.rand((S_q, K), generator=g, device=dev) * thr[:, None]).to(torch.int32)   # K draws below the threshold
                ci = torch.where(torch.arange(K, device=dev)[None, :] < thr[:, None], ci, torch.full_like(ci, -1))
                kw.update(cmp_sparse_indices=ci.view(S_q, 1, K).contiguous())
            t = _time_ms(lambda: dsa.sparse_flash_mla(q, **kw), reps=5, warm=2)
            res[f"{name}_{mode}"] = {"us": t * 1e3}
            if mode == "decode":
                # the same call as replays of a CUDA graph (what a serving loop does with a decode step): device time without
                # the host code between the launches; variants whose front door reads a length on the host cannot be captured
                try:
                    res[f"{name}_{mode}"]["us_graph_replay"] = _time_graph_ms(lambda: dsa.sparse_flash_mla(q, **kw)) * 1e3
                except Exception as exc:  # noqa: BLE001 (the eager figure stands)
                    res[f"{name}_{mode}"]["graph_replay"] = f"not capturable: {type(exc).__name__}"
                    torch.cuda.synchronize()
    assert dsa.kernel_status() == 0
    res["workload"] = "sparse_flash_mla, B=1, 64 heads, D=512, TND, bf16, block 128, window 127, K=512; prefill S=8192, decode 1 token vs 8193 keys"
    res["reference_published_us_tilelang_ascend"] = {"swa_prefill": 1490.9, "hca_prefill": 3141.9, "csa_prefill": 6022.7, "swa_decode": 13.8,
                                                     "hca_decode": 18.6, "csa_decode": 31.7}
    return res


def measure_mla_decode(dev, peaks) -> dict:
    """Dense MLA decode behind the reference's `mla_decode` factory on the largest shape of its layered test
    (examples_experiment/deepseek_mla/example_mla_decode/test_mla_decode.py: B=132, 128 heads, 8192 keys, dim 512 + 64):
    every key of every sequence is read once, kv and k_pe in place; timed as CUDA graph replays."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator(device=dev).manual_seed(17)
    B, H, N, dim, pe = 132, 128, 8192, 512, 64
    q = torch.randn((B, H, dim), generator=g, device=dev).to(torch.bfloat16)
    q_pe = torch.randn((B, H, pe), generator=g, device=dev).to(torch.bfloat16)
    kv = torch.randn((B, N, 1, dim), generator=g, device=dev).to(torch.bfloat16)
    k_pe = torch.randn((B, N, 1, pe), generator=g, device=dev).to(torch.bfloat16)
    kernel = dsa.mla_decode(B, H, 1, N, dim, pe)
    t = _time_graph_ms(lambda: kernel(q, q_pe, kv, k_pe), calls=4, reps=5)
    assert dsa.kernel_status() == 0
    nbytes = B * (N * (dim + pe) * 2 + H * (dim + pe) * 2 + H * dim * 2)
    flop = B * N * H * FLOP_PER_PAIR_HEAD
    return {"us": t * 1e3, "algorithmic_gb_per_s": nbytes / (t * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (t * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "tflops": flop / (t * 1e-3) / 1e12, "frac_of_bf16_peak": flop / (t * 1e-3) / 1e12 / peaks["bf16_tflops"], "timing": "CUDA graph replay",
            "workload": f"mla_decode B={B} heads={H} keys={N} dim={dim}+{pe}, bf16 (KV cache {B * N * (dim + pe) * 2 / 1e9:.2f} GB, read in place)"}


def measure_hisa(dev) -> dict:
    """HISA block-sparse indexer logits on the default shape of the reference's test script
    (examples/HISA/block_sparse_mqa_attn_expert_test.py:670-680: 1024 queries, 128 K keys, 32 heads x 128 dims, 64 selected
    blocks of 128 keys, fp16); synthetic tensors."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator(device=dev).manual_seed(3)
    S, S_kv, H, D, bs, topk = 1024, 128 * 1024, 32, 128, 128, 64
    q = torch.rand((S, H, D), generator=g, device=dev).to(torch.float16)
    k = torch.rand((S_kv, D), generator=g, device=dev).to(torch.float16)
    w = torch.rand((S, H), generator=g, device=dev).to(torch.float16)
    ks = torch.zeros(S, dtype=torch.int32, device=dev)
    ke = (torch.arange(1, S + 1, dtype=torch.int32, device=dev) * (S_kv // S)).clamp(max=S_kv)
    blk = torch.randint(0, S_kv // bs, (S, topk), generator=g, device=dev, dtype=torch.int32)
    kernel = dsa.block_sparse_mqa_attn_return_logits(S, S_kv, bs, topk, H, D)
    t = _time_ms(lambda: kernel(q, k, blk, w, ks, ke), reps=5, warm=2)
    flop = S * topk * bs * H * D * 2
    return {"ms": t, "tflops": flop / (t * 1e-3) / 1e12, "workload": f"S={S} S_kv={S_kv} heads={H} index_dim={D} topk={topk} blocks of {bs} keys, fp16"}


def decode_inputs(dev, B: int, g):
    S_kv, H, topk = 32768, 128, 2048
    qd = torch.randn((B, 1, H, 576), generator=g, device=dev).to(torch.bfloat16)
    kvd = torch.randn((B, S_kv, 1, 576), generator=g, device=dev).to(torch.bfloat16)
    idxd = torch.stack([torch.randperm(S_kv, generator=g, device=dev)[:topk] for _ in range(B)]).to(torch.int32).view(B, 1, 1, topk)
    return qd, kvd, idxd


def decode_bytes(B: int) -> int:
    return B * (2048 * 1152 + 128 * 576 * 2 + 128 * 512 * 2 + 2048 * 4)


def measure_other_stages(dev, peaks, small: bool = False) -> dict:
    """Lightning indexer + top-k (S_q=4096, S_kv=8192, 64x128) and decode (B=64, S_kv=32768) on one GPU.
    small: the last 1024 queries / 16 sequences only (for profiler captures)."""
    import tilelang_ascend_b200 as dsa
    g = torch.Generator(device=dev).manual_seed(7)
    S1, S2, K = (1024 if small else 4096), 8192, 2048
    qi = torch.randn((1, S1, 64, 128), generator=g, device=dev).to(torch.bfloat16)
    ki = torch.randn((1, S2, 1, 128), generator=g, device=dev).to(torch.bfloat16)
    wi = (torch.randn((1, S1, 64), generator=g, device=dev) / 8).float()
    t_sc = _time_ms(lambda: dsa.indexer_scores_raw(qi, ki, wi, sparse_mode=3, fill_masked=False))
    t_all = _time_ms(lambda: dsa.lightning_indexer_raw(qi, ki, wi, sparse_count=K, sparse_mode=3))
    t_all_set = _time_ms(lambda: dsa.lightning_indexer_raw(qi, ki, wi, sparse_count=K, sparse_mode=3, ordered=False))
    pairs = int((np.arange(S1, dtype=np.int64) + (S2 - S1) + 1).sum())
    sc_tflops = pairs * 64 * 256 / (t_sc * 1e-3) / 1e12
    del qi, ki, wi
    B = 16 if small else 64
    qd, kvd, idxd = decode_inputs(dev, B, g)
    dec = lambda n, **kw: dsa.sparse_mla_fwd_raw(qd[:n], kvd[:n], idxd[:n], sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512, **kw)  # noqa: E731
    # decode steps are timed as replays of a CUDA graph (as a serving loop launches them); the eager figure beside it is
    # bounded by the host's launch rate, not by the GPU
    t_dec = _time_graph_ms(lambda: dec(B))
    t_dec_one = _time_graph_ms(lambda: dec(B, nsplit=1))
    t_dec_eager = _time_ms(lambda: dec(B), reps=20)
    dec_gbs = decode_bytes(B) / (t_dec * 1e-3) / 1e9
    # one GPU's share of the same decode case sharded over 8 GPUs: 8 sequences, keys of every query split over work units
    B8 = 8
    t_dec8 = _time_graph_ms(lambda: dec(B8))
    t_dec8_one = _time_graph_ms(lambda: dec(B8, nsplit=1))
    t_dec8_eager = _time_ms(lambda: dec(B8), reps=20)
    del qd, kvd, idxd
    # the whole pipeline on the prefill shape: indexer scores -> top-2048 -> sparse MLA forward on the SELECTED indices,
    # three library calls back to back on one stream (S_q = S_kv = 4096; index heads 64 x 128 as in the indexer case)
    Sp = 1024 if small else WORKLOAD["S"]
    S_kvp = WORKLOAD["S_kv"]
    qi = torch.randn((1, Sp, 64, 128), generator=g, device=dev).to(torch.bfloat16)
    ki = torch.randn((1, S_kvp, 1, 128), generator=g, device=dev).to(torch.bfloat16)
    wi = (torch.randn((1, Sp, 64), generator=g, device=dev) / 8).float()
    qm = torch.randn((1, Sp, WORKLOAD["H"], WORKLOAD["D"]), generator=g, device=dev).to(torch.bfloat16)
    kvm = torch.randn((1, S_kvp, 1, WORKLOAD["D"]), generator=g, device=dev).to(torch.bfloat16)

    def pipeline():
        # the attention does not depend on the order of a query's list: the selector's final sort is left out
        sel, _ = dsa.lightning_indexer_raw(qi, ki, wi, sparse_count=WORKLOAD["topk"], sparse_mode=3, ordered=False)
        return dsa.sparse_mla_fwd_raw(qm, kvm, sel.view(1, Sp, 1, WORKLOAD["topk"]), sm_scale=WORKLOAD["D"] ** -0.5, q_start=S_kvp - Sp,
                                      causal=True, dv=WORKLOAD["DV"])
    t_pipe = _time_ms(pipeline)
    pp = np.arange(Sp, dtype=np.int64) + (S_kvp - Sp) + 1                       # candidates per query (causal)
    pipe_flop = int(pp.sum()) * 64 * 256 + int(np.minimum(pp, WORKLOAD["topk"]).sum()) * WORKLOAD["H"] * FLOP_PER_PAIR_HEAD
    pipe_tflops = pipe_flop / (t_pipe * 1e-3) / 1e12
    del qi, ki, wi, qm, kvm
    backward = measure_backward(dev, peaks, 256 if small else WORKLOAD["S"])
    assert dsa.kernel_status() == 0
    return {
        "backward": backward,
        **({} if small else {"mla_decode": measure_mla_decode(dev, peaks)}),
        "pipeline": {"ms": t_pipe, "tokens_per_s": Sp / (t_pipe * 1e-3), "tflops": pipe_tflops, "frac_of_bf16_peak": pipe_tflops / peaks["bf16_tflops"],
                     "roofline": {"bound": "tensor", "achieved": pipe_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                  "frac": pipe_tflops / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst)",
                                  "algorithmic_flop": pipe_flop,
                                  "counts": "indexer 2*128*64 FLOP per candidate pair + forward 2176 FLOP per (selected pair, head); nothing for the selector"},
                     "workload": f"indexer (64 x 128) -> top-2048 (index sets, ascending) -> sparse MLA forward on the selected indices, S_q={Sp}, S_kv={S_kvp}, one stream"},
        "indexer_scores": {"ms": t_sc, "tflops": sc_tflops, "frac_of_bf16_peak": sc_tflops / peaks["bf16_tflops"],
                           "workload": f"S_q={S1} S_kv=8192 64 heads x 128, causal"},
        "indexer_plus_topk": {"ms": t_all, "ms_index_sets_only": t_all_set, "tokens_per_s": S1 / (t_all * 1e-3), "top_k": K},
        "decode": {"us": t_dec * 1e3, "us_one_unit_per_query": t_dec_one * 1e3, "us_eager_calls": t_dec_eager * 1e3, "timing": "CUDA graph replay", "tokens_per_s": B / (t_dec * 1e-3), "algorithmic_gb_per_s": dec_gbs,
                   "frac_of_hbm_peak": dec_gbs / peaks["hbm_gbs"], "algorithmic_bytes": decode_bytes(B),
                   "workload": f"B={B} x 1 token, S_kv=32768, H=128, topk=2048 (KV cache {B * 32768 * 1152 / 1e9:.1f} GB, larger than L2)"},
        "decode_8_sequences": {"us": t_dec8 * 1e3, "us_one_unit_per_query": t_dec8_one * 1e3, "us_eager_calls": t_dec8_eager * 1e3, "timing": "CUDA graph replay", "tokens_per_s": B8 / (t_dec8 * 1e-3),
                               "workload": "8 of those sequences (one GPU's share at 8 GPUs), split-KV chosen by the library"},
    }


def measure_sustained(kernel, q, kv, idx, q_start, flop: float, local_rank: int, peaks, seconds: float = 2.5) -> dict:
    """The forward repeated back to back for `seconds`: average step time together with the SM clock sampled meanwhile
    (a seconds-long run settles at the power-capped clock, the 20-step headline runs at the boost clock)."""
    t1 = _time_ms(lambda: kernel(q, kv, idx, q_start_index_s=q_start), reps=5, warm=1)
    reps = max(20, int(seconds * 1e3 / max(t1, 1e-3)))
    with ClockSampler(local_rank) as clk:
        ms = _time_ms(lambda: kernel(q, kv, idx, q_start_index_s=q_start), reps=reps, warm=0)
    c = clk.summary()
    tf = flop / (ms * 1e-3) / 1e12
    return {"ms_per_step": ms, "steps": reps, "tflops": tf, "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
            "sm_mhz": c["sm_mhz"], "reasons": c["reasons"], "ms_times_mhz": ms * c["sm_mhz"] if c["sm_mhz"] else None}


def measure_copy_peak(dev) -> dict:
    """Pinned host <-> device copy bandwidth of this box (256 MB, both directions at once on two streams): the ceiling of
    the end-to-end number, whose every step moves its inputs in and its results out."""
    n = 256 << 20
    h_in = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n, dtype=torch.uint8).pin_memory()
    d_in, d_out = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def both():
        s1.wait_stream(torch.cuda.current_stream(dev))
        s2.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s1):
            d_in.copy_(h_in, non_blocking=True)
        with torch.cuda.stream(s2):
            h_out.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream(dev).wait_stream(s1)
        torch.cuda.current_stream(dev).wait_stream(s2)
    t_h2d = _time_ms(lambda: d_in.copy_(h_in, non_blocking=True), reps=5, warm=2)
    t_d2h = _time_ms(lambda: h_out.copy_(d_out, non_blocking=True), reps=5, warm=2)
    t_both = _time_ms(both, reps=5, warm=2)
    return {"h2d_gb_per_s": n / t_h2d / 1e6, "d2h_gb_per_s": n / t_d2h / 1e6, "both_directions_gb_per_s_each": n / t_both / 1e6}


# ------------------------------------------------------------------------------------------------- CPU arm
def find_reference_golden():
    """The reference's own torch golden of the forward when a checkout of the reference is at hand (DSA_REFERENCE_ROOT, or a
    copy under baseline/_ref): its FunctionDef is compiled on its own with `ast`, nothing else of the file runs.  None when
    there is no checkout (the GPU box): the oracle port is timed instead."""
    for root in (os.environ.get("DSA_REFERENCE_ROOT"), os.path.join(ROOT, "baseline", "_ref")):
        if not root:
            continue
        path = os.path.join(root, "examples/sparse_flash_attention/example_sparse_flash_attn_dynamic_shape.py")
        if os.path.isfile(path):
            try:
                sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
                from make_golden import load_functions
                return load_functions(path, ["ref_sparse_attention_fwd_interface"])["ref_sparse_attention_fwd_interface"]
            except Exception:
                return None
    return None


def cpu_sample_starts(S: int) -> np.ndarray:
    nblk = max(1, min(CPU_SAMPLE_BLOCKS, S // CPU_SAMPLE_BLOCK))
    return np.unique((np.linspace(0, S - CPU_SAMPLE_BLOCK, nblk).astype(np.int64) // CPU_SAMPLE_BLOCK) * CPU_SAMPLE_BLOCK)


def cpu_forward_sample(q, kv, idx, starts: np.ndarray, block: int, golden=None):
    """CPU forward (the reference golden when given, else the oracle port) on blocks of `block` consecutive query rows starting
    at `starts`, all host cores: (row numbers, out, lse-or-None, seconds, threads)."""
    from oracle import dsa_oracle as orc
    w = WORKLOAD
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    outs, lses, rows = [], [], []
    t0 = time.perf_counter()
    for s0 in starts.tolist():
        e0 = min(s0 + block, w["S"])
        qs = (w["S_kv"] - w["S"]) + s0
        if golden is not None:
            ix = idx[:, s0:e0]
            o = golden(q[:, s0:e0], kv, torch.where(ix < 0, torch.full_like(ix, w["S_kv"]), ix), qs, kv_stride=1).float()
            l = None
        else:
            o, l = orc.sparse_mla_fwd(q[:, s0:e0], kv, idx[:, s0:e0], q_start_index_s=qs, q_chunk=32)
        outs.append(o)
        lses.append(l)
        rows.append(np.arange(s0, e0))
    dt = time.perf_counter() - t0
    return np.concatenate(rows), torch.cat(outs, 1), (None if lses[0] is None else torch.cat(lses, 1)), dt, threads


def make_inputs_cpu_rows(starts: np.ndarray, block: int, seed: int):
    """The workload's tensors on the CPU with only the sampled query rows filled in (same distributions as the GPU arm's
    data: q, kv ~ N(0,1) bf16, row t = distinct indices drawn from its causal range, -1 padded); the other rows are never read."""
    w = WORKLOAD
    g = torch.Generator().manual_seed(seed)
    kv = torch.randn((w["B"], w["S_kv"], 1, w["D"]), generator=g).to(torch.bfloat16)
    q = torch.zeros((w["B"], w["S"], w["H"], w["D"]), dtype=torch.bfloat16)
    idx = torch.full((w["B"], w["S"], 1, w["topk"]), -1, dtype=torch.int32)
    for s0 in starts.tolist():
        e0 = min(s0 + block, w["S"])
        q[:, s0:e0] = torch.randn((w["B"], e0 - s0, w["H"], w["D"]), generator=g).to(torch.bfloat16)
        for b in range(w["B"]):
            for t in range(s0, e0):
                sel = torch.randperm((w["S_kv"] - w["S"]) + t + 1, generator=g)[: w["topk"]]
                idx[b, t, 0, : sel.numel()] = sel.to(torch.int32)
    return q, kv, idx


def cpu_sample_text(n_rows: int, n_blocks: int, kind: str) -> str:
    what = "the reference's torch golden ref_sparse_attention_fwd_interface" if kind == "reference" else "fp32 torch port of the reference golden"
    return f"{n_rows} queries ({n_blocks} evenly spaced blocks of {CPU_SAMPLE_BLOCK}) of the same workload per step, {what}"


def run_reference_arm(args, rank: int, world: int) -> None:
    """The reference's CPU implementation of the path on the host cores: rank 0 alone runs it; every step is the same evenly
    spaced sample of the workload's queries (tokens/s does not depend on which N the GPU arm runs at)."""
    if rank != 0:
        return
    w = WORKLOAD
    q, kv, idx = make_inputs_cpu_rows(cpu_sample_starts(w["S"]), CPU_SAMPLE_BLOCK, seed=0)
    golden = find_reference_golden()
    kind = "reference" if golden is not None else "port"
    starts = cpu_sample_starts(w["S"])
    times, rows, threads = [], None, 1
    for it in range(args.warmup + args.steps):
        rows, _, _, sec, threads = cpu_forward_sample(q, kv, idx, starts, CPU_SAMPLE_BLOCK, golden)
        if it >= args.warmup:
            times.append(sec)
    sec = sum(times) / len(times)
    value = len(rows) / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": cpu_sample_text(len(rows), len(starts), kind)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------------------------------- multi-GPU extras
def gather_shards(t: torch.Tensor, spans, world: int, dim: int = 1):
    """All-gather of per-rank blocks of different lengths along `dim` (padded to the longest): the full tensor on every rank."""
    import torch.distributed as dist
    pad = max(e - s for s, e in spans)
    shape = list(t.shape)
    shape[dim] = pad
    buf = torch.zeros(shape, dtype=t.dtype, device=t.device)
    buf.narrow(dim, 0, t.shape[dim]).copy_(t)
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf)
    return torch.cat([p.narrow(dim, 0, e - s) for p, (s, e) in zip(parts, spans)], dim=dim)


def measure_sharded_extras(dev, rank: int, world: int, peaks, q, kv, idx, spans) -> dict:
    """At N > 1: the decode case sharded by sequences (64 / N per GPU) and the backward sharded by queries with its one
    exchange -- the NCCL all-reduce of the fp32 key gradient -- inside the timed region, checked against the unsharded run."""
    import torch.distributed as dist
    import tilelang_ascend_b200 as dsa
    res = {}

    def max_over_ranks(ms: float) -> float:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- decode: B = 64 sequences, 64 / N per GPU ----
    B = 64
    s, e = dsa.shard_range(B, rank, world)
    g = torch.Generator(device=dev).manual_seed(7 + 100 * rank)
    qd, kvd, idxd = decode_inputs(dev, e - s, g)
    fn = lambda: dsa.sparse_mla_fwd_raw(qd, kvd, idxd, sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512)  # noqa: E731
    dist.barrier()
    us = max_over_ranks(_time_graph_ms(fn)) * 1e3
    gbs = decode_bytes(B) / (us * 1e-6) / 1e9
    res["decode_sharded"] = {"us": us, "tokens_per_s": B / (us * 1e-6), "algorithmic_gb_per_s_all_gpus": gbs,
                             "frac_of_hbm_peak_per_gpu": gbs / world / peaks["hbm_gbs"],
                             "timing": "CUDA graph replay",
                             "workload": f"B=64 x 1 token, S_kv=32768, topk=2048: {e - s} sequences on this GPU, max over ranks"}
    del qd, kvd, idxd

    # ---- backward: dQ per query block, dKV summed by one all-reduce ----
    w = WORKLOAD
    lo, hi = spans[rank]
    qs, ixs = q[:, lo:hi].contiguous(), idx[:, lo:hi].contiguous()
    scale, q0 = w["D"] ** -0.5, (w["S_kv"] - w["S"]) + lo
    out_s, lse_s = dsa.sparse_mla_fwd_raw(qs, kv, ixs, sm_scale=scale, q_start=q0, causal=True, dv=w["DV"])
    gd = torch.Generator(device=dev).manual_seed(13)
    d_out = torch.randn((w["B"], w["S"], w["H"], w["DV"]), generator=gd, device=dev).to(torch.bfloat16)
    d_out_s = d_out[:, lo:hi].contiguous()
    step = lambda: dsa.sparse_mla_bwd_sharded(qs, kv, ixs, out_s, lse_s, d_out_s, sm_scale=scale, q_start_index_s=q0)  # noqa: E731
    dist.barrier()
    ms = max_over_ranks(_time_ms(step, reps=5, warm=2))
    d_q_s, d_kv = step()
    flop = valid_pairs(w["S"], w["S_kv"], w["topk"]) * w["H"] * 5504
    entry = {"ms": ms, "tokens_per_s": w["S"] / (ms * 1e-3), "tflops_all_gpus": flop / (ms * 1e-3) / 1e12,
             "all_reduce_bytes": d_kv.numel() * 4,
             "workload": "sparse MLA backward of the prefill shape, queries sharded as the forward, NCCL all-reduce of the fp32 key gradient inside the timed step"}
    d_q_full = gather_shards(d_q_s, spans, world)
    if rank == 0:   # unsharded run on this GPU: dQ must be bit-equal (per-query work), dKV equal up to the order of the fp32 atomics
        out_f, lse_f = dsa.sparse_mla_fwd_raw(q, kv, idx, sm_scale=scale, q_start=w["S_kv"] - w["S"], causal=True, dv=w["DV"])
        dq_ref, dkv_ref = dsa.sparse_mla_bwd_raw(q, kv, idx, out_f, lse_f, d_out, sm_scale=scale, q_start=w["S_kv"] - w["S"], causal=True)
        err = float((d_kv - dkv_ref).abs().max())
        entry["check"] = {"dq_bit_equal_to_unsharded": bool(torch.equal(d_q_full, dq_ref)), "dkv_max_abs_diff": err,
                          "dkv_max_abs": float(dkv_ref.abs().max()), "ok": bool(err <= 1e-3 * float(dkv_ref.abs().max()) + 1e-3)}
    res["backward_sharded"] = entry
    assert dsa.kernel_status() == 0
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-chunks", type=int, default=16, help="query blocks of the host-buffer pipeline")
    ap.add_argument("--stage", default="all", choices=["all", "prefill", "others", "backward", "decode", "mla", "v4", "hisa"],
                    help="'all' (default): the headline measurement plus the other stages of the path; profiling aids: 'prefill' "
                         "leaves the other stages out, 'others' runs only the indexer / top-k / decode / backward measurements, 'backward' only the backward (two calls), 'decode' three eager decode steps of --queries sequences (default 64), 'mla' the dense MLA decode factory on the reference test's largest shape, 'v4' the DeepSeek-V4 sparse_flash_mla front door on the reference's benchmark shapes, 'hisa' the block-sparse indexer logits")
    ap.add_argument("--cpu-sample", type=int, default=1, help="0 leaves the CPU baseline / parity sample out")
    ap.add_argument("--sustained-seconds", type=float, default=2.5, help="length of the back-to-back run behind `sustained` (0 leaves it out)")
    ap.add_argument("--queries", type=int, default=0,
                    help="profiling aid: run only the LAST n queries of the workload (a small case for ncu captures); "
                         "the printed line is then not a benchmark result")
    args = ap.parse_args()
    claim_stdout()
    if args.queries:
        WORKLOAD["S"] = args.queries
    else:
        args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    import tilelang_ascend_b200 as dsa
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the kernels)")
    cores = bind_to_local_cores(local_rank, local_world) if world > 1 else []
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    w = WORKLOAD
    peaks = load_peaks()
    if args.stage == "hisa":
        if rank == 0:
            emit({"hisa_block_sparse_logits": measure_hisa(dev)})
        return
    if args.stage == "mla":
        if rank == 0:
            emit({"mla_decode": measure_mla_decode(dev, peaks)})
        return
    if args.stage == "v4":
        if rank == 0:
            emit({"sparse_flash_mla_v4": measure_v4(dev)})
        return
    if args.stage == "backward":
        if rank == 0:
            emit({"backward": measure_backward(dev, peaks, w["S"], reps=1, warm=1)})
        return
    if args.stage == "decode":
        if rank == 0:
            g = torch.Generator(device=dev).manual_seed(7)
            Bd = args.queries or 64
            qd, kvd, idxd = decode_inputs(dev, Bd, g)
            t = _time_ms(lambda: dsa.sparse_mla_fwd_raw(qd, kvd, idxd, sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512), reps=2, warm=1)
            emit({"decode_eager": {"us": t * 1e3, "sequences": Bd, "algorithmic_bytes": decode_bytes(Bd)}})
        return
    if args.stage == "others":
        if rank == 0:
            emit({"other_stages": measure_other_stages(dev, peaks, small=bool(args.queries))})
        return

    # every rank builds the same tensors (same seed, same generator, same GPU model) and keeps its block of the queries
    q, kv, idx = make_inputs_cuda(1000, dev)
    costs = dsa.causal_query_costs(w["S"], w["S_kv"], w["topk"])
    # one (query, 128 heads) unit per SM pair and round: blocks are cut so that the slowest rank's rounds take least time
    sm_pairs = max(1, torch.cuda.get_device_properties(dev).multi_processor_count // 2)
    # (a block may end in a round whose queries are split into shares of their keys, so that half and third rounds exist)
    spans = dsa.shard_ranges_by_rounds(costs, world, sm_pairs, tail_split=world > 1)
    tails = [dsa.tail_split_plan(costs, s, e, sm_pairs)[:2] if world > 1 else (0, 1) for s, e in spans]
    split_tail = tails[rank]
    lo, hi = spans[rank]
    q_s, idx_s = (q, idx) if world == 1 else (q[:, lo:hi].contiguous(), idx[:, lo:hi].contiguous())
    q0 = (w["S_kv"] - w["S"]) + lo
    kernel = dsa.sparse_attention_fwd(heads=w["H"], dim=w["DV"], tail_dim=w["D"] - w["DV"], topk=w["topk"], kv_stride=1,
                                      return_softmax_lse=True)
    out = lse = None
    for _ in range(args.warmup):
        out, lse = kernel(q_s, kv, idx_s, q_start_index_s=q0, split_tail=split_tail)
    torch.cuda.synchronize()
    assert dsa.kernel_status() == 0, "kernel reported a failed wait during warm-up"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_and_all(ms: float):
        t = torch.zeros(world, device=dev, dtype=torch.float64)
        t[rank] = ms
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        per = [float(x) for x in t.tolist()]
        return max(per), per

    # ---- timed region: K steps, inputs resident in HBM, CUDA events on the launching stream ----------
    # A step is one replay of a CUDA graph that holds the step's launches (the forward kernel, and the combine kernel of a
    # split last round): at 8 GPUs a step lasts a quarter of a millisecond and eight Python processes issuing eager calls
    # left gaps between the steps that belong to the host, not to the path.
    step_graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            out, lse = kernel(q_s, kv, idx_s, q_start_index_s=q0, split_tail=split_tail)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph):
            out, lse = kernel(q_s, kv, idx_s, q_start_index_s=q0, split_tail=split_tail)
        step_graph.replay()
        torch.cuda.synchronize()
    except Exception as exc:  # noqa: BLE001 (eager steps then)
        print(f"[bench] CUDA graph capture of the step failed ({type(exc).__name__}: {exc}); timing eager calls", file=sys.stderr)
        step_graph = None
        torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            if step_graph is not None:
                step_graph.replay()
            else:
                out, lse = kernel(q_s, kv, idx_s, q_start_index_s=q0, split_tail=split_tail)
        ev1.record()
        barrier()
    ms_total, per_rank_total = max_and_all(ev0.elapsed_time(ev1))
    ms_step = ms_total / args.steps
    assert dsa.kernel_status() == 0, "kernel reported a failed wait during the timed region"

    # ---- verification (N > 1): reassemble the shards and compare with the unsharded run, bit for bit ------------
    verify = None
    if world > 1:
        full_o, full_l = gather_shards(out, spans, world), gather_shards(lse, spans, world)
        if rank == 0:
            ref_o, ref_l = kernel(q, kv, idx)
            # rows of split tails are sums of fp32 partial results (tolerance); every other row must be bit-equal
            whole = torch.ones(w["S"], dtype=torch.bool, device=dev)
            for (s0, _e0), (m_t, n_t) in zip(spans, tails):
                if n_t > 1:
                    whole[s0:s0 + m_t] = False
            split_rows = int((~whole).sum().item())
            diff_o = (full_o[:, ~whole].float() - ref_o[:, ~whole].float()).abs().max().item() if split_rows else 0.0
            diff_l = (full_l[:, ~whole] - ref_l[:, ~whole]).abs().max().item() if split_rows else 0.0
            verify = {"out_bit_equal_to_unsharded": bool(torch.equal(full_o[:, whole], ref_o[:, whole])),
                      "lse_bit_equal_to_unsharded": bool(torch.equal(full_l[:, whole], ref_l[:, whole])),
                      "rows_compared_bitwise": w["S"] - split_rows, "rows_of_split_tails": split_rows,
                      "split_tails_max_abs_diff_out": diff_o, "split_tails_max_abs_diff_lse": diff_l,
                      "split_tails_ok": bool(diff_o <= 2e-2 and diff_l <= 1e-3),
                      "how": "NCCL all-gather of every rank's out / lse block after the timing, against rank 0's own run over all queries; "
                             "queries of a rank's split last round are combined from fp32 partial results and compared within 2e-2"}
            del ref_o, ref_l
        del full_o, full_l

    # ---- end to end: pinned host inputs -> device -> kernel -> host result, every step (this rank's block only) ----
    q_h = torch.empty(q_s.shape, dtype=q.dtype, pin_memory=True).copy_(q_s)
    kv_h = torch.empty(kv.shape, dtype=kv.dtype, pin_memory=True).copy_(kv)
    idx_h = torch.empty(idx_s.shape, dtype=idx.dtype, pin_memory=True).copy_(idx_s)
    out_h = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
    lse_h = torch.empty(lse.shape, dtype=lse.dtype, pin_memory=True)
    # the package's host-buffer entry: query chunks are copied in, computed and copied out on three streams
    host_fwd = dsa.HostPipelinedForward(kernel, q_s.shape, kv.shape, idx_s.shape, w["DV"], chunks=max(2, args.e2e_chunks // world), device=dev,
                                        q_start_index_s=q0)
    e2e_ms = float("nan")
    if args.e2e_steps > 0:
        host_fwd(q_h, kv_h, idx_h, out_h, lse_h)
        barrier()
        ev0.record()
        for _ in range(args.e2e_steps):
            host_fwd(q_h, kv_h, idx_h, out_h, lse_h)
        ev1.record()
        barrier()
        e2e_total, _ = max_and_all(ev0.elapsed_time(ev1))
        e2e_ms = e2e_total / args.e2e_steps
        # (the resident run may have split the queries of its last round; the pipeline's chunks are never split)
        cut = split_tail[0] if split_tail[1] > 1 else 0
        res = out.cpu()
        assert torch.equal(out_h[:, cut:], res[:, cut:]), "host-buffer pipeline result differs from the resident run"
        assert cut == 0 or (out_h[:, :cut].float() - res[:, :cut].float()).abs().max().item() <= 2e-2, "split tail differs from the pipeline's rows"
    bytes_t = torch.tensor([q_h.numel() * 2 + kv_h.numel() * 2 + idx_h.numel() * 4, out_h.numel() * 2 + lse_h.numel() * 4], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(bytes_t, op=dist.ReduceOp.SUM)
    h2d, d2h = int(bytes_t[0].item()), int(bytes_t[1].item())

    tokens = w["B"] * w["S"]
    pairs = valid_pairs(w["S"], w["S_kv"], w["topk"])
    flop = pairs * w["H"] * FLOP_PER_PAIR_HEAD
    achieved = flop / (ms_step * 1e-3) / 1e12 / world           # per GPU
    dram_per_query = (DRAM_CAPTURE["read"] + DRAM_CAPTURE["write"]) / DRAM_CAPTURE["queries"]
    line = {
        "metric": METRIC, "value": tokens / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
        "tflops_per_gpu": achieved,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["bf16_tflops"], "traffic": dram_per_query * w["B"] * w["S"] / world,
                     "traffic_source": f"ncu dram__bytes_read.sum + dram__bytes_write.sum of a {DRAM_CAPTURE['queries']}-query launch "
                                       f"({DRAM_CAPTURE['summary']}), scaled by the queries of one launch",
                     "peak_source": peaks["source"] + " (burst)",
                     "kernel": "sparse_mla_fwd_pair_kernel", "algorithmic_flop_per_launch": flop / world},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms},
        "gpu_launches": args.steps * sum(2 if n_t > 1 else 1 for _m, n_t in tails),   # the forward kernel, + the combine kernel of a split last round
        "step_launch": "CUDA graph replay" if step_graph is not None else "eager call",
        "clocks": clocks.summary(),
    }
    if world > 1:
        line["per_rank"] = {"queries": [e - s for s, e in spans], "split_tail_queries_and_shares": [list(t) for t in tails],
                            "ms_per_step": [t / args.steps for t in per_rank_total],
                            "cores_of_rank0": cores}
        line["verify"] = verify
        # the replicated measurement of earlier builds, kept beside the sharded one: every rank the WHOLE workload
        rep = _time_ms(lambda: kernel(q, kv, idx), reps=args.steps, warm=2)
        rep_ms, _ = max_and_all(rep)
        line["replicas"] = {"ms_per_step": rep_ms, "tokens_per_s_all_gpus": tokens * world / (rep_ms * 1e-3),
                            "what": "every GPU runs all 4096 queries (N independent copies): weak scaling, no shared resource"}
        try:
            extras = measure_sharded_extras(dev, rank, world, peaks, q, kv, idx, spans)
        except Exception as exc:  # an optional stage must not lose the headline line
            extras = {"error": f"{type(exc).__name__}: {exc}"}
        line["other_stages"] = extras

    if rank == 0 and world == 1 and not args.queries and args.sustained_seconds > 0:
        try:
            line["sustained"] = measure_sustained(kernel, q, kv, idx, q0, flop, local_rank, peaks, seconds=args.sustained_seconds)
            copy_peak = measure_copy_peak(dev)
            line["e2e"]["pinned_copy_peak"] = copy_peak
            # a step moves h2d bytes in and d2h bytes out concurrently: bound = the slower direction at the both-directions rate
            bound_ms = max(h2d, d2h) / (copy_peak["both_directions_gb_per_s_each"] * 1e6)
            line["e2e"]["copy_bound_ms"] = bound_ms
            line["e2e"]["frac_of_copy_bound"] = bound_ms / e2e_ms
        except Exception as exc:
            line["sustained_error"] = f"{type(exc).__name__}: {exc}"

    # ---- the rest of the path on its named shapes (N=1 only; reported beside the headline, not part of it) ----
    if rank == 0 and world == 1 and not args.queries and args.stage == "all":
        line["other_stages"] = measure_other_stages(dev, peaks)

    # ---- CPU baseline (rank 0, N=1 only): the CPU forward on a bounded sample; doubles as a parity check -----
    if rank == 0 and world == 1 and args.cpu_sample > 0:
        golden = find_reference_golden()
        kind = "reference" if golden is not None else "port"
        starts = cpu_sample_starts(w["S"])
        rows, ref_o, ref_l, sec, threads = cpu_forward_sample(q.cpu(), kv.cpu(), idx.cpu(), starts, CPU_SAMPLE_BLOCK, golden)
        sel = torch.from_numpy(rows).to(dev)
        got_o = out[:, sel].float().cpu()
        err_o = float((got_o - ref_o).abs().max())
        ok = err_o <= 2e-2 + 1e-2 * float(ref_o.abs().max())
        par = {"queries": len(rows), "max_abs_err_out": err_o}
        if ref_l is not None:
            err_l = float((lse[:, sel].cpu() - ref_l).abs().max())
            par["max_abs_err_lse"] = err_l
            ok = ok and err_l <= 2e-2 + 1e-2 * float(ref_l.abs().max())
        par["ok"] = bool(ok)
        line["cpu_baseline"] = {"value": len(rows) / sec, "unit": UNIT, "cores": threads, "kind": kind,
                                "sample": cpu_sample_text(len(rows), len(starts), kind) + f", {sec:.1f} s"}
        line["parity_sample"] = par
    if rank == 0:
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
