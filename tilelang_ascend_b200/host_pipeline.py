"""Forward pass from HOST buffers: chunks of queries are copied in, computed and copied out on three CUDA streams so
that PCIe traffic in both directions overlaps the kernel.

The reference adapter only accepts device tensors (tilelang/jit/adapter/cython/cython_wrapper.pyx:164-174); a caller that
holds its activations in pinned host memory would otherwise pay copy-in + compute + copy-out back to back.  This helper
keeps the kernel and its results unchanged: every chunk is an ordinary call of the kernel returned by
``sparse_attention_fwd`` with ``q_start_index_s`` shifted by the chunk start.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


class HostPipelinedForward:
    """Runs ``kernel`` (built with ``return_softmax_lse=True``) over pinned host tensors in ``chunks`` query blocks.

    q_h [B,S,H,D], kv_h [B,S_kv,1,D], idx_h [B,S,1,topk] -> out_h [B,S,H,dv], lse_h [B,S,H]; all host tensors must be
    pinned.  Device staging buffers (three per tensor) are allocated once and reused by every call.
    """

    def __init__(self, kernel, q_shape, kv_shape, idx_shape, dv: int, dtype=torch.bfloat16, chunks: int = 8,
                 device: Optional[torch.device] = None, q_start_index_s: Optional[int] = None):
        self.kernel = kernel
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        B, S, H, D = q_shape
        self.B, self.S, self.H, self.D, self.dv = B, S, H, D, dv
        self.S_kv, self.topk = kv_shape[1], idx_shape[3]
        # causal position of query 0 of q_h: S_kv - S unless the caller holds a block of a longer sequence (a rank's shard)
        self.q_start = self.S_kv - S if q_start_index_s is None else int(q_start_index_s)
        self.chunks = max(1, min(int(chunks), S))
        self.bounds = [(S * i // self.chunks, S * (i + 1) // self.chunks) for i in range(self.chunks)]
        cmax = max(e - s for s, e in self.bounds)
        nbuf = 3
        self.q_d = [torch.empty((B, cmax, H, D), dtype=dtype, device=self.dev) for _ in range(nbuf)]
        self.idx_d = [torch.empty((B, cmax, 1, self.topk), dtype=torch.int32, device=self.dev) for _ in range(nbuf)]
        self.kv_d = torch.empty(kv_shape, dtype=dtype, device=self.dev)
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        self.nbuf = nbuf

    def __call__(self, q_h, kv_h, idx_h, out_h, lse_h) -> Tuple[torch.Tensor, torch.Tensor]:
        for t in (q_h, kv_h, idx_h, out_h, lse_h):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("HostPipelinedForward takes pinned host tensors")
        main = torch.cuda.current_stream(self.dev)
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        with torch.cuda.stream(self.s_in):
            self.kv_d.copy_(kv_h, non_blocking=True)
        ready = [torch.cuda.Event() for _ in self.bounds]     # chunk inputs on the device
        done = [torch.cuda.Event() for _ in self.bounds]      # chunk computed
        drained = [torch.cuda.Event() for _ in self.bounds]   # chunk results copied out (staging buffers reusable)
        keep = []
        for i, (s, e) in enumerate(self.bounds):
            b = i % self.nbuf
            n = e - s
            with torch.cuda.stream(self.s_in):
                if i >= self.nbuf:
                    self.s_in.wait_event(done[i - self.nbuf])  # the kernel that read this staging buffer has finished
                self.q_d[b][:, :n].copy_(q_h[:, s:e], non_blocking=True)
                self.idx_d[b][:, :n].copy_(idx_h[:, s:e], non_blocking=True)
                ready[i].record(self.s_in)
            main.wait_event(ready[i])
            qc = self.q_d[b][:, :n] if n == self.q_d[b].shape[1] else self.q_d[b][:, :n].contiguous()
            ic = self.idx_d[b][:, :n] if n == self.idx_d[b].shape[1] else self.idx_d[b][:, :n].contiguous()
            o, l = self.kernel(qc, self.kv_d, ic, q_start_index_s=self.q_start + s)
            done[i].record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done[i])
                out_h[:, s:e].copy_(o, non_blocking=True)
                lse_h[:, s:e].copy_(l, non_blocking=True)
                drained[i].record(self.s_out)
            o.record_stream(self.s_out)
            l.record_stream(self.s_out)
            keep.append((o, l))
        main.wait_stream(self.s_out)
        main.wait_stream(self.s_in)
        return out_h, lse_h
