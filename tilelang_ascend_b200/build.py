"""Ahead-of-time build of the CUDA library for sm_100a (no JIT, in-tree output).

    python -m tilelang_ascend_b200.build            # builds tilelang_ascend_b200/libdsa_b200.so

nvcc cross-compiles without a GPU.  Objects go to tilelang_ascend_b200/build/ and are rebuilt only
when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
LIB = os.path.join(PKG, "libdsa_b200.so")
SOURCES = ["capi.cu", "sparse_mla_fwd.cu", "sparse_mla_fwd_pair.cu", "sparse_mla_bwd.cu", "sparse_mla_bwd_tc.cu", "indexer.cu", "topk.cu", "no_alloc.cu", "sink_combine.cu", "block_sparse_logits.cu", "selftest.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer_than(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    nvcc = _nvcc()
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    logs = {}

    def compile_one(src: str) -> str:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        path = os.path.join(CSRC, src)
        if force or _newer_than(obj, [path] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", path, "-o", obj]
            res = subprocess.run(cmd, capture_output=True, text=True)
            logs[src] = res.stdout + res.stderr
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{logs[src]}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    if force or _newer_than(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}{res.stderr}")
    if verbose:
        for src, log in logs.items():
            print(f"==== {src}\n{log}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
