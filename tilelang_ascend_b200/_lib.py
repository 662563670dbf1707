"""ctypes binding of ``libdsa_b200.so`` (the C ABI declared in ``include/dsa_b200.h``).

There is no fallback: if the library has not been built, or a call is made without a CUDA device,
the import / call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libdsa_b200.so")

DTYPE_BF16, DTYPE_FP16 = 0, 1
IMPL_AUTO, IMPL_GENERIC, IMPL_TENSOR_CORE = 0, 1, 2

# name -> (restype, argtypes); must list every symbol include/dsa_b200.h declares
SIGNATURES = {
    "dsa_init": (c_int32, []),
    "dsa_get_last_error": (c_char_p, []),
    "dsa_kernel_status": (c_int32, [ctypes.POINTER(c_int32)]),
    "dsa_selftest_bounded_wait": (c_int32, [c_int64, c_void_p, c_void_p]),
    "dsa_topk_select": (c_int32, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int32, c_void_p, c_void_p, c_void_p]),
    "dsa_topk_select_unordered": (c_int32, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int32, c_void_p, c_void_p, c_void_p]),
    "dsa_lightning_indexer_unordered": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                                  c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_size_t,
                                                  c_void_p]),
    "dsa_indexer_scores": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32,
                                     c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_void_p]),
    "dsa_lightning_indexer_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "dsa_lightning_indexer": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                        c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_size_t,
                                        c_void_p]),
    "dsa_lightning_indexer_paged": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                              c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                              c_void_p, c_void_p, c_size_t, c_void_p]),
    "dsa_lightning_indexer_noalloc_max_bytes": (c_size_t, []),
    "dsa_lightning_indexer_noalloc": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32,
                                                c_int32, c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p,
                                                c_void_p]),
    "dsa_sparse_mla_fwd": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                     c_int32, c_int32, c_int32, c_float, c_int32, c_int32, c_int32, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p]),
    "dsa_sparse_mla_fwd_split_tail": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                                c_int32, c_int32, c_int32, c_float, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_size_t, c_void_p]),
    "dsa_sparse_mla_fwd_two_part": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                              c_int32, c_int32, c_int32, c_float, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_int32, c_int32, c_int32, c_void_p, c_size_t, c_void_p]),
    "dsa_sparse_mla_fwd_splitkv_nsplit": (c_int32, [c_int32, c_int32, c_int32, c_int32]),
    "dsa_sparse_mla_fwd_splitkv_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "dsa_sparse_mla_fwd_splitkv": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                             c_int32, c_int32, c_int32, c_float, c_int32, c_int32, c_int32, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_size_t,
                                             c_void_p]),
    "dsa_sparse_mla_bwd": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_float, c_int32,
                                     c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                                     c_void_p]),
    "dsa_block_sparse_logits": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                                          c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p, c_int32, c_int32, c_void_p]),
    "dsa_v4_build_indices": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int32] * 12 + [c_void_p]),
    "dsa_sink_combine": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32,
                                   c_int32, c_void_p]),
    "dsa_sparse_mla_bwd_tc_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "dsa_sparse_mla_bwd_tc": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_float, c_int32,
                                        c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                                        c_void_p, c_size_t, c_int32, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; raise if it is missing (build it with ``python -m tilelang_ascend_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tilelang_ascend_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class DsaError(RuntimeError):
    pass


def check(rc: int) -> None:
    """Raise on a failed call.  With DSA_DEBUG_SYNC=1 in the environment every successful launch is also followed by a
    device synchronisation and a read of the kernels' status word, so that a bounded in-kernel wait that gave up raises
    at the call that caused it (a debugging aid: it serialises host and device)."""
    if rc != 0:
        raise DsaError(load().dsa_get_last_error().decode())
    if os.environ.get("DSA_DEBUG_SYNC") == "1":
        st = kernel_status()
        if st != 0:
            raise DsaError(f"kernel status word = {st}: a bounded in-kernel wait gave up; results of this call are not valid")


def kernel_status() -> int:
    """Synchronise the current device and return (and clear) the kernels' status word."""
    st = c_int32(0)
    check(load().dsa_kernel_status(ctypes.byref(st)))
    return st.value
