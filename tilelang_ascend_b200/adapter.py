"""Host adapter: the checks and allocation rules of the reference's kernel adapter.

The reference adapter (tilelang/jit/adapter/cython/cython_wrapper.pyx:75-203) is handed only the
input tensors, allocates every output with ``torch.empty`` on the device of the first input, rejects
non-contiguous inputs, wrong dtypes and mixed devices with ``ValueError`` before launching, and
launches on the current stream.  The helpers here reproduce those rules for the CUDA library.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16}
_NAMES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "float": torch.float32,
          "int32": torch.int32, "int": torch.int32}


def torch_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _NAMES[str(name)]
    except KeyError:
        raise ValueError(f"unsupported dtype {name!r}") from None


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"kernel supports bfloat16 / float16 inputs, got {dt}") from None


def check_inputs(tensors: Sequence[torch.Tensor], dtypes: Sequence[Optional[torch.dtype]], names: Sequence[str]) -> torch.device:
    """Contiguity / dtype / device checks (ValueError, as the reference adapter raises)."""
    dev = None
    for t, dt, name in zip(tensors, dtypes, names):
        if not isinstance(t, torch.Tensor):
            raise ValueError(f"{name}: expected a torch.Tensor, got {type(t).__name__}")
        if not t.is_contiguous():
            raise ValueError(f"Input tensor {name} must be contiguous")
        if dt is not None and t.dtype != dt:
            raise ValueError(f"Input tensor {name} has dtype {t.dtype}, expected {dt}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"Input tensor {name} is on {t.device}, expected {dev}")
    if dev is None or dev.type != "cuda":
        raise ValueError(f"kernels run on CUDA tensors only (got device {dev}); there is no CPU path")
    return dev


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def current_stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream
