"""dtype / reduce-op tables shared by the Python layer."""
from __future__ import annotations

import torch

from .. import _lib

DTYPE_CODE = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}
OP_CODE = {"sum": _lib.SUM, "add": _lib.SUM, "min": _lib.MIN, "max": _lib.MAX}
ATOL = {torch.float16: 1e-2, torch.bfloat16: 1e-2, torch.float32: 1e-5}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; supported: fp16, bf16, fp32") from None


def op_code(op: str) -> int:
    try:
        return OP_CODE[op.lower()]
    except KeyError:
        raise ValueError(f"unsupported reduce op {op!r}; supported: sum, min, max") from None
