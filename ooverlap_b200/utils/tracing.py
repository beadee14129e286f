"""Optional NVTX ranges around the phases of the model runner and the benchmarks (``OOB_NVTX=1``).

The ranges show up in any CUDA timeline tool and cost nothing when the variable is unset (one shared null
context).  The kernels' own device-side trace (globaltimer stamps per CTA, ``GemmAllReduce.trace_buffer``) is
separate: see ``ooverlap_b200.bench.overlap_trace``.

Capability parity: the reference has no NVTX ranges; it profiles from outside with nsys
(evalution/run_external_p2p_sm_usage.sh:400-428).
"""
from __future__ import annotations

import contextlib

from .config import env_flag

_NULL = contextlib.nullcontext()
_enabled = None


def enabled() -> bool:
    global _enabled
    if _enabled is None:
        _enabled = env_flag("OOB_NVTX", False)
    return _enabled


@contextlib.contextmanager
def _range(name: str):
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_range(name: str):
    """Context manager: an NVTX range called ``name`` when ``OOB_NVTX=1``, nothing otherwise."""
    return _range(name) if enabled() else _NULL
