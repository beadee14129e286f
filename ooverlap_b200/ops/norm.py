"""Residual-add + RMSNorm, stand-alone and fused with the all-reduce / reduce-scatter.

Capability parity: the reference's stand-alone RMSNorm kernels
(src/rmsnorm/rmsnorm.cuh:11-121, not exported to Python there); the fusion with
the collective is new.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib
from ..utils.dtypes import dtype_code
from ..utils.partition import partition


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float,
                      residual: Optional[torch.Tensor] = None):
    """fp32 PyTorch oracle: returns (y, new_residual)."""
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype), xf.to(x.dtype)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None,
            *, out: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None, max_ctas: int = 0):
    """Local ``y = rmsnorm(x + residual) * weight`` (no communication).  Returns ``y`` or ``(y, residual_out)``."""
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous [rows, hidden] tensor")
    rows, hidden = x.shape
    y = out if out is not None else torch.empty_like(x)
    if residual is not None and residual_out is None:
        residual_out = torch.empty_like(x)
    a = _lib.NormArgs()
    a.dtype, a.rows, a.hidden, a.eps = dtype_code(x.dtype), rows, hidden, eps
    a.x_reg, a.x_off = 0, x.data_ptr()  # no communicator: x_off carries the address
    a.residual = residual.data_ptr() if residual is not None else None
    a.weight = weight.data_ptr()
    a.y_local = y.data_ptr()
    a.res_out_reg = -1
    a.res_out_local = residual_out.data_ptr() if residual_out is not None else None
    _lib.check(_lib.lib().oob_fused_norm(None, _lib.NORM_LOCAL, ctypes.byref(a), max_ctas, _stream()))
    return (y, residual_out) if residual is not None else y


def fused_allreduce_rmsnorm(comm, x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                            residual: Optional[torch.Tensor] = None, *, algo: Optional[int] = None,
                            out: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
                            max_ctas: int = 0):
    """``y = rmsnorm(all_reduce(x) + residual) * weight`` in one kernel.

    ``x`` ([rows, hidden], registered memory) holds this rank's partial sums.
    A few rows (up to ``config.ll_max_bytes``, when the communicator has a slot ring) travel as 8-byte cells of data +
    call number and need no barrier at all; decode-sized messages up to ``config.push_max_bytes`` take the push kernel
    (every rank pushes its rows to all ranks, the ranks meet once, every rank sums and normalises every row locally);
    larger ones the two-shot fused
    kernel (rank r reduces and normalises its rows and broadcasts them), through NVLS when the communicator has it;
    fewer rows than ranks the one-shot fused kernel.  ``algo`` forces one of the fused kernels.  Returns ``(y, new_residual)``; with
    the two-shot forms both live in registered memory."""
    if comm.world == 1:
        return rmsnorm(x, weight, eps, residual, out=out, residual_out=residual_out)
    loc = comm._locate(x)
    if loc is None:
        raise ValueError("x must live in registered memory (comm.empty / slot pools / comm.register)")
    rows, hidden = x.shape
    nbytes = x.numel() * x.element_size()
    piece = (nbytes + 255) // 256 * 256
    if algo is None:
        # Decode-sized messages: every rank pushes its rows to all ranks, one barrier, every rank sums and normalises
        # every row locally (measured on 8 x B200 at 16 - 256 KiB: the one-shot fused kernel, whose single CTA per row
        # pulls every peer's copy between two barriers, took 34 - 40 us; push all-reduce + local norm 19 - 22 us).
        ll = getattr(comm, "_ll_arena", None)
        if (not getattr(comm, "emulated", False) and ll is not None and nbytes <= comm.config.ll_max_bytes
                and 2 * piece <= ll[1]):
            algo = _lib.NORM_AR_LL  # a few rows: cells of data + call number, no barrier at all
        elif (not getattr(comm, "emulated", False) and nbytes <= comm.config.push_max_bytes
                and comm._push_staging(piece) is not None):
            algo = _lib.NORM_AR_PUSH_NVLS if comm.nvls else _lib.NORM_AR_PUSH
        elif rows < comm.world:
            algo = _lib.NORM_AR_ONESHOT
        else:
            algo = _lib.NORM_AR_TWOSHOT_NVLS if (comm.nvls and loc[0] == 0) else _lib.NORM_AR_TWOSHOT
    a = _lib.NormArgs()
    a.dtype, a.rows, a.hidden, a.eps = dtype_code(x.dtype), rows, hidden, eps
    a.x_reg, a.x_off = loc
    a.residual = residual.data_ptr() if residual is not None else None
    a.weight = weight.data_ptr()
    a.res_out_reg = -1
    if algo in (_lib.NORM_AR_ONESHOT, _lib.NORM_AR_PUSH, _lib.NORM_AR_PUSH_NVLS, _lib.NORM_AR_LL):
        y = out if out is not None else torch.empty_like(x)
        ro = residual_out if residual_out is not None else torch.empty_like(x)
        a.y_local, a.res_out_local = y.data_ptr(), ro.data_ptr()
        if algo == _lib.NORM_AR_LL:
            ll = getattr(comm, "_ll_arena", None)
            if ll is None or 2 * piece > ll[1]:
                raise ValueError("no flag-in-data staging area of that size (init_round_robin_slots, config.ll_max_bytes)")
            a.stage_reg, a.stage_off, a.piece_bytes = 0, ll[0], ll[1]
        elif algo != _lib.NORM_AR_ONESHOT:
            stage = comm._push_staging(piece)
            if stage is None:
                raise ValueError("message too large for the staging area of the push kernels (config.push_max_bytes)")
            a.stage_reg, a.stage_off, a.piece_bytes = 0, stage, piece
    else:
        y = out if out is not None and comm.heap_offset(out) is not None else comm.scratch_view(
            ("norm_y", x.dtype, tuple(x.shape)), x.shape, x.dtype)
        ro = residual_out if residual_out is not None and comm.heap_offset(residual_out) is not None else (
            comm.scratch_view(("norm_r", x.dtype, tuple(x.shape)), x.shape, x.dtype))
        a.y_reg, a.y_off = 0, comm.heap_offset(y)
        a.res_out_reg, a.res_out_off = 0, comm.heap_offset(ro)
    # One row per CTA at a time: a large message needs many CTAs to keep enough loads in flight through the switch.
    _lib.check(_lib.lib().oob_fused_norm(comm._h, algo, ctypes.byref(a), max_ctas or (32 if nbytes <= (1 << 20) else 128),
                                         _stream()))
    return y, ro


def fused_reduce_scatter_rmsnorm(comm, x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                                 residual: Optional[torch.Tensor] = None, *, max_ctas: int = 0):
    """Sequence-parallel form: rank r gets ``rmsnorm(sum_ranks(x)[rows of r] + residual) * weight``.
    ``residual`` holds only this rank's rows.  Returns ``(y, new_residual)`` of shape [rows_of_rank, hidden]."""
    loc = comm._locate(x)
    if loc is None:
        raise ValueError("x must live in registered memory")
    rows, hidden = x.shape
    b, e = partition(rows, comm.world, comm.rank)
    y = torch.empty((e - b, hidden), dtype=x.dtype, device=x.device)
    ro = torch.empty_like(y)
    a = _lib.NormArgs()
    a.dtype, a.rows, a.hidden, a.eps = dtype_code(x.dtype), rows, hidden, eps
    a.x_reg, a.x_off = loc
    a.residual = residual.data_ptr() if residual is not None else None
    a.weight = weight.data_ptr()
    a.y_local, a.res_out_local = y.data_ptr(), ro.data_ptr()
    a.res_out_reg = -1
    algo = _lib.NORM_RS_NVLS if (comm.nvls and loc[0] == 0) else _lib.NORM_RS
    _lib.check(_lib.lib().oob_fused_norm(comm._h, algo, ctypes.byref(a), max_ctas or 32, _stream()))
    return y, ro
