"""Single-GPU emulation of a multi-rank group.

All ranks' heaps live on one device and every collective (or fused GEMM) is
ONE cooperative launch whose block rows act as the ranks, so the multi-rank
kernels — flags, barriers, peer loads and stores, counters — run unchanged on a
machine with a single GPU.  Separate launches that wait on one another are
never used for this (they are not guaranteed to be co-resident).

"Local" (unregistered) operands of rank r are row r of a stacked tensor.

Capability parity: the reference's same-process multi-device mode
(``oo_group_create_p2p``, src/comm/ooverlap_comm_public.cu:707-849) doubles as
its test and tuning harness; it needs one GPU per rank.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from .comm import tensor_from_ptr
from .utils.dtypes import dtype_code, op_code
from .utils.partition import max_shard


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class EmulatedGroup:
    def __init__(self, world: int, device: int = 0, heap_bytes: int = 256 << 20, timeout_ms: int = 5000):
        self.world = world
        self.device = device
        self.emulated = True
        self.nvls = False
        self.rank = 0
        self._counter_next = 0
        h = ctypes.c_void_p()
        _lib.check(_lib.lib().oob_comm_create_emulated(world, device, heap_bytes, ctypes.byref(h)))
        self._h = h
        _lib.check(_lib.lib().oob_comm_set_timeout_ms(h, timeout_ms))
        info = _lib.CommInfo()
        _lib.check(_lib.lib().oob_comm_info(h, ctypes.byref(info)))
        self.heap_bytes = int(info.heap_bytes)

    def close(self) -> None:
        if self._h is not None:
            _lib.lib().oob_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # heap -----------------------------------------------------------------
    def alloc(self, nbytes: int, align: int = 1024) -> int:
        off = ctypes.c_uint64()
        _lib.check(_lib.lib().oob_alloc(self._h, int(nbytes), int(align), ctypes.byref(off)))
        return int(off.value)

    def free(self, offset: int) -> None:
        _lib.check(_lib.lib().oob_free(self._h, offset))

    def view(self, offset: int, shape, dtype: torch.dtype, rank: int) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        ptr = int(_lib.lib().oob_heap_ptr(self._h, rank, offset))
        return tensor_from_ptr(ptr, nbytes, self.device, self).view(dtype).view(shape)

    def counters(self, rank: int) -> torch.Tensor:
        """The general arrival counters of ``rank``'s signal pad (int32 view): every fused op re-arms the ones it
        used, so they read zero between launches (the check the reference does with
        tool/verify_signal_tile_counts.py:108+ on its tile counters)."""
        lib = _lib.lib()
        return self.view(int(lib.oob_pad_counter_offset()), (int(lib.oob_pad_counter_count()),), torch.int32, rank)

    def views(self, offset: int, shape, dtype: torch.dtype) -> list:
        return [self.view(offset, shape, dtype, r) for r in range(self.world)]

    def reserve_counters(self, n: int) -> int:
        base = self._counter_next
        self._counter_next += n
        return base

    def release_counters(self, base: int) -> None:
        if 0 <= base < self._counter_next:
            self._counter_next = base

    def check_status(self) -> None:
        torch.cuda.synchronize(self.device)
        _lib.check(_lib.lib().oob_comm_status(self._h, None))

    def status(self) -> _lib.DeviceStatus:
        torch.cuda.synchronize(self.device)
        s = _lib.DeviceStatus()
        _lib.lib().oob_comm_status(self._h, ctypes.byref(s))
        return s

    def recover(self) -> None:
        _lib.check(_lib.lib().oob_comm_recover(self._h))

    def set_timeout_ms(self, ms: int) -> None:
        _lib.check(_lib.lib().oob_comm_set_timeout_ms(self._h, ms))

    def bounded_wait_selftest(self) -> None:
        _lib.check(_lib.lib().oob_test_bounded_wait(self._h, _stream()))

    # collectives ------------------------------------------------------------
    def all_reduce(self, in_off: int, count: int, dtype: torch.dtype, op: str = "sum", *, algo: int,
                   out_off: Optional[int] = None, out_local: Optional[torch.Tensor] = None, max_ctas: int = 4) -> None:
        """``out_local`` is a ``[world, count]`` tensor for the one-shot algorithms."""
        _lib.check(_lib.lib().oob_allreduce(
            self._h, dtype_code(dtype), op_code(op), algo, 0, in_off, 0 if out_off is not None else -1, out_off or 0,
            ctypes.c_void_p(out_local.data_ptr()) if out_local is not None else None, count, max_ctas, _stream()))

    def all_reduce_push(self, stage_off: int, piece_bytes: int, x: torch.Tensor, out: torch.Tensor, op: str = "sum", *,
                        max_ctas: int = 4) -> None:
        """One-barrier push all-reduce: ``x`` and ``out`` are ``[world, count]`` (row r = rank r's input / result),
        the staging area is two sets of ``world * piece_bytes`` at ``stage_off`` of every rank's heap (consecutive calls
        alternate between the sets, decided on the device)."""
        assert x.shape[0] == self.world and out.shape == x.shape and x.is_contiguous() and out.is_contiguous()
        _lib.check(_lib.lib().oob_allreduce_push(self._h, dtype_code(x.dtype), op_code(op), 0, stage_off, piece_bytes,
                                                 ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                                 x.shape[1], 0, max_ctas, _stream()))

    def all_reduce_ll(self, stage_off: int, piece_bytes: int, x: torch.Tensor, out: torch.Tensor, op: str = "sum", *,
                      max_ctas: int = 4) -> None:
        """Flag-in-data all-reduce without a barrier: ``x`` and ``out`` are ``[world, count]``; the staging area is two
        sets of ``world * piece_bytes`` (8 bytes per 32-bit word of a row) at ``stage_off`` of every rank's heap and
        must be zero before its first use and again after ``recover()`` (the call numbers restart from zero)."""
        assert x.shape[0] == self.world and out.shape == x.shape and x.is_contiguous() and out.is_contiguous()
        _lib.check(_lib.lib().oob_allreduce_ll(self._h, dtype_code(x.dtype), op_code(op), 0, stage_off, piece_bytes,
                                               ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                               x.shape[1], 0, max_ctas, _stream()))

    def reduce_scatter(self, in_off: int, count: int, dtype: torch.dtype, out_local: torch.Tensor, op: str = "sum", *,
                       algo: int = _lib.RS_P2P, max_ctas: int = 4) -> None:
        """``out_local`` is ``[world, ceil(count / world)]``; row r receives rank r's partition."""
        assert out_local.shape[0] == self.world and out_local.shape[1] == max_shard(count, self.world)
        _lib.check(_lib.lib().oob_reduce_scatter(self._h, dtype_code(dtype), op_code(op), algo, 0, in_off,
                                                 ctypes.c_void_p(out_local.data_ptr()), count, max_ctas, _stream()))

    def all_gather(self, out_off: int, count: int, dtype: torch.dtype, *, src_local: Optional[torch.Tensor] = None,
                   dst_local: Optional[torch.Tensor] = None, algo: int = _lib.AG_PUSH_P2P, max_ctas: int = 4) -> None:
        """Push: ``src_local`` is ``[world, ceil(count / world)]`` (row r = rank r's shard) and the gathered
        buffer is the heap region at ``out_off`` of every rank.  Pull: the heap region holds each rank's shard
        and ``dst_local`` is ``[world, count]``."""
        _lib.check(_lib.lib().oob_all_gather(
            self._h, dtype_code(dtype), algo, 0, out_off,
            ctypes.c_void_p(src_local.data_ptr()) if src_local is not None else None,
            ctypes.c_void_p(dst_local.data_ptr()) if dst_local is not None else None, count, max_ctas, _stream()))

    def all_to_all(self, out_off: int, count_per_peer: int, dtype: torch.dtype, src_local: torch.Tensor, *,
                   max_ctas: int = 4) -> None:
        """``src_local`` is ``[world (sender), world (destination), count_per_peer]``; afterwards the heap region at
        ``out_off`` of rank j holds ``[world (sender), count_per_peer]``."""
        _lib.check(_lib.lib().oob_all_to_all(self._h, dtype_code(dtype), 0, out_off, ctypes.c_void_p(src_local.data_ptr()),
                                             count_per_peer, max_ctas, _stream()))

    def fused_norm(self, algo: int, *, x_off: int, rows: int, hidden: int, dtype: torch.dtype, weight: torch.Tensor,
                   eps: float, residual: Optional[torch.Tensor] = None, y_off: Optional[int] = None,
                   y_local: Optional[torch.Tensor] = None, res_out_off: Optional[int] = None,
                   res_out_local: Optional[torch.Tensor] = None, local_stride_bytes: int = 0, max_ctas: int = 8,
                   stage_off: Optional[int] = None, piece_bytes: int = 0) -> None:
        a = _lib.NormArgs()
        a.dtype, a.rows, a.hidden, a.eps = dtype_code(dtype), rows, hidden, eps
        a.x_reg, a.x_off = 0, x_off
        a.residual = residual.data_ptr() if residual is not None else None
        a.weight = weight.data_ptr()
        a.y_reg, a.y_off = 0, y_off or 0
        a.y_local = y_local.data_ptr() if y_local is not None else None
        a.res_out_reg = 0 if res_out_off is not None else -1
        a.res_out_off = res_out_off or 0
        a.res_out_local = res_out_local.data_ptr() if res_out_local is not None else None
        a.emu_stride_local = local_stride_bytes
        a.stage_reg, a.stage_off, a.piece_bytes = 0, stage_off or 0, piece_bytes  # push algorithms only
        _lib.check(_lib.lib().oob_fused_norm(self._h, algo, ctypes.byref(a), max_ctas, _stream()))
