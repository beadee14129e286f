"""Plain tcgen05 GEMM: ``C[M, N] = A[M, K] @ B[N, K]^T`` (B in torch ``Linear.weight`` layout).

Capability parity: ``gemm_plain_sm90_dispatch`` / the cuBLAS column GEMM of the
reference's legacy binding (src/gemm/gemm_plain_sm90_dispatch.h:19-46,
src/pybind.cpp:266-324).  One hand-written sm_100a kernel replaces the 122
generated CUTLASS instances.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib
from . import solutions
from ..utils.dtypes import dtype_code


def _check_operands(a: torch.Tensor, b: torch.Tensor) -> None:
    if a.dtype not in (torch.float16, torch.bfloat16) or a.dtype != b.dtype:
        raise TypeError("GEMM operands must both be fp16 or both bf16")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"shape mismatch: A {tuple(a.shape)} x B^T {tuple(b.shape)}")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("A and B must be row-major (unit stride along K)")
    if not a.is_cuda or not b.is_cuda:
        raise ValueError("GEMM operands must be CUDA tensors")


def fill_gemm_args(args: _lib.GemmArgs, a: torch.Tensor, b: torch.Tensor) -> None:
    args.dtype = dtype_code(a.dtype)
    args.M, args.K = a.shape
    args.N = b.shape[0]
    args.A, args.lda = a.data_ptr(), a.stride(0)
    args.B, args.ldb = b.data_ptr(), b.stride(0)


def gemm(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *, max_ctas: int = 0,
         splits: int = 0, pair: int = 0, skinny: int = 0, splitk_reduce: int = 0,
         gemv: int = 0, stream_k: int = 0, order: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = a @ b.T`` with fp32 accumulation in TMEM.

    ``order`` (two-SM kernel): an int64 CUDA tensor ``[2 * tiles, 2]`` (``tiles`` = 256x256 tiles of the output) that
    the kernel fills with the tile-order record: per 128-row half of every tile the globaltimer nanoseconds at which
    it was stored and ``pair << 32 | index in the pair's sequence``; see :func:`tile_order`.

    ``splits`` > 1 splits K over that many CTAs per output tile (fp32 partials in the library's workspace,
    summed in split order); 0 picks a split from the shape (small-M problems that would otherwise leave most
    SMs idle), 1 turns it off.

    ``pair`` selects the two-SM kernel (256x256 tiles computed by CTA pairs with ``tcgen05.mma.cta_group::2``; each
    CTA stages half of the B block): 0 uses it for unsplit problems with more than 128 rows, 1 whenever the problem
    is unsplit, -1 never.

    ``stream_k`` (two-SM kernel): when the tile count is not a multiple of the pair count, the last wave and the
    remainder are cut along K into equal ranges, one per pair, so that no pair idles; pairs that compute part of a tile
    park fp32 accumulators in a library-owned workspace and the part that arrives last sums them in pair order
    (bit-reproducible).  0 uses it when the idle share would exceed 3 % of the run, 1 whenever there is a remainder,
    -1 never.

    ``skinny`` selects the weight-streaming kernel for ``M <= 128`` (the weight rows fill the tensor-core
    instruction's 128-row dimension, the tokens are its narrow dimension; stream-K split, deterministic) with 1.
    It is opt-in: measured inside a decode step the tiled split-K path is a little faster at every ``M``.

    ``splitk_reduce`` says where a split-K sum is taken: -1 inside the GEMM kernel (the warp that delivers the last
    partial of a 32-row quadrant), 0 or 1 in a second kernel launched right after it (faster at every ``M``).
    The order of summation, and so the result, is the same.

    ``gemv`` = 1 uses the CUDA-core streaming kernel for ``M <= 4`` (a warp per weight row, no tensor cores, no
    split-K hand-off); 0 uses it where it measured faster (one row; two rows with ``N * K`` up to 12 M), -1 never."""
    _check_operands(a, b)
    M, N = a.shape[0], b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    elif out.shape != (M, N) or out.dtype != a.dtype or out.stride(1) != 1:
        raise ValueError("bad output tensor")
    if not (splits or pair or skinny or gemv or stream_k or max_ctas):
        # Nothing asked for: a profiled configuration for exactly this shape (bench.gemm_profile) beats the rule.
        sol = solutions.lookup_gemm(M, N, a.shape[1], "bf16" if a.dtype == torch.bfloat16 else "fp16")
        if sol is not None:
            splits, pair, skinny = int(sol.get("splits", 0)), int(sol.get("pair", 0)), int(sol.get("skinny", 0))
            gemv, stream_k = int(sol.get("gemv", 0)), int(sol.get("stream_k", 0))
    args = _lib.GemmArgs()
    args.mode = _lib.GEMM_PLAIN
    fill_gemm_args(args, a, b)
    args.C, args.ldc = out.data_ptr(), out.stride(0)
    args.max_ctas = max_ctas
    args.splits = splits
    args.pair = pair
    args.skinny = skinny
    args.splitk_reduce = splitk_reduce
    args.gemv = gemv
    args.stream_k = stream_k
    if order is not None:
        check_order_buffer(order, M, N)
        args.order = order.data_ptr()
    _lib.check(_lib.lib().oob_gemm(None, ctypes.byref(args), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return out


def order_buffer(M: int, N: int, device="cuda") -> torch.Tensor:
    """A zeroed tile-order record for an [M, N] output of the two-SM kernel (``order=`` of :func:`gemm`,
    ``order_buffer`` of the overlap ops)."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    return torch.zeros((2 * tiles, 2), dtype=torch.int64, device=device)


def check_order_buffer(order: torch.Tensor, M: int, N: int) -> None:
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if order.dtype != torch.int64 or not order.is_cuda or not order.is_contiguous() or order.numel() < 4 * tiles:
        raise ValueError(f"order must be a contiguous int64 CUDA tensor of at least {2 * tiles} x 2 words")


def tile_order(order: torch.Tensor) -> list:
    """Decodes a tile-order record into a list of dicts sorted by completion time: ``unit`` (2 * tile's number in the
    schedule + CTA of the pair), ``t_us`` (microseconds after the first completion), ``pair`` and ``index`` (the
    tile's position in that pair's own sequence).  Halves the kernel never wrote (rows past M) are left out.

    Capability parity: the reference records in which order its GEMM finishes tiles to derive reorder hints
    (tool/search.py, the tile-order capture of src/gemm/gemm_with_signal_sm90.h); here the schedule is fixed by the
    kernel (PairSched) and the record shows how the hardware actually ran it."""
    rows = order.detach().cpu().tolist()
    done = [(t, u, w) for u, (t, w) in enumerate(rows) if t > 0]
    if not done:
        return []
    t0 = min(t for t, _, _ in done)
    return [dict(unit=u, t_us=(t - t0) / 1e3, pair=int(w >> 32), index=int(w & 0xFFFFFFFF)) for t, u, w in sorted(done)]


def stable_tile_waves(records, wave: int) -> dict:
    """Compares the tile-order records of several launches of one shape (each the output of :func:`tile_order`, or a
    plain list of unit numbers in completion order) and reports what is reproducible about the order.

    ``wave`` is the number of units that complete together (CTAs of the GEMM grid; for the two-SM kernel
    2 x pairs, since every CTA of a pair records its half).  A unit's wave in a launch is its position in the
    completion order divided by ``wave``.  Returns ``waves`` (per unit: its wave when that is the same in every
    launch, else -1), ``stable_fraction``, ``hint`` (all units ordered by their median wave, then by number: an order
    that a consumer may rely on at wave granularity) and ``min_group_waves`` (the smallest g such that every unit stays
    inside the same group of g consecutive waves in every launch: the finest chunking of the output by completion
    time that holds from launch to launch).

    Capability parity: the monitor rounds of the reference's search (tool/search.py:639-754) keep the tiles that land
    in the same wave window every time and derive a stable order and a minimum group size from them.  The fused
    kernels of this library signal every tile on its own and need no such hint; the analysis is for diagnosis and for
    choosing slab boundaries of the ``chunked`` strategy."""
    if wave < 1:
        raise ValueError("wave must be at least 1")
    orders = [[(r["unit"] if isinstance(r, dict) else int(r)) for r in rec] for rec in records]
    if not orders or not orders[0]:
        return dict(waves=[], stable_fraction=0.0, hint=[], min_group_waves=0)
    units = sorted(orders[0])
    if any(sorted(o) != units for o in orders):
        raise ValueError("the records do not cover the same units")
    pos = [{u: i // wave for i, u in enumerate(o)} for o in orders]
    per_unit = {u: [p[u] for p in pos] for u in units}
    waves = [per_unit[u][0] if len(set(per_unit[u])) == 1 else -1 for u in units]
    n_waves = (len(units) + wave - 1) // wave
    g = 1
    while g < n_waves and any(len({w // g for w in ws}) > 1 for ws in per_unit.values()):
        g += 1
    median = {u: sorted(ws)[len(ws) // 2] for u, ws in per_unit.items()}
    return dict(waves=waves, stable_fraction=sum(1 for w in waves if w >= 0) / len(units),
                hint=sorted(units, key=lambda u: (median[u], u)), min_group_waves=g)


def reserve_workspace(splitk_bytes: int = 0) -> None:
    """Allocates the library's GEMM scratch on the current device now: the stream-K workspace of the two-SM kernel and,
    when ``splitk_bytes`` > 0, a split-K workspace of that size (see :func:`splitk_workspace_bytes`).  Call it before
    capturing a CUDA graph: nothing can be allocated during capture, and a GEMM that would need to grow its workspace
    then fails instead."""
    _lib.check(_lib.lib().oob_gemm_reserve_workspace(int(splitk_bytes)))


def splitk_workspace_bytes(M: int, N: int, K: int, *, max_ctas: int = 0, splits: int = 0) -> int:
    """Split-K workspace bytes :func:`gemm` needs for this shape (0 when the problem is not split)."""
    return int(_lib.lib().oob_gemm_splitk_bytes(M, N, K, max_ctas, splits))


def gemm_plan_splits(M: int, N: int, K: int, *, max_ctas: int = 0, splits: int = 0) -> int:
    """Number of K splits :func:`gemm` uses for this shape (1 = the problem is not split)."""
    return int(_lib.lib().oob_gemm_plan_splits(M, N, K, max_ctas, splits))


def gemm_swiglu(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *, max_ctas: int = 0,
                fused: Optional[bool] = None) -> torch.Tensor:
    """``silu(a @ b[:F].T) * (a @ b[F:].T)`` for a gate/up weight ``b`` of shape [2F, K]; returns [M, F].

    When the GEMM is one that is split over K (every decode-step shape), the activation is applied by the kernel
    that sums the splits: no separate launch and no 16-bit round trip of the [M, 2F] intermediate.  Otherwise, or
    with ``fused=False``, the GEMM is followed by the stand-alone SwiGLU kernel."""
    from .decode import silu_mul
    _check_operands(a, b)
    M, N = a.shape[0], b.shape[0]
    if N % 16 != 0:
        raise ValueError("the gate/up weight must have 2F rows with F a multiple of 8")
    F = N // 2
    if out is None:
        out = torch.empty((M, F), dtype=a.dtype, device=a.device)
    elif out.shape != (M, F) or out.dtype != a.dtype or out.stride(1) != 1 or out.stride(0) % 8 != 0:
        raise ValueError("bad output tensor")
    can_fuse = gemm_plan_splits(M, N, a.shape[1], max_ctas=max_ctas) > 1
    if fused is None:
        fused = can_fuse
    if fused and not can_fuse:
        raise ValueError("this problem is not split over K, so the epilogue has no kernel to run in")
    if not fused:
        return silu_mul(gemm(a, b, max_ctas=max_ctas), out)
    epi = _lib.SwigluEpilogue()
    epi.F = F
    args = _lib.GemmArgs()
    args.mode = _lib.GEMM_PLAIN
    fill_gemm_args(args, a, b)
    args.C, args.ldc = out.data_ptr(), out.stride(0)
    args.max_ctas = max_ctas
    args.skinny = -1
    args.epilogue = _lib.EPILOGUE_SWIGLU
    args.epilogue_args = ctypes.cast(ctypes.pointer(epi), ctypes.c_void_p)
    _lib.check(_lib.lib().oob_gemm(None, ctypes.byref(args), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return out
