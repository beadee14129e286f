"""GEMM + collective overlap ops (one fused sm_100a kernel each).

* :class:`GemmAllReduce` — row-parallel linear: ``C = sum_ranks(A_r @ B_r^T)`` on every rank.
* :class:`GemmReduceScatterNorm` — ``y_rows_of_rank = rmsnorm(sum_ranks(A_r @ B_r^T) + residual) * w``.
* :class:`AllGatherGemm` — column-parallel linear: ``C = allgather_rows(A_shard) @ B^T``.

Each object owns the registered buffers (tile-packed partial products, output,
gathered operand) and the arrival counters of its shape, so calls are a single
kernel launch with fixed addresses (CUDA-graph friendly).

Capability parity: ``OverlapImpl::GemmAllReduceOverlap`` /
``GemmReduceScatterOverlap`` of the reference (src/overlap_impl.cu:450-706) and
its Python driver (test/test.py:509-676).  The segment search, reorder maps and
the separate wait kernel are gone: the GEMM epilogue signals per tile and
reducer CTAs of the same launch stream the reduction over NVSwitch.  The
RMSNorm tail and AllGather->GEMM have no counterpart there.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib
from ..utils.logging import logger
from ..utils.partition import partition
from .gemm import _check_operands, fill_gemm_args, gemm

TILE_M = 128


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _emulated(comm) -> bool:
    return bool(getattr(comm, "emulated", False))


def _use_nvls(comm, choice) -> int:
    """NVLS (in-switch reduction / broadcast) pays off from four ranks on; between two GPUs plain peer
    stores are faster.  ``choice`` overrides the default: False / 0 = peer pushes only, True / 1 = peer pushes of the
    partial tiles + multimem.st of the result, 2 = partial tiles stay local and the owner reduces them inside the
    switch (multimem.ld_reduce), which moves the message once per direction instead of 1.75 times."""
    if not getattr(comm, "nvls", False):
        return 0
    if choice is None:
        return 2 if comm.world >= 4 else 0
    if choice is True:
        return 1
    return int(choice)  # 0 = peer pushes only, 1 = push + multimem.st, 2 = in-switch reduce (pull) + multimem.st


_KERNELS = {None: 0, "auto": 0, "pair": 1, "one_sm": -1}


def _kernel_code(kernel) -> int:
    """``kernel``: None / "auto" = the two-SM (CTA pair, 256x256 tiles) kernel whenever it supports the shape, "pair" =
    the same, asked for explicitly, "one_sm" = the one-SM kernel (128x256 tiles; partial tiles are pushed to their owner
    rank with bulk tensor stores)."""
    if kernel not in _KERNELS:
        raise ValueError(f"kernel must be one of {sorted(k for k in _KERNELS if k)}")
    return _KERNELS[kernel]


def _operands(comm, a: torch.Tensor, b: torch.Tensor):
    """In emulation ``a`` and ``b`` are stacked ``[world, ...]``; returns (a0, b0, a_stride, b_stride)."""
    if _emulated(comm):
        if a.dim() != 3 or b.dim() != 3 or a.shape[0] != comm.world or b.shape[0] != comm.world:
            raise ValueError("emulated group: operands must be stacked [world, rows, K]")
        return a[0], b[0], a.stride(0) * a.element_size(), b.stride(0) * b.element_size()
    return a, b, 0, 0


def plan_gemm_all_reduce(world: int, M: int, N: int, emulated: bool, strategy: str = "auto", chunks: Optional[int] = None,
                         use_nvls=None, comm_ctas: Optional[int] = None, solution: Optional[dict] = None,
                         kernel: Optional[str] = None):
    """Resolves what :class:`GemmAllReduce` will run: ``(strategy, chunks, use_nvls, comm_ctas, kernel)`` with
    ``strategy`` one of fused / unfused / chunked and ``kernel`` one of None (the library's default), "pair", "one_sm".
    Pure function of its arguments (``solution`` is a tuned entry for the shape, or None), so that the rule can be read
    and tested without a GPU.  What the caller fixed (``use_nvls``, ``comm_ctas``, ``kernel``) is never overridden."""
    if strategy not in ("auto", "fused", "unfused", "chunked"):
        raise ValueError(strategy)
    if strategy == "auto" and solution is not None and not emulated:
        strategy = solution.get("strategy", "auto")
        if strategy not in ("auto", "fused", "unfused", "chunked"):
            raise ValueError(f"solution names an unknown strategy {strategy!r}")
        if comm_ctas is None and solution.get("comm_ctas"):
            comm_ctas = int(solution["comm_ctas"])
        if use_nvls is None and "use_nvls" in solution and solution["use_nvls"] is not None:
            use_nvls = int(solution["use_nvls"])
        if chunks is None and solution.get("chunks"):
            chunks = int(solution["chunks"])
        if kernel is None and solution.get("kernel"):
            kernel = str(solution["kernel"])
    if strategy == "auto":
        strategy, nv, ctas, kern = _auto_rule(world, M * N * 2, emulated)
        if use_nvls is None:
            use_nvls = nv
        if comm_ctas is None:
            comm_ctas = ctas
        if kernel is None:
            kernel = kern
    if strategy == "chunked":
        if chunks is None:
            chunks = M // 2048 if M % 2048 == 0 else 1  # slabs of 2048 rows: several waves of tiles each
        if chunks < 1 or M % chunks:
            raise ValueError("M must be a multiple of the number of chunks")
        if emulated:
            strategy = "fused"  # one launch per op in emulation
        elif world < 2 or chunks == 1:
            strategy = "unfused"  # nothing to pipeline against
    if strategy != "chunked":
        chunks = 1
    return strategy, chunks, use_nvls, comm_ctas, kernel


def _auto_rule(world: int, out_bytes: int, emulated: bool):
    """The measured choices on B200 / NVSwitch: (strategy, use_nvls, comm_ctas, kernel); None = the op's default.

    * emulation: one launch per op, so always fused;
    * two ranks: fused; outputs of 64 MiB and more on the two-SM kernel reducing in place through the switch with 24
      communication CTAs, smaller ones on the one-SM kernel that pushes partial tiles (it starts reducing earlier, which
      is what counts for one or two waves of tiles);
    * four ranks (measured): up to 16 MiB the one-SM kernel with pushed tiles (59 us at M = 512); above that the two-SM
      kernel reducing in place through the switch with 16 communication CTAs (130 / 360 us at M = 2048 / 8192 against
      150 / 500 us for the GEMM followed by the all-reduce);
    * eight ranks (measured): up to 16 MiB the one-SM kernel with the in-switch pull (59 against 78 us unfused at
      M = 512); up to 64 MiB this library's GEMM followed by its in-switch all-reduce (131 us at M = 2048; the fused
      variants are within 2 %); above that the two-SM kernel reducing in place through the switch with 8 communication
      CTAs (374 against 393 us unfused at M = 8192)."""
    big = out_bytes > (64 << 20)
    if emulated:
        return "fused", None, None, None
    if world < 4:
        return ("fused", 1, 24, "pair") if big else ("fused", None, 16, "one_sm")
    if world < 8:
        return ("fused", 0, 16, "one_sm") if out_bytes <= (16 << 20) else ("fused", 1, 16, "pair")
    if big:
        return "fused", 1, 8, "pair"
    if out_bytes <= (16 << 20):
        return "fused", 2, 16, "one_sm"
    return "unfused", None, None, None


class GemmAllReduce:
    """Row-parallel linear: ``C = sum_ranks(A_r @ B_r^T)`` in every rank's registered memory.

    ``strategy``:
      * ``"fused"``   one kernel: the epilogue pushes partial tiles to their owner rank, communication CTAs (and GEMM
                      CTAs that ran out of tiles) reduce and broadcast them while later tiles still compute;
      * ``"unfused"`` this library's GEMM writes into the registered output, then its all-reduce kernel runs on it
                      (the policy picks one-shot / two-shot / NVLS and the CTA budget);
      * ``"chunked"`` the rows are cut into ``chunks`` slabs (default: slabs of 2048 rows; a single slab means unfused); slab i is computed by this library's GEMM on the
                      caller's stream and all-reduced (in-switch two-shot, a handful of CTAs) on a side stream while
                      the GEMM of slab i + 1 runs on the other SMs: the all-reduce moves each byte once per direction
                      through the switch, which the fused kernel's peer pushes cannot, and only the first GEMM slab
                      is exposed.  For large M from four ranks on;
      * ``"autotune"`` decided at the first call: every fused variant and the unfused pair are checked and timed on the
                      real operands, all ranks agree on the fastest (see ``_autotune``; ``tuning`` holds the table);
      * ``"auto"``    (default) a tuned solution for the shape when one is packaged or named by
                      ``OOB_OVERLAP_SOLUTIONS``, else the rule derived from the measurements on B200 / NVSwitch
                      (``_auto_rule``): small outputs on the one-SM fused kernel, large ones on the two-SM fused kernel
                      that reduces in place through the switch, and at eight ranks the unfused pair in between.

    ``kernel`` picks the fused kernel: "pair" (two-SM mainloop, 256x256 tiles; the epilogue writes the partial product
    into this rank's copy of the output, reducers reduce it in place: ``use_nvls`` 1 = through the switch, 0 = peer
    loads and stores) or "one_sm" (128x256 tiles pushed to their owner rank; ``use_nvls`` 0 = peer pushes + peer
    broadcast, 1 = multimem broadcast of the result, 2 = tiles stay local and the owner pulls their in-switch sum).
    """

    def __init__(self, comm, M: int, N: int, dtype: torch.dtype, *, comm_ctas: Optional[int] = None, max_ctas: int = 0,
                 use_nvls=None, strategy: str = "auto", chunks: Optional[int] = None, kernel: Optional[str] = None):
        self.comm, self.M, self.N, self.dtype = comm, M, N, dtype
        self.max_ctas = max_ctas
        self.kernel = _kernel_code(kernel)
        self.multi = comm.world > 1
        self._tuned = None
        self.tuning = None
        if strategy == "autotune":
            if self.multi and not _emulated(comm):
                # Decided at the first call, on the real operands (K is not known before): see _autotune.
                self.strategy, self.chunks, self.use_nvls = "autotune", 1, use_nvls
                self.comm_ctas = comm_ctas or 0
                self._tune_args = dict(max_ctas=max_ctas, kernel=kernel)
                return
            strategy = "auto"
        sol = None
        if strategy == "auto" and not _emulated(comm):
            # A tuned solution for this shape (OOB_OVERLAP_SOLUTIONS, written by bench.tune_overlap) wins.
            from . import solutions
            sol = solutions.lookup("gemm_ar", M, N, 0, comm.world, "bf16" if dtype == torch.bfloat16 else "fp16")
        strategy, chunks, use_nvls, comm_ctas, planned_kernel = plan_gemm_all_reduce(
            comm.world, M, N, _emulated(comm), strategy, chunks, use_nvls, comm_ctas, sol, kernel)
        self.kernel = _kernel_code(planned_kernel)
        self.chunks = chunks
        self.strategy = strategy
        self.use_nvls = use_nvls
        self.comm_ctas = comm_ctas if comm_ctas is not None else (20 if comm.world < 4 else 16)
        if self.multi:
            lib = _lib.lib()
            self.c_off = comm.alloc(M * N * 2)
            self._out = None if _emulated(comm) else comm.view(self.c_off, (M, N), dtype)
            if self.strategy == "fused":
                try:
                    self.partial_off = comm.alloc(int(lib.oob_gemm_partial_bytes(M, N)))
                    try:
                        self.counter_base = comm.reserve_counters(lib.oob_gemm_counters_needed(_lib.GEMM_AR, M, N, comm.world))
                    except Exception:
                        comm.free(self.partial_off)
                        raise
                except Exception:  # nothing of a half-built op stays allocated (every rank fails alike)
                    comm.free(self.c_off)
                    self.multi = False
                    raise
            if self.strategy == "chunked":
                self._side = torch.cuda.Stream()
                self._slab_done = [torch.cuda.Event() for _ in range(self.chunks)]
                self._joined = torch.cuda.Event()

    @property
    def fused(self) -> bool:
        return self.multi and self.strategy == "fused"

    # ------------------------------------------------------------------------------------------------ autotune
    def _candidates(self):
        """(strategy, kernel, use_nvls, comm_ctas) to try: the unfused pair; the two-SM kernel over a few CTA budgets,
        through the switch when the heap has a multicast alias (and with peer loads/stores between two ranks, where
        both move the same bytes); the one-SM kernel with pushed partial tiles (and, from four ranks on, with the
        in-switch pull); from four ranks on and for tall outputs also the slab pipeline on two streams."""
        nvls = bool(getattr(self.comm, "nvls", False))
        world = self.comm.world
        cands = [("unfused", None, None, None)]
        budgets = [4, 8, 16, 24, 32]
        aligned = wave_aligned_comm_ctas(self.M, self.N)
        if aligned not in budgets:
            budgets = sorted(budgets + [aligned])  # the largest budget that costs the GEMM no extra wave of tiles
        for c in budgets:
            if nvls:
                cands.append(("fused", "pair", 1, c))
            if not nvls or world == 2:
                cands.append(("fused", "pair", 0, c))
        cands.append(("fused", "one_sm", 0, 16))
        if nvls and world >= 4:
            cands.append(("fused", "one_sm", 2, 16))
            if self.M % 2048 == 0 and self.M >= 4096:
                cands.append(("chunked", None, None, None))
        return cands

    def _autotune(self, a: torch.Tensor, b: torch.Tensor):
        """First call of ``strategy="autotune"``: every candidate is built, checked against the unfused pair's result
        and timed on the real operands (CUDA events).  The ranks exchange their times on the host; a candidate counts
        with its slowest rank, and one that raised, failed its check or hit a device timeout on ANY rank is out (after
        a timeout all ranks recover the communicator together before the next candidate).  The fastest one is kept, so
        all ranks take the same decision.  Costs a few tens of milliseconds and synchronises the device: the first
        call must not be inside a CUDA-graph capture."""
        comm = self.comm
        cands = self._candidates()
        agreed = []
        ref = None
        iters = 10
        INF = 1 << 60
        def agree(value: int) -> list:
            """Host-side exchange of one value per rank; recovers the communicator on all ranks if any rank's device
            side reports a timeout.  Returns (values, any_timeout)."""
            rows = comm.host_all_gather([value, 0 if comm.status_ok() else 1])
            timed_out = any(r[1] for r in rows)
            if timed_out:
                comm.recover()
            return [r[0] for r in rows], timed_out

        for strat, kern, nv, c in cands:
            op, ok = None, False
            try:
                op = GemmAllReduce(comm, self.M, self.N, self.dtype, comm_ctas=c, use_nvls=nv, strategy=strat, kernel=kern,
                                   max_ctas=self._tune_args["max_ctas"])
                out = op(a, b)
                torch.cuda.synchronize()
                comm.check_status()
                if ref is None:
                    ref = out.clone()
                    ok = True
                else:
                    scale = max(1.0, float(ref.float().abs().max()))
                    ok = bool((out.float() - ref.float()).abs().max() <= 2e-2 * scale)
            except Exception as e:  # noqa: BLE001 - any failure of a candidate takes the candidate out, on every rank
                logger.info("autotune: %s/%s/nvls=%s/ctas=%s failed on rank %d: %s", strat, kern, nv, c, comm.rank, e)
                ok = False
            oks, timed_out = agree(1 if ok else 0)
            ns = INF
            if all(oks) and not timed_out:
                try:
                    op(a, b)
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(iters):
                        op(a, b)
                    e1.record()
                    torch.cuda.synchronize()
                    comm.check_status()
                    ns = int(e0.elapsed_time(e1) / iters * 1e6)
                except Exception as e:  # noqa: BLE001
                    logger.info("autotune: timing %s/%s/nvls=%s/ctas=%s failed on rank %d: %s", strat, kern, nv, c, comm.rank, e)
                    ns = INF
                times, timed_out = agree(ns)
                ns = INF if timed_out else max(times)
            if op is not None:
                op.release()
            agreed.append(ns)
        if min(agreed) >= INF:
            raise _lib.OobError(_lib.ERR_UNSUPPORTED, "autotune: no candidate ran correctly on every rank")
        best = min(range(len(cands)), key=lambda i: agreed[i])
        strat, kern, nv, c = cands[best]
        self.tuning = [dict(strategy=s_, kernel=k_, use_nvls=n_, comm_ctas=c_, us=round(t / 1e3, 1) if t < INF else None)
                       for (s_, k_, n_, c_), t in zip(cands, agreed)]
        self._tuned = GemmAllReduce(comm, self.M, self.N, self.dtype, comm_ctas=c, use_nvls=nv, strategy=strat, kernel=kern,
                                    max_ctas=self._tune_args["max_ctas"])
        self.strategy, self.comm_ctas, self.use_nvls = self._tuned.strategy, self._tuned.comm_ctas, self._tuned.use_nvls
        self.kernel = self._tuned.kernel
        self.chunks = self._tuned.chunks
        return self._tuned

    def output(self, rank: Optional[int] = None) -> torch.Tensor:
        """The [M, N] result buffer in registered memory (of ``rank`` in emulation)."""
        if self._tuned is not None:
            return self._tuned.output(rank)
        if _emulated(self.comm):
            return self.comm.view(self.c_off, (self.M, self.N), self.dtype, rank or 0)
        return self._out

    def release(self) -> None:
        """Gives the op's registered buffers and counters back (collective by convention)."""
        if not self.multi:
            return
        if self._tuned is not None or self.strategy == "autotune":
            if self._tuned is not None:
                self._tuned.release()
            self.multi = False
            return
        if self.strategy == "fused":
            self.comm.free(self.partial_off)
            self.comm.release_counters(self.counter_base)
        self.comm.free(self.c_off)
        self.multi = False

    def __call__(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        if not self.multi:
            return gemm(a, b, max_ctas=self.max_ctas)
        if self._tuned is not None:
            return self._tuned(a, b)
        if self.strategy == "autotune":
            return self._autotune(a, b)(a, b)
        if self.strategy == "unfused":
            gemm(a, b, out=self._out, max_ctas=self.max_ctas, splits=1)
            return self.comm.all_reduce(self._out)
        if self.strategy == "chunked":
            # Every collective of this op is issued on the side stream, in slab order, on every rank; the caller's
            # stream only computes, and joins the side stream at the end.
            main = torch.cuda.current_stream()
            rows = self.M // self.chunks
            for i in range(self.chunks):
                sl = slice(i * rows, (i + 1) * rows)
                gemm(a[sl], b, out=self._out[sl], max_ctas=self.max_ctas, splits=1)
                self._slab_done[i].record(main)
                self._side.wait_event(self._slab_done[i])
                with torch.cuda.stream(self._side):
                    self.comm.all_reduce(self._out[sl])
            self._joined.record(self._side)
            main.wait_event(self._joined)
            return self._out
        a0, b0, sa, sb = _operands(self.comm, a, b)
        _check_operands(a0, b0)
        if a0.shape[0] != self.M or b0.shape[0] != self.N:
            raise ValueError("operand shapes do not match this op")
        args = _lib.GemmArgs()
        args.mode = _lib.GEMM_AR
        fill_gemm_args(args, a0, b0)
        args.a_emu_stride, args.b_emu_stride = sa, sb
        args.comm_ctas, args.max_ctas = self.comm_ctas, self.max_ctas
        args.pair = self.kernel
        args.use_nvls = _use_nvls(self.comm, self.use_nvls)
        args.no_join = 0 if getattr(self, "join", True) else 1
        trace = getattr(self, "trace_buffer", None)  # [ctas, 8] int64 device tensor: per-CTA phase stamps
        args.trace = trace.data_ptr() if trace is not None else None
        order = getattr(self, "order_buffer", None)  # tile-order record of the two-SM kernel (ops.gemm.order_buffer)
        args.order = order.data_ptr() if order is not None else None
        args.partial_reg, args.partial_off = 0, self.partial_off
        args.c_reg, args.c_off = 0, self.c_off
        args.counter_base = self.counter_base
        _lib.check(_lib.lib().oob_gemm(self.comm._h, ctypes.byref(args), _stream()))
        return self.output()


def wave_aligned_comm_ctas(M: int, N: int, sms: int = 148, lo: int = 4, hi: int = 24) -> int:
    """Communication CTAs for a fused op on the two-SM kernel such that the GEMM loses no wave to them: the GEMM runs
    on ``sms / 2 - c / 2`` CTA pairs and takes ``ceil(tiles / pairs)`` waves of 256 x 256 tiles; among the budgets
    ``lo .. hi`` (even) that reach the smallest wave count the LARGEST is returned, since those reducers are free.
    Example: 4096 x 8192 is 512 tiles; 74 .. 65 pairs need 8 waves and so do 64 pairs, so 20 CTAs cost the GEMM nothing."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    best, best_waves = lo, None
    for c in range(lo, hi + 1, 2):
        pairs = (sms - c) // 2
        if pairs < 1:
            break
        waves = -(-tiles // pairs)
        if best_waves is None or waves < best_waves or (waves == best_waves and c > best):
            best, best_waves = c, waves
    return best


class GemmReduceScatterNorm:
    """``weight=None`` gives the plain GEMM->reduce-scatter (+ optional residual add).  Defaults from the 8-GPU
    measurements of the 70B FFN shapes: the two-SM kernel, reduction through the switch, 8 communication CTAs (more
    only take SMs from the GEMM, which is the longer part: 280 us with 8 against 298 us with 16)."""

    def __init__(self, comm, M: int, N: int, dtype: torch.dtype, *, eps: float = 1e-6, comm_ctas: int = 8,
                 use_nvls: Optional[bool] = None,
                 max_ctas: int = 0, kernel: Optional[str] = None):
        self.kernel = _kernel_code(kernel)
        if comm.world < 2:
            raise ValueError("needs at least two ranks")
        if M % comm.world or (M // comm.world) % TILE_M:
            raise ValueError(f"M / world must be a multiple of {TILE_M}")
        self.comm, self.M, self.N, self.dtype, self.eps = comm, M, N, dtype, eps
        self.use_nvls = use_nvls
        self.comm_ctas, self.max_ctas = comm_ctas, max_ctas
        lib = _lib.lib()
        self.partial_off = comm.alloc(int(lib.oob_gemm_partial_bytes(M, N)))
        self.counter_base = comm.reserve_counters(lib.oob_gemm_counters_needed(_lib.GEMM_RS_NORM, M, N, comm.world))
        self.rows = M // comm.world

    def release(self) -> None:
        """Gives the op's registered buffer and counters back (collective by convention)."""
        if self.partial_off is not None:
            self.comm.free(self.partial_off)
            self.comm.release_counters(self.counter_base)
            self.partial_off = None

    def __call__(self, a: torch.Tensor, b: torch.Tensor, weight: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, *, y: Optional[torch.Tensor] = None,
                 residual_out: Optional[torch.Tensor] = None):
        """Returns ``(y, residual_out)``; in emulation both are stacked ``[world, rows, N]``."""
        a0, b0, sa, sb = _operands(self.comm, a, b)
        _check_operands(a0, b0)
        emu = _emulated(self.comm)
        shape = (self.comm.world, self.rows, self.N) if emu else (self.rows, self.N)
        if y is None:
            y = torch.empty(shape, dtype=self.dtype, device=a.device)
        if residual_out is None and residual is not None:
            residual_out = torch.empty(shape, dtype=self.dtype, device=a.device)
        args = _lib.GemmArgs()
        args.mode = _lib.GEMM_RS_NORM
        fill_gemm_args(args, a0, b0)
        args.a_emu_stride, args.b_emu_stride = sa, sb
        args.comm_ctas, args.max_ctas = self.comm_ctas, self.max_ctas
        args.pair = self.kernel
        args.use_nvls = _use_nvls(self.comm, self.use_nvls)
        args.no_join = 0 if getattr(self, "join", True) else 1
        trace = getattr(self, "trace_buffer", None)  # [ctas, 8] int64 device tensor: per-CTA phase stamps
        args.trace = trace.data_ptr() if trace is not None else None
        order = getattr(self, "order_buffer", None)  # tile-order record of the two-SM kernel (ops.gemm.order_buffer)
        args.order = order.data_ptr() if order is not None else None
        args.partial_reg, args.partial_off = 0, self.partial_off
        args.counter_base = self.counter_base
        args.residual = residual.data_ptr() if residual is not None else None
        args.weight = weight.data_ptr() if weight is not None else None
        args.eps = self.eps
        args.y_local = y.data_ptr()
        args.res_out_local = residual_out.data_ptr() if residual_out is not None else None
        args.rs_emu_stride = self.rows * self.N * 2 if emu else 0
        _lib.check(_lib.lib().oob_gemm(self.comm._h, ctypes.byref(args), _stream()))
        return y, residual_out


class AllGatherGemm:
    """Defaults from the measurements of the 70B FFN shapes: the two-SM kernel, 8 pusher CTAs; the stream-K tail by the
    plain-GEMM rule up to four ranks (381 against 448 us at tp4) and whole tiles only from eight on (242 against
    296 us at tp8, where a tail makes the last pairs depend on several late chunks at once).  ``stream_k``: None = that
    default, 0 = the plain-GEMM rule, 1 = always, -1 = never."""

    def __init__(self, comm, M: int, K: int, dtype: torch.dtype, *, comm_ctas: int = 8, max_ctas: int = 0,
                 use_nvls: Optional[bool] = None, kernel: Optional[str] = None, stream_k: Optional[int] = None):
        if stream_k is None:
            stream_k = 0 if comm.world <= 4 else -1
        self.use_nvls = use_nvls
        self.kernel = _kernel_code(kernel)
        self.stream_k = stream_k
        if comm.world < 2:
            raise ValueError("needs at least two ranks")
        if M % comm.world or (M // comm.world) % TILE_M:
            raise ValueError(f"M / world must be a multiple of {TILE_M}")
        self.comm, self.M, self.K, self.dtype = comm, M, K, dtype
        self.comm_ctas, self.max_ctas = comm_ctas, max_ctas
        self.a_full_off = comm.alloc(M * K * 2)
        self.counter_base = comm.reserve_counters(_lib.lib().oob_gemm_counters_needed(_lib.GEMM_AG, M, 8, comm.world))

    def release(self) -> None:
        """Gives the gathered buffer and the chunk flags back (collective by convention)."""
        if self.a_full_off is not None:
            self.comm.free(self.a_full_off)
            self.comm.release_counters(self.counter_base)
            self.a_full_off = None

    def gathered(self, rank: Optional[int] = None) -> torch.Tensor:
        """The gathered A ([M, K]) as it landed in this rank's registered memory.  Rows of the rank's own
        shard are only present there when the broadcast went through NVLS."""
        if _emulated(self.comm):
            return self.comm.view(self.a_full_off, (self.M, self.K), self.dtype, rank or 0)
        return self.comm.view(self.a_full_off, (self.M, self.K), self.dtype)

    def __call__(self, a_shard: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``a_shard``: [M / world, K]; ``b``: [N_local, K].  Returns C [M, N_local] (stacked in emulation)."""
        a0, b0, sa, sb = _operands(self.comm, a_shard, b)
        _check_operands(a0, b0)
        emu = _emulated(self.comm)
        N = b0.shape[0]
        shape = (self.comm.world, self.M, N) if emu else (self.M, N)
        if out is None:
            out = torch.empty(shape, dtype=self.dtype, device=b.device)
        args = _lib.GemmArgs()
        args.mode = _lib.GEMM_AG
        fill_gemm_args(args, a0, b0)
        args.M = self.M  # logical problem: the gathered operand
        args.C, args.ldc = out.data_ptr(), N
        args.a_emu_stride, args.b_emu_stride = sa, sb
        args.c_emu_stride = self.M * N * 2 if emu else 0
        args.comm_ctas, args.max_ctas = self.comm_ctas, self.max_ctas
        args.pair, args.stream_k = self.kernel, self.stream_k
        args.use_nvls = _use_nvls(self.comm, self.use_nvls)
        args.no_join = 0 if getattr(self, "join", True) else 1
        trace = getattr(self, "trace_buffer", None)  # [ctas, 8] int64 device tensor: per-CTA phase stamps
        args.trace = trace.data_ptr() if trace is not None else None
        order = getattr(self, "order_buffer", None)  # tile-order record of the two-SM kernel (ops.gemm.order_buffer)
        args.order = order.data_ptr() if order is not None else None
        args.a_full_reg, args.a_full_off = 0, self.a_full_off
        args.counter_base = self.counter_base
        _lib.check(_lib.lib().oob_gemm(self.comm._h, ctypes.byref(args), _stream()))
        return out


def gemm_all_reduce_unfused(comm, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Our GEMM followed by our all-reduce as two kernels (comparison point for the fused op)."""
    out = comm.empty((a.shape[0], b.shape[0]), a.dtype) if comm.world > 1 else None
    c = gemm(a, b, out=out)
    return comm.all_reduce(c) if comm.world > 1 else c


__all__ = ["GemmAllReduce", "GemmReduceScatterNorm", "AllGatherGemm", "gemm_all_reduce_unfused", "partition"]
