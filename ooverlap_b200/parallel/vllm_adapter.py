"""vLLM tensor-parallel backend hook.

``OoverlapAllReduce`` is a drop-in for vLLM's ``CustomAllreduce`` (the object
``CudaCommunicator.ca_comm`` of vLLM 0.22: ``disabled``, ``should_custom_ar``,
``custom_all_reduce``, ``capture``, ``close``) whose all-reduces run on this
library's kernels, plus the extras of the reference adapter: ``all_gather``
along any dimension, a direct-slot row-parallel linear (the GEMM writes straight
into the registered slot that is then reduced in place), and ``destroy``.

``install()`` wires it into vLLM without touching vLLM's files: it wraps
``CudaCommunicator.__init__`` so that, when ``VLLM_FORCE_ALLREDUCE_BACKEND``
is ``ooverlap``, ``ca_comm`` is an ``OoverlapAllReduce`` and the other
fast paths (quick all-reduce, FlashInfer, torch symmetric memory) are turned
off; failing to build the communicator raises instead of silently falling back,
as the reference's forced-backend switch does.

Environment (names follow the reference's ``VLLM_OOVERLAP_*`` family):

  VLLM_FORCE_ALLREDUCE_BACKEND   auto | ooverlap | custom | pynccl | nccl_symm  (``auto`` / unset: leave vLLM alone).
                                 A forced backend serves EVERY tensor-parallel all-reduce or the call raises: nothing
                                 falls through to another backend unnoticed.  ``custom`` = vLLM's own CustomAllreduce,
                                 ``pynccl`` = NCCL through vLLM's PyNccl wrapper, ``nccl_symm`` = NCCL on symmetric
                                 memory (needs vLLM's ``VLLM_USE_NCCL_SYMM_MEM`` machinery to load); these three are the
                                 comparison arms of the serving benchmark.
  VLLM_OOVERLAP_STRICT           1 (default): a tensor the ooverlap backend cannot take raises; 0: it is counted as
                                 declined and handed to vLLM's own chain (the counts are logged when the group closes)
  VLLM_OOVERLAP_RR_SLOTS         all-reduce ring slots (default 16)
  VLLM_OOVERLAP_RR_CAPACITY_BYTES  bytes per slot (default 128 MiB)
  VLLM_OOVERLAP_RR_DTYPE         bf16 | fp16 | fp32 (default bf16)
  VLLM_OOVERLAP_AG_SLOTS / _AG_CAPACITY_BYTES / _AG_DTYPE   all-gather pool (4 x 64 MiB, bf16)
  VLLM_OOVERLAP_BROKER_KEY       fixed rendezvous key (default: a UUID broadcast over the CPU group)
  VLLM_OOVERLAP_ROW_PARALLEL     1: bias-free, unquantised ``RowParallelLinear`` layers (o_proj, down_proj) run as
                                 this library's GEMM into a registered slot + in-place all-reduce (default 0)
  VLLM_OOVERLAP_DEBUG            verbose logging

Capability parity: patches/vllm/v0.25.0/vllm/distributed/device_communicators/ooverlap_all_reduce.py:44-704
(adapter), cuda_communicator.py:52-60,99-107,160-169,311-343,451-472 (forced backend), and
model_executor/models/qwen2.py:84-120 (direct-slot row-parallel) of the reference.  The reference overwrites vLLM
0.25.0 source files guarded by git-blob hashes; the vLLM installed here is 0.22, so the hook is a run-time patch.
"""
from __future__ import annotations

import contextlib
import os
import uuid
from typing import Optional

import torch

from ..comm import Communicator
from ..utils.logging import logger

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
           "half": torch.float16, "fp32": torch.float32, "float32": torch.float32}


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return int(v) if v not in (None, "") else default


def _env_dtype(name: str, default: str) -> torch.dtype:
    v = os.environ.get(name, default).lower()
    if v not in _DTYPES:
        raise ValueError(f"{name}={v!r}: expected one of {sorted(_DTYPES)}")
    return _DTYPES[v]


def forced_backend() -> str:
    v = os.environ.get("VLLM_FORCE_ALLREDUCE_BACKEND", "auto").strip().lower()
    if v not in ("auto", "ooverlap", "custom", "pynccl", "nccl_symm"):
        raise ValueError(f"VLLM_FORCE_ALLREDUCE_BACKEND={v!r} is not one of auto, ooverlap, custom, pynccl, nccl_symm")
    return v


def short_broker_key(seed: str) -> str:
    """A rendezvous key short enough for a socket name (the reference keeps its prefix under 90 characters)."""
    clean = "".join(c if c.isalnum() else "_" for c in seed)
    return ("vllm_" + clean)[:48]


class OoverlapAllReduce:
    """All-reduce / all-gather backend for one tensor-parallel group (one process per GPU)."""

    def __init__(self, group=None, device: Optional[torch.device | int | str] = None, *,
                 communicator: Optional[Communicator] = None, max_size: Optional[int] = None):
        self.disabled = True
        self._IS_CAPTURING = False
        self.comm: Optional[Communicator] = None
        self.group = group
        self.debug = os.environ.get("VLLM_OOVERLAP_DEBUG", "0") not in ("", "0")
        self.rr_dtype = _env_dtype("VLLM_OOVERLAP_RR_DTYPE", "bf16")
        # Ring of result / staging slots.  A slot holds 8192 tokens of a hidden-8192 model (8192 x 16 KiB = 128 MiB), so
        # that a prefill chunk of that size is one copy into the slot and one in-place all-reduce whose result is handed
        # out as it lies in the slot; a larger tensor is reduced in slot-sized pieces (a 16384-token chunk: two pieces
        # and two copies out; VLLM_OOVERLAP_RR_CAPACITY_BYTES=268435456 with VLLM_OOVERLAP_RR_SLOTS=8 makes it one, a
        # setting that has not run inside the engine yet).  Decode-sized messages go through the flag-in-data / push
        # kernels and only land in a slot.
        self.rr_slots = _env_int("VLLM_OOVERLAP_RR_SLOTS", 16)
        self.rr_capacity = _env_int("VLLM_OOVERLAP_RR_CAPACITY_BYTES", 128 << 20)
        self.ag_dtype = _env_dtype("VLLM_OOVERLAP_AG_DTYPE", "bf16")
        self.ag_slots = _env_int("VLLM_OOVERLAP_AG_SLOTS", 4)
        self.ag_capacity = _env_int("VLLM_OOVERLAP_AG_CAPACITY_BYTES", 64 << 20)
        self.max_size = max_size if max_size is not None else self.rr_capacity
        # What this backend did for its group: all-reduces served from a ring slot, served in slot-sized pieces
        # (tensors larger than a slot), and declined by reason.  Logged at close; read with stats().
        self.served = 0
        self.served_chunked = 0
        self.declined: dict[str, int] = {}
        if communicator is None:
            communicator = self._build_communicator(group, device)
        self.comm = communicator
        self.rank, self.world_size = communicator.rank, communicator.world
        self.device = torch.device("cuda", communicator.device)
        if self.world_size == 1:
            return  # nothing to reduce: stay disabled, callers fall through
        communicator.init_round_robin_slots(self.rr_dtype, self.rr_capacity, self.rr_slots)
        communicator.init_all_gather_slots(self.ag_dtype, self.ag_capacity, self.ag_slots)
        self.disabled = False
        logger.info("ooverlap backend ready: rank %d/%d on %s, %d x %d MiB all-reduce slots (%s), NVLS %s", self.rank,
                    self.world_size, self.device, self.rr_slots, self.rr_capacity >> 20, self.rr_dtype, communicator.nvls)

    # ------------------------------------------------------------------ setup
    def _build_communicator(self, group, device) -> Communicator:
        import torch.distributed as dist
        if group is None:
            group = dist.group.WORLD
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        if device is None:
            device = torch.cuda.current_device()
        index = torch.device(device).index if not isinstance(device, int) else device
        if index is None:
            index = torch.cuda.current_device()
        # Every rank learns every rank's device index through the (CPU) group.
        devices = [None] * world
        dist.all_gather_object(devices, int(index), group=group)
        key = os.environ.get("VLLM_OOVERLAP_BROKER_KEY")
        if key is None:
            box = [uuid.uuid4().hex if rank == 0 else None]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0), group=group)
            key = box[0]
        heap = (self.rr_slots * self.rr_capacity + self.ag_slots * self.ag_capacity + (256 << 20))
        return Communicator(devices, rank, short_broker_key(key), heap_bytes=heap)

    # ---------------------------------------------------- vLLM CustomAllreduce
    def why_not(self, inp: torch.Tensor) -> Optional[str]:
        """None when a ring slot can take ``inp`` as it is, else the reason it cannot."""
        if self.disabled:
            return "backend disabled"
        if not inp.is_cuda or inp.device != self.device:
            return "not on this rank's device"
        if inp.dtype != self.rr_dtype:
            return f"dtype {inp.dtype} is not the pool's {self.rr_dtype}"
        if not inp.is_contiguous():
            return "not contiguous"
        nbytes = inp.numel() * inp.element_size()
        if nbytes == 0:
            return "empty"
        if nbytes % 16:
            return "size is not a multiple of 16 bytes"
        if nbytes > self.max_size:
            return "larger than a slot"
        return None

    def should_custom_ar(self, inp: torch.Tensor) -> bool:
        return self.why_not(inp) is None

    should_ooverlap_ar = should_custom_ar

    def all_reduce(self, inp: torch.Tensor) -> Optional[torch.Tensor]:
        """Copy into the next ring slot, reduce in place, return the slot view (it aliases pool memory and
        stays valid until the ring wraps: ``VLLM_OOVERLAP_RR_SLOTS`` later all-reduces).  None when the tensor
        is not eligible (see :meth:`why_not`)."""
        why = self.why_not(inp)
        if why is not None:
            self.declined[why] = self.declined.get(why, 0) + 1
            return None
        self.served += 1
        return self.comm.all_reduce_round_robin(inp)

    def all_reduce_any_size(self, inp: torch.Tensor) -> Optional[torch.Tensor]:
        """Like :meth:`all_reduce`, and a tensor that is only too large for a slot is reduced in slot-sized pieces of
        whole rows into a fresh tensor (prefill batches; the ring stays the only registered memory)."""
        why = self.why_not(inp)
        if why is None:
            self.served += 1
            return self.comm.all_reduce_round_robin(inp)
        row_bytes = (inp.numel() // max(1, inp.shape[0])) * inp.element_size() if inp.dim() > 0 else 0
        if why != "larger than a slot" or row_bytes == 0 or row_bytes > self.max_size or row_bytes % 16:
            self.declined[why] = self.declined.get(why, 0) + 1
            return None
        rows = max(1, self.max_size // row_bytes)
        out = torch.empty_like(inp)
        for r0 in range(0, inp.shape[0], rows):
            out[r0:r0 + rows].copy_(self.comm.all_reduce_round_robin(inp[r0:r0 + rows]))
        self.served_chunked += 1
        return out

    def stats(self) -> dict:
        return {"served": self.served, "served_in_pieces": self.served_chunked, "declined": dict(self.declined)}

    def custom_all_reduce(self, inp: torch.Tensor) -> Optional[torch.Tensor]:
        out = self.all_reduce(inp)
        if self.debug and out is not None:
            logger.debug("all_reduce %s %s capturing=%s", tuple(inp.shape), inp.dtype, self._IS_CAPTURING)
        return out

    @contextlib.contextmanager
    def capture(self):
        """vLLM wraps CUDA-graph capture in this.  Slots have fixed addresses and the epoch counters of the
        kernels live on the device, so nothing needs registering afterwards."""
        self._IS_CAPTURING = True
        try:
            yield
        finally:
            self._IS_CAPTURING = False

    def close(self) -> None:
        if self.comm is not None:
            logger.info("ooverlap backend rank %d: all-reduces served %d (+%d in slot-sized pieces), declined %s",
                        self.rank, self.served, self.served_chunked, self.declined or "none")
            path = os.environ.get("VLLM_OOVERLAP_STATS_FILE")
            if path:  # one JSON line per rank, for the serving benchmark's record
                import json
                with open(path, "a") as f:
                    f.write(json.dumps({"rank": self.rank, "world": self.world_size, **self.stats()}) + "\n")
            self.comm.close()
            self.comm = None
        self.disabled = True

    destroy = close

    # ----------------------------------------------------------- all-gather
    def should_all_gather(self, inp: torch.Tensor) -> bool:
        if self.disabled or not inp.is_cuda or inp.dtype != self.ag_dtype:
            return False
        return inp.numel() * inp.element_size() * self.world_size <= self.ag_capacity

    def all_gather(self, inp: torch.Tensor, dim: int = -1) -> Optional[torch.Tensor]:
        """Gather along ``dim``: rank-major gather through the slot pool, then a ``movedim``/``reshape`` to put the
        gathered axis in place (same data flow as the reference adapter)."""
        if not self.should_all_gather(inp):
            return None
        if dim < 0:
            dim += inp.dim()
        x = inp.contiguous()
        lead = x.reshape(1, -1) if x.dim() == 0 else x.reshape(x.shape[0], -1) if x.dim() > 1 else x.reshape(-1, 1)
        gathered = self.comm.all_gather_round_robin(lead)           # [world * d0, rest]
        gathered = gathered.reshape((self.world_size,) + tuple(x.shape))
        gathered = gathered.movedim(0, dim)                          # [..., world, d_dim, ...]
        shape = list(x.shape)
        shape[dim] *= self.world_size
        return gathered.reshape(shape)

    # ------------------------------------------------ direct-slot row-parallel
    def row_parallel(self, x: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
        """``all_reduce(x @ weight.T)`` for a bias-free, unquantised row-parallel layer: the GEMM (this library's
        tcgen05 kernel) writes straight into the next registered slot, which is then reduced in place."""
        from ..ops import gemm
        if self.disabled or x.dtype != self.rr_dtype or weight.dtype != self.rr_dtype:
            return None
        x2 = x.reshape(-1, x.shape[-1])
        out_shape = (x2.shape[0], weight.shape[0])
        nbytes = out_shape[0] * out_shape[1] * x.element_size()
        if nbytes > self.rr_capacity or x2.shape[1] % 8 or not x2.is_contiguous() or x2.shape[0] == 0:
            return None
        slot = self.comm.acquire_all_reduce_slot(out_shape)
        gemm(x2, weight, out=slot)
        out = self.comm.all_reduce_preloaded_slot(slot)
        return out.reshape(tuple(x.shape[:-1]) + (weight.shape[0],))

    qwen_row_parallel = row_parallel


# --------------------------------------------------------------------------------------------------------------------
# Direct-slot row-parallel linear as a torch custom op, so that a compiled vLLM model can call it.
# --------------------------------------------------------------------------------------------------------------------
_row_parallel_backend: Optional["OoverlapAllReduce"] = None  # the tensor-parallel group's backend in this process


@torch.library.custom_op("ooverlap_b200::row_parallel_linear", mutates_args=())
def row_parallel_linear_op(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``all_reduce(x @ weight.T)`` over the tensor-parallel group through the registered backend.  The result lives
    in a slot of the backend's ring: it must be consumed before the ring wraps (16 slots by default)."""
    backend = _row_parallel_backend
    out = backend.row_parallel(x, weight) if backend is not None else None
    if out is None:
        raise RuntimeError("row_parallel_linear: no backend, or the operands do not fit a slot (check the caller's "
                           "eligibility test)")
    return out


@row_parallel_linear_op.register_fake
def _row_parallel_linear_fake(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return x.new_empty(tuple(x.shape[:-1]) + (weight.shape[0],))


def row_parallel_eligible(layer, x: torch.Tensor, backend) -> bool:
    """True when a vLLM ``RowParallelLinear`` call can take the direct-slot path: the reference restricts it to
    bias-free, unquantised layers whose result is reduced (model_executor/models/qwen2.py:84-120)."""
    if not isinstance(backend, OoverlapAllReduce) or backend.disabled:
        return False
    if not getattr(layer, "reduce_results", False) or getattr(layer, "tp_size", 1) <= 1:
        return False
    if not getattr(layer, "input_is_parallel", False) or getattr(layer, "bias", None) is not None:
        return False
    if type(getattr(layer, "quant_method", None)).__name__ != "UnquantizedLinearMethod":
        return False
    w = getattr(layer, "weight", None)
    if w is None or w.dtype != backend.rr_dtype or x.dtype != backend.rr_dtype or not x.is_cuda:
        return False
    rows = x.numel() // max(1, x.shape[-1])
    if rows == 0 or x.shape[-1] % 8 or not x.is_contiguous():
        return False
    return rows * w.shape[0] * x.element_size() <= backend.rr_capacity


def _patch_row_parallel_linear() -> bool:
    """Routes eligible ``RowParallelLinear.forward`` calls through :func:`row_parallel_linear_op`."""
    from vllm.distributed.parallel_state import get_tp_group
    from vllm.model_executor.layers import linear as vl

    original_forward = vl.RowParallelLinear.forward

    def patched_forward(self, input_):
        try:
            backend = getattr(get_tp_group().device_communicator, "ca_comm", None)
        except Exception:  # noqa: BLE001  (group not built yet)
            backend = None
        if row_parallel_eligible(self, input_, backend):
            global _row_parallel_backend
            _row_parallel_backend = backend
            out = torch.ops.ooverlap_b200.row_parallel_linear(input_, self.weight)
            if not self.return_bias:
                return out
            return out, None
        return original_forward(self, input_)

    vl.RowParallelLinear.forward = patched_forward
    return True


_installed = False


def _strict() -> bool:
    return os.environ.get("VLLM_OOVERLAP_STRICT", "1") not in ("0", "")


def forced_all_reduce(self, input_, mode: str, original_all_reduce):
    """``CudaCommunicator.all_reduce`` under a forced backend (the reference's ``_all_reduce_forced``,
    cuda_communicator.py:328-343): the named backend serves the tensor, or the call raises.  ``self`` is the vLLM
    communicator.  Pure dispatch, so that it can be tested with stand-ins."""
    if mode == "ooverlap":
        ca = getattr(self, "ca_comm", None)
        if not isinstance(ca, OoverlapAllReduce):
            raise RuntimeError("VLLM_FORCE_ALLREDUCE_BACKEND=ooverlap, but this group has no ooverlap backend")
        out = ca.all_reduce_any_size(input_)
        if out is not None:
            return out
        if _strict():
            raise RuntimeError(f"VLLM_FORCE_ALLREDUCE_BACKEND=ooverlap: tensor {tuple(input_.shape)} {input_.dtype} cannot "
                               f"be served ({ca.why_not(input_)}); set VLLM_OOVERLAP_RR_DTYPE / "
                               "VLLM_OOVERLAP_RR_CAPACITY_BYTES to fit the model, or VLLM_OOVERLAP_STRICT=0 to let such "
                               "tensors fall through to vLLM's own chain (they are counted)")
        return original_all_reduce(self, input_)
    if mode == "custom":
        ca = getattr(self, "ca_comm", None)
        if ca is None or ca.disabled or not ca.should_custom_ar(input_):
            raise RuntimeError(f"VLLM_FORCE_ALLREDUCE_BACKEND=custom: vLLM's custom all-reduce cannot take tensor "
                               f"{tuple(input_.shape)} {input_.dtype}")
        out = ca.custom_all_reduce(input_)
        if out is None:
            raise RuntimeError("VLLM_FORCE_ALLREDUCE_BACKEND=custom: custom_all_reduce declined the tensor")
        return out
    if mode == "pynccl":
        nc = getattr(self, "pynccl_comm", None)
        if nc is None or nc.disabled:
            raise RuntimeError("VLLM_FORCE_ALLREDUCE_BACKEND=pynccl: this group has no PyNccl communicator")
        out = nc.all_reduce(input_)
        if out is None:
            raise RuntimeError("VLLM_FORCE_ALLREDUCE_BACKEND=pynccl: PyNccl declined the tensor")
        return out
    if mode == "nccl_symm":
        from vllm.distributed.device_communicators.pynccl_allocator import is_symmetric_memory_enabled
        if not is_symmetric_memory_enabled() or getattr(self, "pynccl_comm", None) is None:
            raise RuntimeError("VLLM_FORCE_ALLREDUCE_BACKEND=nccl_symm: NCCL symmetric memory is not available in this "
                               "vLLM process (VLLM_USE_NCCL_SYMM_MEM machinery did not load)")
        out = torch.ops.vllm.all_reduce_symmetric_with_copy(input_)
        if out is None:
            raise RuntimeError("VLLM_FORCE_ALLREDUCE_BACKEND=nccl_symm: the symmetric-memory all-reduce declined the tensor")
        return out
    return original_all_reduce(self, input_)


def install() -> bool:
    """Patches vLLM's ``CudaCommunicator`` in this process according to ``VLLM_FORCE_ALLREDUCE_BACKEND``.  Returns
    True when a backend is forced and the patch is in place.  Call before vLLM builds its distributed groups (the
    ``vllm.general_plugins`` entry point of this package does, in every engine and worker process)."""
    global _installed
    mode = forced_backend()
    if mode == "auto":
        return False
    if _installed:
        return True
    if mode == "nccl_symm":
        os.environ.setdefault("VLLM_USE_NCCL_SYMM_MEM", "1")
    from vllm.distributed.device_communicators import cuda_communicator as cc

    original_init = cc.CudaCommunicator.__init__
    original_all_reduce = cc.CudaCommunicator.all_reduce
    original_all_gather = cc.CudaCommunicator.all_gather
    original_destroy = cc.CudaCommunicator.destroy

    def drop(self, names):
        for name in names:
            other = getattr(self, name, None)
            if other is not None and hasattr(other, "destroy"):
                try:
                    other.destroy()
                except Exception:  # noqa: BLE001
                    pass
            setattr(self, name, None)

    def patched_init(self, *args, **kwargs):
        original_init(self, *args, **kwargs)
        if getattr(self, "world_size", 1) <= 1:
            return
        self._oob_forced = mode
        if mode == "ooverlap":
            # Forced: no silent fallback.  Any failure to build the backend propagates.
            old = getattr(self, "ca_comm", None)
            if old is not None and hasattr(old, "close"):
                try:
                    old.close()
                except Exception:  # noqa: BLE001
                    pass
            self.ca_comm = OoverlapAllReduce(group=self.cpu_group, device=self.device)
            drop(self, ("qr_comm", "fi_ar_comm", "symm_mem_comm"))
        elif mode == "custom":
            drop(self, ("qr_comm", "fi_ar_comm", "symm_mem_comm"))
            if getattr(self, "ca_comm", None) is None or self.ca_comm.disabled:
                raise RuntimeError("VLLM_FORCE_ALLREDUCE_BACKEND=custom, but vLLM's custom all-reduce is not available "
                                   "for this group")
        elif mode in ("pynccl", "nccl_symm"):
            drop(self, ("qr_comm", "fi_ar_comm", "symm_mem_comm"))
            old = getattr(self, "ca_comm", None)
            if old is not None and hasattr(old, "close"):
                try:
                    old.close()
                except Exception:  # noqa: BLE001
                    pass
            self.ca_comm = None
        logger.info("vLLM all-reduce backend forced to %s", mode)

    def patched_all_reduce(self, input_):
        forced = getattr(self, "_oob_forced", None)
        if forced is None:
            return original_all_reduce(self, input_)
        return forced_all_reduce(self, input_, forced, original_all_reduce)

    def patched_all_gather(self, input_, dim: int = -1):
        ca = getattr(self, "ca_comm", None)
        if isinstance(ca, OoverlapAllReduce):
            out = ca.all_gather(input_, dim)
            if out is not None:
                return out
        return original_all_gather(self, input_, dim)

    def patched_destroy(self):
        ca = getattr(self, "ca_comm", None)
        if isinstance(ca, OoverlapAllReduce):
            ca.close()
            self.ca_comm = None
        return original_destroy(self)

    cc.CudaCommunicator.__init__ = patched_init
    cc.CudaCommunicator.all_reduce = patched_all_reduce
    cc.CudaCommunicator.all_gather = patched_all_gather
    cc.CudaCommunicator.destroy = patched_destroy
    if mode == "ooverlap" and _env_int("VLLM_OOVERLAP_ROW_PARALLEL", 0):
        _patch_row_parallel_linear()
        logger.info("vLLM RowParallelLinear routed through the direct-slot GEMM + all-reduce")
    _installed = True
    return True
