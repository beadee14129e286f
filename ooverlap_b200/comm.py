"""``Communicator``: the torch-collectives API on registered buffers.

GPU tensors go through the native library (symmetric heap + sm_100a kernels
that load/store peer memory or use NVLS multimem); CPU tensors go through a
gloo-backed fallback with the same partition semantics, so the plumbing can be
tested without a GPU.

Capability parity: ``ooverlap_torch_ext.Communicator`` of the reference
(src/torch_collectives_pybind.cpp:79-152 construction, :212-404 all_reduce
flavours, :408-529 round-robin slot pools, :531-839 all-gather, :868-907
bindings).  Added on top: ``reduce_scatter``, the CPU fallback, the fused
all-reduce + residual + RMSNorm, and zero-copy tensors allocated straight from
the registered heap.
"""
from __future__ import annotations

import ctypes
import os
import threading
import uuid
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from .utils.config import Config
from .utils.dtypes import dtype_code, op_code
from .utils.logging import logger
from .utils.partition import max_shard, partition


class _DeviceMemory:
    """Exposes a raw device address range through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner  # keeps the communicator alive while views exist
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, device: int, owner=None) -> torch.Tensor:
    """uint8 tensor aliasing ``nbytes`` of device memory at ``ptr``."""
    return torch.as_tensor(_DeviceMemory(ptr, nbytes, owner), device=torch.device("cuda", device))


@dataclass
class SlotPool:
    """A ring of equally sized registered buffers (graph-friendly: fixed addresses)."""
    dtype: torch.dtype
    capacity_bytes: int
    offsets: list
    next_index: int = 0

    def advance(self) -> int:
        i = self.next_index
        self.next_index = (i + 1) % len(self.offsets)
        return i


_policy_lock = threading.Lock()


def _current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class Communicator:
    """One per rank process.

    ``Communicator(devices, local_rank, broker_key)`` mirrors the reference's
    constructor: ``devices[i]`` is the CUDA device of rank ``i``, and
    ``broker_key`` names the node-local rendezvous.  When ``devices`` is None
    the object is a CPU communicator that runs over the default (gloo)
    ``torch.distributed`` process group.
    """

    def __init__(self, devices: Optional[Sequence[int]] = None, local_rank: Optional[int] = None,
                 broker_key: Optional[str] = None, *, heap_bytes: Optional[int] = None, config: Optional[Config] = None,
                 cpu_group=None):
        self.config = config or Config.from_env()
        self._h = None
        self._cpu_group = cpu_group
        self._scratch = {}
        self._view_cache = {}
        self._ipc_cache = {}
        self._ar_pool: Optional[SlotPool] = None
        self._ag_pool: Optional[SlotPool] = None
        self._push_arena = None  # (heap offset, piece capacity) of the push kernels' staging area
        self._ll_arena = None    # (heap offset, piece capacity) of the flag-in-data kernel's staging area
        self._counter_next = 0
        if devices is None:
            import torch.distributed as dist
            if not dist.is_initialized():
                raise RuntimeError("CPU Communicator needs an initialised torch.distributed (gloo) process group")
            self.rank = dist.get_rank(cpu_group)
            self.world = dist.get_world_size(cpu_group)
            self.device = None
            self.nvls = False
            return
        if local_rank is None:
            raise ValueError("local_rank is required with devices")
        if broker_key is None:
            broker_key = os.environ.get("OOB_BROKER_KEY")
        if broker_key is None:
            broker_key = self._key_from_process_group()
        self.rank = int(local_rank)
        self.world = len(devices)
        self.device = int(devices[self.rank])
        # The kernels load and store peer memory directly: every other rank's GPU must be reachable from this one
        # (NVLink / NVSwitch, or at least PCIe peer access).  There is no host-staged path: say so instead of failing
        # later inside the memory mapping.
        if torch.cuda.is_available():
            for r, d in enumerate(devices):
                if r != self.rank and int(d) != self.device and not torch.cuda.can_device_access_peer(self.device, int(d)):
                    raise _lib.OobError(_lib.ERR_UNSUPPORTED,
                                        f"unsupported topology: cuda:{self.device} (rank {self.rank}) has no peer access to "
                                        f"cuda:{int(d)} (rank {r}); see `oob_topology` for the link table")
        flags = 0
        if self.config.disable_nvls:
            flags |= _lib.FLAG_NO_NVLS
        if self.config.legacy_ipc:
            flags |= _lib.FLAG_LEGACY_IPC
        lib = _lib.lib()
        # OOB_TUNING_POLICY names a policy file; without it the policy measured on B200 / NVSwitch that ships
        # with the package is used ("builtin" selects the compiled-in size rule instead).
        policy = self.config.tuning_policy
        if not policy:
            packaged = os.path.join(os.path.dirname(os.path.abspath(__file__)), "policy", "b200_nvswitch.json")
            policy = packaged if os.path.exists(packaged) else ""
        if policy and policy != "builtin":
            with _policy_lock:  # the table is process-wide; several ranks of one process may be created at once
                _lib.check(lib.oob_policy_load(policy.encode()))
        handle = ctypes.c_void_p()
        _lib.check(lib.oob_comm_create(self.rank, self.world, self.device, broker_key.encode(),
                                       heap_bytes or self.config.heap_bytes, flags, self.config.timeout_ms,
                                       ctypes.byref(handle)))
        self._h = handle
        _lib.check(lib.oob_comm_set_timeout_ms(self._h, self.config.timeout_ms))
        info = _lib.CommInfo()
        _lib.check(lib.oob_comm_info(self._h, ctypes.byref(info)))
        self.info = info
        self.nvls = bool(info.nvls)
        self.heap_bytes = int(info.heap_bytes)
        self._heap_base = int(lib.oob_heap_ptr(self._h, self.rank, 0))
        # Allocated on EVERY rank up front: heap offsets stay identical only if all ranks allocate alike.
        self._dummy_off = self.alloc(1024)
        logger.info("rank %d/%d on cuda:%d: heap %d MiB, memory kind %d, NVLS %s", self.rank, self.world, self.device,
                    self.heap_bytes >> 20, info.memory_kind, self.nvls)

    # ------------------------------------------------------------------ setup
    @staticmethod
    def _key_from_process_group() -> str:
        """A short rendezvous key agreed on through torch.distributed (rank 0 draws it)."""
        import torch.distributed as dist
        if not dist.is_initialized():
            raise ValueError("broker_key is required when torch.distributed is not initialised")
        box = [uuid.uuid4().hex[:24] if dist.get_rank() == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return "pg_" + box[0]

    @property
    def is_cpu(self) -> bool:
        return self._h is None

    def close(self) -> None:
        if self._h is not None:
            _lib.lib().oob_comm_destroy(self._h)
            self._h = None

    destroy = close

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------ heap memory
    def alloc(self, nbytes: int, align: int = 1024) -> int:
        """Collective by convention: every rank must allocate in the same order.  Returns the heap offset."""
        off = ctypes.c_uint64()
        _lib.check(_lib.lib().oob_alloc(self._h, int(nbytes), int(align), ctypes.byref(off)))
        return int(off.value)

    def free(self, offset: int) -> None:
        _lib.check(_lib.lib().oob_free(self._h, int(offset)))

    def view(self, offset: int, shape, dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        """Tensor view of the heap of ``rank`` (default: this rank) at ``offset``."""
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        r = self.rank if rank is None else rank
        ptr = int(_lib.lib().oob_heap_ptr(self._h, r, int(offset)))
        if nbytes == 0:
            return torch.empty(shape, dtype=dtype, device=torch.device("cuda", self.device))
        return tensor_from_ptr(ptr, nbytes, self.device, self).view(dtype).view(shape)

    def empty(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor in registered (symmetric) memory.  Collective by convention."""
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        n = 1
        for s in shape:
            n *= s
        off = self.alloc(max(16, n * torch.empty((), dtype=dtype).element_size()))
        return self.view(off, shape, dtype)

    def heap_offset(self, t: torch.Tensor) -> Optional[int]:
        """Offset of ``t`` inside this rank's heap, or None when it lives elsewhere."""
        if self._h is None or not t.is_cuda:
            return None
        p = t.data_ptr()
        if self._heap_base <= p < self._heap_base + self.heap_bytes:
            return p - self._heap_base
        return None

    def _locate(self, t: torch.Tensor):
        """(registration id, offset) of a registered tensor, or None."""
        off = self.heap_offset(t)
        if off is not None:
            return 0, off
        hit = self._ipc_cache.get(t.data_ptr())
        if hit is not None and hit[1] >= t.numel() * t.element_size():
            return hit[0], 0
        return None

    def register(self, t: torch.Tensor) -> int:
        """Registers a tensor that was not allocated from the heap (legacy CUDA IPC, base + offset).
        Collective; cached by data pointer like the reference's ``all_reduce_inplace_cached``."""
        loc = self._locate(t)
        if loc is not None:
            return loc[0]
        if not t.is_contiguous():
            raise ValueError("only contiguous tensors can be registered")
        reg = ctypes.c_int()
        nbytes = t.numel() * t.element_size()
        _lib.check(_lib.lib().oob_register_ipc(self._h, ctypes.c_void_p(t.data_ptr()), nbytes, ctypes.byref(reg)))
        self._ipc_cache[t.data_ptr()] = (reg.value, nbytes, t)
        return reg.value

    def reserve_counters(self, n: int) -> int:
        """Reserves ``n`` general arrival counters of the signal pad (fused GEMM ops)."""
        base = self._counter_next
        if base + n > 16384 - 1:
            raise RuntimeError("out of arrival counters")
        self._counter_next += n
        return base

    def release_counters(self, base: int) -> None:
        """Gives back every counter reserved at or after ``base`` (stack discipline; counters are zero
        between calls because their consumers re-arm them)."""
        if 0 <= base < self._counter_next:
            self._counter_next = base

    # ------------------------------------------------------------- host sync
    def barrier(self) -> None:
        if self._h is None:
            import torch.distributed as dist
            dist.barrier(self._cpu_group)
            return
        _lib.check(_lib.lib().oob_comm_barrier(self._h))

    def host_all_gather(self, values: Sequence[int]) -> list:
        """Host-side all-gather of a few 64-bit integers per rank through the rendezvous: ``result[r]`` is rank r's
        list.  No kernel runs, so ranks can still agree on what to do while the device side is poisoned by a timeout."""
        vals = [int(v) for v in values]
        n = len(vals)
        if self.world == 1:
            return [vals]
        if self._h is None:  # CPU fallback: through the gloo group
            parts = self._cpu_gather_all(torch.tensor(vals, dtype=torch.int64))
            return [p.tolist() for p in parts]
        mine = (ctypes.c_int64 * n)(*vals)
        out = (ctypes.c_int64 * (n * self.world))()
        _lib.check(_lib.lib().oob_comm_host_allgather(self._h, mine, out, n * 8))
        return [list(out[r * n:(r + 1) * n]) for r in range(self.world)]

    def status_ok(self) -> bool:
        """True when no kernel of this rank has given up a wait since the last ``recover``."""
        try:
            self.check_status()
            return True
        except _lib.OobError:
            return False

    def check_status(self) -> None:
        """Raises ``DeviceTimeout`` when a kernel of this rank gave up waiting."""
        if self._h is not None:
            _lib.check(_lib.lib().oob_comm_status(self._h, None))

    def recover(self) -> None:
        """Collective: clears flags and status on every rank after a device timeout.

        The call numbers of the flag-in-data all-reduce start again from zero, so its cells are zeroed too: a cell
        left over from before the recovery could otherwise show the number of a later call that has not written it
        yet.  The ranks meet on the host first (no kernel of any rank still stores into this rank's cells) and again
        inside the native call (no rank launches before every rank's cells are zero)."""
        if self._h is None:
            return
        if self._ll_arena is not None:
            torch.cuda.synchronize()
            self.barrier()
            off, piece = self._ll_arena
            self.view(off, (2 * self.world * piece,), torch.uint8).zero_()
            torch.cuda.synchronize()
        _lib.check(_lib.lib().oob_comm_recover(self._h))

    def set_timeout_ms(self, ms: int) -> None:
        """Budget of every device-side wait of this communicator."""
        _lib.check(_lib.lib().oob_comm_set_timeout_ms(self._h, int(ms)))

    # ------------------------------------------------------------- scratch
    def _scratch_for(self, key, nbytes: int) -> int:
        hit = self._scratch.get(key)
        if hit is not None and hit[1] >= nbytes:
            return hit[0]
        if hit is not None:
            self.free(hit[0])
        off = self.alloc(max(nbytes, 16))
        self._scratch[key] = (off, nbytes)
        return off

    def scratch_view(self, key, shape, dtype: torch.dtype) -> torch.Tensor:
        """A cached registered scratch tensor for ``key`` (same call order on every rank)."""
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = self._scratch_for(key, nbytes)
        ck = (off, shape, dtype)
        hit = self._view_cache.get(ck)
        if hit is None:
            hit = self._view_cache[ck] = self.view(off, shape, dtype)
        return hit

    # ------------------------------------------------------------ all-reduce
    def all_reduce(self, x: torch.Tensor, op: str = "sum", *, algo: int = _lib.ALGO_AUTO, max_ctas: int = 0) -> torch.Tensor:
        """Sum (min, max) of ``x`` over all ranks.

        A tensor that already lives in registered memory is reduced in place
        and returned.  Any other CUDA tensor is copied into a cached registered
        scratch buffer keyed by dtype and shape, reduced there, and the scratch
        view is returned (same contract as the reference's ``all_reduce``)."""
        if not x.is_cuda:
            return self._cpu_all_reduce(x, op)
        loc = self._locate(x) if x.is_contiguous() else None
        if loc is None:
            off = self._scratch_for(("ar", x.dtype, tuple(x.shape)), x.numel() * x.element_size())
            buf = self.view(off, x.shape, x.dtype)
            buf.copy_(x)
            x, loc = buf, (0, off)
        self._launch_ar(x, loc, loc, None, op, algo, max_ctas)
        return x

    def all_reduce_out(self, x: torch.Tensor, out: torch.Tensor, op: str = "sum", *, algo: int = _lib.ALGO_AUTO,
                       max_ctas: int = 0) -> torch.Tensor:
        """``x`` must be registered; ``out`` may be any CUDA tensor (one-shot) or registered (two-shot)."""
        if not x.is_cuda:
            out.copy_(self._cpu_all_reduce(x.clone(), op))
            return out
        loc = self._locate(x)
        if loc is None:
            raise ValueError("all_reduce_out needs an input in registered memory; use all_reduce")
        oloc = self._locate(out)
        self._launch_ar(x, loc, oloc, out, op, algo, max_ctas)
        return out

    def all_reduce_inplace(self, x: torch.Tensor, op: str = "sum", **kw) -> torch.Tensor:
        """In place on ``x``; a tensor outside the heap is registered first (collective, cached)."""
        if not x.is_cuda:
            x.copy_(self._cpu_all_reduce(x.clone(), op))
            return x
        if self._locate(x) is None:
            self.register(x)
        return self.all_reduce(x, op, **kw)

    all_reduce_inplace_cached = all_reduce_inplace

    def _launch_ar(self, x, in_loc, out_loc, out_local, op, algo, max_ctas):
        lib = _lib.lib()
        out_reg, out_off = out_loc if out_loc is not None else (-1, 0)
        local_ptr = ctypes.c_void_p(out_local.data_ptr()) if out_local is not None else None
        if algo == _lib.ALGO_AUTO and in_loc[0] != 0:
            # IPC-registered (non-heap) memory has no multicast alias.
            algo = _lib.AR_TWOSHOT_P2P if out_loc is not None else _lib.AR_ONESHOT_P2P
        if out_loc is not None and out_loc == in_loc and algo in (_lib.AR_ONESHOT_P2P, _lib.AR_ONESHOT_NVLS):
            raise ValueError("one-shot all-reduce cannot run in place")
        if out_loc is not None and out_loc == in_loc:
            local_ptr = None  # in place: only the two-shot family applies
        _lib.check(lib.oob_allreduce(self._h, dtype_code(x.dtype), op_code(op), algo, in_loc[0], in_loc[1], out_reg,
                                     out_off, local_ptr, x.numel(), max_ctas or self.config.max_ctas,
                                     ctypes.c_void_p(_current_stream_ptr())))

    # -------------------------------------------------------- reduce-scatter
    def reduce_scatter(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, op: str = "sum", *,
                       algo: int = _lib.ALGO_AUTO, max_ctas: int = 0) -> torch.Tensor:
        """Rank r receives the reduction of elements ``partition(numel, world, r)`` of the flattened ``x``.

        With ``out=None`` the result is written in place into the rank's own
        partition of ``x`` (the reference's in-place slice semantics,
        include/ooverlap/comm.h ``oo_tensor_slice_t``) and that slice is returned."""
        if not x.is_cuda:
            return self._cpu_reduce_scatter(x, out, op)
        flat_in = x
        loc = self._locate(x) if x.is_contiguous() else None
        if loc is None:
            off = self._scratch_for(("rs", x.dtype, tuple(x.shape)), x.numel() * x.element_size())
            flat_in = self.view(off, x.shape, x.dtype)
            flat_in.copy_(x)
            loc = (0, off)
        b, e = partition(x.numel(), self.world, self.rank)
        if out is None:
            out = flat_in.view(-1)[b:e]
        elif out.numel() != e - b:
            raise ValueError(f"out has {out.numel()} elements, this rank's partition has {e - b}")
        if loc[0] != 0 and algo == _lib.ALGO_AUTO:
            algo = _lib.RS_P2P
        if e > b:
            _lib.check(_lib.lib().oob_reduce_scatter(self._h, dtype_code(x.dtype), op_code(op), algo, loc[0], loc[1],
                                                     ctypes.c_void_p(out.data_ptr()), x.numel(),
                                                     max_ctas or self.config.max_ctas,
                                                     ctypes.c_void_p(_current_stream_ptr())))
        else:
            # Nothing owned (more ranks than elements): still take part in the barriers.
            dummy = self._dummy_off
            _lib.check(_lib.lib().oob_reduce_scatter(self._h, dtype_code(x.dtype), op_code(op), algo, loc[0], loc[1],
                                                     ctypes.c_void_p(self._heap_base + dummy), x.numel(),
                                                     max_ctas or self.config.max_ctas,
                                                     ctypes.c_void_p(_current_stream_ptr())))
        return out

    # ------------------------------------------------------------ all-gather
    def all_gather(self, shard: torch.Tensor, out: Optional[torch.Tensor] = None, *, total: Optional[int] = None,
                   algo: int = _lib.ALGO_AUTO, max_ctas: int = 0) -> torch.Tensor:
        """Concatenates every rank's ``shard`` (flattened) in rank order.

        ``total`` is the gathered element count when shards are uneven
        (partition rule ``base + 1`` for the first ranks); by default every
        rank contributes ``shard.numel()`` elements.  The result lives in
        registered memory (``out`` if it is registered, else a cached scratch)."""
        if not shard.is_cuda:
            return self._cpu_all_gather(shard, out, total)
        count = total if total is not None else shard.numel() * self.world
        b, e = partition(count, self.world, self.rank)
        if e - b != shard.numel():
            raise ValueError(f"this rank's partition has {e - b} elements, shard has {shard.numel()}")
        esize = shard.element_size()
        if out is not None and self._locate(out) is not None and out.is_contiguous():
            loc = self._locate(out)
            result = out
        else:
            off = self._scratch_for(("ag", shard.dtype, count), count * esize)
            loc = (0, off)
            result = self.view(off, (count,), shard.dtype)
        if loc[0] != 0 and algo == _lib.ALGO_AUTO:
            algo = _lib.AG_PUSH_P2P
        src = shard if shard.is_contiguous() else shard.contiguous()
        src_ptr = src.data_ptr() if src.numel() else self._heap_base
        _lib.check(_lib.lib().oob_all_gather(self._h, dtype_code(shard.dtype), algo, loc[0], loc[1],
                                             ctypes.c_void_p(src_ptr), None, count,
                                             max_ctas or self.config.max_ctas, ctypes.c_void_p(_current_stream_ptr())))
        if out is not None and result is not out:
            out.view(-1).copy_(result)
            return out
        if out is None and total is None and shard.dim() >= 1:
            return result.view((self.world * shard.shape[0],) + tuple(shard.shape[1:]))
        return result

    # ------------------------------------------------------------ all-to-all
    def all_to_all(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, *, max_ctas: int = 0) -> torch.Tensor:
        """``x`` is ``[world, ...]``: slice j goes to rank j.  Returns ``[world, ...]`` whose slice i came from rank i
        (registered memory: ``out`` if it is registered, else a cached scratch).  Every rank must pass the same shape."""
        if x.shape[0] != self.world:
            raise ValueError("the first dimension must be the number of ranks")
        if not x.is_cuda:
            return self._cpu_all_to_all(x, out)
        src = x if x.is_contiguous() else x.contiguous()
        per = src[0].numel()
        if out is not None and self._locate(out) is not None and out.is_contiguous() and out.shape == x.shape:
            loc, result = self._locate(out), out
        else:
            off = self._scratch_for(("a2a", x.dtype, tuple(x.shape)), x.numel() * x.element_size())
            loc, result = (0, off), self.view(off, tuple(x.shape), x.dtype)
        if per:
            _lib.check(_lib.lib().oob_all_to_all(self._h, dtype_code(x.dtype), loc[0], loc[1], ctypes.c_void_p(src.data_ptr()),
                                                 per, max_ctas or self.config.max_ctas, ctypes.c_void_p(_current_stream_ptr())))
        if out is not None and result is not out:
            out.copy_(result)
            return out
        return result

    def _cpu_all_to_all(self, x: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
        import torch.distributed as dist
        result = out if out is not None else torch.empty_like(x)
        # gloo has no all_to_all: gather everybody's tensor and keep the slices addressed to this rank
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self._cpu_group)
        for i in range(self.world):
            result[i].copy_(parts[i][self.rank])
        return result

    # ------------------------------------------------------ round-robin pools
    def init_round_robin_slots(self, dtype: torch.dtype, capacity_bytes: int, slot_count: int) -> None:
        """All-reduce slot ring: ``slot_count`` registered buffers of ``capacity_bytes``.  Collective."""
        if self._ar_pool is not None:
            for off in self._ar_pool.offsets:
                self.free(off)
        self._ar_pool = SlotPool(dtype, int(capacity_bytes), [self.alloc(capacity_bytes) for _ in range(slot_count)])
        if self._ll_arena is None and self.config.ll_max_bytes > 0 and self.world > 1:
            # Staging area of the flag-in-data all-reduce: 8 bytes per 32-bit word of the message, two sets of `world`
            # pieces.  It must read as zero on every rank before any rank stores into it: zero, then meet on the host.
            piece = (2 * self.config.ll_max_bytes + 255) // 256 * 256
            off = self.alloc(2 * self.world * piece)
            self.view(off, (2 * self.world * piece,), torch.uint8).zero_()
            torch.cuda.synchronize()
            self.barrier()
            self._ll_arena = (off, piece)

    def init_all_gather_slots(self, dtype: torch.dtype, capacity_bytes: int, slot_count: int) -> None:
        if self._ag_pool is not None:
            for off in self._ag_pool.offsets:
                self.free(off)
        self._ag_pool = SlotPool(dtype, int(capacity_bytes), [self.alloc(capacity_bytes) for _ in range(slot_count)])

    def _pool_view(self, pool: Optional[SlotPool], shape, what: str) -> torch.Tensor:
        if pool is None:
            raise RuntimeError(f"{what} slot pool is not initialised")
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=pool.dtype).element_size()
        if nbytes > pool.capacity_bytes:
            raise ValueError(f"{nbytes} bytes do not fit a {pool.capacity_bytes}-byte slot")
        # Views are cached per (slot, shape): the hot path (and CUDA-graph capture) then creates no tensors.
        key = (pool.offsets[pool.next_index], tuple(int(s) for s in shape), pool.dtype)
        hit = self._view_cache.get(key)
        if hit is None:
            if len(self._view_cache) > 4096:
                self._view_cache.clear()
            hit = self._view_cache[key] = self.view(key[0], key[1], pool.dtype)
        return hit

    def acquire_all_reduce_slot(self, shape) -> torch.Tensor:
        """View of the NEXT slot; a producer (e.g. a GEMM) writes its output straight into it."""
        return self._pool_view(self._ar_pool, shape, "all-reduce")

    def all_reduce_preloaded_slot(self, view: torch.Tensor, op: str = "sum", **kw) -> torch.Tensor:
        """All-reduces the slot returned by ``acquire_all_reduce_slot`` in place and advances the ring.
        The returned tensor aliases pool memory and stays valid until the ring wraps."""
        pool = self._ar_pool
        if pool is None or self.heap_offset(view) != pool.offsets[pool.next_index]:
            raise ValueError("tensor is not the current all-reduce slot")
        pool.advance()
        return self.all_reduce(view, op, **kw)

    def all_reduce_slot_capacity(self) -> int:
        """Bytes per slot of the all-reduce ring (0 when the ring is not initialised)."""
        return self._ar_pool.capacity_bytes if self._ar_pool is not None else 0

    def commit_all_reduce_slot(self, view: torch.Tensor) -> torch.Tensor:
        """Hands the slot returned by ``acquire_all_reduce_slot`` over to an op that reduces it itself (for instance
        the fused all-reduce + RMSNorm): checks that ``view`` is the current slot and advances the ring, so that
        the next ``acquire`` returns a different buffer.  The ring's bookkeeping stays in this class."""
        pool = self._ar_pool
        if pool is None or self.heap_offset(view) != pool.offsets[pool.next_index]:
            raise ValueError("tensor is not the current all-reduce slot")
        pool.advance()
        return view

    def all_reduce_round_robin(self, x: torch.Tensor, op: str = "sum", **kw) -> torch.Tensor:
        """All-reduce of an ordinary tensor through the next slot of the ring; the result aliases the slot and stays
        valid until the ring wraps.  Small messages (``OOB_PUSH_MAX_BYTES``, 256 KiB by default) take the one-barrier
        push kernel: no copy into the slot first, the ranks' inputs land in a staging area of their own and the sum is
        written into the slot.  Larger ones are copied into the slot and reduced in place."""
        out = self.all_reduce_push(x, op) if not kw else None
        if out is not None:
            return out
        slot = self.acquire_all_reduce_slot(x.shape)
        slot.copy_(x)
        return self.all_reduce_preloaded_slot(slot, op, **kw)

    def _push_staging(self, piece: int) -> Optional[int]:
        """Heap offset of the staging area of the push kernels (two sets of ``world`` pieces; allocated at the first
        use, on every rank alike, sized for ``config.push_max_bytes``).  None when ``piece`` does not fit."""
        if self._push_arena is None:
            cap = (max(self.config.push_max_bytes, 4096) + 255) // 256 * 256
            self._push_arena = (self.alloc(2 * self.world * cap), cap)
        off, cap = self._push_arena
        return off if piece <= cap else None

    def all_reduce_push(self, x: torch.Tensor, op: str = "sum", *, max_ctas: int = 0,
                        use_nvls: Optional[bool] = None) -> Optional[torch.Tensor]:
        """Low-latency all-reduce of a small tensor into the next ring slot, which is returned (valid until the ring
        wraps).  Up to ``config.ll_max_bytes`` (64 KiB) the flag-in-data kernel (``oob_allreduce_ll``: 8-byte cells of
        data + call number, receivers spin on the cells, no barrier); above that the one-barrier push kernel
        (``oob_allreduce_push``): every rank pushes ``x`` into its piece of a staging area on all ranks, the ranks meet
        once, each sums the pieces locally.  The staging area belongs to the push kernels alone and
        holds two sets of pieces that consecutive calls alternate between (decided on the device), so calls may follow
        one another at once, also as replays of captured CUDA graphs, as long as a rank's calls run one after the
        other (one stream, or streams ordered by events).  None when the push path does not apply: no
        ring, a message above ``config.push_max_bytes``, or one that does not fit a slot."""
        pool = self._ar_pool
        if pool is None or not x.is_cuda or not x.is_contiguous() or x.dtype != pool.dtype:
            return None
        nbytes = x.numel() * x.element_size()
        piece = (nbytes + 255) // 256 * 256
        if nbytes == 0 or nbytes > self.config.push_max_bytes or piece > pool.capacity_bytes:
            return None
        use_ll = self._ll_arena is not None and nbytes <= self.config.ll_max_bytes and 2 * piece <= self._ll_arena[1]
        stage = None if use_ll else self._push_staging(piece)
        if stage is None and not use_ll:
            return None
        off = pool.offsets[pool.next_index]
        key = ("push", off, tuple(x.shape), x.dtype)
        out = self._view_cache.get(key)
        if out is None:
            if len(self._view_cache) > 4096:
                self._view_cache.clear()
            out = self._view_cache[key] = self.view(off, tuple(x.shape), x.dtype)
        pool.advance()
        nvls = self.nvls if use_nvls is None else (bool(use_nvls) and self.nvls)
        if use_ll:
            # A few KiB to a few tens of KiB: cells of 4 data bytes + 4 flag bytes, no barrier (see oob_allreduce_ll).
            _lib.check(_lib.lib().oob_allreduce_ll(self._h, dtype_code(x.dtype), op_code(op), 0, self._ll_arena[0],
                                                   self._ll_arena[1], ctypes.c_void_p(x.data_ptr()),
                                                   ctypes.c_void_p(out.data_ptr()), x.numel(),
                                                   1 if (use_nvls and self.nvls) else 0,  # peer stores unless asked
                                                   max_ctas or self.config.max_ctas, ctypes.c_void_p(_current_stream_ptr())))
            return out
        _lib.check(_lib.lib().oob_allreduce_push(self._h, dtype_code(x.dtype), op_code(op), 0, stage, piece,
                                                 ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), x.numel(),
                                                 1 if nvls else 0, max_ctas or self.config.max_ctas,
                                                 ctypes.c_void_p(_current_stream_ptr())))
        return out

    def acquire_all_gather_slot(self, shard_shape) -> torch.Tensor:
        """View of this rank's part of the next all-gather slot (shape ``shard_shape``)."""
        shard_shape = tuple(int(s) for s in shard_shape)
        full = (self.world * shard_shape[0],) + shard_shape[1:]
        whole = self._pool_view(self._ag_pool, full, "all-gather")
        return whole[self.rank * shard_shape[0]:(self.rank + 1) * shard_shape[0]]

    def all_gather_preloaded_slot(self, shard_view: torch.Tensor, **kw) -> torch.Tensor:
        pool = self._ag_pool
        if pool is None:
            raise RuntimeError("all-gather slot pool is not initialised")
        full_shape = (self.world * shard_view.shape[0],) + tuple(shard_view.shape[1:])
        whole = self.view(pool.offsets[pool.next_index], full_shape, pool.dtype)
        pool.advance()
        return self.all_gather(shard_view, out=whole, **kw).view(full_shape)

    def all_gather_round_robin(self, shard: torch.Tensor, **kw) -> torch.Tensor:
        slot = self.acquire_all_gather_slot(shard.shape)
        slot.copy_(shard)
        return self.all_gather_preloaded_slot(slot, **kw)

    # ------------------------------------------------------------ CPU fallback
    def _cpu_gather_all(self, flat: torch.Tensor) -> list:
        import torch.distributed as dist
        parts = [torch.empty_like(flat) for _ in range(self.world)]
        dist.all_gather(parts, flat, group=self._cpu_group)
        return parts

    @staticmethod
    def _cpu_combine(parts: list, op: str) -> torch.Tensor:
        acc = parts[0].to(torch.float32) if parts[0].dtype in (torch.float16, torch.bfloat16) else parts[0].clone()
        for p in parts[1:]:
            q = p.to(acc.dtype)
            if op in ("sum", "add"):
                acc = acc + q
            elif op == "min":
                acc = torch.minimum(acc, q)
            elif op == "max":
                acc = torch.maximum(acc, q)
            else:
                raise ValueError(op)
        return acc.to(parts[0].dtype)

    def _cpu_all_reduce(self, x: torch.Tensor, op: str) -> torch.Tensor:
        op_code(op)
        flat = x.contiguous().view(-1)
        # Same data flow as the two-shot kernels: reduce the owned partition in rank order, then gather.
        parts = self._cpu_gather_all(flat)
        b, e = partition(flat.numel(), self.world, self.rank)
        mine = self._cpu_combine([p[b:e] for p in parts], op)
        gathered = self._cpu_all_gather(mine, None, flat.numel())
        x.copy_(gathered.view(x.shape))
        return x

    def _cpu_reduce_scatter(self, x: torch.Tensor, out: Optional[torch.Tensor], op: str) -> torch.Tensor:
        op_code(op)
        flat = x.contiguous().view(-1)
        parts = self._cpu_gather_all(flat)
        b, e = partition(flat.numel(), self.world, self.rank)
        mine = self._cpu_combine([p[b:e] for p in parts], op)
        if out is None:
            if x.is_contiguous():
                x.view(-1)[b:e] = mine
                return x.view(-1)[b:e]
            return mine
        out.view(-1).copy_(mine)
        return out

    def _cpu_all_gather(self, shard: torch.Tensor, out: Optional[torch.Tensor], total: Optional[int]) -> torch.Tensor:
        import torch.distributed as dist
        flat = shard.contiguous().view(-1)
        count = total if total is not None else flat.numel() * self.world
        b, e = partition(count, self.world, self.rank)
        if e - b != flat.numel():
            raise ValueError(f"this rank's partition has {e - b} elements, shard has {flat.numel()}")
        pad = max_shard(count, self.world)
        padded = torch.zeros(pad, dtype=flat.dtype)
        padded[:flat.numel()] = flat
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(parts, padded, group=self._cpu_group)
        pieces = []
        for r in range(self.world):
            rb, re = partition(count, self.world, r)
            pieces.append(parts[r][:re - rb])
        result = torch.cat(pieces)
        if out is not None:
            out.view(-1).copy_(result)
            return out
        if total is None and shard.dim() >= 1:
            return result.view((self.world * shard.shape[0],) + tuple(shard.shape[1:]))
        return result
