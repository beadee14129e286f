"""All GPUs of a node driven by ONE process: a list of communicators, one per device, that a single host thread
launches on in turn.

    group = LocalGroup([0, 1, 2, 3], heap_bytes=1 << 30)
    xs = group.empty((n,), torch.bfloat16)            # one registered tensor per device
    ...fill xs[r] on device r...
    ys = group.all_reduce(xs)                         # one launch per device, back to back, no host synchronisation
    group.synchronize(); group.check_status(); group.close()

Every rank is an ordinary :class:`Communicator` (same heap, same NVLS alias, same kernels); only the host side differs:
the rendezvous runs between threads of this process, and calls that are collective ON THE HOST (creation, barrier,
recover, IPC registration, destruction) are issued from one thread per rank at the same time.  Kernel launches are
asynchronous, so one thread can issue a collective on device 0, 1, 2, ... in turn: each device's kernel waits (with
its usual bounded wait) until its peers' kernels have been launched too.  Nothing synchronous may sit between those
launches; ``each`` keeps to that.

Use it for tuning sweeps and tests that want one process, and for applications that drive a whole node from one
process.  Production serving with one process per GPU uses :class:`Communicator` directly.

Capability parity: oo_group_create_p2p (src/comm/ooverlap_comm_public.cu:707-849) and the single-process sweep
harness of the reference (src/test/external_p2p_collective_sweep_sm90.cu:87-185).
"""
from __future__ import annotations

import threading
import uuid
from typing import Callable, List, Optional, Sequence

import torch

from .comm import Communicator
from .utils.config import Config


class LocalGroup:
    def __init__(self, devices: Optional[Sequence[int]] = None, *, heap_bytes: Optional[int] = None,
                 config: Optional[Config] = None):
        if devices is None:
            devices = list(range(torch.cuda.device_count()))
        self.devices = [int(d) for d in devices]
        if len(set(self.devices)) != len(self.devices) or not self.devices:
            raise ValueError("devices must be distinct CUDA device indices")
        self.world = len(self.devices)
        self.comms: List[Optional[Communicator]] = [None] * self.world
        key = "lg_" + uuid.uuid4().hex[:20]

        def make(r: int):
            torch.cuda.set_device(self.devices[r])
            self.comms[r] = Communicator(self.devices, r, key, heap_bytes=heap_bytes, config=config)

        self._host_collective(make)
        self.nvls = all(c.nvls for c in self.comms)

    # ------------------------------------------------------------------ plumbing
    def _host_collective(self, fn: Callable[[int], object]) -> list:
        """Runs ``fn(rank)`` for every rank at the same time, one thread per rank (for calls that rendezvous on the
        host).  The first exception is re-raised after all threads have ended."""
        results, errors = [None] * self.world, [None] * self.world

        def run(r: int):
            try:
                torch.cuda.set_device(self.devices[r])
                results[r] = fn(r)
            except BaseException as e:  # noqa: BLE001 - handed to the caller below
                errors[r] = e

        threads = [threading.Thread(target=run, args=(r,), name=f"oob-rank{r}") for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        for e in errors:
            if e is not None:
                raise e
        return results

    def each(self, fn: Callable[[int, Communicator], object]) -> list:
        """Runs ``fn(rank, comm)`` for every rank in turn on the calling thread with the rank's device current.  For
        kernel launches (asynchronous); ``fn`` must not synchronise with the device."""
        out = []
        for r, c in enumerate(self.comms):
            with torch.cuda.device(self.devices[r]):
                out.append(fn(r, c))
        return out

    def synchronize(self) -> None:
        for d in self.devices:
            torch.cuda.synchronize(d)

    # ------------------------------------------------------------------ memory
    def empty(self, shape, dtype: torch.dtype) -> List[torch.Tensor]:
        """One registered tensor per device, at the same heap offset on every rank."""
        return self.each(lambda r, c: c.empty(shape, dtype))

    def free(self, tensors: Sequence[torch.Tensor]) -> None:
        self.each(lambda r, c: c.free(c.heap_offset(tensors[r])))

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, xs: Sequence[torch.Tensor], op: str = "sum", **kw) -> List[torch.Tensor]:
        return self.each(lambda r, c: c.all_reduce(xs[r], op, **kw))

    def reduce_scatter(self, xs: Sequence[torch.Tensor], outs: Optional[Sequence[torch.Tensor]] = None, op: str = "sum",
                       **kw) -> List[torch.Tensor]:
        return self.each(lambda r, c: c.reduce_scatter(xs[r], None if outs is None else outs[r], op, **kw))

    def all_gather(self, shards: Sequence[torch.Tensor], outs: Optional[Sequence[torch.Tensor]] = None,
                   **kw) -> List[torch.Tensor]:
        return self.each(lambda r, c: c.all_gather(shards[r], None if outs is None else outs[r], **kw))

    def all_to_all(self, xs: Sequence[torch.Tensor], outs: Optional[Sequence[torch.Tensor]] = None,
                   **kw) -> List[torch.Tensor]:
        return self.each(lambda r, c: c.all_to_all(xs[r], None if outs is None else outs[r], **kw))

    # ------------------------------------------------------------------ host-side collectives
    def init_round_robin_slots(self, dtype: torch.dtype, capacity_bytes: int, slot_count: int) -> None:
        """Slot ring on every rank (the ranks meet on the host while they set it up)."""
        self._host_collective(lambda r: self.comms[r].init_round_robin_slots(dtype, capacity_bytes, slot_count))

    def barrier(self) -> None:
        self._host_collective(lambda r: self.comms[r].barrier())

    def check_status(self) -> None:
        self.synchronize()
        for c in self.comms:
            c.check_status()

    def recover(self) -> None:
        self._host_collective(lambda r: self.comms[r].recover())

    def close(self) -> None:
        if any(c is not None and not c.is_cpu for c in self.comms):
            self.synchronize()
            self._host_collective(lambda r: self.comms[r].close() if self.comms[r] is not None else None)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
