"""Host <-> device staging for a stepped workload: the next step's inputs travel from pinned host memory while the
current step computes, and a step's result is read back without stalling the launch of the next step.

    io = HostPipeline({"x": (rows, k)}, torch.float16, depth=2)
    io.feed({"x": host_batch_0})                    # H2D of step 0 starts on the copy stream
    for i in range(steps):
        dev = io.take()                             # compute stream waits for step i's copy only
        if i + 1 < steps:
            io.feed({"x": host_batches[i + 1]})     # H2D of step i + 1 overlaps step i's kernels
        y = op(dev["x"], w)
        io.done()                                   # step i's buffers may be overwritten once its kernels finished
        fut = io.read_back(y[0], pinned_row)        # D2H on the copy stream, after step i's kernels
        ...                                         # fut.wait() one step later (or at the end)

Everything is ordered with CUDA events; no call blocks the host except ``ReadBack.wait``.

Capability parity: none in the reference (its benchmarks create their operands on the device); this is what a serving
or training loop around the overlap ops needs so that PCIe traffic hides behind the kernels.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch


class ReadBack:
    """A device-to-host copy in flight."""

    def __init__(self, event: "torch.cuda.Event", host: torch.Tensor):
        self._event, self.host = event, host

    def wait(self) -> torch.Tensor:
        self._event.synchronize()
        return self.host

    def ready(self) -> bool:
        return self._event.query()


class HostPipeline:
    def __init__(self, shapes: Dict[str, Sequence[int]], dtype: torch.dtype, *, depth: int = 2,
                 device: Optional[torch.device] = None):
        if depth < 2:
            raise ValueError("depth must be at least 2 (one buffer in use, one being filled)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.depth = depth
        self.copy_stream = torch.cuda.Stream(device=self.device)   # host -> device
        self.back_stream = torch.cuda.Stream(device=self.device)   # device -> host (its own queue: a read-back never
                                                                   # waits behind the next step's input copy)
        self._bufs = [{k: torch.empty(tuple(s), dtype=dtype, device=self.device) for k, s in shapes.items()}
                      for _ in range(depth)]
        self._filled = [torch.cuda.Event() for _ in range(depth)]   # H2D into buffer j finished
        self._free = [None] * depth                                 # kernels that read buffer j finished
        self._fed = 0      # feeds so far
        self._taken = 0    # takes so far
        self._doned = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._snap = {}    # (shape, dtype) -> ring of [staging tensor, event of its last read-back]

    def feed(self, host: Dict[str, torch.Tensor]) -> None:
        """Starts the copy of one step's inputs (pinned host tensors) into the next free buffer."""
        if self._fed - self._doned >= self.depth:
            raise RuntimeError("every buffer is in use: call done() for an earlier step first")
        j = self._fed % self.depth
        with torch.cuda.stream(self.copy_stream):
            if self._free[j] is not None:
                self.copy_stream.wait_event(self._free[j])
            for k, dst in self._bufs[j].items():
                src = host[k]
                if not src.is_pinned():
                    raise ValueError(f"input {k!r} must be in pinned host memory")
                dst.copy_(src, non_blocking=True)
                self.h2d_bytes += src.numel() * src.element_size()
            self._filled[j].record(self.copy_stream)
        self._fed += 1

    def take(self) -> Dict[str, torch.Tensor]:
        """The device tensors of the oldest fed step; the current stream waits for their copy."""
        if self._taken >= self._fed:
            raise RuntimeError("take() without a matching feed()")
        j = self._taken % self.depth
        torch.cuda.current_stream(self.device).wait_event(self._filled[j])
        self._taken += 1
        return self._bufs[j]

    def done(self) -> None:
        """Marks the kernels enqueued so far on the current stream as the last readers of the oldest taken step."""
        if self._doned >= self._taken:
            raise RuntimeError("done() without a matching take()")
        j = self._doned % self.depth
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._free[j] = ev
        self._doned += 1

    def read_back(self, src: torch.Tensor, host: torch.Tensor, *, snapshot: bool = True) -> ReadBack:
        """Copies ``src`` (device) into ``host`` (pinned) on the read-back stream once the kernels enqueued so far on the
        current stream have finished.  With ``snapshot`` (default) ``src`` is first copied, on the current stream,
        into a small staging tensor owned by the pipeline, so that later kernels may overwrite ``src`` at once;
        without it ``src`` must stay untouched until the returned handle is ready."""
        if not host.is_pinned():
            raise ValueError("the destination must be in pinned host memory")
        cur = torch.cuda.current_stream(self.device)
        if snapshot:
            key = (tuple(src.shape), src.dtype)
            ring = self._snap.setdefault(key, [])
            slot = None
            for ent in ring:  # a staging tensor whose earlier read-back has finished
                if ent[1] is None or ent[1].query():
                    slot = ent
                    break
            if slot is None:
                if len(ring) >= 2 * self.depth:  # bounded: reuse the oldest, ordered behind its copy
                    slot = ring[0]
                    cur.wait_event(slot[1])
                    ring.append(ring.pop(0))
                else:
                    slot = [torch.empty_like(src, memory_format=torch.contiguous_format), None]
                    ring.append(slot)
            slot[0].copy_(src)
            src = slot[0]
        ready = torch.cuda.Event()
        ready.record(cur)
        done = torch.cuda.Event()
        with torch.cuda.stream(self.back_stream):
            self.back_stream.wait_event(ready)
            host.copy_(src, non_blocking=True)
            done.record(self.back_stream)
        if snapshot:
            slot[1] = done
        self.d2h_bytes += src.numel() * src.element_size()
        return ReadBack(done, host)
