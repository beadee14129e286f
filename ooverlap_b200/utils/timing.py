"""Device-side timing helpers and a clock/throttle sampler.

Capability parity: include/ooverlap/testing/timing.cuh:13-42 and
two_gpu_test_utils.cuh:21-84 (CUDA events per rank, maximum over ranks).
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable

import torch


def flush_l2(buf: torch.Tensor | None = None) -> torch.Tensor:
    """Overwrites a buffer larger than the 126 MB L2 so that the next kernel starts cold."""
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    buf.fill_(1)
    return buf


def time_cuda(fn: Callable[[], None], iters: int, warmup: int = 3, flush: torch.Tensor | None = None) -> list[float]:
    """Per-iteration device time in milliseconds (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        out.append(a.elapsed_time(b))
    return out


def max_over_ranks(value: float, group=None) -> float:
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized():
        return value
    dev = "cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0, period_ms: int = 100):
        self.device_index = device_index
        self.period_ms = period_ms
        self._proc = None
        self._lines: list[str] = []
        self._thread = None

    def start(self) -> "ClockSampler":
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def pump():
            assert self._proc is not None and self._proc.stdout is not None
            for line in self._proc.stdout:
                self._lines.append(line.strip())

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        if self._proc is not None:
            time.sleep(self.period_ms / 1000.0)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thread is not None:
                self._thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}
