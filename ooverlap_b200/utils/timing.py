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


def percentiles(samples: list[float]) -> dict:
    """p50 / p90 / p99 / mean of a list of latencies (nearest-rank), as the reference's benches report them
    (test/test.py:331-353, tool/bandwidth.py:107-253)."""
    if not samples:
        return {"p50": None, "p90": None, "p99": None, "mean": None, "n": 0}
    xs = sorted(samples)

    def rank(q):
        return xs[min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))]

    return {"p50": rank(0.5), "p90": rank(0.9), "p99": rank(0.99), "mean": sum(xs) / len(xs), "n": len(xs)}


def graph_timed(fn: Callable[[], None], iters: int, warmup: int, *, per_graph: int = 5, min_ms: float = 30.0,
                max_reps: int = 400, use_graph: bool = True) -> dict:
    """Times ``fn`` on every rank of the default process group and returns microseconds per call as the maximum over
    ranks: ``us`` (the median of three back-to-back runs of ``reps`` graph replays) and ``p50`` / ``p90`` / ``p99``
    over the individual replays of those runs (each replay is ``per_graph`` calls, timed with its own pair of CUDA
    events).  Calls are replayed from a CUDA graph so that small operations measure the kernels, not the Python launch
    path; a measurement lasts at least ``min_ms`` of device time so that the start skew between ranks is amortised."""
    import torch.distributed as dist
    multi = dist.is_available() and dist.is_initialized()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = None
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(per_graph):
                    fn()
            graph.replay()
        except Exception:  # capture refused: eager launches
            graph = None
    torch.cuda.synchronize()

    def rank_max(v: float) -> float:
        if not multi:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def once(reps: int):
        if multi:
            dist.barrier()
        torch.cuda.synchronize()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        evs[0].record()
        for i in range(reps):
            if graph is not None:
                graph.replay()
            else:
                for _ in range(per_graph):
                    fn()
            evs[i + 1].record()
        torch.cuda.synchronize()
        each = [evs[i].elapsed_time(evs[i + 1]) / per_graph * 1e3 for i in range(reps)]
        return evs[0].elapsed_time(evs[reps]) / (reps * per_graph) * 1e3, each

    pilot, _ = once(max(1, iters // per_graph))
    pilot = rank_max(pilot)
    reps = max(1, int(min(max_reps, max(iters // per_graph, min_ms * 1e3 / max(pilot * per_graph, 1.0)))))
    runs, every = [], []
    for _ in range(3):
        us, each = once(reps)
        runs.append(rank_max(us))
        every += each
    runs.sort()
    pc = percentiles(every)
    return {"us": runs[1], "best_us": runs[0], "p50": rank_max(pc["p50"]), "p90": rank_max(pc["p90"]),
            "p99": rank_max(pc["p99"]), "replays": pc["n"], "per_replay": per_graph, "graph": graph is not None}


class NvmlClockSampler:
    """Samples the SM clock, power and clock-event reasons of one GPU through NVML (read-only queries) from a thread,
    every ``period_ms``.  ``begin()`` / ``end()`` bracket the timed region: only samples taken between them are
    summarised, so that a short region is not diluted by the idle clocks around it.  ``available`` is False when NVML
    (the ``pynvml`` module) cannot be used; the nvidia-smi based :class:`ClockSampler` is the fallback then."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, cuda_index: int = 0, period_ms: float = 2.0):
        self.period = period_ms / 1000.0
        self._samples: list[tuple[float, int, int, float]] = []  # (time, sm MHz, reasons, watts)
        self._stop = threading.Event()
        self._thread = None
        self._t0 = self._t1 = None
        self._max_mhz = None
        self.available = False
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:
                uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
            self._nvml, self._handle = pynvml, handle
            self._reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons")
            self._max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self._read()
            self.available = True
        except Exception:
            self.available = False

    def _read(self):
        n = self._nvml
        mhz = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
        reasons = int(self._reasons_fn(self._handle))
        try:
            watts = n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
        except Exception:
            watts = 0.0
        return time.perf_counter(), int(mhz), reasons, watts

    def start(self) -> "NvmlClockSampler":
        if not self.available:
            return self

        def loop():
            while not self._stop.is_set():
                try:
                    self._samples.append(self._read())
                except Exception:
                    pass
                time.sleep(self.period)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def begin(self) -> None:
        self._t0 = time.perf_counter()

    def end(self) -> None:
        self._t1 = time.perf_counter()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        t0 = self._t0 if self._t0 is not None else 0.0
        t1 = self._t1 if self._t1 is not None else float("inf")
        inside = [s for s in self._samples if t0 <= s[0] <= t1]
        used = inside if len(inside) >= 3 else self._samples  # a very short region: report what there is
        bits = 0
        for s in used:
            bits |= s[2]
        return {"sm_mhz": statistics.median([s[1] for s in used]) if used else None, "sm_max_mhz": self._max_mhz,
                "reasons": sorted(name for bit, name in self.REASONS.items() if bits & bit),
                "samples": len(inside), "samples_total": len(self._samples),
                "power_w_max": round(max((s[3] for s in used), default=0.0), 1), "source": "nvml"}


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
