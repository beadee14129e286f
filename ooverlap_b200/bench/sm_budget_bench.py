"""A collective on a few CTAs running BESIDE a GEMM on the remaining SMs: what each loses to the other.

The point of SM-efficient collectives is that a GEMM can keep almost every SM while the collective runs.  For every
CTA budget ``c`` this tool times, on every rank (CUDA events, max over ranks, CUDA-graph replay):

* the GEMM alone on all SMs and alone on ``148 - c`` SMs,
* the collective alone with ``c`` CTAs,
* both together: the collective on a side stream (launched first, ``c`` CTAs), the GEMM on the main stream with the
  remaining SMs; the time of each inside the pair and the time until both are done,

and reports the slow-down of each (together / alone) and how much of the shorter one is hidden
(``(gemm_alone + coll_alone - both) / min(gemm_alone, coll_alone)``).  NCCL's all-reduce beside cuBLAS is measured
the same way (NCCL picks its own CTA count) as the comparison point.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \\
        -m ooverlap_b200.bench.sm_budget_bench --bytes 67108864 --ctas 4,8,16,32 --gemm 8192,8192,1024

Capability parity: evalution/run_external_p2p_sm_usage.sh:400-428 and tool/nsys_sm_usage.py:38-78 of the reference
measure the median "SMs Active" of its collectives with nsys (not installed here); active_sm_count
(src/gemm/gemm_with_signal_sm90.h:408-410) is its knob for leaving SMs to the communication.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import Communicator
from ..ops import gemm

PER_GRAPH = 4


def _time_pair(main_fn, side_fn, side_stream, reps):
    """Runs side_fn on the side stream and main_fn on the current stream, forked from one event and joined at the end,
    from a CUDA graph.  Returns (us_main, us_side, us_both) per call, max over ranks."""
    fork, joined = torch.cuda.Event(), torch.cuda.Event()
    ev = {k: [torch.cuda.Event(enable_timing=True) for _ in range(2)] for k in ("main", "side")}

    def body(timed: bool):
        # The stream that is current NOW: inside torch.cuda.graph(...) that is the capture stream, and only work forked
        # from it is captured.
        main = torch.cuda.current_stream()
        fork.record(main)
        if side_fn is not None:
            side_stream.wait_event(fork)
            with torch.cuda.stream(side_stream):
                if timed:
                    ev["side"][0].record(side_stream)
                side_fn()
                if timed:
                    ev["side"][1].record(side_stream)
                joined.record(side_stream)
        if main_fn is not None:
            if timed:
                ev["main"][0].record(main)
            main_fn()
            if timed:
                ev["main"][1].record(main)
        if side_fn is not None:
            main.wait_event(joined)

    for _ in range(3):
        body(False)
    torch.cuda.synchronize()
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(PER_GRAPH):
                body(False)
        graph.replay()
    except Exception:
        graph = None
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        if graph is not None:
            graph.replay()
        else:
            for _ in range(PER_GRAPH):
                body(False)
    b.record()
    torch.cuda.synchronize()
    both = a.elapsed_time(b) / (reps * PER_GRAPH) * 1e3
    # the split between the two, from one eager pass with events on both streams
    dist.barrier()
    body(True)
    torch.cuda.synchronize()
    t_main = ev["main"][0].elapsed_time(ev["main"][1]) * 1e3 if main_fn is not None else 0.0
    t_side = ev["side"][0].elapsed_time(ev["side"][1]) * 1e3 if side_fn is not None else 0.0
    t = torch.tensor([t_main, t_side, both], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1]), float(t[2])


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--bytes", type=int, default=64 << 20, help="all-reduce message")
    p.add_argument("--ctas", default="4,8,16,32")
    p.add_argument("--gemm", default="8192,8192,1024", help="M,N,K of the GEMM that runs beside the collective")
    p.add_argument("--reps", type=int, default=20)
    p.add_argument("--out", default="")
    args = p.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(list(range(world)), rank, heap_bytes=args.bytes + (256 << 20))
    sms = torch.cuda.get_device_properties(local).multi_processor_count
    M, N, K = (int(v) for v in args.gemm.split(","))
    dt = torch.bfloat16
    a = torch.randn(M, K, device="cuda").to(dt)
    b = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dt)
    c = torch.empty(M, N, device="cuda", dtype=dt)
    n = args.bytes // 2
    sym = comm.empty((n,), dt)
    sym.fill_(0.001)
    nccl_buf = torch.full((n,), 0.001, device="cuda", dtype=dt)
    side = torch.cuda.Stream()
    lines = []

    def emit(rec):
        lines.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    base = dict(bench="sm_budget", world=world, sms=sms, gemm=[M, N, K], bytes=args.bytes, nvls=int(comm.nvls))
    g_full, _, _ = _time_pair(lambda: gemm(a, b, out=c, splits=1), None, side, args.reps)
    emit({**base, "arm": "gemm_alone", "ctas_gemm": sms, "us": round(g_full, 1)})
    for ctas in [int(v) for v in args.ctas.split(",")]:
        rest = (sms - ctas) // 2 * 2
        g_rest, _, _ = _time_pair(lambda: gemm(a, b, out=c, splits=1, max_ctas=rest), None, side, args.reps)
        _, c_alone, _ = _time_pair(None, lambda: comm.all_reduce(sym, max_ctas=ctas), side, args.reps)
        sym.fill_(0.001)
        g_in, c_in, both = _time_pair(lambda: gemm(a, b, out=c, splits=1, max_ctas=rest),
                                      lambda: comm.all_reduce(sym, max_ctas=ctas), side, args.reps)
        sym.fill_(0.001)
        emit({**base, "arm": "ours", "ctas_coll": ctas, "ctas_gemm": rest, "gemm_alone_all_sms_us": round(g_full, 1),
              "gemm_alone_us": round(g_rest, 1), "coll_alone_us": round(c_alone, 1), "gemm_beside_us": round(g_in, 1),
              "coll_beside_us": round(c_in, 1), "both_us": round(both, 1),
              "gemm_slowdown": round(g_in / g_full, 3), "coll_slowdown": round(c_in / c_alone, 3),
              "hidden_fraction": round((g_rest + c_alone - both) / max(1e-9, min(g_rest, c_alone)), 3)})
        comm.check_status()
    # NCCL beside cuBLAS (NCCL chooses its own CTA count)
    mm_alone, _, _ = _time_pair(lambda: torch.matmul(a, b.t(), out=c), None, side, args.reps)
    _, n_alone, _ = _time_pair(None, lambda: dist.all_reduce(nccl_buf), side, args.reps)
    nccl_buf.fill_(0.001)
    mm_in, n_in, both = _time_pair(lambda: torch.matmul(a, b.t(), out=c), lambda: dist.all_reduce(nccl_buf), side, args.reps)
    emit({**base, "arm": "nccl+cublas", "gemm_alone_us": round(mm_alone, 1), "coll_alone_us": round(n_alone, 1),
          "gemm_beside_us": round(mm_in, 1), "coll_beside_us": round(n_in, 1), "both_us": round(both, 1),
          "gemm_slowdown": round(mm_in / mm_alone, 3), "coll_slowdown": round(n_in / n_alone, 3),
          "hidden_fraction": round((mm_alone + n_alone - both) / max(1e-9, min(mm_alone, n_alone)), 3)})
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for rec in lines:
                f.write(json.dumps(rec) + "\n")
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
