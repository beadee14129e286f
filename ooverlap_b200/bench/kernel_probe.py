"""Runs one kernel of the library a few times on one GPU and prints its CUDA-event time.

Small enough to sit under a profiler::

    python -m ooverlap_b200.bench.kernel_probe --op gemm --m 8192 --n 8192 --k 8192 --iters 3
    python -m ooverlap_b200.bench.kernel_probe --op gemm_splitk --m 64 --n 8192 --k 8192
    python -m ooverlap_b200.bench.kernel_probe --op rmsnorm --m 16384 --n 8192
    python -m ooverlap_b200.bench.kernel_probe --op allreduce --world 8 --bytes 67108864     (emulated ranks)
    python -m ooverlap_b200.bench.kernel_probe --op gemm_ar --world 2 --m 2048 --n 2048 --k 1024  (emulated ranks)

Each run prints a JSON line with the time per call, the achieved TFLOP/s or GB/s and the fraction of the
measured peak (``MEASURED_PEAKS.json`` beside the repository root when present, else 1629.9 TFLOP/s and
6546 GB/s).

Capability parity: test/bench_gemm_sm90.py:101-190 of the reference (GEMM timing against cuBLAS).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1629.9, 6546.2, "fallback"


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ms.append(a.elapsed_time(b))
    ms.sort()
    return ms[len(ms) // 2]


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--op", default="gemm", choices=["gemm", "gemm_splitk", "cublas", "rmsnorm", "allreduce", "gemm_ar"])
    p.add_argument("--m", type=int, default=8192)
    p.add_argument("--n", type=int, default=8192)
    p.add_argument("--k", type=int, default=8192)
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--world", type=int, default=8)
    p.add_argument("--bytes", type=int, default=64 << 20)
    p.add_argument("--splits", type=int, default=0)
    p.add_argument("--no-flush", action="store_true")
    args = p.parse_args()

    from .. import EmulatedGroup, _lib
    from ..ops import GemmAllReduce, gemm, rmsnorm
    torch.cuda.set_device(0)
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    tf_peak, bw_peak, src = peaks()
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rec = {"op": args.op, "dtype": args.dtype, "peaks": src}
    if args.op in ("gemm", "gemm_splitk", "cublas"):
        a = torch.randn(args.m, args.k, device="cuda").to(dt)
        b = (torch.randn(args.n, args.k, device="cuda") / args.k ** 0.5).to(dt)
        out = torch.empty(args.m, args.n, device="cuda", dtype=dt)
        if args.op == "cublas":
            fn = lambda: torch.matmul(a, b.t(), out=out)  # noqa: E731
        else:
            splits = args.splits if args.op == "gemm_splitk" else 1
            fn = lambda: gemm(a, b, out=out, splits=splits)  # noqa: E731
        ms = timed(fn, args.iters, args.warmup, flush)
        tflops = 2.0 * args.m * args.n * args.k / (ms * 1e-3) / 1e12
        gbs = (args.m * args.k + args.n * args.k + args.m * args.n) * 2 / (ms * 1e-3) / 1e9
        rec.update(M=args.m, N=args.n, K=args.k, us=round(ms * 1e3, 2), tflops=round(tflops, 1),
                   frac_of_peak_tflops=round(tflops / tf_peak, 3), min_traffic_gbs=round(gbs, 1),
                   frac_of_peak_hbm=round(gbs / bw_peak, 3))
    elif args.op == "rmsnorm":
        x = torch.randn(args.m, args.n, device="cuda").to(dt)
        r = torch.randn(args.m, args.n, device="cuda").to(dt)
        w = torch.ones(args.n, device="cuda", dtype=dt)
        y, ro = torch.empty_like(x), torch.empty_like(x)
        ms = timed(lambda: rmsnorm(x, w, 1e-6, r, out=y, residual_out=ro), args.iters, args.warmup, flush)
        gbs = 4.0 * x.numel() * 2 / (ms * 1e-3) / 1e9
        rec.update(rows=args.m, hidden=args.n, us=round(ms * 1e3, 2), gbs=round(gbs, 1), frac_of_peak_hbm=round(gbs / bw_peak, 3))
    elif args.op == "allreduce":
        g = EmulatedGroup(args.world, heap_bytes=args.bytes + (32 << 20))
        n = args.bytes // 2
        off = g.alloc(args.bytes)
        for r in range(args.world):
            g.view(off, (n,), dt, r).fill_(0.001 * (r + 1))
        ms = timed(lambda: g.all_reduce(off, n, dt, algo=_lib.AR_TWOSHOT_P2P, out_off=off, max_ctas=148 // args.world),
                   args.iters, args.warmup, flush)
        g.check_status()
        # every emulated rank reads all ranks' shards and writes them back to all ranks (all on this GPU)
        gbs = 2.0 * args.world * args.bytes / (ms * 1e-3) / 1e9
        rec.update(world=args.world, bytes=args.bytes, us=round(ms * 1e3, 2), local_traffic_gbs=round(gbs, 1),
                   frac_of_peak_hbm=round(gbs / bw_peak, 3))
        g.close()
    else:
        g = EmulatedGroup(args.world, heap_bytes=(args.m * args.n * 2) * 3 + (64 << 20))
        op = GemmAllReduce(g, args.m, args.n, dt, comm_ctas=4)
        a = torch.randn(args.world, args.m, args.k, device="cuda").to(dt)
        b = (torch.randn(args.world, args.n, args.k, device="cuda") / args.k ** 0.5).to(dt)
        ms = timed(lambda: op(a, b), args.iters, args.warmup, flush)
        g.check_status()
        tflops = 2.0 * args.world * args.m * args.n * args.k / (ms * 1e-3) / 1e12
        rec.update(world=args.world, M=args.m, N=args.n, K=args.k, us=round(ms * 1e3, 2), tflops_all_ranks=round(tflops, 1))
        g.close()
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
