"""GEMM configuration profiler: for a list of shapes, times every way this library can run a plain GEMM and records
the fastest per shape in a table that ``ops.gemm`` loads back (``OOB_GEMM_SOLUTIONS`` or the packaged
``ooverlap_b200/policy/gemm_solutions.json``).

    python -m ooverlap_b200.bench.gemm_profile --shapes 512x8192x8192,2048x8192x8192,64x8192x3584 --out gemm_solutions.json

Candidates per shape (each verified against an fp32 reference before it is timed):

* the two-SM kernel (CTA pairs, 256x256 tiles) without and with the stream-K tail,
* the one-SM kernel (128x256 tiles) unsplit and with K split 2 / 4 / 8 / 16 ways (fp32 partials, summed by a second
  kernel) where K allows,
* the weight-streaming kernel for M <= 128 and the CUDA-core kernel for M <= 4,
* the library's own rule (all arguments 0) and cuBLAS (``torch.matmul``) as the yardsticks.

Timing: CUDA-graph replay, CUDA events, ``--rotate`` operand sets cycled inside the graph so that shapes smaller than
L2 are not measured L2-warm (set ``--rotate 1`` to measure the warm case on purpose); the candidates are measured round
robin in ``--rounds`` passes and the median per candidate is kept, so that clock drift over the run is not credited to a
kernel.

Capability parity: tool/gen_config_sm90.py:175-357 and the profiling pass of src/gemm/gemm_with_signal_sm90.h:238-292
in the reference pick one of its generated tile / cluster / stream-K instances per shape; here the instances are the
kernels above and the choice is stored per shape in the same way.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from ..ops import gemm
from ..ops import solutions
from ..utils.timing import graph_timed

L2_BYTES = 126 << 20


def candidates(M: int, N: int, K: int):
    out = [dict(name="rule", kw={})]
    if M > 128:
        out.append(dict(name="pair", kw=dict(pair=1, splits=1, stream_k=-1)))
        out.append(dict(name="pair+stream_k", kw=dict(pair=1, splits=1, stream_k=1)))
    out.append(dict(name="one_sm", kw=dict(pair=-1, splits=1)))
    for s in (2, 4, 8, 16):
        if K // s >= 256 and (K // 64) % s == 0:
            out.append(dict(name=f"one_sm/split{s}", kw=dict(pair=-1, splits=s)))
    if M <= 128:
        out.append(dict(name="weight_streaming", kw=dict(skinny=1)))
    if M <= 4:
        out.append(dict(name="cuda_core", kw=dict(gemv=1)))
    return out


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--shapes", default="512x8192x8192,2048x8192x8192,8192x8192x8192", help="MxNxK, comma separated")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--rounds", type=int, default=3, help="round-robin passes over the candidates (median is kept)")
    p.add_argument("--rotate", type=int, default=0, help="operand sets cycled per graph (0 = enough to exceed L2)")
    p.add_argument("--out", default="gemm_solutions.json")
    p.add_argument("--log", default="", help="append one JSON line per measured candidate")
    p.add_argument("--force", action="store_true")
    args = p.parse_args()
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    table = dict(solutions.load(args.out)) if os.path.exists(args.out) else {}
    for shape in args.shapes.split(","):
        M, N, K = (int(v) for v in shape.split("x"))
        key = solutions.gemm_key(M, N, K, args.dtype)
        if key in table and not args.force:
            continue
        per_set = (M * K + N * K + M * N) * 2
        rotate = args.rotate or max(1, min(8, -(-2 * L2_BYTES // per_set)))
        g = torch.Generator(device="cuda").manual_seed(M + 3 * N + 7 * K)
        a = [torch.randn(M, K, device="cuda", generator=g).to(dt) for _ in range(rotate)]
        b = [(torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dt) for _ in range(rotate)]
        out = torch.empty(M, N, device="cuda", dtype=dt)
        want = a[0].float() @ b[0].float().t()
        scale = max(1.0, want.abs().max().item())
        rows = []

        def run_all(fn):
            for i in range(rotate):
                fn(a[i], b[i])

        runnable = []
        for cand in candidates(M, N, K):
            kw = cand["kw"]
            try:
                got = gemm(a[0], b[0], **kw)
                torch.cuda.synchronize()
            except Exception as e:  # a kernel that does not take this shape
                rows.append(dict(name=cand["name"], us=None, error=str(e)[:120]))
                continue
            err = (got.float() - want).abs().max().item()
            if not err <= 1e-2 * scale:
                rows.append(dict(name=cand["name"], us=None, error=f"max abs err {err:.3g}"))
                continue
            runnable.append(cand)
        # Round robin over the candidates, several rounds, median per candidate: the GPU's clock state drifts over a run
        # (power cap, temperature), and measuring one candidate after the other would credit that drift to the kernels.
        samples = {c["name"]: [] for c in runnable}
        samples["cublas"] = []
        for _ in range(args.rounds):
            for cand in runnable:
                kw = cand["kw"]
                t = graph_timed(lambda: run_all(lambda x, w: gemm(x, w, out=out, **kw)), args.iters, 2, per_graph=2,
                                min_ms=8.0)
                samples[cand["name"]].append(t["us"] / rotate)
            t = graph_timed(lambda: run_all(lambda x, w: torch.matmul(x, w.t(), out=out)), args.iters, 2, per_graph=2,
                            min_ms=8.0)
            samples["cublas"].append(t["us"] / rotate)
        med = {k: sorted(v)[len(v) // 2] for k, v in samples.items()}
        for cand in runnable:
            rows.append(dict(name=cand["name"], kw=cand["kw"], us=round(med[cand["name"]], 2),
                             spread=round(max(samples[cand["name"]]) - min(samples[cand["name"]]), 2)))
        cublas_us = round(med["cublas"], 2)
        ok = [r for r in rows if r.get("us") and r["name"] != "rule"]
        best = min(ok, key=lambda r: r["us"])
        rule = next((r for r in rows if r["name"] == "rule"), None)
        flops = 2.0 * M * N * K
        entry = dict(best["kw"], name=best["name"], us=best["us"], tflops=round(flops / best["us"] / 1e6, 1),
                     rule_us=rule.get("us") if rule else None, cublas_us=cublas_us, rotate=rotate,
                     candidates={r["name"]: r.get("us") for r in rows})
        table[key] = entry
        line = json.dumps({"shape": key, **entry})
        print(line, flush=True)
        if args.log:
            with open(args.log, "a") as f:
                f.write(line + "\n")
        solutions.save(args.out, table)
        del a, b, want
    return 0


if __name__ == "__main__":
    sys.exit(main())
