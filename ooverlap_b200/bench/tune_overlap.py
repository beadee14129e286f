"""Tuner / evaluation driver for the overlap ops: finds the fastest way to run GEMM->AllReduce for a list of shapes and
keeps it per shape in a solution file that the library loads back (``OOB_OVERLAP_SOLUTIONS``, or the packaged
``ooverlap_b200/policy/overlap_solutions.json``).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \\
        -m ooverlap_b200.bench.tune_overlap --shapes 512x8192x8192,2048x8192x8192,8192x8192x8192 --out solutions.json

Search.  Per shape the tuner first measures the two building blocks alone: this library's GEMM on all SMs and its
all-reduce of the output with a few CTA budgets.  From those it PREDICTS every candidate with a small latency model

* unfused pair      ``t_gemm + t_ar``
* fused kernel      ``max(t_gemm * sms / (sms - c), t_ar(c)) + t_first``   (``c`` communication CTAs; the GEMM runs on
                    the remaining SMs, the reduction streams behind it; ``t_first`` = one wave of tiles plus a flag
                    round trip, the part that cannot overlap)

and then MEASURES the candidates in order of predicted time, stopping when the prediction of the next one is more than
``--slack`` (15 %) above the best time measured so far.  ``--exhaustive`` measures them all.  Every measured candidate
is verified against an fp32 reference first.  The run is resumable: shapes already present in the output file are
skipped unless ``--force``.

Capability parity: tool/search.py:1288-1400 (latency model: interpolated communication curve + wave-scaled GEMM time),
:1475-1638 (exhaustive / predictive search, solution JSON) and the resumable scenario loop of
tool/evaluate_sm90.py:787-1084 in the reference.  The search space is different by construction: no segment
partitions or tile-order hints exist here; the knobs are the strategy, the kernel, the CTA split and the data path.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import Communicator
from ..ops import GemmAllReduce, gemm, solutions
from .overlap_bench import check, timed


def predict_us(cand: dict, t_gemm: float, t_ar: dict, sms: int, t_first: float) -> float:
    """Latency model of one candidate (see the module docstring).  ``t_ar`` maps a CTA budget to the measured
    all-reduce time; budgets in between take the nearest measured one."""
    if cand["strategy"] == "unfused":
        return t_gemm + min(t_ar.values())
    if cand["strategy"] == "chunked":
        slabs = max(1, cand.get("slabs", 4))
        return t_gemm / slabs + max(t_gemm * (slabs - 1) / slabs, min(t_ar.values())) + 10.0
    c = cand["comm_ctas"]
    nearest = min(t_ar, key=lambda k: abs(k - c))
    comm = t_ar[nearest] * (1.75 if not cand["use_nvls"] else 1.0)  # peer stores move 1.75 x the bytes of the switch path
    return max(t_gemm * sms / max(1, sms - c), comm) + t_first


def candidates(comm_ctas, nvls_paths, kernels, M=0, world=0):
    out = [dict(strategy="unfused", kernel="", comm_ctas=0, use_nvls=0)]
    for k in kernels:
        for c in comm_ctas:
            for nv in nvls_paths:
                if k == "pair" and nv == 2:
                    continue  # the two-SM kernel has one switch path (in-place reduce), selected by 1
                out.append(dict(strategy="fused", kernel=k, comm_ctas=c, use_nvls=nv))
    if world >= 4 and M >= 4096 and M % 2048 == 0:
        out.append(dict(strategy="chunked", kernel="", comm_ctas=0, use_nvls=1))  # slab pipeline on two streams
    return out


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--shapes", default="512x8192x8192,2048x8192x8192,8192x8192x8192", help="MxNxK (global K)")
    p.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    p.add_argument("--comm-ctas", default="8,16,24,32")
    p.add_argument("--kernels", default="pair,one_sm")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--slack", type=float, default=0.15)
    p.add_argument("--exhaustive", action="store_true")
    p.add_argument("--out", default="overlap_solutions.json")
    p.add_argument("--log", default="", help="append one JSON line per measured candidate")
    p.add_argument("--force", action="store_true")
    args = p.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(list(range(world)), rank, heap_bytes=2 << 30)
    sms = torch.cuda.get_device_properties(local).multi_processor_count
    dt = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    table = dict(solutions.load(args.out)) if os.path.exists(args.out) else {}
    ctas = [int(v) for v in args.comm_ctas.split(",")]
    paths = [0] + ([1, 2] if comm.nvls else [])
    kernels = [k for k in args.kernels.split(",") if k]
    for shape in args.shapes.split(","):
        M, N, K = (int(v) for v in shape.split("x"))
        k = solutions.key("gemm_ar", M, N, K, world, args.dtype)
        if k in table and not args.force:
            continue
        a = torch.randn(M, K // world, device="cuda").to(dt)
        b = (torch.randn(N, K // world, device="cuda") / K ** 0.5).to(dt)
        want = a.float() @ b.float().t()
        dist.all_reduce(want)
        # building blocks alone
        sym = comm.empty((M, N), dt)
        t_gemm = timed(lambda: gemm(a, b, out=sym, splits=1), args.iters, 3)["us"]
        t_ar = {c: timed(lambda: comm.all_reduce(sym, max_ctas=c), args.iters, 3)["us"] for c in ctas}
        comm.free(comm.heap_offset(sym))
        tiles = ((M + 255) // 256) * ((N + 255) // 256)
        waves = max(1.0, tiles / (sms / 2))
        t_first = t_gemm / waves + 5.0
        cands = candidates(ctas, paths, kernels, M, world)
        for c in cands:
            if c["strategy"] == "chunked":
                c["slabs"] = M // 2048
        for c in cands:
            c["predicted_us"] = round(predict_us(c, t_gemm, t_ar, sms, t_first), 1)
        cands.sort(key=lambda c: c["predicted_us"])
        best, measured = None, 0
        for cand in cands:
            if not args.exhaustive and best is not None and cand["predicted_us"] > best["us"] * (1.0 + args.slack):
                break
            op = GemmAllReduce(comm, M, N, dt, comm_ctas=cand["comm_ctas"] or None,
                               use_nvls=cand["use_nvls"] if cand["strategy"] == "fused" else None,
                               strategy=cand["strategy"], kernel=cand["kernel"] or None)
            check(f"{k} {cand}", op(a, b), want)
            t = timed(lambda: op(a, b), args.iters, 3)
            op.release()
            measured += 1
            rec = dict(cand, us=t["us"], p50=t["p50"], p90=t["p90"], p99=t["p99"])
            if best is None or rec["us"] < best["us"]:
                best = rec
            if rank == 0:
                print(json.dumps({"shape": k, **rec}), flush=True)
                if args.log:
                    with open(args.log, "a") as f:
                        f.write(json.dumps({"shape": k, **rec}) + "\n")
        best = dict(best, gemm_alone_us=t_gemm, allreduce_alone_us=min(t_ar.values()), candidates=len(cands), measured=measured)
        table[k] = best
        if rank == 0:
            solutions.save(args.out, table)
        del want
        dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
