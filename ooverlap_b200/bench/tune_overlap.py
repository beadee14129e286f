"""Tuner / evaluation driver for the overlap ops: measures every strategy of GEMM->AllReduce for a list of shapes
and keeps the best one per shape in a solution file that the library loads back (``OOB_OVERLAP_SOLUTIONS``).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        -m ooverlap_b200.bench.tune_overlap --shapes 512x8192x8192,2048x8192x8192,8192x8192x8192 --out solutions.json

Candidates per shape: the unfused pair (GEMM + policy-selected all-reduce) and the fused kernel over
``--comm-ctas`` x {peer pushes, pushes + multicast result, in-switch reduction}.  The run is resumable: shapes
already present in the output file are skipped unless ``--force``.

Capability parity: tool/search.py:1475-1693 (candidate enumeration, measurement, solution JSON) and the resumable
scenario loop of tool/evaluate_sm90.py:787-1084 in the reference.  The search space is different by construction:
no segment partitions or tile-order hints exist here, the knobs are the strategy, the CTA split and the data path.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

from .. import Communicator
from ..ops import GemmAllReduce, solutions
from .overlap_bench import timed


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--shapes", default="512x8192x8192,2048x8192x8192,8192x8192x8192", help="MxNxK (global K)")
    p.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    p.add_argument("--comm-ctas", default="8,16,24")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--out", default="overlap_solutions.json")
    p.add_argument("--force", action="store_true")
    args = p.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(list(range(world)), rank, heap_bytes=2 << 30)
    dt = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    table = dict(solutions.load(args.out)) if os.path.exists(args.out) else {}
    for shape in args.shapes.split(","):
        M, N, K = (int(v) for v in shape.split("x"))
        k = solutions.key("gemm_ar", M, N, K, world, args.dtype)
        if k in table and not args.force:
            continue
        a = torch.randn(M, K // world, device="cuda").to(dt)
        b = (torch.randn(N, K // world, device="cuda") / K ** 0.5).to(dt)
        cands = [dict(strategy="unfused", comm_ctas=0, use_nvls=0)]
        paths = [0] + ([1, 2] if comm.nvls else [])
        for c in (int(v) for v in args.comm_ctas.split(",")):
            cands += [dict(strategy="fused", comm_ctas=c, use_nvls=nv) for nv in paths]
        best = None
        for cand in cands:
            op = GemmAllReduce(comm, M, N, dt, comm_ctas=cand["comm_ctas"] or None, use_nvls=cand["use_nvls"],
                               strategy=cand["strategy"])
            us = timed(lambda: op(a, b), args.iters, 3)
            op.release()
            if best is None or us < best["us"]:
                best = dict(cand, us=round(us, 1))
            if rank == 0:
                print(f"{k} {cand} {us:.1f} us", flush=True)
        table[k] = best
        if rank == 0:
            solutions.save(args.out, table)
        dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
