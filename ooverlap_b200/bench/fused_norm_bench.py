"""Latency of the fused all-reduce + residual + RMSNorm op at decode and prefill-chunk sizes, against NCCL all-reduce
followed by PyTorch's residual add and RMSNorm.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \\
        -m ooverlap_b200.bench.fused_norm_bench --hidden 8192 --rows 1,4,16,64,256,1024 --out fused_norm.jsonl

For every row count (message = rows x hidden bf16: 16 KiB for one token of a hidden-8192 model, 4 MiB for 256) the
tool times, from CUDA graphs, with CUDA events, as the maximum over ranks and with p50 / p90 / p99 over the replays:

* ``ours_fused``     one kernel: all-reduce of the registered partial sums + residual add + RMSNorm (what
                     ``fused_allreduce_rmsnorm`` picks for the size)
* ``ours_push+norm`` the one-barrier push all-reduce into a ring slot, then the stand-alone residual + RMSNorm kernel
                     (messages up to ``OOB_PUSH_MAX_BYTES``)
* ``ours_unfused``   this library's in-place all-reduce, then its stand-alone residual + RMSNorm kernel
* ``nccl+torch``     ``dist.all_reduce`` + ``residual.add_`` + ``torch.nn.functional.rms_norm``

and checks each arm's output against an fp32 reference first.

Capability parity: the reference times its all-reduce against NCCL with mean / median / p90 (tool/bandwidth.py:107-253,
test/test.py:331-353); it has no fused normalisation (its RMSNorm kernels are stand-alone, src/rmsnorm/rmsnorm.cuh).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import Communicator
from ..ops import fused_allreduce_rmsnorm, rmsnorm
from ..utils.timing import graph_timed


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--hidden", type=int, default=8192)
    p.add_argument("--rows", default="1,4,16,64,256,1024")
    p.add_argument("--iters", type=int, default=50)
    p.add_argument("--eps", type=float, default=1e-6)
    p.add_argument("--out", default="")
    args = p.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(list(range(world)), rank, heap_bytes=1 << 30)
    comm.init_round_robin_slots(torch.bfloat16, 32 << 20, 4)
    dt = torch.bfloat16
    H = args.hidden
    gen = torch.Generator(device="cuda").manual_seed(7 + rank)
    w = (1 + 0.02 * torch.randn(H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))).to(dt)
    lines = []
    for rows in [int(r) for r in args.rows.split(",")]:
        part = torch.randn(rows, H, device="cuda", generator=gen).to(dt)
        res = torch.randn(rows, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(11)).to(dt)
        x = comm.empty((rows, H), dt)
        x.copy_(part)
        want_sum = part.float().clone()
        dist.all_reduce(want_sum)
        s = (want_sum + res.float()).to(dt).float()
        want = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + args.eps) * w.float()
        nccl_buf = part.clone()

        def ours_fused():
            return fused_allreduce_rmsnorm(comm, x, w, args.eps, res)

        def ours_unfused():
            x.copy_(part)  # the in-place all-reduce overwrites its input
            return rmsnorm(comm.all_reduce(x), w, args.eps, res)

        def ours_push_norm():
            return rmsnorm(comm.all_reduce_push(x), w, args.eps, res)

        def nccl_torch():
            nccl_buf.copy_(part)
            dist.all_reduce(nccl_buf)
            h = nccl_buf + res
            return torch.nn.functional.rms_norm(h, (H,), w, args.eps), h

        base = dict(bench="fused_allreduce_rmsnorm", world=world, rows=rows, hidden=H, bytes=rows * H * 2, dtype="bf16",
                    nvls=int(comm.nvls))
        def ours_fused_32():
            return fused_allreduce_rmsnorm(comm, x, w, args.eps, res, max_ctas=32)

        arms = [("ours_fused", ours_fused), ("ours_unfused", ours_unfused), ("nccl+torch", nccl_torch)]
        if rows * H * 2 > (1 << 20):
            arms.insert(1, ("ours_fused_32ctas", ours_fused_32))
        if rows * H * 2 <= comm.config.push_max_bytes:
            arms.insert(1, ("ours_push+norm", ours_push_norm))
        for name, fn in arms:
            y = fn()[0]
            torch.cuda.synchronize()
            err = (y.float() - want).abs().max().item()
            ok = torch.tensor([1 if err <= 6e-2 * max(1.0, want.abs().max().item()) else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if not ok.item():
                raise RuntimeError(f"{name} rows={rows}: result check failed (this rank: max abs err {err:.4g})")
            t = graph_timed(fn, args.iters, 5, per_graph=5, min_ms=10.0, max_reps=200)
            rec = {**base, "impl": name, "us": round(t["us"], 2), "p50": round(t["p50"], 2), "p90": round(t["p90"], 2),
                   "p99": round(t["p99"], 2), "max_abs_err": round(err, 4)}
            lines.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
        comm.free(comm.heap_offset(x))
        comm.check_status()
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
