"""Headline benchmark: GEMM -> AllReduce (row-parallel tensor-parallel linear), fp16.

One step = the three shapes of the headline config run back to back:
``A[M, K/tp] @ B[N, K/tp]^T`` summed over the ``tp`` ranks for M in {512, 2048, 8192},
N = K = 8192.  The reported value is the latency of one step in microseconds
(lower is better); total work is fixed as ``tp`` grows (strong scaling).

``--impl ours``         fused tcgen05 GEMM + in-kernel all-reduce of this repository (default)
``--impl nccl_cublas``  torch.matmul (cuBLAS) followed by NCCL all-reduce: the path the reference's
                        BaselineImpl takes (src/baseline_impl.cu:55-106), measured on this machine
``--impl reference``    the unmodified reference package; it cannot be built offline, so this arm prints
                        why and exits 0

Launch: ``python bench.py`` for one GPU, or through ``python -m torch.distributed.run --nproc-per-node N``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

MS = (512, 2048, 8192)
N_DIM = 8192
K_DIM = 8192
ROTATE = 4  # operand sets cycled between steps so that no step finds its inputs in L2

REFERENCE_UNAVAILABLE = (
    "reference cannot be installed offline: pip reports that the reference tree has neither setup.py nor pyproject.toml, "
    "its CMake build needs the empty submodules src/third-party/{cutlass,nccl,nlohmann_json}, and its device code "
    "is compute_90a only (WGMMA GEMMs do not run on sm_100)")


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl_cublas"])
    p.add_argument("--comm-ctas", type=int, default=int(os.environ.get("OOB_BENCH_COMM_CTAS", "0")),
                   help="communication CTAs of the fused kernel (0 = the library's choice per shape)")
    p.add_argument("--strategy", default="auto", choices=["auto", "fused", "unfused", "chunked"])
    return p.parse_args()


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:  # one line per job, also when launched as several ranks
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be launched with torch.distributed.run", file=sys.stderr)
            return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from ooverlap_b200 import Communicator
    from ooverlap_b200.ops import GemmAllReduce, gemm
    from ooverlap_b200.utils.timing import ClockSampler

    dtype = torch.float16
    k_local = K_DIM // world
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    # Host copies of the activations in pinned memory (end-to-end arm copies them in every step).
    a_host = {m: torch.randn(m, k_local, generator=torch.Generator().manual_seed(rank * 7 + m)).to(dtype).pin_memory()
              for m in MS}
    a_dev = {m: [a_host[m].to(dev, non_blocking=True).clone() for _ in range(ROTATE)] for m in MS}
    weights = [(torch.randn(N_DIM, k_local, device=dev, generator=gen) / K_DIM ** 0.5).to(dtype) for _ in range(ROTATE)]

    comm = None
    ops = {}
    launches_per_step = 0
    if args.impl == "ours":
        if world > 1:
            heap = sum(2 * m * N_DIM * 2 for m in MS) + (64 << 20)
            comm = Communicator(list(range(world)), rank, heap_bytes=heap)
            for m in MS:
                ops[m] = GemmAllReduce(comm, m, N_DIM, dtype, comm_ctas=args.comm_ctas or None, strategy=args.strategy)
        per_op = {"unfused": lambda op: 2, "chunked": lambda op: 2 * op.chunks}
        launches_per_step = sum(per_op.get(ops[m].strategy, lambda op: 1)(ops[m]) if m in ops else 1 for m in MS)

    outs = {m: torch.empty(m, N_DIM, dtype=dtype, device=dev) for m in MS}

    def step(i: int, a_of=None):
        w = weights[i % ROTATE]
        for m in MS:
            a = a_of[m] if a_of is not None else a_dev[m][i % ROTATE]
            if args.impl == "ours":
                if world > 1:
                    outs[m] = ops[m](a, w)
                else:
                    gemm(a, w, out=outs[m])
            else:
                torch.matmul(a, w.t(), out=outs[m])
                if world > 1:
                    dist.all_reduce(outs[m])

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- correctness spot check (outside the timed region) ----------------
    step(0)
    fence()
    ref = a_dev[512][0].float() @ weights[0].float().t()
    if world > 1:
        dist.all_reduce(ref)
    err = (outs[512].float() - ref).abs().max().item()
    if not err <= 2e-2 * max(1.0, ref.abs().max().item()):
        print(f"rank {rank}: result check failed, max abs err {err}", file=sys.stderr)
        return 1

    # ---- device-timed arm ---------------------------------------------------
    # The clock sampler runs from the warm-up on (nvidia-smi needs a moment to start) and is stopped right
    # after the timed loop, so its samples are taken under this load.
    sampler = ClockSampler(local_rank, period_ms=50).start() if rank == 0 else None
    for i in range(max(3, args.warmup)):
        step(i)
    fence()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per_shape = {m: 0.0 for m in MS}
    start.record()
    for i in range(args.steps):
        step(i)
    end.record()
    fence()
    total_ms = start.elapsed_time(end)
    clocks = sampler.stop() if sampler is not None else None

    # per-shape breakdown (separate pass, informational)
    for m in MS:
        w = weights[0]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        fence()
        ev[0].record()
        for i in range(args.steps):
            a, w = a_dev[m][i % ROTATE], weights[i % ROTATE]
            if args.impl == "ours":
                if world > 1:
                    ops[m](a, w)
                else:
                    gemm(a, w, out=outs[m])
            else:
                torch.matmul(a, w.t(), out=outs[m])
                if world > 1:
                    dist.all_reduce(outs[m])
        ev[1].record()
        fence()
        per_shape[m] = ev[0].elapsed_time(ev[1]) / args.steps * 1e3

    # ---- end-to-end arm: inputs from pinned host memory, one result row back per shape ----------------------
    stage = {m: torch.empty(m, k_local, dtype=dtype, device=dev) for m in MS}
    back = {m: torch.empty(N_DIM, dtype=dtype).pin_memory() for m in MS}

    def e2e_step(i: int):
        for m in MS:
            stage[m].copy_(a_host[m], non_blocking=True)
        step(i, stage)
        for m in MS:
            back[m].copy_(outs[m][0], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    fence()
    t0 = time.perf_counter()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for i in range(args.steps):
        e2e_step(i)
    e2.record()
    fence()
    e2e_ms = max(s2.elapsed_time(e2), 0.0)
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3

    def rank_max(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    total_ms = rank_max(total_ms)
    e2e_ms = rank_max(max(e2e_ms, e2e_wall_ms))
    per_shape = {m: rank_max(v) for m, v in per_shape.items()}
    status_ok = True
    if comm is not None:
        comm.check_status()

    if rank == 0:
        ms_per_step = total_ms / args.steps
        flops = sum(2.0 * m * N_DIM * K_DIM for m in MS)
        line = {
            "metric": "gemm_allreduce_overlap_latency_us",
            "value": round(ms_per_step * 1e3, 2),
            "unit": "us per step (M=512,2048,8192 back to back)",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(3, args.warmup),
            "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": False,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "fp16",
            "data": "synthetic (A ~ N(0,1), B ~ N(0,1/K), seeded per rank; random-init weights)",
            "impl": args.impl,
            "config": {"model": "row-parallel TP linear GEMM->AllReduce", "M": list(MS), "N": N_DIM, "K": K_DIM,
                       "global_batch": sum(MS), "seq_len": 1, "parallelism": f"tp{world}",
                       "l2": f"{ROTATE} operand sets rotated between steps; per-step working set exceeds the 126 MB L2",
                       "strategy": {str(m): (ops[m].strategy if m in ops else "gemm") for m in MS},
                       "comm_ctas": {str(m): (ops[m].comm_ctas if m in ops and ops[m].strategy == "fused" else 0) for m in MS}},
            "per_shape_us": {str(m): round(v, 2) for m, v in per_shape.items()},
            "tflops_aggregate": round(flops / (ms_per_step * 1e-3) / 1e12, 1),
            "clocks": clocks,
            "e2e": {"value": round(e2e_ms / args.steps * 1e3, 2), "unit": "us per step",
                    "h2d_bytes_per_step": sum(m * k_local * 2 for m in MS),
                    "d2h_bytes_per_step": len(MS) * N_DIM * 2},
            "gpu_launches": launches_per_step * args.steps if args.impl == "ours" else 0,
            "status_ok": status_ok,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        if comm is not None:
            comm.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
