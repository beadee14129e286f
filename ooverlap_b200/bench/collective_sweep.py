"""Collective latency / bus-bandwidth sweep: this library's kernels against NCCL.

Launch with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m ooverlap_b200.bench.collective_sweep --min-bytes 1024 --max-bytes 1073741824 --out sweep.jsonl

For every power-of-two message size and each of all-reduce / reduce-scatter /
all-gather on bf16 buffers (values ~U(-1,1), seed = rank) it times every
applicable algorithm of this library over a few CTA budgets, and NCCL through
``torch.distributed`` on the same buffers, with CUDA events per rank and the
maximum over ranks.  Rank 0 writes one JSON line per measurement and, with
``--policy``, the best (algorithm, CTAs) per size as a tuning-policy file.

Capability parity: test/sweep_tma_collectives.py:29-109,357-746 (CTA-policy
sweep -> policy JSON), tool/bandwidth.py:107-275 (latency / bus-bandwidth
curves) and test/test_external_p2p_collective_sweep.py of the reference.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import Communicator, _lib
from ..utils.partition import bus_bandwidth_gbs, partition

AR_NAMES = {_lib.AR_ONESHOT_P2P: "oneshot_p2p", _lib.AR_TWOSHOT_P2P: "twoshot_p2p", _lib.AR_TWOSHOT_NVLS: "twoshot_nvls",
            _lib.AR_ONESHOT_NVLS: "oneshot_nvls"}
RS_NAMES = {_lib.RS_P2P: "p2p", _lib.RS_NVLS: "nvls"}
AG_NAMES = {_lib.AG_PUSH_P2P: "push_p2p", _lib.AG_PUSH_NVLS: "push_nvls"}


USE_GRAPH = True
PER_GRAPH = 10


def timed(fn, iters, warmup, world):
    """Seconds per call, device-timed, max over ranks.  Calls are replayed from a CUDA graph (ten per
    graph) so that small-message numbers measure the kernels, not the Python launch path."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = None
    if USE_GRAPH:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(PER_GRAPH):
                    fn()
            graph.replay()
        except Exception:  # capture refused: fall back to eager launches
            graph = None
            torch.cuda.synchronize()
    def once(reps):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            if graph is not None:
                graph.replay()
            else:
                for _ in range(PER_GRAPH):
                    fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / (reps * PER_GRAPH)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e-3  # seconds per call, max over ranks

    # The start skew between ranks is paid once per measurement: run long enough (>= ~5 ms) to amortise it.
    pilot = once(max(1, iters // PER_GRAPH))
    reps = max(1, int(min(200, max(iters // PER_GRAPH, 5e-3 / max(pilot * PER_GRAPH, 1e-7)))))
    return min(once(reps), once(reps))


def latency_stats(fn, iters, warmup) -> dict:
    """p50 / p90 / p99 of the per-replay latencies (microseconds per call, max over ranks), for the latency tables."""
    from ..utils.timing import graph_timed
    t = graph_timed(fn, iters, warmup, per_graph=PER_GRAPH, min_ms=5.0, max_reps=200)
    return {k: round(t[k], 2) for k in ("p50", "p90", "p99")}


def merge_policies(paths, out_path: str, comment: str = "") -> int:
    """Merges policy files (as written by ``--policy``) into one: points of the same (world, collective, nvls, bytes)
    are replaced by the later file's.  Returns the number of points."""
    merged = {}
    for path in paths:
        with open(path) as f:
            data = json.load(f)
        comment = comment or data.get("comment", "")
        for pt in data["points"]:
            merged[(pt["world"], pt["collective"], pt["nvls"], pt["bytes"])] = pt
    pts = [merged[k] for k in sorted(merged)]
    with open(out_path, "w") as f:
        json.dump({"comment": comment, "points": pts}, f, indent=1)
    return len(pts)


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--merge", nargs="+", default=None, metavar="POLICY.json",
                   help="no measurement: merge these policy files (later files win) into --policy and exit")
    p.add_argument("--min-bytes", type=int, default=1 << 10)
    p.add_argument("--max-bytes", type=int, default=1 << 30)
    p.add_argument("--iters", type=int, default=50)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--ctas", default="4,8,16,32,64")
    p.add_argument("--collectives", default="all_reduce,reduce_scatter,all_gather")
    p.add_argument("--out", default="")
    p.add_argument("--policy", default="")
    p.add_argument("--stats-max-bytes", type=int, default=0,
                   help="for messages up to this size also report p50 / p90 / p99 of the best configuration and of NCCL")
    args = p.parse_args()
    if args.merge:
        if not args.policy:
            raise SystemExit("--merge needs --policy OUT.json")
        print(f"{merge_policies(args.merge, args.policy)} points -> {args.policy}")
        return 0

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(list(range(world)), rank, heap_bytes=2 * args.max_bytes + (64 << 20))
    dtype = torch.bfloat16
    max_elems = args.max_bytes // 2
    gen = torch.Generator(device="cuda").manual_seed(rank)
    src = (torch.rand(max_elems, device="cuda", generator=gen) * 2 - 1).to(dtype)
    sym_in = comm.empty((max_elems,), dtype)
    sym_out = comm.empty((max_elems,), dtype)
    sym_in.copy_(src)
    nccl_buf = src.clone()
    nccl_out = torch.empty_like(src)
    cta_list = [int(c) for c in args.ctas.split(",")]
    lines, best = [], {}
    comm.init_round_robin_slots(dtype, 8 << 20, 8)  # the ring behind all_reduce_round_robin / the push kernel

    def record(coll, nbytes, impl, algo_name, algo, ctas, sec):
        rec = {"collective": coll, "world": world, "bytes": nbytes, "impl": impl, "algo": algo_name, "ctas": ctas,
               "us": round(sec * 1e6, 2), "bus_gbs": round(bus_bandwidth_gbs(coll, world, nbytes, sec), 1),
               "nvls": int(comm.nvls)}
        lines.append(rec)
        if impl == "ours":  # registered-buffer algorithms only: the ring arms are not policy candidates
            # Two policies: for communicators with an NVLS alias (any algorithm may win) and without one.
            for has_nvls in ((1, 0) if "nvls" not in algo_name else (1,)):
                if has_nvls and not comm.nvls:
                    continue
                key = (coll, nbytes, has_nvls)
                if key not in best or sec < best[key][0]:
                    best[key] = (sec, algo, ctas)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    size = args.min_bytes
    while size <= args.max_bytes:
        n = size // 2
        iters = args.iters if size <= (64 << 20) else max(5, args.iters // 5)
        if "all_reduce" in args.collectives:
            sec = timed(lambda: dist.all_reduce(nccl_buf[:n]), iters, args.warmup, world)
            record("all_reduce", size, "nccl", "nccl", -1, 0, sec)
            algos = [_lib.AR_TWOSHOT_P2P] + ([_lib.AR_TWOSHOT_NVLS] if comm.nvls else [])
            if size <= (8 << 20):
                algos += [_lib.AR_ONESHOT_P2P] + ([_lib.AR_ONESHOT_NVLS] if comm.nvls else [])
            for algo in algos:
                for ctas in cta_list:
                    if ctas != cta_list[0] and ctas * 512 * 16 > max(size, 8192) * 4:
                        continue  # more CTAs than work
                    if algo in (_lib.AR_ONESHOT_P2P, _lib.AR_ONESHOT_NVLS):
                        fn = lambda: comm.all_reduce_out(sym_in[:n], sym_out[:n], algo=algo, max_ctas=ctas)  # noqa: E731
                    else:
                        fn = lambda: comm.all_reduce(sym_in[:n], algo=algo, max_ctas=ctas)  # noqa: E731
                    record("all_reduce", size, "ours", AR_NAMES[algo], algo, ctas, timed(fn, iters, args.warmup, world))
            sym_in.copy_(src)  # in-place sums grow; refresh
            # The ring path an application (the vLLM hook) takes for an ordinary tensor: the one-barrier push kernel
            # for small messages, else copy into the slot + in-place all-reduce.
            if size <= (8 << 20) // (world + 1):
                x = src[:n]
                if comm.all_reduce_push(x) is not None:
                    record("all_reduce", size, "ours_ring", "push", -2, 0,
                           timed(lambda: comm.all_reduce_push(x), iters, args.warmup, world))
                saved = comm.config.push_max_bytes
                comm.config.push_max_bytes = 0
                record("all_reduce", size, "ours_ring", "copy+inplace", -3, 0,
                       timed(lambda: comm.all_reduce_round_robin(x), iters, args.warmup, world))
                comm.config.push_max_bytes = saved
            if size <= args.stats_max_bytes:
                x = src[:n]
                arms = {"nccl": lambda: dist.all_reduce(nccl_buf[:n]), "ours_ring": lambda: comm.all_reduce_round_robin(x)}
                key = ("all_reduce", size, 1 if comm.nvls else 0)
                if key in best:
                    _, b_algo, b_ctas = best[key]
                    if b_algo in (_lib.AR_ONESHOT_P2P, _lib.AR_ONESHOT_NVLS):
                        arms["ours_best"] = lambda: comm.all_reduce_out(sym_in[:n], sym_out[:n], algo=b_algo, max_ctas=b_ctas)
                    else:
                        arms["ours_best"] = lambda: comm.all_reduce(sym_in[:n], algo=b_algo, max_ctas=b_ctas)
                for name, fn in arms.items():
                    rec = {"collective": "all_reduce", "world": world, "bytes": size, "impl": name, "stat": "latency_us",
                           **latency_stats(fn, iters, args.warmup)}
                    lines.append(rec)
                    if rank == 0:
                        print(json.dumps(rec), flush=True)
                sym_in.copy_(src)
        if "reduce_scatter" in args.collectives and n >= world:
            b, e = partition(n, world, rank)
            sec = timed(lambda: dist.reduce_scatter_tensor(nccl_out[: n // world], nccl_buf[: n // world * world]), iters,
                        args.warmup, world)
            record("reduce_scatter", size, "nccl", "nccl", -1, 0, sec)
            out = nccl_out[: e - b]
            for algo in [_lib.RS_P2P] + ([_lib.RS_NVLS] if comm.nvls else []):
                for ctas in cta_list:
                    if ctas != cta_list[0] and ctas * 512 * 16 > max(size, 8192) * 4:
                        continue
                    fn = lambda: comm.reduce_scatter(sym_in[:n], out=out, algo=algo, max_ctas=ctas)  # noqa: E731
                    record("reduce_scatter", size, "ours", RS_NAMES[algo], algo, ctas, timed(fn, iters, args.warmup, world))
        if "all_gather" in args.collectives and n >= world:
            shard = n // world
            sec = timed(lambda: dist.all_gather_into_tensor(nccl_out[: shard * world], nccl_buf[:shard]), iters,
                        args.warmup, world)
            record("all_gather", size, "nccl", "nccl", -1, 0, sec)
            for algo in [_lib.AG_PUSH_P2P] + ([_lib.AG_PUSH_NVLS] if comm.nvls else []):
                for ctas in cta_list:
                    if ctas != cta_list[0] and ctas * 512 * 16 > max(size, 8192) * 4:
                        continue
                    fn = lambda: comm.all_gather(src[:shard], out=sym_out[: shard * world], algo=algo, max_ctas=ctas)  # noqa: E731
                    record("all_gather", size, "ours", AG_NAMES[algo], algo, ctas, timed(fn, iters, args.warmup, world))
        torch.cuda.synchronize()
        comm.check_status()
        size *= 2

    if rank == 0:
        if args.out:
            with open(args.out, "w") as f:
                for rec in lines:
                    f.write(json.dumps(rec) + "\n")
        if args.policy:
            pts = [{"world": world, "collective": coll, "nvls": nv, "bytes": nbytes, "algo": algo, "ctas": ctas}
                   for (coll, nbytes, nv), (_, algo, ctas) in sorted(best.items())]
            with open(args.policy, "w") as f:
                json.dump({"points": pts}, f, indent=1)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
