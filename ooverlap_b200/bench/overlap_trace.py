"""Phase timeline of one fused GEMM->AllReduce (or GEMM->RS+norm) launch from the kernel's device-side trace.

Launch with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m ooverlap_b200.bench.overlap_trace --op gemm_ar --M 8192 --comm-ctas 16

Every CTA of the launch records ``globaltimer`` stamps (kernel entry, GEMM tiles done, first reduction item ready,
last reduction item finished, after the final rank barrier) plus how many reduction items it processed and how long
it waited for arrival counters.  Rank 0 prints, relative to the earliest CTA start, the min / median / max of each
stamp for GEMM CTAs and for dedicated communication CTAs: enough to see whether the reduction really runs under
the GEMM or only after it.

Capability parity: the reference's GEMM "monitor" mode records the completion order of tiles
(src/epilogue/reorder_epilogue.h:549-588) and its tuner consumes it (tool/search.py:564-636).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

from .. import Communicator
from ..ops.gemm import order_buffer, tile_order
from ..ops import GemmAllReduce, GemmReduceScatterNorm


def summarize(name, vals):
    vals = [v for v in vals if v is not None]
    if not vals:
        return {name: None}
    return {name: {"min": round(min(vals), 1), "med": round(statistics.median(vals), 1), "max": round(max(vals), 1)}}


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--op", default="gemm_ar", choices=["gemm_ar", "gemm_rs_norm"])
    p.add_argument("--M", dest="m", type=int, default=8192)
    p.add_argument("--N", dest="n", type=int, default=8192)
    p.add_argument("--K", dest="k", type=int, default=8192, help="global K (split over ranks)")
    p.add_argument("--comm-ctas", type=int, default=16)
    p.add_argument("--nvls", default="auto", choices=["auto", "on", "off", "pull"])
    p.add_argument("--no-join", action="store_true")
    p.add_argument("--kernel", default=None, choices=["pair", "one_sm"], help="fused kernel (default: the library's choice)")
    args = p.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(list(range(world)), rank, heap_bytes=1 << 30)
    nv = {"auto": None, "on": True, "off": False, "pull": 2}[args.nvls]
    dt = torch.float16 if args.op == "gemm_ar" else torch.bfloat16
    kl = args.k // world
    a = torch.randn(args.m, kl, device="cuda").to(dt)
    b = (torch.randn(args.n, kl, device="cuda") / args.k ** 0.5).to(dt)
    if args.op == "gemm_ar":
        op = GemmAllReduce(comm, args.m, args.n, dt, comm_ctas=args.comm_ctas, use_nvls=nv, strategy="fused", kernel=args.kernel)
        run = lambda: op(a, b)  # noqa: E731
    else:
        op = GemmReduceScatterNorm(comm, args.m, args.n, dt, comm_ctas=args.comm_ctas, use_nvls=nv, kernel=args.kernel)
        w = torch.ones(args.n, device="cuda", dtype=dt)
        res = torch.zeros(args.m // world, args.n, device="cuda", dtype=dt)
        run = lambda: op(a, b, w, res)  # noqa: E731
    op.join = not args.no_join
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    trace = torch.zeros(160, 8, dtype=torch.int64, device="cuda")
    op.trace_buffer = trace
    if (args.kernel or "pair") == "pair":
        op.order_buffer = order_buffer(args.m, args.n)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run()
    e1.record()
    torch.cuda.synchronize()
    comm.check_status()
    t = trace.cpu()
    used = t[t[:, 0] > 0]
    t0 = int(used[:, 0].min())
    rel = lambda col, rows: [(int(v) - t0) / 1e3 if int(v) > 0 else None for v in rows[:, col]]  # noqa: E731
    gemm_rows, comm_rows = used[used[:, 7] == 0], used[used[:, 7] == 1]
    out = {"rank": rank, "op": args.op, "M": args.m, "N": args.n, "K": args.k, "tp": world, "comm_ctas": args.comm_ctas,
           "nvls": args.nvls, "join": not args.no_join, "kernel": args.kernel or "auto", "kernel_us": round(e0.elapsed_time(e1) * 1e3, 1),
           "ctas": int(used.shape[0]), "gemm_ctas": int(gemm_rows.shape[0])}
    out.update(summarize("gemm_done_us", rel(1, gemm_rows)))
    out.update(summarize("gemm_cta_first_reduce_ready_us", rel(2, gemm_rows)))
    out.update(summarize("gemm_cta_reduce_done_us", rel(3, gemm_rows)))
    out.update(summarize("gemm_cta_end_us", rel(4, gemm_rows)))
    out.update(summarize("comm_cta_first_ready_us", rel(2, comm_rows)))
    out.update(summarize("comm_cta_done_us", rel(3, comm_rows)))
    out.update(summarize("comm_cta_end_us", rel(4, comm_rows)))
    out["items_by_comm_ctas"] = int(comm_rows[:, 5].sum())
    out["items_by_gemm_ctas"] = int(gemm_rows[:, 5].sum())
    out["comm_cta_wait_us_med"] = round(statistics.median([int(v) / 1e3 for v in comm_rows[:, 6]]), 1) if len(comm_rows) else None
    if getattr(op, "order_buffer", None) is not None:
        rec = tile_order(op.order_buffer)
        if rec:
            # Tile-order record of the two-SM kernel: when each 128-row half-tile was published to its reducer.
            out["half_tiles_published"] = len(rec)
            out["publish_order_first_units"] = [r["unit"] for r in rec[:16]]
            out["publish_span_us"] = round(rec[-1]["t_us"], 1)
            out["publish_us_quartiles"] = [round(rec[len(rec) * q // 4 - (1 if q == 4 else 0)]["t_us"], 1) for q in (1, 2, 3, 4)]
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        for g in gathered[:2] + gathered[-1:]:
            print(json.dumps(g), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
