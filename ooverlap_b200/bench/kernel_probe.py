"""Runs one kernel of the library a few times on one GPU and prints its CUDA-event time.

Small enough to sit under a profiler::

    python -m ooverlap_b200.bench.kernel_probe --op gemm --m 8192 --n 8192 --k 8192 --iters 3
    python -m ooverlap_b200.bench.kernel_probe --op gemm_splitk --m 64 --n 8192 --k 8192
    python -m ooverlap_b200.bench.kernel_probe --op rmsnorm --m 16384 --n 8192
    python -m ooverlap_b200.bench.kernel_probe --op allreduce --world 8 --bytes 67108864     (emulated ranks)
    python -m ooverlap_b200.bench.kernel_probe --op gemm_ar --world 2 --m 2048 --n 2048 --k 1024  (emulated ranks)
    python -m ooverlap_b200.bench.kernel_probe --op attn_decode --m 64 --heads 8 --kv-heads 1 --ctx 1088
    python -m ooverlap_b200.bench.kernel_probe --specs '[{"op": "gemm", "m": 2048, "pair": 1}, {"op": "cublas", "m": 2048}]'

``--specs`` runs several probes in one process (each entry overrides the command-line values).

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


OPS = ["gemm", "gemm_splitk", "cublas", "rmsnorm", "allreduce", "reduce_scatter", "all_gather", "fused_norm_ar", "gemm_ar",
       "gemm_rs", "ag_gemm", "attn_decode", "sdpa_decode", "silu_mul", "rope"]


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--op", default="gemm", choices=OPS)
    p.add_argument("--m", type=int, default=8192)
    p.add_argument("--n", type=int, default=8192)
    p.add_argument("--k", type=int, default=8192)
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--world", type=int, default=8)
    p.add_argument("--bytes", type=int, default=64 << 20)
    p.add_argument("--splits", type=int, default=0)
    p.add_argument("--pair", type=int, default=0, help="plain GEMM: 1 = two-SM kernel, -1 = one-SM kernel, 0 = auto")
    p.add_argument("--stream-k", type=int, default=0, help="two-SM kernel: 1 = stream-K tail, -1 = whole tiles only, 0 = auto")
    p.add_argument("--kernel", default=None, choices=["pair", "one_sm"], help="fused ops: two-SM or one-SM kernel")
    p.add_argument("--algo", type=int, default=1, help="emulated collectives: algorithm number of the C API")
    p.add_argument("--ctas", type=int, default=0, help="emulated collectives: CTAs per rank (0 = 148 / world)")
    p.add_argument("--comm-ctas", type=int, default=4, help="fused ops: communication CTAs per rank")
    p.add_argument("--skinny", type=int, default=0, help="plain GEMM, M <= 128: 1 = weight-streaming kernel, -1 = never")
    p.add_argument("--splitk-reduce", type=int, default=0, help="split-K sum: 1 = second kernel, -1 = inside the GEMM kernel")
    p.add_argument("--gemv", type=int, default=0, help="plain GEMM, M <= 4: 1 = CUDA-core streaming kernel")
    p.add_argument("--heads", type=int, default=8)
    p.add_argument("--kv-heads", type=int, default=1)
    p.add_argument("--ctx", type=int, default=1088, help="attention: context length (keys attended)")
    p.add_argument("--no-flush", action="store_true")
    p.add_argument("--specs", default="", help="JSON list of probes; each entry overrides these options")
    args = p.parse_args()
    torch.cuda.set_device(0)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if not args.specs:
        print(json.dumps(probe(args, flush)))
        return 0
    for spec in json.loads(args.specs):
        one = argparse.Namespace(**vars(args))
        for k, v in spec.items():
            if not hasattr(one, k.replace("-", "_")):
                raise SystemExit(f"unknown probe option {k!r}")
            setattr(one, k.replace("-", "_"), v)
        if one.op not in OPS:
            raise SystemExit(f"unknown op {one.op!r}")
        print(json.dumps(probe(one, flush)), flush=True)
        torch.cuda.empty_cache()
    return 0


def probe(args, flush) -> dict:
    from .. import EmulatedGroup, _lib
    from ..ops import GemmAllReduce, attn_decode, gemm, rmsnorm, rope_kv_write, rope_tables, silu_mul
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    tf_peak, bw_peak, src = peaks()
    rec = {"op": args.op, "dtype": args.dtype, "peaks": src}
    if args.op in ("gemm", "gemm_splitk", "cublas"):
        a = torch.randn(args.m, args.k, device="cuda").to(dt)
        b = (torch.randn(args.n, args.k, device="cuda") / args.k ** 0.5).to(dt)
        out = torch.empty(args.m, args.n, device="cuda", dtype=dt)
        if args.op == "cublas":
            fn = lambda: torch.matmul(a, b.t(), out=out)  # noqa: E731
        else:
            splits = args.splits if args.op == "gemm_splitk" else 1
            rec["pair"], rec["skinny"], rec["splitk_reduce"], rec["gemv"] = args.pair, args.skinny, args.splitk_reduce, args.gemv
            rec["stream_k"] = args.stream_k
            fn = lambda: gemm(a, b, out=out, splits=splits, pair=args.pair, skinny=args.skinny,  # noqa: E731
                              splitk_reduce=args.splitk_reduce, gemv=args.gemv, stream_k=args.stream_k)
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
    elif args.op in ("attn_decode", "sdpa_decode"):
        # args.m sequences, one new token each, against `ctx` cached keys per sequence.
        B, H, KV, L = args.m, args.heads, args.kv_heads, args.ctx
        max_len = (L + 127) // 128 * 128
        q = torch.randn(B, H, 128, device="cuda").to(dt)
        kc = torch.randn(B, KV, max_len, 128, device="cuda").to(dt)
        vc = torch.randn(B, KV, max_len, 128, device="cuda").to(dt)
        pos = torch.full((1,), L - 1, dtype=torch.long, device="cuda")
        if args.op == "attn_decode":
            out = torch.empty(B, H * 128, device="cuda", dtype=dt)
            fn = lambda: attn_decode(q, kc, vc, pos, out=out, splits=args.splits)  # noqa: E731
        else:
            mask = torch.full((1, 1, 1, max_len), float("-inf"), device="cuda", dtype=dt)
            mask[..., :L] = 0
            fn = lambda: torch.nn.functional.scaled_dot_product_attention(  # noqa: E731
                q.view(B, H, 1, 128), kc, vc, attn_mask=mask, enable_gqa=True)
        ms = timed(fn, args.iters, args.warmup, flush)
        gbs = 2.0 * B * KV * L * 128 * 2 / (ms * 1e-3) / 1e9
        rec.update(B=B, heads=H, kv_heads=KV, ctx=L, us=round(ms * 1e3, 2), kv_gbs=round(gbs, 1),
                   frac_of_peak_hbm=round(gbs / bw_peak, 3))
    elif args.op == "silu_mul":
        gu = torch.randn(args.m, 2 * args.n, device="cuda").to(dt)
        out = torch.empty(args.m, args.n, device="cuda", dtype=dt)
        ms = timed(lambda: silu_mul(gu, out), args.iters, args.warmup, flush)
        gbs = 3.0 * args.m * args.n * 2 / (ms * 1e-3) / 1e9
        rec.update(rows=args.m, F=args.n, us=round(ms * 1e3, 2), gbs=round(gbs, 1), frac_of_peak_hbm=round(gbs / bw_peak, 3))
    elif args.op == "rope":
        B, H, KV = args.m, args.heads, args.kv_heads
        qkv = torch.randn(B, (H + 2 * KV) * 128, device="cuda").to(dt)
        kc = torch.zeros(B, KV, 256, 128, device="cuda", dtype=dt)
        vc = torch.zeros_like(kc)
        cos, sin = rope_tables(256, 128, 500000.0, qkv.device)
        pos = torch.full((1,), 100, dtype=torch.long, device="cuda")
        qo = torch.empty(B, H * 128, device="cuda", dtype=dt)
        ms = timed(lambda: rope_kv_write(qkv, B, 1, H, KV, kc, vc, cos, sin, pos, q_out=qo), args.iters, args.warmup, flush)
        rec.update(B=B, heads=H, kv_heads=KV, us=round(ms * 1e3, 2))
    elif args.op == "allreduce":
        g = EmulatedGroup(args.world, heap_bytes=args.bytes + (32 << 20))
        n = args.bytes // 2
        off = g.alloc(args.bytes)
        for r in range(args.world):
            g.view(off, (n,), dt, r).fill_(0.001 * (r + 1))
        ctas = args.ctas or 148 // args.world
        if args.algo in (_lib.AR_ONESHOT_P2P,):
            out_local = torch.empty(args.world, n, device="cuda", dtype=dt)
            fn = lambda: g.all_reduce(off, n, dt, algo=args.algo, out_local=out_local, max_ctas=ctas)  # noqa: E731
        else:
            fn = lambda: g.all_reduce(off, n, dt, algo=_lib.AR_TWOSHOT_P2P, out_off=off, max_ctas=ctas)  # noqa: E731
        rec["algo"], rec["ctas"] = args.algo, ctas
        ms = timed(fn, args.iters, args.warmup, flush)
        g.check_status()
        # every emulated rank reads all ranks' shards and writes them back to all ranks (all on this GPU)
        gbs = 2.0 * args.world * args.bytes / (ms * 1e-3) / 1e9
        rec.update(world=args.world, bytes=args.bytes, us=round(ms * 1e3, 2), local_traffic_gbs=round(gbs, 1),
                   frac_of_peak_hbm=round(gbs / bw_peak, 3))
        g.close()
    elif args.op in ("reduce_scatter", "all_gather"):
        g = EmulatedGroup(args.world, heap_bytes=args.bytes + (32 << 20))
        n = args.bytes // 2
        shard = (n + args.world - 1) // args.world
        off = g.alloc(args.bytes)
        for r in range(args.world):
            g.view(off, (n,), dt, r).fill_(0.001 * (r + 1))
        local = torch.full((args.world, shard), 0.5, device="cuda", dtype=dt)
        ctas = args.ctas or 148 // args.world
        if args.op == "reduce_scatter":
            fn = lambda: g.reduce_scatter(off, n, dt, local, algo=_lib.RS_P2P, max_ctas=ctas)  # noqa: E731
            traffic = args.world * args.bytes + args.bytes  # every rank reads its shard of all ranks, writes its shard
        else:
            fn = lambda: g.all_gather(off, n, dt, src_local=local, algo=_lib.AG_PUSH_P2P, max_ctas=ctas)  # noqa: E731
            traffic = args.bytes + args.world * args.bytes  # every rank reads its shard, writes it to all ranks
        ms = timed(fn, args.iters, args.warmup, flush)
        g.check_status()
        gbs = traffic / (ms * 1e-3) / 1e9
        rec.update(world=args.world, bytes=args.bytes, ctas=ctas, us=round(ms * 1e3, 2), local_traffic_gbs=round(gbs, 1),
                   frac_of_peak_hbm=round(gbs / bw_peak, 3))
        g.close()
    elif args.op == "fused_norm_ar":
        # all-reduce (two-shot, peer loads) + residual + RMSNorm of [m, n] per rank, emulated ranks
        rows, hidden = args.m, args.n
        nbytes = rows * hidden * 2
        g = EmulatedGroup(args.world, heap_bytes=3 * nbytes + (32 << 20))
        x_off, y_off, ro_off = g.alloc(nbytes), g.alloc(nbytes), g.alloc(nbytes)
        for r in range(args.world):
            g.view(x_off, (rows, hidden), dt, r).normal_()
        res = torch.randn(args.world, rows, hidden, device="cuda").to(dt)
        w = torch.ones(hidden, device="cuda", dtype=dt)
        ctas = args.ctas or 148 // args.world
        fn = lambda: g.fused_norm(_lib.NORM_AR_TWOSHOT, x_off=x_off, rows=rows, hidden=hidden, dtype=dt, weight=w,  # noqa: E731
                                  eps=1e-6, residual=res, y_off=y_off, res_out_off=ro_off,
                                  local_stride_bytes=nbytes, max_ctas=ctas)
        ms = timed(fn, args.iters, args.warmup, flush)
        g.check_status()
        gbs = (args.world * nbytes + nbytes + 2 * args.world * nbytes) / (ms * 1e-3) / 1e9
        rec.update(world=args.world, rows=rows, hidden=hidden, ctas=ctas, us=round(ms * 1e3, 2),
                   local_traffic_gbs=round(gbs, 1), frac_of_peak_hbm=round(gbs / bw_peak, 3))
        g.close()
    elif args.op in ("gemm_rs", "ag_gemm"):
        from ..ops import AllGatherGemm, GemmReduceScatterNorm
        g = EmulatedGroup(args.world, heap_bytes=(args.m * max(args.n, args.k) * 2) * 3 + (64 << 20))
        rows = args.m // args.world
        if args.op == "gemm_rs":
            op = GemmReduceScatterNorm(g, args.m, args.n, dt, comm_ctas=args.comm_ctas, kernel=args.kernel)
            a = torch.randn(args.world, args.m, args.k, device="cuda").to(dt)
            b = (torch.randn(args.world, args.n, args.k, device="cuda") / args.k ** 0.5).to(dt)
            res = torch.randn(args.world, rows, args.n, device="cuda").to(dt)
            w = torch.ones(args.n, device="cuda", dtype=dt)
            fn = lambda: op(a, b, w, res)  # noqa: E731
        else:
            op = AllGatherGemm(g, args.m, args.k, dt, comm_ctas=args.comm_ctas, kernel=args.kernel)
            a = torch.randn(args.world, rows, args.k, device="cuda").to(dt)
            b = (torch.randn(args.world, args.n, args.k, device="cuda") / args.k ** 0.5).to(dt)
            out = torch.empty(args.world, args.m, args.n, device="cuda", dtype=dt)
            fn = lambda: op(a, b, out=out)  # noqa: E731
        ms = timed(fn, args.iters, args.warmup, flush)
        g.check_status()
        tflops = 2.0 * args.world * args.m * args.n * args.k / (ms * 1e-3) / 1e12
        rec.update(world=args.world, M=args.m, N=args.n, K=args.k, kernel=args.kernel or "auto", comm_ctas=args.comm_ctas,
                   us=round(ms * 1e3, 2), tflops_all_ranks=round(tflops, 1))
        g.close()
    else:
        g = EmulatedGroup(args.world, heap_bytes=(args.m * args.n * 2) * 3 + (64 << 20))
        op = GemmAllReduce(g, args.m, args.n, dt, comm_ctas=args.comm_ctas, kernel=args.kernel)
        rec["kernel"], rec["comm_ctas"] = args.kernel or "auto", args.comm_ctas
        a = torch.randn(args.world, args.m, args.k, device="cuda").to(dt)
        b = (torch.randn(args.world, args.n, args.k, device="cuda") / args.k ** 0.5).to(dt)
        ms = timed(lambda: op(a, b), args.iters, args.warmup, flush)
        g.check_status()
        tflops = 2.0 * args.world * args.m * args.n * args.k / (ms * 1e-3) / 1e12
        rec.update(world=args.world, M=args.m, N=args.n, K=args.k, us=round(ms * 1e3, 2), tflops_all_ranks=round(tflops, 1))
        g.close()
    return rec


if __name__ == "__main__":
    sys.exit(main())
