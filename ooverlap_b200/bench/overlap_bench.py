"""GEMM + collective overlap benchmark: fused kernels of this library against cuBLAS + NCCL.

Launch with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m ooverlap_b200.bench.overlap_bench --ops gemm_ar,gemm_rs_norm,ag_gemm --out overlap.jsonl

Ops and shapes (tp = number of ranks):

* ``gemm_ar``       fp16 ``A[M, 8192/tp] @ B[8192, 8192/tp]^T`` summed over ranks, M in {512, 2048, 8192}
* ``gemm_rs_norm``  bf16 M = 4096 tokens, hidden 8192, K = 28672/tp, + residual + RMSNorm (eps 1e-6) on the rank's rows
* ``ag_gemm``       bf16 all-gather of A[4096/tp, 8192] then ``@ B[28672/tp, 8192]^T``
* ``gemm_a2a``      baseline only (cuBLAS GEMM + NCCL all-to-all of row blocks), as in the reference; not in the default list

For each it times (CUDA-graph replay, CUDA events, max over ranks): the fused kernel over a few
communication-CTA budgets and with/without NVLS, this library's unfused GEMM + collective, and
torch.matmul (cuBLAS) + NCCL (+ a PyTorch RMSNorm for the tail).  Every line carries the roofline: the slower
of FLOPs at the measured GEMM peak and bytes over NVLink at the measured link bandwidth.

Capability parity: test/test.py:509-1043 (perf_overlap / baselines / speed-up summary) and
tool/evaluate_sm90.py of the reference.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import Communicator
from ..ops import AllGatherGemm, GemmAllReduce, GemmReduceScatterNorm, gemm, rmsnorm_reference

GEMM_PEAK_TFLOPS = 1629.9   # measured cuBLAS bf16 burst on this machine class
LINK_GBS = 770.0            # measured peer copy, per direction per GPU
PER_GRAPH = 5
TOL = 1e-2                  # the reference's tolerance for 16-bit results (include/ooverlap/testing/test_utils.cuh:87-110)


def timed(fn, iters, warmup) -> dict:
    """Microseconds per call (max over ranks): ``us`` = median of three runs, plus p50 / p90 / p99 over the replays."""
    from ..utils.timing import graph_timed
    t = graph_timed(fn, iters, warmup, per_graph=PER_GRAPH, min_ms=30.0)
    return {"us": round(t["us"], 1), "p50": round(t["p50"], 1), "p90": round(t["p90"], 1), "p99": round(t["p99"], 1)}


def check(name: str, got: torch.Tensor, want: torch.Tensor, tol: float = TOL) -> float:
    """Max abs error of a result against its fp32 reference; raises when any rank is outside the tolerance."""
    err = (got.float() - want).abs().max().item()
    ok = err <= tol * max(1.0, want.abs().max().item())
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if not flag.item():
        raise RuntimeError(f"{name}: result check failed on some rank (this rank: max abs err {err:.4g})")
    return err


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--ops", default="gemm_ar,gemm_rs_norm,ag_gemm")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--comm-ctas", default="8,20,32")
    p.add_argument("--nvls", default="auto", help="auto | on | off | both")
    p.add_argument("--join", default="on", help="on | off | both: GEMM CTAs join the reduction when out of tiles")
    p.add_argument("--ms", default="512,2048,8192")
    p.add_argument("--out", default="")
    p.add_argument("--extra", default="", help="comma list of additional arms: chunked (GemmAllReduce strategy 'chunked')")
    p.add_argument("--kernels", default="pair", help="comma list of fused kernels to time: pair (two-SM, CTA pairs), one_sm")
    p.add_argument("--no-baselines", action="store_true", help="skip the cuBLAS + NCCL arms")
    args = p.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(list(range(world)), rank, heap_bytes=3 << 30)
    ctas = [int(c) for c in args.comm_ctas.split(",")]
    nvls_opts = {"auto": [None], "on": [True], "off": [False], "pull": [2], "both": [True, False], "all": [2, True, False]}[args.nvls]
    join_opts = {"on": [True], "off": [False], "both": [True, False]}[args.join]
    kernels = [k for k in args.kernels.split(",") if k]
    lines = []
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)

    def emit(rec):
        lines.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    def roofline_us(flops_per_rank, link_bytes):
        return max(flops_per_rank / (GEMM_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e6

    if "gemm_ar" in args.ops:
        N = K = 8192
        k_local = K // world
        dt = torch.float16
        for M in [int(m) for m in args.ms.split(",")]:
            a = torch.randn(M, k_local, device="cuda", generator=gen).to(dt)
            b = (torch.randn(N, k_local, device="cuda", generator=gen) / K ** 0.5).to(dt)
            msg = M * N * 2
            roof = roofline_us(2.0 * M * N * k_local, 2.0 * (world - 1) / world * msg)
            roof_nvls = roofline_us(2.0 * M * N * k_local, float(msg))
            base = dict(op="gemm_ar", M=M, N=N, K=K, tp=world, dtype="fp16", roofline_p2p_us=round(roof, 1),
                        roofline_nvls_us=round(roof_nvls, 1))
            out = torch.empty(M, N, dtype=dt, device="cuda")
            want = a.float() @ b.float().t()
            dist.all_reduce(want)

            def cublas_nccl():
                torch.matmul(a, b.t(), out=out)
                dist.all_reduce(out)
            if not args.no_baselines:
                emit({**base, "impl": "cublas+nccl", **timed(cublas_nccl, args.iters, args.warmup)})
                emit({**base, "impl": "cublas_gemm_only", **timed(lambda: torch.matmul(a, b.t(), out=out), args.iters, args.warmup)})
            sym = comm.empty((M, N), dt)

            def ours_unfused():
                gemm(a, b, out=sym, splits=1)
                comm.all_reduce(sym)
            ours_unfused()
            check(f"gemm_ar M={M} unfused", sym, want)
            emit({**base, "impl": "ours_unfused", **timed(ours_unfused, args.iters, args.warmup)})
            emit({**base, "impl": "ours_gemm_only", **timed(lambda: gemm(a, b, out=sym, splits=1), args.iters, args.warmup)})
            for kernel in kernels:
                for c in ctas:
                    for nv in nvls_opts:
                        for jn in (join_opts if kernel == "one_sm" else [True]):
                            if kernel == "pair" and nv == 2:
                                continue
                            op = GemmAllReduce(comm, M, N, dt, comm_ctas=c, use_nvls=nv, strategy="fused", kernel=kernel)
                            op.join = jn
                            err = check(f"gemm_ar M={M} {kernel} ctas={c} nvls={nv}", op(a, b), want)
                            t = timed(lambda: op(a, b), args.iters, args.warmup)
                            emit({**base, "impl": "ours_fused", "kernel": kernel, "comm_ctas": c, "nvls": nv, "join": jn, **t,
                                  "max_abs_err": round(err, 5),
                                  "roofline_frac": round((roof_nvls if comm.nvls and nv is not False and nv != 0 else roof) / t["us"], 3)})
                            op.release()
            op = GemmAllReduce(comm, M, N, dt)  # the library's own choice for this shape
            check(f"gemm_ar M={M} auto", op(a, b), want)
            emit({**base, "impl": "ours_auto", "strategy": op.strategy, **timed(lambda: op(a, b), args.iters, args.warmup)})
            op.release()
            if "chunked" in args.extra:
                # slab GEMMs on this stream, in-switch all-reduce of each finished slab on a side stream
                op = GemmAllReduce(comm, M, N, dt, strategy="chunked")
                if op.strategy == "chunked":
                    check(f"gemm_ar M={M} chunked", op(a, b), want)
                    t = timed(lambda: op(a, b), args.iters, args.warmup)
                    emit({**base, "impl": "ours_chunked", "chunks": op.chunks, **t, "roofline_frac": round(roof_nvls / t["us"], 3)})
                op.release()
            comm.free(comm.heap_offset(sym))
            del want
            torch.cuda.synchronize()
            comm.check_status()

    if "gemm_a2a" in args.ops and world > 1:
        # Baseline only, as in the reference (BaselineImpl::GemmAll2All, src/baseline_impl.cu:178-267): cuBLAS GEMM,
        # then every rank sends row block r of its output to rank r.  This library has no all-to-all of its own.
        N, K, dt = 8192, 8192, torch.float16
        for M in [int(m) for m in args.ms.split(",")]:
            if M % world:
                continue
            a = torch.randn(M, K, device="cuda", generator=gen).to(dt)
            b = (torch.randn(N, K, device="cuda", generator=gen) / K ** 0.5).to(dt)
            out = torch.empty(M, N, dtype=dt, device="cuda")
            recv = torch.empty_like(out)

            def cublas_a2a():
                torch.matmul(a, b.t(), out=out)
                dist.all_to_all_single(recv, out)
            emit(dict(op="gemm_a2a", M=M, N=N, K=K, tp=world, dtype="fp16", impl="cublas+nccl_all_to_all",
                      **timed(cublas_a2a, args.iters, args.warmup)))

    if "gemm_rs_norm" in args.ops and 4096 % (128 * world) == 0:
        M, H, K = 4096, 8192, 28672 // world
        dt = torch.bfloat16
        a = torch.randn(M, K, device="cuda", generator=gen).to(dt)
        b = (torch.randn(H, K, device="cuda", generator=gen) / 28672 ** 0.5).to(dt)
        rows = M // world
        res = torch.randn(rows, H, device="cuda", generator=gen).to(dt)
        w = (1 + 0.02 * torch.randn(H, device="cuda", generator=gen)).to(dt)
        roof = roofline_us(2.0 * M * H * K, (world - 1) / world * M * H * 2)
        base = dict(op="gemm_rs_norm", M=M, N=H, K=K * world, tp=world, dtype="bf16", roofline_us=round(roof, 1))
        full = torch.empty(M, H, dtype=dt, device="cuda")
        shard = torch.empty(rows, H, dtype=dt, device="cuda")

        def cublas_nccl_rs():
            torch.matmul(a, b.t(), out=full)
            dist.reduce_scatter_tensor(shard, full)
            return rmsnorm_reference(shard, w, 1e-6, res)
        if not args.no_baselines:
            emit({**base, "impl": "cublas+nccl_rs+torch_norm", **timed(cublas_nccl_rs, args.iters, args.warmup)})
            emit({**base, "impl": "cublas_gemm_only", **timed(lambda: torch.matmul(a, b.t(), out=full), args.iters, args.warmup)})
        # fp32 reference of this rank's rows: sum over ranks of the partial products, + residual, RMSNorm
        part = a[:, :].float() @ b.float().t()
        dist.all_reduce(part)
        srow = (part[rank * rows:(rank + 1) * rows] + res.float()).to(dt).float()
        del part
        want_y = srow * torch.rsqrt(srow.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
        for kernel in kernels:
            for c in ctas:
                for nv in nvls_opts:
                    if kernel == "pair" and nv == 2:
                        continue
                    op = GemmReduceScatterNorm(comm, M, H, dt, eps=1e-6, comm_ctas=c, use_nvls=nv, kernel=kernel)
                    y = torch.empty(rows, H, dtype=dt, device="cuda")
                    ro = torch.empty(rows, H, dtype=dt, device="cuda")
                    op(a, b, w, res, y=y, residual_out=ro)
                    err = check(f"gemm_rs_norm {kernel} ctas={c} nvls={nv}", y, want_y, tol=6e-2)
                    t = timed(lambda: op(a, b, w, res, y=y, residual_out=ro), args.iters, args.warmup)
                    emit({**base, "impl": "ours_fused", "kernel": kernel, "comm_ctas": c, "nvls": nv, **t,
                          "max_abs_err": round(err, 5), "roofline_frac": round(roof / t["us"], 3)})
                    op.release()
        torch.cuda.synchronize()
        comm.check_status()

    if "ag_gemm" in args.ops and 4096 % (128 * world) == 0 and world > 1:
        M, K, N = 4096, 8192, 28672 // world
        dt = torch.bfloat16
        rows = M // world
        a_shard = torch.randn(rows, K, device="cuda", generator=gen).to(dt)
        b = (torch.randn(N, K, device="cuda", generator=gen) / K ** 0.5).to(dt)
        roof = roofline_us(2.0 * M * N * K, (world - 1) / world * M * K * 2)
        base = dict(op="ag_gemm", M=M, N=N * world, K=K, tp=world, dtype="bf16", roofline_us=round(roof, 1))
        a_full = torch.empty(M, K, dtype=dt, device="cuda")
        out = torch.empty(M, N, dtype=dt, device="cuda")

        def nccl_ag_cublas():
            dist.all_gather_into_tensor(a_full, a_shard)
            torch.matmul(a_full, b.t(), out=out)
        nccl_ag_cublas()
        want_c = a_full.float() @ b.float().t()
        if not args.no_baselines:
            emit({**base, "impl": "nccl_ag+cublas", **timed(nccl_ag_cublas, args.iters, args.warmup)})
            emit({**base, "impl": "cublas_gemm_only", **timed(lambda: torch.matmul(a_full, b.t(), out=out), args.iters, args.warmup)})
        for kernel in kernels:
            for c in ctas:
                for nv in nvls_opts:
                    if kernel == "pair" and nv == 2:
                        continue
                    for sk in ([0, -1] if kernel == "pair" else [0]):
                        op = AllGatherGemm(comm, M, K, dt, comm_ctas=c, use_nvls=nv, kernel=kernel, stream_k=sk)
                        out.zero_()
                        op(a_shard, b, out=out)
                        err = check(f"ag_gemm {kernel} ctas={c} nvls={nv} stream_k={sk}", out, want_c)
                        t = timed(lambda: op(a_shard, b, out=out), args.iters, args.warmup)
                        emit({**base, "impl": "ours_fused", "kernel": kernel, "comm_ctas": c, "nvls": nv, "stream_k": sk, **t,
                              "max_abs_err": round(err, 5), "roofline_frac": round(roof / t["us"], 3)})
                        op.release()
        torch.cuda.synchronize()
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
