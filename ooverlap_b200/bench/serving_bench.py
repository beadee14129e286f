"""Tensor-parallel serving benchmark: output tokens per second of a Llama-architecture model.

Launch with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        -m ooverlap_b200.bench.serving_bench --model llama3-70b --batches 1,16,64,256 --in-len 1024 --out-len 128

Random-init bf16 weights of the named architecture, uniform-random token-id prompts, greedy decoding.  For every
batch size it runs the ``ours`` backend (tcgen05 GEMMs, fused all-reduce + residual + RMSNorm over NVLink) and the
``nccl`` backend (cuBLAS + NCCL all-reduce + PyTorch RMSNorm), BOTH with the decode step replayed from a CUDA graph
(``--no-graph`` runs both eagerly; a backend whose capture fails is re-run eagerly and its line says so), and
prints one JSON line per (backend, batch) with the
wall time of prefill + decode, the decode-only time, and output tokens per second (batch * out_len / total).

Capability parity: test/benchmark_vllm_paperlike.py:1-140 and evalution/run_vllm_paperlike.sh:7-120 of the
reference (fresh runs per backend x batch x workload, output tok/s).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

from .. import Communicator
from ..models.llama import LLAMA3_8B, LLAMA3_70B, TINY, LlamaConfig, LlamaTP

MODELS = {"llama3-70b": LLAMA3_70B, "llama3-8b": LLAMA3_8B, "tiny": TINY}


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="llama3-70b", choices=sorted(MODELS))
    p.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the model's own)")
    p.add_argument("--batches", default="1,16,64,256")
    p.add_argument("--in-len", type=int, default=1024)
    p.add_argument("--out-len", type=int, default=128)
    p.add_argument("--backends", default="nccl,ours")
    p.add_argument("--no-graph", action="store_true")
    p.add_argument("--out", default="")
    args = p.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = MODELS[args.model]
    if args.layers:
        cfg = LlamaConfig(**{**cfg.__dict__, "layers": args.layers})
    batches = [int(b) for b in args.batches.split(",")]
    max_b = max(batches)
    comm = None
    if world > 1 and "ours" in args.backends:
        comm = Communicator(list(range(world)), rank, heap_bytes=3 << 30)
        comm.init_round_robin_slots(torch.bfloat16, 8 << 20, 8)
    lines = []
    for backend in args.backends.split(","):
        torch.cuda.empty_cache()
        model = LlamaTP(cfg, comm if backend == "ours" else None, rank=rank, world=world, backend=backend,
                        max_batch=max_b, max_len=args.in_len + args.out_len, device=dev)
        for b in batches:
            prompts = torch.randint(0, cfg.vocab, (b, args.in_len), device=dev,
                                    generator=torch.Generator(device=dev).manual_seed(b))
            # warm-up run of the same shape (loads kernels, sizes scratch buffers)
            model.generate(prompts, min(4, args.out_len), use_graph=False)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            first = model.generate(prompts, 1)
            torch.cuda.synchronize()
            t_prefill = time.perf_counter() - t0
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            graphed = not args.no_graph
            try:
                toks = model.generate(prompts, args.out_len, use_graph=graphed)
            except Exception as e:  # capture refused (e.g. a collective that cannot be captured): measure eagerly
                if not graphed:
                    raise
                if rank == 0:
                    print(f"{backend}: CUDA-graph capture failed ({type(e).__name__}: {e}); eager run", file=sys.stderr)
                graphed = False
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                t0 = time.perf_counter()
                toks = model.generate(prompts, args.out_len, use_graph=False)
            torch.cuda.synchronize()
            total = time.perf_counter() - t0
            t = torch.tensor([total, t_prefill], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total, t_prefill = float(t[0]), float(t[1])
            rec = {"bench": "serving", "model": args.model, "layers": cfg.layers, "tp": world, "backend": backend,
                   "batch": b, "in_len": args.in_len, "out_len": args.out_len, "total_s": round(total, 4),
                   "prefill_s": round(t_prefill, 4), "decode_ms_per_token": round((total - t_prefill) / max(1, args.out_len - 1) * 1e3, 3),
                   "output_tok_s": round(b * args.out_len / total, 1), "dtype": "bf16", "data": "synthetic",
                   "decode_graph": graphed,
                   "checksum": int(toks.sum().item()) % 1000003, "first": int(first[0, 0]),
                   # switches that change which kernels run (recorded so that lines from different runs can be told apart)
                   "switches": {k: os.environ[k] for k in ("OOB_FUSED_EPILOGUES", "OOB_PREFILL_CHUNKS", "OOB_GEMM_GEMV",
                                                           "OOB_ATTN_STAGES", "OOB_GEMM_SKINNY", "OOB_GEMM_PAIR",
                                                           "OOB_SPLITK_REDUCE_MIN_M") if k in os.environ}}
            lines.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
            if comm is not None:
                comm.check_status()
        del model
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for rec in lines:
                f.write(json.dumps(rec) + "\n")
    if world > 1:
        dist.barrier()
        if comm is not None:
            comm.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
