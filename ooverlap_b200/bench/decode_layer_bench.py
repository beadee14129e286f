"""Time of one decode step per transformer layer at tensor-parallel SHARD shapes on one GPU.

The model is one rank's share of a ``--tp``-way group (heads, KV heads, FFN and vocabulary divided; see
``LlamaConfig.shard``) with a few layers, run without communication: what is left is exactly the kernels one rank
executes per layer in a served model, so the number shows how close the decode path is to the memory roofline
(weights + KV cache read once per step) independently of the interconnect.

    python -m ooverlap_b200.bench.decode_layer_bench --model 70b --tp 8 --layers 4 --batch 1,64,256 --ctx 1088

Prints one JSON line per (backend, batch): microseconds per layer of a graph-replayed decode step, the bytes a
layer must read, and the fraction of the measured HBM bandwidth (``MEASURED_PEAKS.json`` when present).

Capability parity: the reference measures serving only end to end through vLLM
(test/benchmark_vllm_paperlike.py:1-140); this is the per-layer view of the same step.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .kernel_probe import peaks


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="70b", choices=["70b", "8b"])
    p.add_argument("--tp", type=int, default=8)
    p.add_argument("--layers", type=int, default=4)
    p.add_argument("--batch", default="1,64,256")
    p.add_argument("--ctx", type=int, default=1088, help="keys attended per sequence")
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--backends", default="ours,nccl")
    p.add_argument("--kernels", action="store_true",
                   help="also list the kernels of one replayed step with their device time (CUPTI activity records "
                        "through torch.profiler: for shares and gaps, not for reported numbers)")
    args = p.parse_args()

    from ..models import LLAMA3_8B, LLAMA3_70B, LlamaTP
    torch.cuda.set_device(0)
    full = LLAMA3_70B if args.model == "70b" else LLAMA3_8B
    cfg = full.shard(args.tp, args.layers)
    _, bw_peak, src = peaks()
    hd = cfg.head_dim
    w_bytes = 2 * ((cfg.heads + 2 * cfg.kv_heads) * hd * cfg.hidden + cfg.hidden * cfg.heads * hd
                   + 2 * cfg.ffn * cfg.hidden + cfg.hidden * cfg.ffn)
    max_len = (args.ctx + 1 + 127) // 128 * 128
    for backend in args.backends.split(","):
        for B in [int(x) for x in args.batch.split(",")]:
            m = LlamaTP(cfg, None, backend=backend, max_batch=B, max_len=max_len, seed=1)
            m.k_cache.normal_()
            m.v_cache.normal_()
            pos = torch.full((1,), args.ctx - 1, dtype=torch.long, device="cuda")
            mask = torch.full((1, 1, 1, max_len), float("-inf"), device="cuda", dtype=m.dtype)
            mask[..., :args.ctx] = 0
            tok = torch.randint(0, cfg.vocab, (B, 1), device="cuda")
            with torch.no_grad():
                m.forward(tok, pos, attn_mask=mask)  # eager warm-up: sizes scratch, loads kernels
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    m.forward(tok, pos, attn_mask=mask)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                graph.replay()
            b.record()
            b.synchronize()
            us_layer = a.elapsed_time(b) * 1e3 / args.steps / cfg.layers
            kv_bytes = 2 * B * cfg.kv_heads * args.ctx * hd * 2
            floor_us = (w_bytes + kv_bytes) / (bw_peak * 1e9) * 1e6
            print(json.dumps({"bench": "decode_layer", "model": args.model, "tp": args.tp, "backend": backend, "batch": B,
                              "ctx": args.ctx, "layers": cfg.layers, "us_per_layer": round(us_layer, 1),
                              "weight_mb": round(w_bytes / 1e6, 1), "kv_mb": round(kv_bytes / 1e6, 1),
                              "hbm_floor_us": round(floor_us, 1), "frac_of_hbm_floor": round(floor_us / us_layer, 3),
                              "peaks": src,
                              "l2": "weights of the layers (%.0f MB) exceed the 126 MB L2" % (w_bytes * cfg.layers / 1e6)}),
                  flush=True)
            if args.kernels:
                from torch.profiler import ProfilerActivity, profile
                with profile(activities=[ProfilerActivity.CUDA]) as prof:
                    for _ in range(3):
                        graph.replay()
                    torch.cuda.synchronize()
                evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                             key=lambda e: e.time_range.start)
                n = len(evs) // 3
                step = evs[2 * n:]  # the last of the three replays
                per = {}
                for e in step:
                    d = per.setdefault(e.name[:60], [0, 0.0])
                    d[0] += 1
                    d[1] += e.time_range.end - e.time_range.start
                busy = sum(v[1] for v in per.values())
                span = step[-1].time_range.end - step[0].time_range.start if step else 0.0
                print(json.dumps({"bench": "decode_step_kernels", "backend": backend, "batch": B, "kernels_per_step": len(step),
                                  "busy_us": round(busy, 1), "span_us": round(span, 1),
                                  "by_kernel_us": {k: [v[0], round(v[1], 1)] for k, v in
                                                   sorted(per.items(), key=lambda kv: -kv[1][1])}}), flush=True)
            del m, graph
            torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    sys.exit(main())
