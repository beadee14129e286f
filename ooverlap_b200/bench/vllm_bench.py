"""Serving throughput through the vLLM engine with this library as the tensor-parallel all-reduce backend.

One fresh process per backend (``--per-batch-engines`` makes it one per backend and batch, as the reference does):
the engine is built on a Llama-architecture model with random weights (``load_format="dummy"``, a config written to
a temporary directory, no tokenizer); for every batch size, ``batch`` prompts of ``--in-len`` uniform-random token
ids are generated to ``--out-len`` tokens with greedy sampling, and the process prints one JSON line per batch with
output tokens per second.  Backends:

``ooverlap``  ``VLLM_FORCE_ALLREDUCE_BACKEND=ooverlap``: this library, loaded in every vLLM process through the
              ``vllm.general_plugins`` entry point that ``pyproject.toml`` declares.  For a run from the source tree
              (nothing installed) the driver writes that entry point's metadata into a temporary directory and puts it,
              and the repository root, on ``PYTHONPATH`` of the child.  The line carries how many all-reduces the
              backend served and declined (forced mode raises on a tensor it cannot serve).
``default``   vLLM as it comes (its own choice among custom all-reduce, symmetric memory and NCCL)
``custom``    vLLM's own custom all-reduce, forced
``pynccl``    NCCL, forced

    python -m ooverlap_b200.bench.vllm_bench --model llama3-70b --tp 8 --batches 1,64,256 --backends pynccl,custom,ooverlap

``--orders`` runs the backends in every listed order (the reference runs all permutations, with a cool-down
between runs, so that no backend always runs on a cold or a hot machine); ``ooverlap_b200.bench.aggregate`` merges
the lines.

Capability parity: test/benchmark_vllm_paperlike.py:1-140 and evalution/run_vllm_paperlike.sh:1-140 of the
reference (fresh ``vllm bench throughput`` subprocess per model, backend, device set, batch and workload).
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import subprocess
import sys
import tempfile
import time

MODELS = {
    # name: (layers, hidden, heads, kv_heads, ffn, vocab)
    "llama3-70b": (80, 8192, 64, 8, 28672, 128256),
    "llama3-8b": (32, 4096, 32, 8, 14336, 128256),
    "tiny": (2, 1024, 8, 2, 2048, 1024),
}
BACKENDS = ("ooverlap", "default", "custom", "pynccl", "nccl_symm")


def write_model_dir(path: str, model: str, layers: int = 0, max_len: int = 4096) -> str:
    """Writes a Hugging Face ``config.json`` of the named Llama architecture into ``path`` (no weights: the engine
    is started with ``load_format="dummy"``)."""
    n_layers, hidden, heads, kv_heads, ffn, vocab = MODELS[model]
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": hidden,
        "intermediate_size": ffn, "num_hidden_layers": layers or n_layers, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "vocab_size": vocab, "max_position_embeddings": max(max_len, 8192),
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "hidden_act": "silu", "tie_word_embeddings": False,
        "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2, "attention_bias": False, "mlp_bias": False,
    }
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return path


def write_plugin_metadata(path: str) -> str:
    """Writes ``ooverlap_b200-<version>.dist-info`` with the ``vllm.general_plugins`` entry point into ``path``: what an
    installation of this package (``pip install .``, see pyproject.toml) puts into site-packages.  With ``path`` on
    ``PYTHONPATH``, vLLM's plugin loader finds the hook in every process it starts, although nothing is installed."""
    from .. import __version__
    d = os.path.join(path, f"ooverlap_b200-{__version__}.dist-info")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "METADATA"), "w") as f:
        f.write(f"Metadata-Version: 2.1\nName: ooverlap-b200\nVersion: {__version__}\n")
    with open(os.path.join(d, "entry_points.txt"), "w") as f:
        f.write("[vllm.general_plugins]\nooverlap_b200 = ooverlap_b200.parallel.vllm_adapter:install\n")
    with open(os.path.join(d, "RECORD"), "w") as f:
        f.write("")
    return path


def child_env(backend: str, repo_root: str, base: dict | None = None, plugin_dir: str = "", stats_file: str = "") -> dict:
    """Environment of one benchmark process."""
    env = dict(os.environ if base is None else base)
    parts = [p for p in (plugin_dir, repo_root, env.get("PYTHONPATH", "")) if p]
    env["PYTHONPATH"] = os.pathsep.join(parts)
    env["VLLM_WORKER_MULTIPROC_METHOD"] = "spawn"
    env["MASTER_ADDR"] = "127.0.0.1"
    env["VLLM_HOST_IP"] = "127.0.0.1"
    if backend == "default":
        env.pop("VLLM_FORCE_ALLREDUCE_BACKEND", None)
    else:
        env["VLLM_FORCE_ALLREDUCE_BACKEND"] = backend
    if stats_file:
        env["VLLM_OOVERLAP_STATS_FILE"] = stats_file
    return env


def child_command(args, backend: str, batches: str, model_dir: str) -> list[str]:
    return [sys.executable, "-m", "ooverlap_b200.bench.vllm_bench", "--worker", "--backend", backend, "--batches", batches,
            "--model-dir", model_dir, "--model", args.model, "--tp", str(args.tp), "--in-len", str(args.in_len),
            "--out-len", str(args.out_len), "--repeats", str(args.repeats), "--graphs", args.graphs] + \
           (["--eager"] if args.eager else [])


def run_worker(args) -> int:
    """Builds one engine and measures ``repeats`` generations of every batch size."""
    import numpy as np
    from vllm import LLM, SamplingParams
    from vllm.inputs import TokensPrompt

    batches = [int(x) for x in args.batches.split(",") if x]
    vocab = MODELS[args.model][5]
    kw = {}
    if not args.eager and args.graphs != "default":
        # CUDA graphs of whole decode steps without the compiler pass (engine start in seconds instead of minutes;
        # the all-reduce backend is captured like any other kernel).
        kw["compilation_config"] = {"mode": 0, "cudagraph_mode": args.graphs.upper(),
                                    "cudagraph_capture_sizes": sorted({1, 2, 4, 8, 16, 32, 64, 128, 256} & set(range(1, max(batches) + 1)) | set(batches))}
    llm = LLM(model=args.model_dir, skip_tokenizer_init=True, tensor_parallel_size=args.tp, dtype="bfloat16",
              load_format="dummy", max_model_len=args.in_len + args.out_len + 16, max_num_seqs=max(max(batches), 1),
              gpu_memory_utilization=0.90, enforce_eager=args.eager, disable_custom_all_reduce=args.backend == "pynccl",
              disable_log_stats=True, seed=0, **kw)
    rng = np.random.default_rng(0)
    sp = SamplingParams(temperature=0.0, max_tokens=args.out_len, ignore_eos=True, detokenize=False)
    for batch in batches:
        prompts = [TokensPrompt(prompt_token_ids=rng.integers(10, vocab - 10, size=args.in_len).tolist())
                   for _ in range(batch)]
        llm.generate(prompts[: min(2, len(prompts))], sp, use_tqdm=False)  # warm-up: graphs, allocator
        best = None
        for _ in range(args.repeats):
            t0 = time.perf_counter()
            outs = llm.generate(prompts, sp, use_tqdm=False)
            dt = time.perf_counter() - t0
            n_out = sum(len(o.outputs[0].token_ids) for o in outs)
            tps = n_out / dt
            best = tps if best is None or tps > best else best
        print(json.dumps({"bench": "vllm_throughput", "model": args.model, "tp": args.tp, "backend": args.backend,
                          "batch": batch, "in_len": args.in_len, "out_len": args.out_len, "repeats": args.repeats,
                          "output_tok_s": round(best, 2), "eager": bool(args.eager), "graphs": args.graphs,
                          "data": "uniform-random token ids", "weights": "random (load_format=dummy)"}), flush=True)
    return 0


def read_stats(path: str) -> dict | None:
    """Sums the per-rank lines the backend wrote at shutdown (served / declined all-reduces)."""
    try:
        lines = [json.loads(ln) for ln in open(path) if ln.strip()]
    except OSError:
        return None
    if not lines:
        return None
    declined: dict = {}
    for ln in lines:
        for k, v in ln.get("declined", {}).items():
            declined[k] = declined.get(k, 0) + v
    return {"ranks": len(lines), "served": sum(ln.get("served", 0) for ln in lines),
            "served_in_pieces": sum(ln.get("served_in_pieces", 0) for ln in lines), "declined": declined}


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="llama3-70b", choices=sorted(MODELS))
    p.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the model's own)")
    p.add_argument("--tp", type=int, default=8)
    p.add_argument("--batches", default="1,64,256")
    p.add_argument("--backends", default="pynccl,custom,ooverlap")
    p.add_argument("--orders", default="given", help="given | all: run the backends in the given order or in every permutation")
    p.add_argument("--in-len", type=int, default=1024)
    p.add_argument("--out-len", type=int, default=128)
    p.add_argument("--repeats", type=int, default=2)
    p.add_argument("--cooldown", type=float, default=5.0, help="seconds between runs")
    p.add_argument("--timeout", type=float, default=1800.0, help="limit of one run, seconds")
    p.add_argument("--eager", action="store_true", help="no CUDA graphs / compilation in the engine")
    p.add_argument("--graphs", default="full_decode_only", help="default = the engine's own compilation + CUDA-graph "
                   "settings; else a cudagraph_mode (full_decode_only, full, piecewise, none) with the compiler pass off")
    p.add_argument("--per-batch-engines", action="store_true", help="a fresh engine per batch size (default: per backend)")
    p.add_argument("--out", default="", help="append the JSON lines to this file")
    p.add_argument("--dry-run", action="store_true", help="print the commands instead of running them")
    # worker mode (one engine, one batch)
    p.add_argument("--worker", action="store_true")
    p.add_argument("--backend", default="ooverlap", choices=BACKENDS)
    p.add_argument("--model-dir", default="")
    args = p.parse_args()
    if args.worker:
        return run_worker(args)

    backends = [b for b in args.backends.split(",") if b]
    for b in backends:
        if b not in BACKENDS:
            raise SystemExit(f"unknown backend {b!r}")
    orders = list(itertools.permutations(backends)) if args.orders == "all" else [tuple(backends)]
    if args.out:
        # what produced the file: command line, versions, GPUs and the environment that steers the backends
        from ..utils.manifest import write_manifest
        write_manifest(args.out + ".manifest.json", extra={"bench": "vllm_throughput", "model": args.model, "tp": args.tp,
                                                           "backends": backends, "orders": len(orders)})
    repo_root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    rc = 0
    with tempfile.TemporaryDirectory(prefix="oob_vllm_") as tmp:
        model_dir = write_model_dir(os.path.join(tmp, args.model), args.model, args.layers, args.in_len + args.out_len + 16)
        plugin_dir = write_plugin_metadata(os.path.join(tmp, "plugin"))
        groups = args.batches.split(",") if args.per_batch_engines else [args.batches]
        for oi, order in enumerate(orders):
            for batches in groups:
                for backend in order:
                    cmd = child_command(args, backend, batches, model_dir)
                    if args.dry_run:
                        print(json.dumps({"order": oi, "backend": backend, "batches": batches, "cmd": cmd}))
                        continue
                    stats_file = os.path.join(tmp, f"stats_{oi}_{backend}_{batches.replace(',', '_')}.jsonl")
                    t0 = time.perf_counter()
                    try:
                        res = subprocess.run(cmd, env=child_env(backend, repo_root, None, plugin_dir, stats_file),
                                             capture_output=True, text=True, timeout=args.timeout)
                    except subprocess.TimeoutExpired:
                        print(json.dumps({"bench": "vllm_throughput", "backend": backend, "batches": batches, "order": oi,
                                          "error": f"no result within {args.timeout:.0f} s"}), flush=True)
                        rc = 1
                        continue
                    wall = time.perf_counter() - t0
                    lines = [ln for ln in res.stdout.splitlines() if ln.startswith('{"bench"')]
                    if res.returncode != 0 or not lines:
                        tail = (res.stderr or res.stdout)[-1500:]
                        print(json.dumps({"bench": "vllm_throughput", "backend": backend, "batches": batches, "order": oi,
                                          "error": f"exit {res.returncode}", "tail": tail}), flush=True)
                        rc = 1
                    stats = read_stats(stats_file)
                    for line in lines:
                        rec = json.loads(line)
                        rec["order"] = oi
                        rec["engine_wall_s"] = round(wall, 1)
                        if backend == "ooverlap":
                            rec["all_reduces"] = stats
                        out = json.dumps(rec)
                        print(out, flush=True)
                        if args.out:
                            with open(args.out, "a") as f:
                                f.write(out + "\n")
                    time.sleep(args.cooldown)
    return rc


if __name__ == "__main__":
    sys.exit(main())
