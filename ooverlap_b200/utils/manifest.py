"""Run manifest: what produced a benchmark file.  One JSON object with the command line, the time, the versions of
Python / torch / CUDA / NCCL / this library, the GPUs and every environment variable that steers this library, the
vLLM hook, NCCL or device visibility; written next to a benchmark's output so that a result can be traced to its
configuration later.

Capability parity: the run manifests with environment capture of the reference's vLLM benchmark driver
(test/benchmark_vllm_paperlike.py:117-140).
"""
from __future__ import annotations

import json
import os
import platform
import sys
import time
from typing import Optional, Sequence

ENV_PREFIXES = ("OOB_", "VLLM_", "NCCL_", "CUDA_", "TORCH_NCCL_", "OMP_NUM_THREADS", "MASTER_", "WORLD_SIZE", "RANK",
                "LOCAL_RANK")
_SECRET_WORDS = ("KEY", "TOKEN", "SECRET", "PASSWORD")


def captured_env(env: Optional[dict] = None) -> dict:
    """The variables of ``env`` (default: this process's) that a manifest records; values of variables whose name looks
    like a credential are replaced by their length."""
    env = os.environ if env is None else env
    out = {}
    for k in sorted(env):
        if not k.startswith(ENV_PREFIXES):
            continue
        v = env[k]
        secret = any(w in k.upper() for w in _SECRET_WORDS) and not k.startswith("VLLM_OOVERLAP_BROKER_KEY")
        out[k] = f"<{len(v)} characters>" if secret else v
    return out


def run_manifest(argv: Optional[Sequence[str]] = None, extra: Optional[dict] = None, env: Optional[dict] = None) -> dict:
    m = {"argv": list(sys.argv if argv is None else argv), "time_utc": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
         "host": platform.node(), "python": platform.python_version(), "env": captured_env(env)}
    try:
        import torch
        m["torch"] = torch.__version__
        m["cuda_runtime"] = torch.version.cuda
        if torch.cuda.is_available():
            m["gpus"] = [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())]
            try:
                m["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version())
            except Exception:
                pass
        else:
            m["gpus"] = []
    except Exception as e:  # a manifest must never stop a run
        m["torch"] = f"unavailable: {e}"
    try:
        from .. import _lib
        m["library"] = _lib.lib().oob_version().decode()
    except Exception as e:
        m["library"] = f"unavailable: {e}"
    try:
        from importlib import metadata
        m["vllm"] = metadata.version("vllm")  # the version only: importing the package costs seconds
    except Exception:
        m["vllm"] = None
    if extra:
        m.update(extra)
    return m


def write_manifest(path: str, argv: Optional[Sequence[str]] = None, extra: Optional[dict] = None) -> dict:
    """Writes the manifest to ``path`` (atomic replace) and returns it."""
    m = run_manifest(argv, extra)
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, "w") as f:
        json.dump(m, f, indent=1, sort_keys=True)
    os.replace(tmp, path)
    return m
