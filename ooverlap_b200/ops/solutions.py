"""Per-shape tuning results ("solutions") for the overlap ops.

A solution file is a JSON object ``{"<op>:<M>x<N>x<K>:tp<world>:<dtype>": {"strategy": ..., "comm_ctas": ...,
"use_nvls": ..., "kernel": ..., "us": ...}, ...}`` written by ``ooverlap_b200.bench.tune_overlap``.  ``GemmAllReduce``
consults the file named by ``OOB_OVERLAP_SOLUTIONS``, else the packaged ``policy/overlap_solutions.json`` (the measured
winners for the headline shapes on 2, 4 and 8 x B200 / NVSwitch), before falling back to its built-in rule;
``OOB_OVERLAP_SOLUTIONS=none`` turns the lookup off.

Capability parity: the reference saves one solution JSON per (M, N, K, backend) with the searched segment sizes,
tile order and SM split (tool/search.py:355-421, test/test.py:805-820) and its benchmark loads it back.
"""
from __future__ import annotations

import json
import os
import tempfile
from typing import Optional

_cache = {}
PACKAGED = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "policy", "overlap_solutions.json")


def key(op: str, M: int, N: int, K: int, world: int, dtype: str) -> str:
    return f"{op}:{M}x{N}x{K}:tp{world}:{dtype}"


def load(path: str) -> dict:
    if path not in _cache:
        try:
            with open(path) as f:
                data = json.load(f)
            if not isinstance(data, dict):
                raise ValueError("solution file must hold a JSON object")
        except FileNotFoundError:
            data = {}
        _cache[path] = data
    return _cache[path]


def lookup(op: str, M: int, N: int, K: int, world: int, dtype: str, path: Optional[str] = None) -> Optional[dict]:
    """The stored solution for a shape; K == 0 matches any K of that (op, M, N)."""
    path = path or os.environ.get("OOB_OVERLAP_SOLUTIONS", "") or PACKAGED
    if path == "none" or not os.path.exists(path):
        return None
    table = load(path)
    hit = table.get(key(op, M, N, K, world, dtype))
    if hit is None and K == 0:
        prefix, suffix = f"{op}:{M}x{N}x", f":tp{world}:{dtype}"
        for k, v in table.items():
            if k.startswith(prefix) and k.endswith(suffix):
                return v
    return hit


PACKAGED_GEMM = os.path.join(os.path.dirname(PACKAGED), "gemm_solutions.json")
_gemm_path = None  # resolved once: "" = no table


def gemm_key(M: int, N: int, K: int, dtype: str) -> str:
    return f"gemm:{M}x{N}x{K}:{dtype}"


def lookup_gemm(M: int, N: int, K: int, dtype: str) -> Optional[dict]:
    """The profiled configuration of a plain GEMM shape (written by ``ooverlap_b200.bench.gemm_profile``): the file
    named by ``OOB_GEMM_SOLUTIONS``, else the packaged ``policy/gemm_solutions.json``; ``OOB_GEMM_SOLUTIONS=none`` turns
    the lookup off.  The path is resolved once per process."""
    global _gemm_path
    if _gemm_path is None:
        path = os.environ.get("OOB_GEMM_SOLUTIONS", "") or PACKAGED_GEMM
        _gemm_path = path if path != "none" and os.path.exists(path) else ""
    if not _gemm_path:
        return None
    return load(_gemm_path).get(gemm_key(M, N, K, dtype))


def reset_gemm_lookup() -> None:
    """Forget the resolved table path (tests change the environment variable)."""
    global _gemm_path
    _gemm_path = None


def save(path: str, table: dict) -> None:
    """Atomic replace, so that an interrupted tuning run never leaves a truncated file."""
    d = os.path.dirname(os.path.abspath(path)) or "."
    fd, tmp = tempfile.mkstemp(prefix=".solutions.", dir=d)
    with os.fdopen(fd, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    os.replace(tmp, path)
    _cache[path] = dict(table)
