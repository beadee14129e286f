"""Environment-variable configuration layer.

Capability parity: the reference is configured through environment variables
only (OOVERLAP_TUNING_POLICY, OOVERLAP_MAX_CTAS, ... in
src/comm/tuning/tuning_policy.cpp:25-29 and the VLLM_OOVERLAP_* family in
patches/vllm/v0.25.0/vllm/distributed/device_communicators/ooverlap_all_reduce.py:44-67).
All names understood by this package are listed here.
"""
from __future__ import annotations

import os
from dataclasses import dataclass


def _int(name: str, default: int) -> int:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    try:
        return int(v)
    except ValueError:
        raise ValueError(f"{name} must be an integer, got {v!r}") from None


def _flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v.strip().lower() not in ("", "0", "false", "no", "off")


def env_int(name: str, default: int) -> int:
    """Integer environment variable (unset or empty: ``default``)."""
    return _int(name, default)


def env_flag(name: str, default: bool = False) -> bool:
    """Boolean environment variable ("", 0, false, no, off are false)."""
    return _flag(name, default)


# Names read directly by the native library (csrc/gemm/gemm.cu) or by single call sites:
#   OOB_GEMM_PAIR=0            plain GEMM: never use the two-SM kernel
#   OOB_GEMM_SKINNY=1          plain GEMM: weight-streaming kernel for M <= 16
#   OOB_GEMM_GEMV=0 / 1        plain GEMM, CUDA-core streaming kernel: 0 = never by default, 1 = for every M <= 4
#                              (unset: M = 1, and M = 2 with a small weight matrix)
#   OOB_SPLITK_REDUCE_MIN_M=n  split-K: sum inside the GEMM kernel below n rows (default 1: always the second kernel)
#   OOB_ATTN_STAGES=3          decode attention: three pipeline stages per warp (192 KiB of shared memory per CTA)
#   OOB_FUSED_EPILOGUES=1      model runner: RoPE + cache write and SwiGLU in the split-K sum of the preceding GEMM
#   OOB_PREFILL_CHUNKS=n       model runner, prefill: row-parallel GEMM in n slabs overlapped with the all-reduce + norm
#   OOB_PREFILL_CHUNK_MIN_ROWS from how many tokens on (default 4096)
#   OOB_NVTX=1                 NVTX ranges around the model runner's layers (utils/tracing.py)


@dataclass
class Config:
    heap_bytes: int            # OOB_HEAP_BYTES: symmetric heap per rank
    timeout_ms: int            # OOB_TIMEOUT_MS: budget of device waits and of the rendezvous
    disable_nvls: bool         # OOB_DISABLE_NVLS
    legacy_ipc: bool           # OOB_LEGACY_IPC: cudaIpc handles instead of VMM file descriptors
    max_ctas: int              # OOB_MAX_CTAS: cap of the CTA budget chosen by the policy (0 = none)
    tuning_policy: str         # OOB_TUNING_POLICY: JSON file
    log_level: str             # OOB_LOG_LEVEL: error / warning / info / debug / trace
    ar_slots: int              # OOB_AR_SLOTS, OOB_AR_SLOT_BYTES: round-robin all-reduce pool
    ar_slot_bytes: int
    ag_slots: int              # OOB_AG_SLOTS, OOB_AG_SLOT_BYTES: all-gather pool
    ag_slot_bytes: int
    ll_max_bytes: int          # OOB_LL_MAX_BYTES: round-robin all-reduces up to this size take the flag-in-data kernel
    push_max_bytes: int        # OOB_PUSH_MAX_BYTES: round-robin all-reduces up to this size take the one-barrier push
                               # kernel (0 = never)

    @staticmethod
    def from_env() -> "Config":
        return Config(
            heap_bytes=_int("OOB_HEAP_BYTES", 1 << 30),
            timeout_ms=_int("OOB_TIMEOUT_MS", 10000),
            disable_nvls=_flag("OOB_DISABLE_NVLS"),
            legacy_ipc=_flag("OOB_LEGACY_IPC"),
            max_ctas=_int("OOB_MAX_CTAS", 0),
            tuning_policy=os.environ.get("OOB_TUNING_POLICY", ""),
            log_level=os.environ.get("OOB_LOG_LEVEL", "warning"),
            ar_slots=_int("OOB_AR_SLOTS", 8),
            ar_slot_bytes=_int("OOB_AR_SLOT_BYTES", 8 << 20),
            ag_slots=_int("OOB_AG_SLOTS", 4),
            ag_slot_bytes=_int("OOB_AG_SLOT_BYTES", 64 << 20),
            ll_max_bytes=_int("OOB_LL_MAX_BYTES", 64 << 10),
            push_max_bytes=_int("OOB_PUSH_MAX_BYTES", 256 << 10),
        )
