"""ctypes binding of ``libooverlap_b200.so`` (the C ABI in ``csrc/api/oob.h``).

The library is built in-tree by :mod:`ooverlap_b200._build`; it is loaded from
``ooverlap_b200/lib`` so that the loaded file is the one that travels with the
source tree.  Loading works on machines without a GPU (the CUDA runtime is
linked statically and the driver is resolved lazily); GPU entry points then
return errors instead of crashing.

Capability parity: the reference exposes its C++ through two pybind11 modules
(src/torch_collectives_pybind.cpp:868-907, src/pybind.cpp:329-648).
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import (POINTER, Structure, byref, c_char_p, c_float, c_int, c_int64, c_uint, c_uint64, c_void_p)

from . import _build

OOB_OK = 0
ERR_INVALID, ERR_CUDA, ERR_BOOTSTRAP, ERR_UNSUPPORTED, ERR_NOMEM, ERR_DEVICE_TIMEOUT, ERR_POISONED = -1, -2, -3, -4, -5, -6, -7

TOPO_PROBES, TOPO_NO_ENABLE_PEER, TOPO_NO_ATOMIC_PROBE, TOPO_NO_COPY_PROBE = 1, 2, 4, 8
TOPO_NO_MULTIMEM_PROBE, TOPO_REQUIRE_PEER, TOPO_TEXT, TOPO_NO_BULK_PROBE = 16, 32, 64, 128

LOG_SINK = ctypes.CFUNCTYPE(None, c_int, c_char_p)
LOG_ERROR, LOG_WARN, LOG_INFO, LOG_DEBUG = 0, 1, 2, 3

F16, BF16, F32 = 0, 1, 2
SUM, MIN, MAX = 0, 1, 2
ALGO_AUTO = -1
AR_ONESHOT_P2P, AR_TWOSHOT_P2P, AR_TWOSHOT_NVLS, AR_ONESHOT_NVLS = 0, 1, 2, 3
RS_P2P, RS_NVLS = 0, 1
AG_PUSH_P2P, AG_PUSH_NVLS, AG_PULL_P2P = 0, 1, 2
NORM_LOCAL, NORM_AR_ONESHOT, NORM_AR_TWOSHOT, NORM_AR_TWOSHOT_NVLS, NORM_RS, NORM_RS_NVLS = range(6)
NORM_AR_PUSH, NORM_AR_PUSH_NVLS, NORM_AR_LL = 6, 7, 8
GEMM_PLAIN, GEMM_AR, GEMM_RS_NORM, GEMM_AG = range(4)
EPILOGUE_NONE, EPILOGUE_SWIGLU, EPILOGUE_ROPE_KV = range(3)
FLAG_NO_NVLS, FLAG_LEGACY_IPC = 1, 2


class OobError(RuntimeError):
    """An entry point of the native library failed."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[oob {code}] {message}")
        self.code = code


class DeviceTimeout(OobError):
    """A kernel gave up waiting for a peer (the communicator is poisoned until ``recover``)."""


class CommInfo(Structure):
    _fields_ = [("rank", c_int), ("world", c_int), ("device", c_int), ("nvls", c_int), ("emulated", c_int),
                ("memory_kind", c_int), ("heap_bytes", c_uint64), ("user_offset", c_uint64), ("timeout_ns", c_uint64)]


class DeviceStatus(Structure):
    _fields_ = [("code", c_int), ("rank", c_int), ("peer", c_int), ("block", c_int), ("expected", c_uint),
                ("observed", c_uint), ("where", c_int), ("pad", c_int)]


class NormArgs(Structure):
    _fields_ = [("dtype", c_int), ("rows", c_int), ("hidden", c_int), ("eps", c_float), ("x_reg", c_int),
                ("x_off", c_uint64), ("residual", c_void_p), ("weight", c_void_p), ("y_reg", c_int),
                ("y_off", c_uint64), ("y_local", c_void_p), ("res_out_reg", c_int), ("res_out_off", c_uint64),
                ("res_out_local", c_void_p), ("emu_stride_local", c_uint64), ("stage_reg", c_int), ("stage_off", c_uint64),
                ("piece_bytes", c_uint64)]


class GemmArgs(Structure):
    _fields_ = [("mode", c_int), ("dtype", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("A", c_void_p),
                ("lda", c_int), ("B", c_void_p), ("ldb", c_int), ("C", c_void_p), ("ldc", c_int),
                ("a_emu_stride", c_uint64), ("b_emu_stride", c_uint64), ("c_emu_stride", c_uint64),
                ("comm_ctas", c_int), ("max_ctas", c_int), ("partial_reg", c_int), ("partial_off", c_uint64),
                ("c_reg", c_int), ("c_off", c_uint64), ("counter_base", c_int), ("residual", c_void_p),
                ("weight", c_void_p), ("eps", c_float), ("y_local", c_void_p), ("res_out_local", c_void_p),
                ("rs_emu_stride", c_uint64), ("a_full_reg", c_int), ("a_full_off", c_uint64), ("use_nvls", c_int),
                ("splits", c_int), ("no_join", c_int), ("trace", c_void_p), ("pair", c_int), ("splitk_reduce", c_int), ("skinny", c_int), ("epilogue", c_int),
                ("epilogue_args", c_void_p), ("gemv", c_int), ("stream_k", c_int), ("order", c_void_p)]


class SwigluEpilogue(Structure):
    _fields_ = [("F", c_int)]


class RopeArgs(Structure):
    _fields_ = [("dtype", c_int), ("B", c_int), ("T", c_int), ("H", c_int), ("KV", c_int), ("hd", c_int),
                ("qkv", c_void_p), ("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("cache_batch_stride", c_int64), ("max_len", c_int), ("batch0", c_int), ("cos_table", c_void_p),
                ("sin_table", c_void_p), ("pos_dev", c_void_p), ("pos0", c_int)]


class AttnDecodeArgs(Structure):
    _fields_ = [("dtype", c_int), ("B", c_int), ("H", c_int), ("KV", c_int), ("q", c_void_p), ("k_cache", c_void_p),
                ("v_cache", c_void_p), ("cache_batch_stride", c_int64), ("max_len", c_int), ("batch0", c_int),
                ("out", c_void_p), ("pos_dev", c_void_p), ("len", c_int), ("scale", c_float), ("splits", c_int),
                ("len_bound", c_int), ("workspace", c_void_p)]


_lock = threading.Lock()
_lib = None


def _declare(lib) -> None:
    P = c_void_p
    lib.oob_last_error.restype = c_char_p
    lib.oob_version.restype = c_char_p
    lib.oob_set_log_level.argtypes = [c_int]
    lib.oob_get_log_level.argtypes = []
    lib.oob_set_log_sink.argtypes = [LOG_SINK]
    lib.oob_log_message.argtypes = [c_int, c_char_p]
    lib.oob_comm_create.argtypes = [c_int, c_int, c_int, c_char_p, c_uint64, c_uint, c_int, POINTER(P)]
    lib.oob_comm_create_emulated.argtypes = [c_int, c_int, c_uint64, POINTER(P)]
    lib.oob_comm_destroy.argtypes = [P]
    lib.oob_comm_info.argtypes = [P, POINTER(CommInfo)]
    lib.oob_comm_set_timeout_ms.argtypes = [P, c_int]
    lib.oob_comm_barrier.argtypes = [P]
    lib.oob_comm_host_allgather.argtypes = [P, ctypes.c_void_p, ctypes.c_void_p, c_uint64]
    lib.oob_comm_status.argtypes = [P, POINTER(DeviceStatus)]
    lib.oob_comm_recover.argtypes = [P]
    lib.oob_alloc.argtypes = [P, c_uint64, c_uint64, POINTER(c_uint64)]
    lib.oob_free.argtypes = [P, c_uint64]
    lib.oob_heap_ptr.argtypes = [P, c_int, c_uint64]
    lib.oob_heap_ptr.restype = P
    lib.oob_heap_mc_ptr.argtypes = [P, c_uint64]
    lib.oob_heap_mc_ptr.restype = P
    lib.oob_register_ipc.argtypes = [P, P, c_uint64, POINTER(c_int)]
    lib.oob_unregister.argtypes = [P, c_int]
    lib.oob_allreduce.argtypes = [P, c_int, c_int, c_int, c_int, c_uint64, c_int, c_uint64, P, c_uint64, c_int, P]
    lib.oob_reduce_scatter.argtypes = [P, c_int, c_int, c_int, c_int, c_uint64, P, c_uint64, c_int, P]
    lib.oob_all_gather.argtypes = [P, c_int, c_int, c_int, c_uint64, P, P, c_uint64, c_int, P]
    lib.oob_all_to_all.argtypes = [P, c_int, c_int, c_uint64, P, c_uint64, c_int, P]
    lib.oob_allreduce_push.argtypes = [P, c_int, c_int, c_int, c_uint64, c_uint64, P, P, c_uint64, c_int, c_int, P]
    lib.oob_allreduce_ll.argtypes = [P, c_int, c_int, c_int, c_uint64, c_uint64, P, P, c_uint64, c_int, c_int, P]
    lib.oob_fused_norm.argtypes = [P, c_int, POINTER(NormArgs), c_int, P]
    lib.oob_gemm.argtypes = [P, POINTER(GemmArgs), P]
    lib.oob_gemm_plan_splits.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.oob_pad_counter_offset.restype = c_uint64
    lib.oob_pad_counter_offset.argtypes = []
    lib.oob_pad_counter_count.argtypes = []
    lib.oob_gemm_counters_needed.argtypes = [c_int, c_int, c_int, c_int]
    lib.oob_test_pair_schedule.argtypes = [c_int] * 8 + [POINTER(c_int), c_int]
    lib.oob_gemm_reserve_workspace.argtypes = [c_uint64]
    lib.oob_gemm_splitk_bytes.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.oob_gemm_splitk_bytes.restype = c_uint64
    lib.oob_gemm_partial_bytes.argtypes = [c_int, c_int]
    lib.oob_gemm_partial_bytes.restype = c_uint64
    lib.oob_rope_kv_write.argtypes = [POINTER(RopeArgs), P]
    lib.oob_silu_mul.argtypes = [c_int, P, c_int64, P, c_int, c_int, P]
    lib.oob_attn_decode.argtypes = [POINTER(AttnDecodeArgs), P]
    lib.oob_attn_decode_auto_splits.argtypes = [c_int, c_int, c_int]
    lib.oob_attn_decode_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.oob_attn_decode_workspace_bytes.restype = c_uint64
    lib.oob_policy_load.argtypes = [c_char_p]
    lib.oob_policy_select.argtypes = [c_int, c_int, c_uint64, c_int, POINTER(c_int), POINTER(c_int)]
    lib.oob_topology_json.argtypes = [c_char_p, c_uint64, c_int]
    lib.oob_topology_describe.argtypes = [c_char_p, c_uint64, c_uint, POINTER(c_int), c_int]
    lib.oob_test_bounded_wait.argtypes = [P, P]
    lib.oob_bootstrap_create.argtypes = [c_int, c_int, c_char_p, c_int, POINTER(P)]
    lib.oob_bootstrap_destroy.argtypes = [P]
    lib.oob_bootstrap_allgather.argtypes = [P, P, P, c_uint64]
    lib.oob_bootstrap_barrier.argtypes = [P]
    lib.oob_bootstrap_exchange_fds.argtypes = [P, c_int, POINTER(c_int)]
    lib.oob_bootstrap_broadcast_fd.argtypes = [P, c_int, POINTER(c_int)]


def lib():
    """The loaded native library (built first if the in-tree binary is missing or stale)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.LIB
                if not _build.is_current():
                    path = _build.build()
                handle = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
                _declare(handle)
                _lib = handle
    return _lib


def last_error() -> str:
    msg = lib().oob_last_error()
    return msg.decode() if msg else ""


def check(code: int) -> None:
    if code == OOB_OK:
        return
    msg = last_error()
    if code in (ERR_DEVICE_TIMEOUT, ERR_POISONED):
        raise DeviceTimeout(code, msg)
    raise OobError(code, msg)


__all__ = [name for name in globals() if name.isupper()] + [
    "lib", "check", "last_error", "OobError", "DeviceTimeout", "CommInfo", "DeviceStatus", "NormArgs", "GemmArgs",
    "byref",
]
