"""Argument checks of the native entry points run before any CUDA call, so they can be exercised without a GPU:
bad arguments must come back as OOB_ERR_INVALID / OOB_ERR_UNSUPPORTED with a message, never as a launch."""
import ctypes

import pytest
import torch

from ooverlap_b200 import _lib


def _err(code):
    assert code < 0
    return _lib.last_error()


def test_rope_and_swiglu_and_attention_reject_bad_arguments():
    lib = _lib.lib()
    a = _lib.RopeArgs()
    a.dtype, a.B, a.T, a.H, a.KV, a.hd = _lib.BF16, 1, 1, 8, 1, 100  # hd not a multiple of 8
    assert lib.oob_rope_kv_write(ctypes.byref(a), None) == _lib.ERR_INVALID and "RoPE" in _err(-1)
    a.hd = 128
    assert lib.oob_rope_kv_write(ctypes.byref(a), None) == _lib.ERR_INVALID and "null" in _err(-1)
    assert lib.oob_rope_kv_write(None, None) == _lib.ERR_INVALID
    assert lib.oob_silu_mul(_lib.F32, 16, 64, 16, 1, 32, None) == _lib.ERR_INVALID          # dtype
    assert lib.oob_silu_mul(_lib.BF16, 16, 64, 16, 1, 30, None) == _lib.ERR_INVALID         # F % 8
    assert lib.oob_silu_mul(_lib.BF16, 16, 32, 16, 1, 32, None) == _lib.ERR_INVALID         # ld < 2F
    assert lib.oob_silu_mul(_lib.BF16, 8, 64, 16, 1, 32, None) == _lib.ERR_INVALID          # alignment
    d = _lib.AttnDecodeArgs()
    d.dtype, d.B, d.H, d.KV = _lib.BF16, 1, 40, 2                                            # 20 query heads per KV head
    assert lib.oob_attn_decode(ctypes.byref(d), None) == _lib.ERR_INVALID and "16" in _err(-1)
    d.H = 8
    assert lib.oob_attn_decode(ctypes.byref(d), None) == _lib.ERR_INVALID and "null" in _err(-1)


def test_gemm_rejects_bad_arguments_before_launching():
    lib = _lib.lib()
    g = _lib.GemmArgs()
    g.mode, g.dtype = _lib.GEMM_PLAIN, _lib.F32
    assert lib.oob_gemm(None, ctypes.byref(g), None) == _lib.ERR_INVALID and "dtype" in _err(-1)
    g.dtype, g.mode = _lib.BF16, _lib.GEMM_AR
    assert lib.oob_gemm(None, ctypes.byref(g), None) == _lib.ERR_INVALID and "communicator" in _err(-1)
    # an epilogue on a problem that is not split over K has no kernel to run in
    g.mode, g.M, g.N, g.K = _lib.GEMM_PLAIN, 8192, 8192, 8192
    epi = _lib.SwigluEpilogue()
    epi.F = 4096
    g.epilogue, g.epilogue_args = _lib.EPILOGUE_SWIGLU, ctypes.cast(ctypes.pointer(epi), ctypes.c_void_p)
    assert lib.oob_gemm_plan_splits(8192, 8192, 8192, 0, 0) == 1
    assert lib.oob_gemm(None, ctypes.byref(g), None) == _lib.ERR_UNSUPPORTED and "not split" in _err(-1)
    # split problem, inconsistent SwiGLU geometry
    g.M, g.N, g.K = 16, 7168, 8192
    assert lib.oob_gemm_plan_splits(16, 7168, 8192, 0, 0) > 1
    assert lib.oob_gemm(None, ctypes.byref(g), None) == _lib.ERR_INVALID and "SwiGLU" in _err(-1)
    g.epilogue_args = None
    assert lib.oob_gemm(None, ctypes.byref(g), None) == _lib.ERR_INVALID and "null epilogue" in _err(-1)


def test_python_wrappers_check_shapes_before_calling_native_code():
    from ooverlap_b200.ops import decode
    q = torch.zeros(2, 8, 64)
    kc = torch.zeros(2, 1, 32, 64)
    with pytest.raises(ValueError):
        decode.attn_decode(q, kc, kc, 3)                       # head size must be 128
    q = torch.zeros(2, 8, 128, dtype=torch.bfloat16)
    kc = torch.zeros(1, 1, 32, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        decode.attn_decode(q, kc, kc, 3)                       # two sequences, one cache slot
    with pytest.raises(ValueError):
        decode.silu_mul(torch.zeros(4, 24))                    # 2F not a multiple of 16
    qkv = torch.zeros(2, 10 * 128, dtype=torch.bfloat16)
    cos, sin = decode.rope_tables(32, 128, 10000.0, "cpu")
    with pytest.raises(ValueError):
        decode.rope_kv_write(qkv, 2, 1, 8, 1, kc, kc, cos, sin, 0)   # cache holds one sequence
    kc2 = torch.zeros(2, 1, 32, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        decode.rope_kv_write(qkv, 2, 1, 8, 1, kc2, kc2, cos[:16], sin[:16], 0)  # tables shorter than the cache
    with pytest.raises(ValueError):
        decode.rope_kv_write(qkv, 2, 1, 8, 1, kc2, kc2, cos, sin, torch.zeros(1, dtype=torch.long))  # pos not on the GPU


def test_collective_entry_points_refuse_a_null_communicator():
    """Every entry point that launches on a communicator answers OOB_ERR_INVALID for a null handle, with a message,
    before it looks at anything else (a caller that lost its handle must not crash the process)."""
    lib = _lib.lib()
    calls = [
        lambda: lib.oob_allreduce(None, _lib.BF16, 0, 0, 0, 0, -1, 0, None, 16, 0, None),
        lambda: lib.oob_reduce_scatter(None, _lib.BF16, 0, 0, 0, 0, None, 16, 0, None),
        lambda: lib.oob_all_gather(None, _lib.BF16, 0, 0, 0, None, None, 16, 0, None),
        lambda: lib.oob_all_to_all(None, _lib.BF16, 0, 0, None, 16, 0, None),
        lambda: lib.oob_allreduce_push(None, _lib.BF16, 0, 0, 0, 4096, None, None, 16, 0, 0, None),
        lambda: lib.oob_allreduce_ll(None, _lib.BF16, 0, 0, 0, 4096, None, None, 16, 0, 0, None),
        lambda: lib.oob_comm_recover(None),
        lambda: lib.oob_comm_barrier(None),
    ]
    for call in calls:
        assert call() == _lib.ERR_INVALID
        assert "null communicator" in _lib.last_error()
