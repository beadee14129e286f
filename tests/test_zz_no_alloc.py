"""The split-K GEMM entry point that allocates nothing (``oob_gemm_splitk_static``).

Some users of this library cannot allocate device memory at the moment they need a GEMM: a serving engine
that gave the whole GPU to its own pool at start-up, a decode step that cannot afford the synchronisation an
allocation may imply, a plug-in whose host forbids allocation in compute callbacks.  For them the library
carries a fixed workspace inside its image.  This test calls the entry point through its exported C symbol,
twice in a row on different inputs (the second call must not see the first call's partial sums or counters),
and compares with the regular entry point, whose workspace comes from ``cudaMalloc``.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other
test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

CAPACITY = 16 << 20


def _symbol():
    from ooverlap_b200 import _lib
    lib = _lib.lib()
    fn = lib.oob_gemm_splitk_static
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    need = lib.oob_gemm_splitk_static_need
    need.argtypes = [ctypes.c_int] * 4
    need.restype = ctypes.c_uint64
    return lib, fn, need


def _call(fn, a, b, out, splits):
    from ooverlap_b200 import _lib
    dtype = _lib.BF16 if a.dtype == torch.bfloat16 else _lib.F16
    return fn(dtype, a.shape[0], b.shape[0], a.shape[1], a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
              out.data_ptr(), out.stride(0), splits, 0, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_matches_allocating_entry_point_on_two_calls_in_a_row(dtype):
    from ooverlap_b200.ops import gemm
    lib, fn, need = _symbol()
    M, N, K, splits = 96, 4096, 2048, 4
    assert need(M, N, K, splits) == 16 * 4 * 128 * 256 * 4 <= CAPACITY
    g = torch.Generator(device="cuda").manual_seed(11)
    pairs = []
    for _ in range(2):
        a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
        b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
        pairs.append((a, b))
    outs = [torch.zeros(M, N, device="cuda", dtype=dtype) for _ in pairs]
    # two calls back to back on one stream, no synchronisation in between
    for (a, b), out in zip(pairs, outs):
        rc = _call(fn, a, b, out, splits)
        assert rc == 0, lib.oob_last_error()
    torch.cuda.synchronize()
    for (a, b), out in zip(pairs, outs):
        want = gemm(a, b, splits=splits)  # existing entry point: workspace from cudaMalloc
        torch.cuda.synchronize()
        ref = a.float() @ b.float().t()
        assert (out.float() - want.float()).abs().max().item() <= 1e-2
        assert (out.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())


def test_other_shape_after_first_use_and_unsplit_call():
    from ooverlap_b200.ops import gemm
    lib, fn, _ = _symbol()
    g = torch.Generator(device="cuda").manual_seed(12)
    for (M, N, K, splits) in [(16, 8192, 1024, 2), (130, 520, 512, 8), (256, 512, 256, 1)]:
        a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
        out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
        assert _call(fn, a, b, out, splits) == 0, lib.oob_last_error()
        want = gemm(a, b, splits=splits)
        torch.cuda.synchronize()
        assert (out.float() - want.float()).abs().max().item() <= 1e-2


def test_rejects_problems_beyond_the_built_in_array():
    from ooverlap_b200 import _lib
    lib, fn, need = _symbol()
    M, N, K, splits = 512, 8192, 4096, 8  # 128 tiles x 8 splits x 128 KiB = 128 MiB
    assert need(M, N, K, splits) > CAPACITY
    a = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
    rc = _call(fn, a, b, out, splits)
    assert rc == _lib.ERR_NOMEM
    msg = lib.oob_last_error().decode()
    assert "built-in array" in msg and "fewer splits" in msg
    torch.cuda.synchronize()
    assert out.min().item() == 7.0  # nothing ran
    # bad arguments are refused as well
    assert fn(_lib.F32, 8, 8, 8, a.data_ptr(), 8, b.data_ptr(), 8, out.data_ptr(), 8, 2, 0, None) == _lib.ERR_INVALID
