"""Residual-add + RMSNorm: stand-alone and fused into all-reduce / reduce-scatter (emulated ranks)."""
import pytest
import torch

from ooverlap_b200 import _lib

pytestmark = pytest.mark.gpu


def _oracle(xs, residual, weight, eps, dtype):
    s = torch.stack([x.float() for x in xs]).sum(0)
    if residual is not None:
        s = (s + residual.float()).to(dtype).float()
    y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y, s


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 64), (37, 8192), (5, 4096 + 8), (3, 16384)])
def test_local_rmsnorm(shape, dtype):
    from ooverlap_b200.ops import rmsnorm
    rows, hidden = shape
    x = torch.randn(rows, hidden, device="cuda").to(dtype)
    res = torch.randn(rows, hidden, device="cuda").to(dtype)
    w = (1 + 0.02 * torch.randn(hidden, device="cuda")).to(dtype)
    y = rmsnorm(x, w, 1e-6)
    want, _ = _oracle([x], None, w, 1e-6, dtype)
    assert (y.float() - want).abs().max().item() <= 2e-2
    y2, r2 = rmsnorm(x, w, 1e-6, res)
    want2, s2 = _oracle([x], res, w, 1e-6, dtype)
    assert (y2.float() - want2).abs().max().item() <= 3e-2
    assert ((r2.float() - s2).abs() <= 1e-2 + s2.abs() * 2 ** -7).all()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", [_lib.NORM_AR_ONESHOT, _lib.NORM_AR_TWOSHOT, _lib.NORM_AR_PUSH, _lib.NORM_AR_LL])
@pytest.mark.parametrize("rows", [1, 5, 64])
def test_allreduce_residual_rmsnorm(world, algo, rows):
    from ooverlap_b200 import EmulatedGroup
    dtype, hidden, eps = torch.bfloat16, 8192, 1e-6
    g = EmulatedGroup(world, heap_bytes=64 << 20)
    nbytes = rows * hidden * 2
    x_off, y_off, r_off = g.alloc(nbytes), g.alloc(nbytes), g.alloc(nbytes)
    xs = []
    for r in range(world):
        x = torch.randn(rows, hidden, device="cuda").to(dtype)
        g.view(x_off, (rows, hidden), dtype, r).copy_(x)
        xs.append(x)
    residual1 = torch.randn(rows, hidden, device="cuda").to(dtype)
    residual = residual1.unsqueeze(0).repeat(world, 1, 1).contiguous()  # replicated on every rank
    w = (1 + 0.02 * torch.randn(hidden, device="cuda")).to(dtype)
    want_y, want_s = _oracle(xs, residual1, w, eps, dtype)
    if algo in (_lib.NORM_AR_ONESHOT, _lib.NORM_AR_PUSH, _lib.NORM_AR_LL):
        y = torch.zeros(world, rows, hidden, device="cuda", dtype=dtype)
        ro = torch.zeros_like(y)
        piece = (nbytes + 255) // 256 * 256 * (2 if algo == _lib.NORM_AR_LL else 1)  # cells: 8 bytes per 4 of data
        stage = g.alloc(2 * world * piece) if algo != _lib.NORM_AR_ONESHOT else None
        if algo == _lib.NORM_AR_LL:  # the flag-in-data staging area must read as zero before its first use
            for r in range(world):
                g.view(stage, (2 * world * piece,), torch.uint8, r).zero_()
            torch.cuda.synchronize()
        for _ in range(1 if algo == _lib.NORM_AR_ONESHOT else 3):  # the push kernels alternate between two sets of pieces
            g.fused_norm(algo, x_off=x_off, rows=rows, hidden=hidden, dtype=dtype, weight=w, eps=eps, residual=residual,
                         y_local=y, res_out_local=ro, local_stride_bytes=nbytes, stage_off=stage, piece_bytes=piece)
            g.check_status()
        ys, rs = [y[r] for r in range(world)], [ro[r] for r in range(world)]
    else:
        g.fused_norm(algo, x_off=x_off, rows=rows, hidden=hidden, dtype=dtype, weight=w, eps=eps, residual=residual,
                     y_off=y_off, res_out_off=r_off, local_stride_bytes=nbytes)
        g.check_status()
        ys = [g.view(y_off, (rows, hidden), dtype, r) for r in range(world)]
        rs = [g.view(r_off, (rows, hidden), dtype, r) for r in range(world)]
    for r in range(world):
        assert (ys[r].float() - want_y).abs().max().item() <= 5e-2, (r, algo)
        assert ((rs[r].float() - want_s).abs() <= 1e-2 + want_s.abs() * 2 ** -7).all()  # one bf16 ulp of slack
        assert torch.equal(ys[r], ys[0])
    g.close()


@pytest.mark.parametrize("world", [2, 4])
def test_reduce_scatter_residual_rmsnorm(world):
    from ooverlap_b200 import EmulatedGroup
    from ooverlap_b200.utils.partition import partition
    dtype, hidden, eps, rows = torch.bfloat16, 4096, 1e-5, 22  # uneven row partition
    g = EmulatedGroup(world, heap_bytes=32 << 20)
    x_off = g.alloc(rows * hidden * 2)
    xs = []
    for r in range(world):
        x = torch.randn(rows, hidden, device="cuda").to(dtype)
        g.view(x_off, (rows, hidden), dtype, r).copy_(x)
        xs.append(x)
    max_rows = -(-rows // world)
    res_full = torch.randn(rows, hidden, device="cuda").to(dtype)
    res = torch.zeros(world, max_rows, hidden, device="cuda", dtype=dtype)
    for r in range(world):
        b, e = partition(rows, world, r)
        res[r, : e - b] = res_full[b:e]
    w = (1 + 0.02 * torch.randn(hidden, device="cuda")).to(dtype)
    y = torch.zeros(world, max_rows, hidden, device="cuda", dtype=dtype)
    ro = torch.zeros_like(y)
    g.fused_norm(_lib.NORM_RS, x_off=x_off, rows=rows, hidden=hidden, dtype=dtype, weight=w, eps=eps, residual=res,
                 y_local=y, res_out_local=ro, local_stride_bytes=max_rows * hidden * 2)
    g.check_status()
    want_y, want_s = _oracle(xs, res_full, w, eps, dtype)
    for r in range(world):
        b, e = partition(rows, world, r)
        assert (y[r, : e - b].float() - want_y[b:e]).abs().max().item() <= 5e-2
        assert ((ro[r, : e - b].float() - want_s[b:e]).abs() <= 1e-2 + want_s[b:e].abs() * 2 ** -7).all()
    g.close()
