"""Fused GEMM + collective kernels with emulated ranks on one GPU (every rank = one block row of a single
cooperative launch).  Oracle: PyTorch fp32 matmul and reductions."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(world, M, N, K, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(world, M, K, device="cuda", generator=g).to(dtype)
    b = (torch.randn(world, N, K, device="cuda", generator=g) / (K * world) ** 0.5).to(dtype)
    return a, b


KERNELS = ["pair", "one_sm"]  # two-SM kernel (CTA pairs, in-place reduction) and one-SM kernel (pushed partial tiles)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("shape", [(256, 512, 256), (1024, 1024, 512), (200, 264, 72), (640, 1280, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_all_reduce(world, shape, dtype, kernel):
    from ooverlap_b200 import EmulatedGroup
    from ooverlap_b200.ops import GemmAllReduce
    M, N, K = shape
    if world == 8 and kernel == "one_sm" and M * N > 256 * 512:
        pytest.skip("eight emulated ranks of the one-SM kernel are covered by the small shape")
    g = EmulatedGroup(world, heap_bytes=64 << 20)
    op = GemmAllReduce(g, M, N, dtype, comm_ctas=4, kernel=kernel)
    a, b = _operands(world, M, N, K, dtype, seed=M + world)
    want = sum(a[r].float() @ b[r].float().t() for r in range(world))
    for it in range(3):  # repeated calls re-arm the tile counters
        for r in range(world):
            op.output(r).zero_()
        op(a, b)
        g.check_status()
        for r in range(world):
            got = op.output(r)
            assert (got.float() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item()), (it, r)
            assert torch.equal(got, op.output(0))
    g.close()


def test_fused_two_sm_kernel_writes_the_tile_order_record():
    """The signal warp stamps every half-tile when it publishes it to its reducer (the emulated ranks share the
    buffer; the last writer's stamp stays)."""
    from ooverlap_b200 import EmulatedGroup
    from ooverlap_b200.ops import GemmAllReduce, order_buffer, tile_order
    world, M, N, K = 2, 1024, 1024, 256
    g = EmulatedGroup(world, heap_bytes=64 << 20)
    op = GemmAllReduce(g, M, N, torch.bfloat16, comm_ctas=4, kernel="pair")
    op.order_buffer = order_buffer(M, N)
    a, b = _operands(world, M, N, K, torch.bfloat16, seed=5)
    op(a, b)
    g.check_status()
    rec = tile_order(op.order_buffer)
    tiles = (M // 256) * (N // 256)
    assert sorted(r["unit"] for r in rec) == list(range(2 * tiles))
    want = sum(a[r].float() @ b[r].float().t() for r in range(world))
    assert (op.output(0).float() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
    g.close()


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("world,blocks,N", [(2, 2, 1024), (4, 2, 1024), (4, 1, 8192), (2, 3, 2560), (8, 1, 512)])
@pytest.mark.parametrize("with_norm", [True, False])
def test_gemm_reduce_scatter_residual_rmsnorm(world, blocks, N, with_norm, kernel):
    from ooverlap_b200 import EmulatedGroup
    from ooverlap_b200.ops import GemmReduceScatterNorm
    dtype, eps = torch.bfloat16, 1e-6
    M, K = 128 * world * blocks, 256
    g = EmulatedGroup(world, heap_bytes=96 << 20)
    op = GemmReduceScatterNorm(g, M, N, dtype, eps=eps, comm_ctas=3, kernel=kernel)
    a, b = _operands(world, M, N, K, dtype, seed=7)
    rows = M // world
    residual = torch.randn(world, rows, N, device="cuda").to(dtype)
    w = (1 + 0.02 * torch.randn(N, device="cuda")).to(dtype) if with_norm else None
    s = sum(a[r].float() @ b[r].float().t() for r in range(world))
    s = (s + residual.reshape(M, N).float()).to(dtype).float()
    want = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * w.float() if with_norm else s
    for it in range(2):
        y, ro = op(a, b, w, residual)
        g.check_status()
        assert (ro.reshape(M, N).float() - s).abs().max().item() <= 3e-2 * max(1.0, s.abs().max().item())
        assert (y.reshape(M, N).float() - want).abs().max().item() <= 6e-2 * max(1.0, want.abs().max().item())
    g.close()


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("world,blocks", [(2, 2), (4, 2), (4, 3), (8, 1)])
def test_all_gather_gemm(world, blocks, kernel):
    from ooverlap_b200 import EmulatedGroup
    from ooverlap_b200.ops import AllGatherGemm
    dtype = torch.bfloat16
    M, N, K = 128 * world * blocks, 520, 320
    g = EmulatedGroup(world, heap_bytes=64 << 20)
    op = AllGatherGemm(g, M, K, dtype, comm_ctas=3, kernel=kernel)
    gen = torch.Generator(device="cuda").manual_seed(3)
    a_full = torch.randn(M, K, device="cuda", generator=gen).to(dtype)
    a_shards = a_full.view(world, M // world, K).contiguous()
    b = (torch.randn(world, N, K, device="cuda", generator=gen) / K ** 0.5).to(dtype)  # each rank its own columns
    for it in range(2):
        out = op(a_shards, b)
        g.check_status()
        for r in range(world):
            want = a_full.float() @ b[r].float().t()
            assert (out[r].float() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item()), (it, r)
    g.close()


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("world", [2, 4])
def test_fused_ops_leave_every_arrival_counter_re_armed(world, kernel):
    """After each fused op (all three kinds, odd and even tile counts) every general counter of every rank's signal
    pad reads zero again: tile arrivals, row-block arrivals, chunk flags and tickets are all re-armed in-kernel."""
    from ooverlap_b200 import EmulatedGroup
    from ooverlap_b200.ops import AllGatherGemm, GemmAllReduce, GemmReduceScatterNorm
    dtype = torch.bfloat16
    g = EmulatedGroup(world, heap_bytes=96 << 20)
    for r in range(world):
        assert int(g.counters(r).abs().max()) == 0
    M, N, K = 128 * world * 2, 768, 256  # 3 column tiles: an odd number of tiles per rank for world = 2
    a, b = _operands(world, M, N, K, dtype, seed=3)
    ar = GemmAllReduce(g, M, N, dtype, comm_ctas=3, kernel=kernel)
    rs = GemmReduceScatterNorm(g, M, N, dtype, eps=1e-6, comm_ctas=2, kernel=kernel)
    ag = AllGatherGemm(g, M, K, dtype, comm_ctas=2, kernel=kernel)
    residual = torch.randn(world, M // world, N, device="cuda").to(dtype)
    a_shards = a[0].reshape(world, M // world, K).contiguous()
    for it in range(2):
        for op in (lambda: ar(a, b), lambda: rs(a, b, None, residual), lambda: ag(a_shards, b)):
            op()
            g.check_status()
            torch.cuda.synchronize()
            for r in range(world):
                c = g.counters(r)
                nz = torch.nonzero(c).flatten().tolist()
                assert not nz, (it, r, nz[:8], c[nz[:8]].tolist())
    g.close()
