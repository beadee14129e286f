"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().t()


def _check(M, N, K, dtype, lda_pad=0):
    from ooverlap_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(M * 131 + N * 17 + K)
    a_full = torch.randn(M, K + lda_pad, device="cuda", generator=g).to(dtype)
    a = a_full[:, :K]
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    c = gemm(a, b)
    torch.cuda.synchronize()
    ref = _ref(a, b)
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * max(1.0, scale), (M, N, K, dtype, err, scale)
    return c


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 256, 64), (128, 256, 512), (256, 512, 1024), (1024, 2048, 4096)])
def test_exact_tiles(shape, dtype):
    _check(*shape, dtype)


@pytest.mark.parametrize("shape", [(1, 256, 64), (100, 200, 72), (129, 257 * 8, 8), (300, 1000, 1096), (5000, 264, 200)])
def test_ragged_shapes(shape):
    _check(*shape, torch.bfloat16)


def test_padded_leading_dimension_and_out():
    from ooverlap_b200.ops import gemm
    _check(256, 512, 256, torch.bfloat16, lda_pad=64)
    a = torch.randn(200, 128, device="cuda").bfloat16()
    b = torch.randn(96, 128, device="cuda").bfloat16()
    big = torch.zeros(200, 128, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, out=big[:, :96])
    assert out.data_ptr() == big.data_ptr()
    torch.cuda.synchronize()
    assert (big[:, :96].float() - _ref(a, b)).abs().max().item() < 0.5
    assert big[:, 96:].abs().max().item() == 0  # nothing written past N


def test_many_tiles_per_cta_and_repeatability():
    # 4096 x 4096 output = 512 tiles on 148 CTAs: exercises the TMEM double buffering and the smem ring wrap.
    c1 = _check(4096, 4096, 1024, torch.bfloat16)
    c2 = _check(4096, 4096, 1024, torch.bfloat16)
    assert torch.equal(c1, c2)


def test_cta_budget():
    from ooverlap_b200.ops import gemm
    a = torch.randn(1024, 512, device="cuda").bfloat16()
    b = torch.randn(1024, 512, device="cuda").bfloat16()
    c_full = gemm(a, b, splits=1)  # same K order in both runs, so the bits must agree
    c_few = gemm(a, b, max_ctas=7, splits=1)
    torch.cuda.synchronize()
    assert torch.equal(c_full, c_few)


@pytest.mark.parametrize("shape", [(16, 8192, 1024), (128, 2048, 4096), (200, 520, 1032), (1, 256, 512)])
@pytest.mark.parametrize("splits", [0, 2, 4, 8])
def test_split_k(shape, splits):
    """K split over several CTAs per tile (fp32 partials in the library workspace, summed in split order)."""
    from ooverlap_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(K + splits)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    ref = _ref(a, b)
    c1 = gemm(a, b, splits=splits)
    c2 = gemm(a, b, splits=splits)  # counters re-armed by the first call
    torch.cuda.synchronize()
    assert (c1.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())
    assert torch.equal(c1, c2)
    # shapes of different size share (and regrow) the workspace
    a2 = torch.randn(64, 2048, device="cuda", generator=g).half()
    b2 = (torch.randn(4096, 2048, device="cuda", generator=g) / 45).half()
    c3 = gemm(a2, b2, splits=4)
    torch.cuda.synchronize()
    assert (c3.float() - _ref(a2, b2)).abs().max().item() <= 2e-2


def test_rejects_bad_operands():
    from ooverlap_b200 import OobError
    from ooverlap_b200.ops import gemm
    a = torch.randn(64, 60, device="cuda").bfloat16()  # K % 8 != 0
    b = torch.randn(64, 60, device="cuda").bfloat16()
    with pytest.raises(OobError):
        gemm(a, b)
    with pytest.raises(TypeError):
        gemm(a.float(), b.float())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(256, 256, 64), (256, 512, 1024), (384, 512, 256), (129, 264, 136), (1000, 200, 72),
                                   (2048, 2048, 2048), (4096, 4096, 1024)])
def test_two_sm_kernel(shape, dtype):
    """256x256 tiles on CTA pairs (tcgen05.mma.cta_group::2) against fp32, and bit-equal to the one-SM kernel: both
    accumulate the K blocks of a tile in the same order in fp32."""
    from ooverlap_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    c_pair = gemm(a, b, splits=1, pair=1, stream_k=-1)
    c_pair2 = gemm(a, b, splits=1, pair=1, stream_k=-1)
    c_one = gemm(a, b, splits=1, pair=-1)
    torch.cuda.synchronize()
    ref = _ref(a, b)
    err = (c_pair.float() - ref).abs().max().item()
    assert err <= 1e-2 * max(1.0, ref.abs().max().item()), (shape, dtype, err)
    assert torch.equal(c_pair, c_pair2)
    assert torch.equal(c_pair, c_one)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,max_ctas", [((512, 8192, 8192), 0), ((2048, 8192, 4096), 0), ((2048, 2048, 2048), 0),
                                            ((1280, 1536, 1024), 0), ((1000, 520, 1096), 0), ((4096, 3584, 2048), 0),
                                            ((768, 768, 4096), 10), ((2304, 1280, 2048), 14), ((256, 512, 8192), 0)])
def test_two_sm_kernel_stream_k_tail(shape, max_ctas, dtype):
    """Stream-K tail of the two-SM kernel: pairs that compute part of a tile park fp32 accumulators in the workspace
    and the last arrival sums them in pair order.  Against fp32; bit-identical from call to call (the order of
    addition is fixed); close to the result without a tail (which adds the same products in a different grouping);
    and calls back to back re-use the workspace flags (they are re-armed in the kernel)."""
    from ooverlap_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    outs = [gemm(a, b, splits=1, pair=1, stream_k=1, max_ctas=max_ctas) for _ in range(3)]
    c_whole = gemm(a, b, splits=1, pair=1, stream_k=-1, max_ctas=max_ctas)
    c_auto = gemm(a, b, max_ctas=max_ctas)
    torch.cuda.synchronize()
    ref = _ref(a, b)
    tol = 1e-2 * max(1.0, ref.abs().max().item())
    assert (outs[0].float() - ref).abs().max().item() <= tol, (shape, dtype)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert (outs[0].float() - c_whole.float()).abs().max().item() <= tol
    assert (c_auto.float() - ref).abs().max().item() <= tol


def test_two_sm_kernel_stream_k_graph_replay_and_reserved_workspace():
    """The stream-K workspace is allocated once per device and never moves: a captured launch stays valid when other
    shapes run in between.  reserve_workspace() makes the allocation happen before the capture."""
    from ooverlap_b200.ops import gemm, reserve_workspace
    reserve_workspace()
    a = torch.randn(512, 2048, device="cuda").bfloat16()
    b = (torch.randn(4096, 2048, device="cuda") / 45.0).bfloat16()
    out = torch.empty(512, 4096, device="cuda", dtype=torch.bfloat16)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gemm(a, b, out=out, splits=1, pair=1, stream_k=1)
    for i in range(3):
        a.normal_()
        other = torch.randn(2048, 1024, device="cuda").bfloat16()
        gemm(other, torch.randn(1536, 1024, device="cuda").bfloat16(), splits=1, pair=1, stream_k=1)
        graph.replay()
        torch.cuda.synchronize()
        ref = _ref(a, b)
        assert (out.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item()), i


def test_split_k_workspace_survives_growth_under_a_captured_graph():
    """A captured split-K GEMM keeps launching with the workspace it was captured with: a later, larger problem gets
    a new block and the old one stays alive.  Growing during capture is refused with a clear error; reserving first
    makes the same capture work."""
    from ooverlap_b200._lib import OobError
    from ooverlap_b200.ops import gemm, reserve_workspace, splitk_workspace_bytes
    a = torch.randn(64, 2048, device="cuda").bfloat16()
    b = (torch.randn(1024, 2048, device="cuda") / 45.0).bfloat16()
    out = torch.empty(64, 1024, device="cuda", dtype=torch.bfloat16)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        gemm(a, b, out=out, splits=4, skinny=-1)  # first use: the workspace exists before the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            gemm(a, b, out=out, splits=4, skinny=-1)
        # a larger split problem on the same stream grows the workspace
        a2 = torch.randn(128, 4096, device="cuda").bfloat16()
        b2 = (torch.randn(8192, 4096, device="cuda") / 64.0).bfloat16()
        c2 = gemm(a2, b2, splits=8, skinny=-1)
        for _ in range(2):
            a.normal_()
            graph.replay()
            s.synchronize()
            assert (out.float() - _ref(a, b)).abs().max().item() <= 1e-2 * max(1.0, _ref(a, b).abs().max().item())
        assert (c2.float() - _ref(a2, b2)).abs().max().item() <= 1e-2 * max(1.0, _ref(a2, b2).abs().max().item())
    # growth during capture: refused, and the capture can be redone after a reservation
    s2 = torch.cuda.Stream()
    a3 = torch.randn(128, 8192, device="cuda").bfloat16()
    b3 = (torch.randn(16384, 8192, device="cuda") / 90.0).bfloat16()
    out3 = torch.empty(128, 16384, device="cuda", dtype=torch.bfloat16)
    need = splitk_workspace_bytes(128, 16384, 8192, splits=16)  # 128 MiB of partial tiles: more than any test before
    assert need > (128 << 20)
    with torch.cuda.stream(s2):
        g2 = torch.cuda.CUDAGraph()
        failed = False
        try:
            with torch.cuda.graph(g2, stream=s2):
                gemm(a3, b3, out=out3, splits=16, skinny=-1)
        except OobError as e:
            failed = True
            assert "oob_gemm_reserve_workspace" in str(e)
        assert failed
    torch.cuda.synchronize()
    reserve_workspace(need)
    with torch.cuda.stream(s2):
        g3 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g3, stream=s2):
            gemm(a3, b3, out=out3, splits=16, skinny=-1)
        g3.replay()
        s2.synchronize()
    assert (out3.float() - _ref(a3, b3)).abs().max().item() <= 1e-2 * max(1.0, _ref(a3, b3).abs().max().item())


def test_two_sm_kernel_cta_budget_and_padded_output():
    from ooverlap_b200.ops import gemm
    a = torch.randn(1024, 512, device="cuda").bfloat16()
    b = torch.randn(1024, 512, device="cuda").bfloat16()
    c_full = gemm(a, b, splits=1, pair=1)
    c_few = gemm(a, b, splits=1, pair=1, max_ctas=6)
    big = torch.zeros(1024, 1280, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=big[:, :1024], splits=1, pair=1)
    torch.cuda.synchronize()
    assert torch.equal(c_full, c_few)
    assert torch.equal(big[:, :1024], c_full)
    assert big[:, 1024:].abs().max().item() == 0


def test_two_sm_kernel_tile_order_record():
    """Every 128-row half of every 256x256 tile reports when it was stored, by which pair and as which of the pair's
    tiles; within a pair the completion times follow the pair's own sequence."""
    from ooverlap_b200.ops import gemm, order_buffer, tile_order
    M, N, K = 2048, 4096, 512
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    order = order_buffer(M, N)
    c = gemm(a, b, splits=1, pair=1, stream_k=-1, max_ctas=32, order=order)
    torch.cuda.synchronize()
    assert torch.equal(c, gemm(a, b, splits=1, pair=1, stream_k=-1))
    rec = tile_order(order)
    tiles = (M // 256) * (N // 256)
    assert len(rec) == 2 * tiles and sorted(r["unit"] for r in rec) == list(range(2 * tiles))
    assert {r["pair"] for r in rec} == set(range(16))  # 32 CTAs = 16 pairs, all of them got tiles
    per_pair = {}
    for r in rec:  # rec is sorted by time
        per_pair.setdefault(r["pair"], []).append(r["index"])
    for pair, idx in per_pair.items():
        assert len(idx) == 2 * tiles // 16
        assert idx == sorted(idx), (pair, idx)
    assert rec[-1]["t_us"] > rec[0]["t_us"]
    with pytest.raises(ValueError):
        gemm(a, b, order=torch.zeros(4, 2, dtype=torch.int64, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 256, 64), (1, 1280, 8192), (7, 7168, 8192), (16, 8192, 1024), (64, 8192, 3584),
                                   (100, 200, 72), (128, 2048, 4096), (33, 1000, 1096), (17, 16032, 2048)])
def test_weight_streaming_kernel(shape, dtype):
    """M <= 128: weight rows on the instruction's 128-row dimension, stream-K split, fp32 partials summed in CTA
    order -- against fp32, and bit-identical from call to call and for any CTA budget that splits K the same way."""
    from ooverlap_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    c1 = gemm(a, b, skinny=1)
    c2 = gemm(a, b, skinny=1)
    c_auto = gemm(a, b)  # the default route: split-K tiles + reduction kernel
    torch.cuda.synchronize()
    ref = _ref(a, b)
    err = (c1.float() - ref).abs().max().item()
    assert err <= 1e-2 * max(1.0, ref.abs().max().item()), (shape, dtype, err)
    assert torch.equal(c1, c2)
    assert (c_auto.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())
    # a small CTA budget changes the split, not the result beyond rounding of the partial sums
    c_few = gemm(a, b, skinny=1, max_ctas=5)
    torch.cuda.synchronize()
    assert (c_few.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())


def test_weight_streaming_kernel_strided_output_and_graph_replay():
    from ooverlap_b200.ops import gemm
    a = torch.randn(5, 512, device="cuda").bfloat16()
    b = torch.randn(264, 512, device="cuda").bfloat16()
    big = torch.zeros(5, 300, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=big[:, :264], skinny=1)
    torch.cuda.synchronize()
    assert (big[:, :264].float() - _ref(a, b)).abs().max().item() < 0.5
    assert big[:, 264:].abs().max().item() == 0
    out = torch.empty(5, 264, device="cuda", dtype=torch.bfloat16)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gemm(a, b, out=out, skinny=1)
    for _ in range(3):
        a.normal_()
        graph.replay()
        torch.cuda.synchronize()
        assert (out.float() - _ref(a, b)).abs().max().item() < 0.5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,splits", [((64, 7168, 8192), 0), ((64, 8192, 3584), 0), ((128, 2048, 4096), 4),
                                          ((200, 520, 1032), 2), ((256, 7168, 2048), 0), ((33, 264, 520), 8),
                                          ((5, 1000, 1096), 3)])
def test_split_k_reduction_kernel_matches_in_kernel_sum(shape, splits, dtype):
    """The sum over the K splits taken by a second kernel equals, bit for bit, the sum taken inside the GEMM kernel
    (same order of addition), and both agree with fp32."""
    from ooverlap_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K + splits)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    c_two = gemm(a, b, splits=splits, skinny=-1, splitk_reduce=1)
    c_in = gemm(a, b, splits=splits, skinny=-1, splitk_reduce=-1)
    c_two2 = gemm(a, b, splits=splits, skinny=-1, splitk_reduce=1)
    torch.cuda.synchronize()
    ref = _ref(a, b)
    assert (c_two.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())
    assert torch.equal(c_two, c_in)
    assert torch.equal(c_two, c_two2)
