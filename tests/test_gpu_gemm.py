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
    c_pair = gemm(a, b, splits=1, pair=1)
    c_pair2 = gemm(a, b, splits=1, pair=1)
    c_one = gemm(a, b, splits=1, pair=-1)
    torch.cuda.synchronize()
    ref = _ref(a, b)
    err = (c_pair.float() - ref).abs().max().item()
    assert err <= 1e-2 * max(1.0, ref.abs().max().item()), (shape, dtype, err)
    assert torch.equal(c_pair, c_pair2)
    assert torch.equal(c_pair, c_one)


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
