"""CUDA-core streaming GEMM for one to four rows against a plain PyTorch fp32 reference and against the
tensor-core path."""
import pytest
import torch

pytestmark = [pytest.mark.gpu]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 1280, 8192), (1, 8192, 1024), (1, 7168, 8192), (2, 8192, 3584), (3, 1000, 1096),
                                   (4, 16032, 8192), (1, 7, 8), (4, 257, 72)])
def test_gemv(shape, dtype):
    from ooverlap_b200.ops import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    c1 = gemm(a, b, gemv=1)
    c2 = gemm(a, b, gemv=1)
    c_tc = gemm(a, b, gemv=-1)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    scale = max(1.0, ref.abs().max().item())
    assert (c1.float() - ref).abs().max().item() <= 1e-2 * scale, (shape, dtype)
    assert torch.equal(c1, c2)
    assert (c1.float() - c_tc.float()).abs().max().item() <= 2e-2 * scale


def test_gemv_strided_operands_and_graph_replay():
    from ooverlap_b200.ops import gemm
    a_full = torch.randn(2, 1024 + 64, device="cuda").bfloat16()
    a = a_full[:, :1024]
    b = torch.randn(264, 1024, device="cuda").bfloat16()
    big = torch.zeros(2, 300, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=big[:, :264], gemv=1)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    assert (big[:, :264].float() - ref).abs().max().item() < 0.5
    assert big[:, 264:].abs().max().item() == 0
    out = torch.empty(2, 264, device="cuda", dtype=torch.bfloat16)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gemm(a, b, out=out, gemv=1)
    for _ in range(3):
        a_full.normal_()
        graph.replay()
        torch.cuda.synchronize()
        assert (out.float() - a.float() @ b.float().t()).abs().max().item() < 0.5
