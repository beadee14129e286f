"""Epilogues applied by the kernel that sums the K splits of a GEMM (SwiGLU; RoPE + KV-cache write), against plain
PyTorch fp32 references and against the unfused pair of kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,F,K", [(1, 3584, 8192), (16, 3584, 8192), (64, 1024, 2048), (200, 520, 1032), (256, 3584, 1024)])
def test_gemm_swiglu(M, F, K, dtype):
    from ooverlap_b200.ops import gemm_plan_splits, gemm_swiglu
    g = torch.Generator(device="cuda").manual_seed(M + F + K)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(2 * F, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    assert gemm_plan_splits(M, 2 * F, K) > 1
    fused = gemm_swiglu(x, w, fused=True)
    unfused = gemm_swiglu(x, w, fused=False)
    torch.cuda.synchronize()
    gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-3
    scale = max(1.0, ref.abs().max().item())
    assert (fused.float() - ref).abs().max().item() <= tol * scale
    # the unfused pair rounds the [M, 2F] intermediate to 16 bits first: close, not identical
    assert (fused.float() - unfused.float()).abs().max().item() <= 2 * tol * scale


def test_gemm_swiglu_falls_back_when_not_split():
    from ooverlap_b200.ops import gemm_plan_splits, gemm_swiglu
    M, F, K = 2048, 2048, 512  # 256 tiles: more than the SMs, so the problem is not split
    assert gemm_plan_splits(M, 2 * F, K) == 1
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(2 * F, K, device="cuda") / K ** 0.5).bfloat16()
    out = gemm_swiglu(x, w)
    torch.cuda.synchronize()
    gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    with pytest.raises(ValueError):
        gemm_swiglu(x, w, fused=True)


def _rope_ref(x, cos, sin):
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,T,H,KV,hd,K,pos,dev_pos", [(2, 1, 8, 1, 128, 8192, 37, True), (64, 1, 8, 1, 128, 8192, 5, True),
                                                        (3, 4, 4, 2, 64, 1024, 9, False)])
def test_gemm_rope_kv_write(B, T, H, KV, hd, K, pos, dev_pos, dtype):
    from ooverlap_b200.ops import gemm_plan_splits, gemm_rope_kv_write, rope_tables
    max_len, batch0 = 96, 1
    N = (H + 2 * KV) * hd
    assert gemm_plan_splits(B * T, N, K) > 1
    g = torch.Generator(device="cuda").manual_seed(B * 100 + T)
    x = torch.randn(B * T, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    kc = torch.full((B + 2, KV, max_len, hd), 7.0, device="cuda", dtype=dtype)
    vc = torch.full_like(kc, -3.0)
    kc2, vc2 = kc.clone(), vc.clone()
    cos, sin = rope_tables(max_len, hd, 10000.0, x.device)
    p = torch.full((1,), pos, dtype=torch.long, device="cuda") if dev_pos else pos
    q = gemm_rope_kv_write(x, w, B, T, H, KV, kc, vc, cos, sin, p, batch0=batch0, fused=True)
    q2 = gemm_rope_kv_write(x, w, B, T, H, KV, kc2, vc2, cos, sin, p, batch0=batch0, fused=False)
    torch.cuda.synchronize()
    qkv = (x.float() @ w.float().t()).view(B, T, H + 2 * KV, hd)
    c, s = cos[pos:pos + T][None, :, None, :], sin[pos:pos + T][None, :, None, :]
    q_ref = _rope_ref(qkv[:, :, :H], c, s).reshape(B * T, H * hd)
    k_ref = _rope_ref(qkv[:, :, H:H + KV], c, s).transpose(1, 2)
    v_ref = qkv[:, :, H + KV:].transpose(1, 2)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    for got, ref in ((q.float(), q_ref), (kc[batch0:batch0 + B, :, pos:pos + T].float(), k_ref),
                     (vc[batch0:batch0 + B, :, pos:pos + T].float(), v_ref)):
        assert (got - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    assert (q.float() - q2.float()).abs().max().item() <= 2 * tol * max(1.0, q_ref.abs().max().item())
    untouched = torch.ones_like(kc, dtype=torch.bool)
    untouched[batch0:batch0 + B, :, pos:pos + T] = False
    assert (kc[untouched] == 7.0).all() and (vc[untouched] == -3.0).all()


def test_model_with_fused_epilogues_matches_unfused(monkeypatch):
    from ooverlap_b200.models import TINY128, LlamaTP
    prompts = torch.randint(0, TINY128.vocab, (3, 40), device="cuda")
    monkeypatch.setenv("OOB_FUSED_EPILOGUES", "0")
    plain = LlamaTP(TINY128, None, backend="ours", max_batch=3, max_len=96, seed=5)
    monkeypatch.setenv("OOB_FUSED_EPILOGUES", "1")
    fused = LlamaTP(TINY128, None, backend="ours", max_batch=3, max_len=96, seed=5)
    assert fused.fused_epilogues and not plain.fused_epilogues
    nxt = torch.randint(0, TINY128.vocab, (3, 1), device="cuda")
    pos = torch.full((1,), 40, dtype=torch.long, device="cuda")
    with torch.no_grad():
        p1, p2 = plain.forward(prompts, 0), fused.forward(prompts, 0)
        d1, d2 = plain.forward(nxt, pos), fused.forward(nxt, pos)
    cosf = torch.nn.functional.cosine_similarity
    assert cosf(p1.float(), p2.float(), dim=-1).min().item() > 0.998
    assert cosf(d1.float(), d2.float(), dim=-1).min().item() > 0.998
    t_graph = fused.generate(prompts, 8, use_graph=True)
    t_eager = fused.generate(prompts, 8, use_graph=False)
    assert torch.equal(t_graph, t_eager)
