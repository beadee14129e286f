"""The model runner's glue (which op is called with what, cache bookkeeping, the fused-epilogue switch) checked on
the CPU: this library's kernels are replaced by plain PyTorch functions with the same contracts, and the model is
compared with its own PyTorch arm."""
import math

import pytest
import torch

from ooverlap_b200.models import llama as L
from ooverlap_b200.ops.decode import attn_decode_reference


def _gemm(a, b, out=None, **kw):
    c = (a.float() @ b.float().t()).to(a.dtype)
    if out is not None:
        out.copy_(c)
        return out
    return c


def _rmsnorm(x, w, eps=1e-6, residual=None, **kw):
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)
    return (y, xf.to(x.dtype)) if residual is not None else y


def _rope_kv_write(qkv, B, T, H, KV, kc, vc, cos, sin, pos, *, batch0=0, q_out=None):
    hd = qkv.shape[1] // (H + 2 * KV)
    p0 = int(pos.item()) if isinstance(pos, torch.Tensor) else int(pos)
    x = qkv.float().view(B, T, H + 2 * KV, hd)
    c, s = cos[p0:p0 + T][None, :, None, :], sin[p0:p0 + T][None, :, None, :]

    def rot(v):
        v1, v2 = v[..., 0::2], v[..., 1::2]
        return torch.stack((v1 * c - v2 * s, v1 * s + v2 * c), dim=-1).flatten(-2)

    kc[batch0:batch0 + B, :, p0:p0 + T] = rot(x[:, :, H:H + KV]).transpose(1, 2).to(qkv.dtype)
    vc[batch0:batch0 + B, :, p0:p0 + T] = x[:, :, H + KV:].transpose(1, 2).to(qkv.dtype)
    return rot(x[:, :, :H]).reshape(B * T, H * hd).to(qkv.dtype)


def _attn_decode(q, kc, vc, pos, *, batch0=0, **kw):
    p = int(pos.item()) if isinstance(pos, torch.Tensor) else int(pos)
    return attn_decode_reference(q, kc, vc, p, batch0=batch0).to(q.dtype)


def _silu_mul(gu, out=None):
    F = gu.shape[1] // 2
    return (torch.nn.functional.silu(gu[:, :F].float()) * gu[:, F:].float()).to(gu.dtype)


def _gemm_swiglu(a, b, out=None, **kw):
    return _silu_mul(_gemm(a, b))


def _gemm_rope_kv_write(x, w, B, T, H, KV, kc, vc, cos, sin, pos, *, batch0=0, q_out=None, fused=None):
    return _rope_kv_write(_gemm(x, w), B, T, H, KV, kc, vc, cos, sin, pos, batch0=batch0)


@pytest.fixture
def cpu_kernels(monkeypatch):
    for name, fn in (("gemm", _gemm), ("rmsnorm", _rmsnorm), ("rope_kv_write", _rope_kv_write), ("attn_decode", _attn_decode),
                     ("silu_mul", _silu_mul), ("gemm_swiglu", _gemm_swiglu), ("gemm_rope_kv_write", _gemm_rope_kv_write)):
        monkeypatch.setattr(L, name, fn)


@pytest.mark.parametrize("cfg_name,fused", [("TINY128", "0"), ("TINY128", "1"), ("TINY", "0")])
def test_model_glue_matches_the_pytorch_arm(cpu_kernels, monkeypatch, cfg_name, fused):
    monkeypatch.setenv("OOB_FUSED_EPILOGUES", fused)
    cfg = getattr(L, cfg_name)
    dev = torch.device("cpu")
    ours = L.LlamaTP(cfg, None, backend="ours", max_batch=3, max_len=48, seed=5, device=dev, dtype=torch.float32)
    ref = L.LlamaTP(cfg, None, backend="nccl", max_batch=3, max_len=48, seed=5, device=dev, dtype=torch.float32)
    assert ours.fused_epilogues == (fused == "1")
    prompts = torch.randint(0, cfg.vocab, (2, 20), generator=torch.Generator().manual_seed(0))
    nxt = torch.randint(0, cfg.vocab, (2, 1), generator=torch.Generator().manual_seed(1))
    pos = torch.full((1,), 20, dtype=torch.long)
    mask = torch.full((1, 1, 1, 48), float("-inf"))
    mask[..., :21] = 0
    with torch.no_grad():
        p1, p2 = ours.forward(prompts, 0, batch0=1), ref.forward(prompts, 0, batch0=1)
        d1, d2 = ours.forward(nxt, pos, attn_mask=mask, batch0=1), ref.forward(nxt, pos, attn_mask=mask, batch0=1)
    assert torch.allclose(p1, p2, atol=2e-4, rtol=1e-3)
    assert torch.allclose(d1, d2, atol=2e-4, rtol=1e-3)
    # both arms filled the same cache slots (sequences 1..2, positions 0..20) and nothing else
    assert torch.allclose(ours.k_cache, ref.k_cache, atol=1e-4) and torch.allclose(ours.v_cache, ref.v_cache, atol=1e-5)
    assert ours.k_cache[:, 0].abs().max() == 0 and ours.k_cache[:, 1:, :, 21:].abs().max() == 0


def test_generate_glue_matches_the_pytorch_arm(cpu_kernels, monkeypatch):
    """Prefill in batch slices + eager decode loop: same greedy tokens from both arms (fp32, no graphs on the CPU)."""
    monkeypatch.setenv("OOB_FUSED_EPILOGUES", "1")
    cfg = L.TINY128
    dev = torch.device("cpu")
    ours = L.LlamaTP(cfg, None, backend="ours", max_batch=3, max_len=40, seed=7, device=dev, dtype=torch.float32)
    ref = L.LlamaTP(cfg, None, backend="nccl", max_batch=3, max_len=40, seed=7, device=dev, dtype=torch.float32)
    prompts = torch.randint(0, cfg.vocab, (3, 12), generator=torch.Generator().manual_seed(3))
    t1 = ours.generate(prompts, 6, prefill_chunk_tokens=24, use_graph=False)  # two sequences per prefill slice
    t2 = ref.generate(prompts, 6, prefill_chunk_tokens=24, use_graph=False)
    assert t1.shape == (3, 6) and torch.equal(t1, t2)
