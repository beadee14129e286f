"""Llama-architecture tensor-parallel decoder for the serving benchmark (random-init weights).

Every linear layer is this library's tcgen05 GEMM; each transformer layer has two row-parallel projections
(``o_proj`` and ``down_proj``) whose all-reduce is fused with the residual add and the following RMSNorm, i.e. 160
all-reduces per token step for the 80-layer 70B configuration.  A decode step of a layer is nine kernels of this
library: QKV GEMM, RoPE + KV-cache write, grouped-query decode attention over the static cache (head size 128),
output GEMM, all-reduce + residual + RMSNorm, gate/up GEMM, SwiGLU, down GEMM, all-reduce + residual + RMSNorm.
Prefill attention uses PyTorch's causal ``scaled_dot_product_attention`` (the reference has no attention kernels;
it only replaces the tensor-parallel communication of a served model).  The decode step has static shapes (the
position is a device tensor) and is replayed from one CUDA graph.

``backend="nccl"`` runs the same model with ``torch.mm`` (cuBLAS) + ``torch.distributed.all_reduce`` (NCCL) +
PyTorch RMSNorm: the comparison arm of the serving benchmark.

Capability parity: the reference serves Qwen2.5 through vLLM with its all-reduce backend
(patches/vllm/v0.25.0/vllm/model_executor/models/qwen2.py, evalution/run_vllm_paperlike.sh:7-120).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import (attn_decode, fused_allreduce_rmsnorm, gemm, gemm_rope_kv_write, gemm_swiglu, rmsnorm, rope_kv_write,
                   rope_tables, silu_mul)
from ..utils.config import env_flag, env_int
from ..utils.tracing import nvtx_range


@dataclass
class LlamaConfig:
    layers: int = 80
    hidden: int = 8192
    heads: int = 64
    kv_heads: int = 8
    ffn: int = 28672
    vocab: int = 128256
    eps: float = 1e-5
    rope_theta: float = 500000.0
    head_size: int = 0  # 0 = hidden / heads

    @property
    def head_dim(self) -> int:
        return self.head_size or self.hidden // self.heads

    def shard(self, world: int, layers: int = 0) -> "LlamaConfig":
        """The configuration one rank of a ``world``-way tensor-parallel group computes (heads, KV heads, FFN and
        vocabulary divided, head size kept): lets one GPU run a rank's kernels at their real shapes, without the
        communication."""
        return LlamaConfig(layers=layers or self.layers, hidden=self.hidden, heads=self.heads // world,
                           kv_heads=max(1, self.kv_heads // world), ffn=self.ffn // world, vocab=self.vocab // world,
                           eps=self.eps, rope_theta=self.rope_theta, head_size=self.head_dim)


LLAMA3_70B = LlamaConfig()
LLAMA3_8B = LlamaConfig(layers=32, hidden=4096, heads=32, kv_heads=8, ffn=14336)
TINY = LlamaConfig(layers=2, hidden=512, heads=8, kv_heads=2, ffn=1024, vocab=1024)
TINY128 = LlamaConfig(layers=2, hidden=1024, heads=8, kv_heads=2, ffn=2048, vocab=1024)  # head size 128


def _apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x: [B, T, H, hd]; cos/sin: [T, hd/2]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1).flatten(-2)


class LlamaTP:
    """One rank of a tensor-parallel Llama decoder with a static KV cache."""

    def __init__(self, cfg: LlamaConfig, comm, *, rank: int = 0, world: int = 1, dtype=torch.bfloat16,
                 device: Optional[torch.device] = None, backend: str = "ours", max_batch: int = 1, max_len: int = 2048,
                 seed: int = 0, nccl_group=None):
        if cfg.heads % world or cfg.kv_heads % world or cfg.ffn % world or cfg.vocab % world:
            raise ValueError("heads, kv_heads, ffn and vocab must be divisible by the tensor-parallel size")
        if backend not in ("ours", "nccl"):
            raise ValueError(backend)
        self.cfg, self.comm, self.rank, self.world, self.dtype, self.backend = cfg, comm, rank, world, dtype, backend
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nccl_group = nccl_group
        self.h_local, self.kv_local = cfg.heads // world, cfg.kv_heads // world
        hd = cfg.head_dim
        g = torch.Generator(device=self.device).manual_seed(seed * 1000 + rank)      # sharded weights
        gn = torch.Generator(device=self.device).manual_seed(seed * 1000 + 999)      # replicated weights

        def w(rows, cols, fan_in):
            return (torch.randn(rows, cols, device=self.device, generator=g, dtype=torch.float32) / fan_in ** 0.5).to(dtype)

        def norm():
            return (1 + 0.02 * torch.randn(cfg.hidden, device=self.device, generator=gn)).to(dtype)

        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append({
                "wqkv": w((self.h_local + 2 * self.kv_local) * hd, cfg.hidden, cfg.hidden),
                "wo": w(cfg.hidden, self.h_local * hd, cfg.hidden),
                "wgu": w(2 * cfg.ffn // world, cfg.hidden, cfg.hidden),
                "wd": w(cfg.hidden, cfg.ffn // world, cfg.ffn),
                "norm1": norm(), "norm2": norm(),
            })
        self.final_norm = norm()
        self.embed = (torch.randn(cfg.vocab, cfg.hidden, device=self.device, generator=gn) * 0.02).to(dtype)
        self.lm_head = w(cfg.vocab // world, cfg.hidden, cfg.hidden)
        self.max_batch, self.max_len = max_batch, max_len
        self.k_cache = torch.zeros(cfg.layers, max_batch, self.kv_local, max_len, hd, device=self.device, dtype=dtype)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=self.device, dtype=torch.float32) / hd))
        ang = torch.arange(max_len, device=self.device, dtype=torch.float32).unsqueeze(-1) * inv
        self.rope_cos, self.rope_sin = ang.cos().to(dtype), ang.sin().to(dtype)  # [max_len, hd/2]
        if backend == "ours":
            self.rope_cos32, self.rope_sin32 = rope_tables(max_len, hd, cfg.rope_theta, self.device)
        # RoPE + cache write and SwiGLU applied by the kernel that sums the K splits of the preceding GEMM (two
        # launches fewer per layer in a decode step).  Off unless OOB_FUSED_EPILOGUES=1.
        self.fused_epilogues = backend == "ours" and env_flag("OOB_FUSED_EPILOGUES", False)
        # Prefill: row-parallel projections of at least OOB_PREFILL_CHUNK_MIN_ROWS tokens are computed in
        # OOB_PREFILL_CHUNKS slabs whose all-reduce + norm overlaps the next slab's GEMM (1 = off).
        self.prefill_chunks = max(1, env_int("OOB_PREFILL_CHUNKS", 1)) if backend == "ours" else 1
        self.prefill_chunk_min_rows = env_int("OOB_PREFILL_CHUNK_MIN_ROWS", 4096)
        self._side, self._joined, self._slab_events = None, None, []

    # ------------------------------------------------------------ primitives
    def _mm(self, x, wt):
        if self.backend == "ours":
            return gemm(x, wt)
        return torch.mm(x, wt.t())

    def _norm(self, x, wt):
        if self.backend == "ours":
            return rmsnorm(x, wt, self.cfg.eps)
        return F.rms_norm(x, (x.shape[-1],), wt, self.cfg.eps)

    def _row_parallel_norm(self, x, wt, residual, norm_w):
        """(rmsnorm(residual + all_reduce(x @ wt^T)) * norm_w, new residual)."""
        if self.backend == "ours":
            if self.world == 1:
                return rmsnorm(gemm(x, wt), norm_w, self.cfg.eps, residual)
            nbytes = x.shape[0] * wt.shape[0] * x.element_size()
            if nbytes <= self.comm.all_reduce_slot_capacity():
                slot = self.comm.commit_all_reduce_slot(self.comm.acquire_all_reduce_slot((x.shape[0], wt.shape[0])))
            else:  # prefill chunks larger than a slot: a cached registered scratch of that shape
                slot = self.comm.scratch_view(("rp", x.shape[0], wt.shape[0]), (x.shape[0], wt.shape[0]), x.dtype)
            chunks = self.prefill_chunks
            if chunks > 1 and x.shape[0] >= self.prefill_chunk_min_rows and x.shape[0] % chunks == 0:
                return self._row_parallel_norm_chunked(x, wt, residual, norm_w, slot, chunks)
            gemm(x, wt, out=slot)
            return fused_allreduce_rmsnorm(self.comm, slot, norm_w, self.cfg.eps, residual)
        part = torch.mm(x, wt.t())
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(part, group=self.nccl_group)
        h = part + residual
        return F.rms_norm(h, (h.shape[-1],), norm_w, self.cfg.eps), h

    def _row_parallel_norm_chunked(self, x, wt, residual, norm_w, slot, chunks):
        """Prefill-sized inputs: the rows are cut into slabs; the GEMM of slab i runs on the caller's stream while
        the all-reduce + residual + RMSNorm of slab i - 1 runs on a side stream (a handful of CTAs next to the
        GEMM's), so that only the first GEMM slab and the last all-reduce are exposed."""
        if self._side is None:
            self._side = torch.cuda.Stream()
            self._joined = torch.cuda.Event()
        while len(self._slab_events) < chunks:
            self._slab_events.append(torch.cuda.Event())
        main = torch.cuda.current_stream()
        rows = x.shape[0] // chunks
        # Outputs in registered memory (the two-shot all-reduce + norm broadcasts into them); one pair per shape,
        # reused by the next projection of the same shape exactly as the unchunked path reuses its scratch.
        shape = (x.shape[0], wt.shape[0])
        y = self.comm.scratch_view(("rp_y",) + shape, shape, x.dtype)
        h = self.comm.scratch_view(("rp_h",) + shape, shape, x.dtype)
        for i in range(chunks):
            sl = slice(i * rows, (i + 1) * rows)
            gemm(x[sl], wt, out=slot[sl])
            self._slab_events[i].record(main)
            self._side.wait_event(self._slab_events[i])
            with torch.cuda.stream(self._side):
                ys, hs = fused_allreduce_rmsnorm(self.comm, slot[sl], norm_w, self.cfg.eps, residual[sl], out=y[sl],
                                                 residual_out=h[sl])
                if ys.data_ptr() != y[sl].data_ptr():  # small slabs take the one-shot form with its own outputs
                    y[sl].copy_(ys)
                    h[sl].copy_(hs)
        self._joined.record(self._side)
        main.wait_event(self._joined)
        return y, h

    # --------------------------------------------------------------- forward
    def forward(self, tokens: torch.Tensor, pos, attn_mask: Optional[torch.Tensor] = None, batch0: int = 0):
        """tokens: [B, T].  Prefill: ``pos`` is the int start position (0) and attention is causal over the chunk.
        Decode: T == 1, ``pos`` is a device LongTensor of shape [1] and ``attn_mask`` masks the unused tail of
        the static cache.  Returns the normalised final hidden state [B*T, hidden]."""
        cfg, hd = self.cfg, self.cfg.head_dim
        B, T = tokens.shape
        decode = isinstance(pos, torch.Tensor)
        ours = self.backend == "ours"
        if not ours:
            if decode:
                cos, sin = self.rope_cos.index_select(0, pos), self.rope_sin.index_select(0, pos)
            else:
                cos, sin = self.rope_cos[pos:pos + T], self.rope_sin[pos:pos + T]
        h = self.embed[tokens.reshape(-1)]  # [B*T, hidden]  residual stream
        x = self._norm(h, self.layers[0]["norm1"])
        sl = slice(batch0, batch0 + B)
        for li, layer in enumerate(self.layers):
            with nvtx_range("layer"):
                if ours and self.fused_epilogues:
                    kc, vc = self.k_cache[li], self.v_cache[li]
                    q = gemm_rope_kv_write(x, layer["wqkv"], B, T, self.h_local, self.kv_local, kc, vc, self.rope_cos32,
                                           self.rope_sin32, pos, batch0=batch0)
                else:
                    qkv = self._mm(x, layer["wqkv"])
                if ours:
                    # One kernel rotates q and k and writes k, v into the cache.
                    if not self.fused_epilogues:
                        kc, vc = self.k_cache[li], self.v_cache[li]
                        q = rope_kv_write(qkv, B, T, self.h_local, self.kv_local, kc, vc, self.rope_cos32, self.rope_sin32,
                                          pos, batch0=batch0)
                    if decode and hd == 128:
                        att = attn_decode(q.view(B, self.h_local, hd), kc, vc, pos, batch0=batch0)
                    elif decode:
                        att = F.scaled_dot_product_attention(q.view(B, 1, self.h_local, hd).transpose(1, 2), kc[sl], vc[sl],
                                                             attn_mask=attn_mask, enable_gqa=True)
                        att = att.transpose(1, 2).reshape(B * T, self.h_local * hd)
                    else:
                        att = F.scaled_dot_product_attention(q.view(B, T, self.h_local, hd).transpose(1, 2),
                                                             kc[sl, :, pos:pos + T], vc[sl, :, pos:pos + T],
                                                             is_causal=True, enable_gqa=True)
                        att = att.transpose(1, 2).reshape(B * T, self.h_local * hd)
                else:
                    qkv = qkv.view(B, T, self.h_local + 2 * self.kv_local, hd)
                    q = _apply_rope(qkv[:, :, : self.h_local], cos, sin).transpose(1, 2)
                    k = _apply_rope(qkv[:, :, self.h_local: self.h_local + self.kv_local], cos, sin).transpose(1, 2)
                    v = qkv[:, :, self.h_local + self.kv_local:].transpose(1, 2)
                    if decode:
                        self.k_cache[li, sl].index_copy_(2, pos, k)
                        self.v_cache[li, sl].index_copy_(2, pos, v)
                        att = F.scaled_dot_product_attention(q, self.k_cache[li, sl], self.v_cache[li, sl],
                                                             attn_mask=attn_mask, enable_gqa=True)
                    else:
                        self.k_cache[li, sl, :, pos:pos + T] = k
                        self.v_cache[li, sl, :, pos:pos + T] = v
                        att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                    att = att.transpose(1, 2).reshape(B * T, self.h_local * hd)
                x, h = self._row_parallel_norm(att, layer["wo"], h, layer["norm2"])
                if ours and self.fused_epilogues:
                    act = gemm_swiglu(x, layer["wgu"])
                elif ours:
                    act = silu_mul(self._mm(x, layer["wgu"]))
                else:
                    gu = self._mm(x, layer["wgu"])
                    half = gu.shape[1] // 2
                    act = F.silu(gu[:, :half]) * gu[:, half:]
                next_norm = self.layers[li + 1]["norm1"] if li + 1 < len(self.layers) else self.final_norm
                x, h = self._row_parallel_norm(act, layer["wd"], h, next_norm)
        return x

    def greedy_token(self, hidden_last: torch.Tensor) -> torch.Tensor:
        """Greedy next token from the column-parallel LM head: local arg-max, then the global one from an
        all-gather of (value, index) pairs."""
        logits = self._mm(hidden_last, self.lm_head).float()  # [B, vocab / tp]
        val, idx = logits.max(dim=-1)
        if self.world == 1:
            return idx
        idx = idx + self.rank * (self.cfg.vocab // self.world)
        pair = torch.stack((val, idx.float()), dim=-1).contiguous()  # [B, 2] fp32
        if self.backend == "ours":
            allp = self.comm.all_gather(pair).view(self.world, -1, 2)
        else:
            import torch.distributed as dist
            allp = torch.empty(self.world, pair.shape[0], 2, device=self.device)
            dist.all_gather_into_tensor(allp, pair, group=self.nccl_group)
        best = allp[:, :, 0].argmax(dim=0)
        return allp[best, torch.arange(pair.shape[0], device=self.device), 1].long()

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, new_tokens: int, *, prefill_chunk_tokens: int = 8192,
                 use_graph: bool = True) -> torch.Tensor:
        """Greedy decoding.  prompts: [B, T_in].  Returns [B, new_tokens]."""
        B, T_in = prompts.shape
        assert B <= self.max_batch and T_in + new_tokens <= self.max_len
        # Prefill in batch slices of at most prefill_chunk_tokens tokens.
        rows = max(1, prefill_chunk_tokens // T_in)
        last = torch.empty(B, self.cfg.hidden, device=self.device, dtype=self.dtype)
        for b0 in range(0, B, rows):
            b1 = min(B, b0 + rows)
            hs = self.forward(prompts[b0:b1], 0, batch0=b0)
            last[b0:b1] = hs.view(b1 - b0, T_in, -1)[:, -1]
        out = torch.empty(B, new_tokens, dtype=torch.long, device=self.device)
        tok = self.greedy_token(last)
        out[:, 0] = tok
        if new_tokens == 1:
            return out
        # Decode: one token per step against the masked full-length cache; position and mask are device tensors
        # so that every step has the same shapes and addresses.
        mask = torch.full((1, 1, 1, self.max_len), float("-inf"), device=self.device, dtype=self.dtype)
        mask[..., :T_in] = 0
        pos = torch.full((1,), T_in, dtype=torch.long, device=self.device)
        cur = tok.view(B, 1).clone()
        nxt = torch.empty(B, dtype=torch.long, device=self.device)

        def step():
            mask.index_fill_(3, pos, 0.0)
            hs = self.forward(cur, pos, attn_mask=mask)
            nxt.copy_(self.greedy_token(hs))
            cur.copy_(nxt.view(B, 1))
            pos.add_(1)

        graph = None
        first = 1
        if use_graph and new_tokens > 3:
            step()  # eager warm-up: sizes scratch buffers and loads kernels before capture
            out[:, 1] = nxt
            first = 2
            torch.cuda.synchronize()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
            except Exception:
                graph = None
                torch.cuda.synchronize()
                raise
        for i in range(first, new_tokens):
            if graph is not None:
                graph.replay()
            else:
                step()
            out[:, i] = nxt
        return out
