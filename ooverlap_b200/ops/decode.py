"""Decode-path kernels of the model runner: RoPE fused with the KV-cache write, SwiGLU, grouped-query decode
attention over a static cache.

Capability parity: the reference leaves the model's own ops to vLLM
(patches/vllm/v0.25.0/vllm/model_executor/models/qwen2.py); this library's serving path needs them so that one
decode step is a fixed sequence of kernels (nine per transformer layer) that a CUDA graph replays.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from .. import _lib
from ..utils.dtypes import dtype_code


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def rope_tables(max_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos`` / ``sin`` tables of shape [max_len, head_dim / 2] for rotation pairs (2i, 2i + 1)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(max_len, device=device, dtype=torch.float32).unsqueeze(-1) * inv
    return ang.cos().contiguous(), ang.sin().contiguous()


def _rope_args(dtype, B: int, T: int, heads: int, kv_heads: int, hd: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
               cos: torch.Tensor, sin: torch.Tensor, pos, batch0: int, q_out: torch.Tensor) -> "_lib.RopeArgs":
    if k_cache.shape[-1] != hd or k_cache.shape != v_cache.shape:
        raise ValueError("head geometry does not match the cache")
    if k_cache.dim() != 4 or k_cache.shape[1] != kv_heads or k_cache.stride(3) != 1 or k_cache.stride(2) != hd \
            or k_cache.stride(1) != k_cache.shape[2] * hd or v_cache.stride() != k_cache.stride():
        raise ValueError("cache must be [batch, kv_heads, max_len, hd] with contiguous (kv_heads, max_len, hd)")
    if batch0 + B > k_cache.shape[0]:
        raise ValueError("sequences outside the cache")
    max_len = k_cache.shape[2]
    if cos.dtype != torch.float32 or cos.shape != (max_len, hd // 2) or not cos.is_contiguous() or sin.shape != cos.shape:
        raise ValueError("cos / sin must be contiguous fp32 [max_len, hd/2] tables")
    a = _lib.RopeArgs()
    a.dtype, a.B, a.T, a.H, a.KV, a.hd = dtype_code(dtype), B, T, heads, kv_heads, hd
    a.qkv, a.q_out = None, q_out.data_ptr()
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.cache_batch_stride, a.max_len, a.batch0 = k_cache.stride(0), max_len, batch0
    a.cos_table, a.sin_table = cos.data_ptr(), sin.data_ptr()
    if isinstance(pos, torch.Tensor):
        if pos.dtype != torch.int64 or pos.numel() != 1 or not pos.is_cuda:
            raise ValueError("pos must be a one-element int64 CUDA tensor")
        a.pos_dev, a.pos0 = pos.data_ptr(), 0
    else:
        a.pos_dev, a.pos0 = None, int(pos)
    return a


def rope_kv_write(qkv: torch.Tensor, B: int, T: int, heads: int, kv_heads: int, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos, *, batch0: int = 0,
                  q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotates the query and key heads of ``qkv`` ([B*T, (heads + 2*kv_heads) * hd]) and writes keys and values
    into one layer's cache ([batch, kv_heads, max_len, hd]) at positions ``pos .. pos + T - 1`` of sequences
    ``batch0 .. batch0 + B - 1``.  ``pos`` is an int, or a device ``int64`` tensor with one element (read by the
    kernel, so a captured launch follows it).  Returns the rotated queries, [B*T, heads * hd]."""
    if qkv.dim() != 2 or not qkv.is_contiguous() or qkv.shape[0] != B * T:
        raise ValueError("qkv must be a contiguous [B*T, (heads + 2*kv_heads) * hd] tensor")
    hd = qkv.shape[1] // (heads + 2 * kv_heads)
    if hd * (heads + 2 * kv_heads) != qkv.shape[1]:
        raise ValueError("head geometry does not match qkv")
    if q_out is None:
        q_out = torch.empty((B * T, heads * hd), dtype=qkv.dtype, device=qkv.device)
    a = _rope_args(qkv.dtype, B, T, heads, kv_heads, hd, k_cache, v_cache, cos, sin, pos, batch0, q_out)
    a.qkv = qkv.data_ptr()
    _lib.check(_lib.lib().oob_rope_kv_write(ctypes.byref(a), _stream()))
    return q_out


def gemm_rope_kv_write(x: torch.Tensor, wqkv: torch.Tensor, B: int, T: int, heads: int, kv_heads: int,
                       k_cache: torch.Tensor, v_cache: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos, *,
                       batch0: int = 0, q_out: Optional[torch.Tensor] = None, fused: Optional[bool] = None) -> torch.Tensor:
    """``rope_kv_write(x @ wqkv.T, ...)``: the QKV projection followed by the rotation and the cache write.

    When the GEMM is one that is split over K (every decode-step shape), rotation and cache write are done by the
    kernel that sums the splits, from the fp32 sums; otherwise (or with ``fused=False``) the GEMM is followed by
    :func:`rope_kv_write`.  Returns the rotated queries, [B*T, heads * hd]."""
    from .gemm import _check_operands, fill_gemm_args, gemm, gemm_plan_splits
    _check_operands(x, wqkv)
    M, N, K = x.shape[0], wqkv.shape[0], x.shape[1]
    if M != B * T:
        raise ValueError("x must have B*T rows")
    hd = N // (heads + 2 * kv_heads)
    if hd * (heads + 2 * kv_heads) != N or hd % 8 != 0:
        raise ValueError("head geometry does not match the QKV weight")
    can_fuse = gemm_plan_splits(M, N, K) > 1
    if fused is None:
        fused = can_fuse
    if fused and not can_fuse:
        raise ValueError("this problem is not split over K, so the epilogue has no kernel to run in")
    if not fused:
        return rope_kv_write(gemm(x, wqkv), B, T, heads, kv_heads, k_cache, v_cache, cos, sin, pos, batch0=batch0,
                             q_out=q_out)
    if q_out is None:
        q_out = torch.empty((M, heads * hd), dtype=x.dtype, device=x.device)
    r = _rope_args(x.dtype, B, T, heads, kv_heads, hd, k_cache, v_cache, cos, sin, pos, batch0, q_out)
    args = _lib.GemmArgs()
    args.mode = _lib.GEMM_PLAIN
    fill_gemm_args(args, x, wqkv)
    args.C, args.ldc = q_out.data_ptr(), N  # C itself is not written; a valid aligned pointer keeps the checks uniform
    args.skinny = -1
    args.epilogue = _lib.EPILOGUE_ROPE_KV
    args.epilogue_args = ctypes.cast(ctypes.pointer(r), ctypes.c_void_p)
    _lib.check(_lib.lib().oob_gemm(None, ctypes.byref(args), _stream()))
    return q_out


def silu_mul(gu: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gu[:, :F]) * gu[:, F:]`` for a [rows, 2F] tensor with unit column stride."""
    if gu.dim() != 2 or gu.stride(1) != 1 or gu.shape[1] % 16 != 0:
        raise ValueError("gu must be [rows, 2F] with F a multiple of 8 and unit column stride")
    rows, F = gu.shape[0], gu.shape[1] // 2
    if out is None:
        out = torch.empty((rows, F), dtype=gu.dtype, device=gu.device)
    elif out.shape != (rows, F) or not out.is_contiguous() or out.dtype != gu.dtype:
        raise ValueError("bad output tensor")
    _lib.check(_lib.lib().oob_silu_mul(dtype_code(gu.dtype), ctypes.c_void_p(gu.data_ptr()), gu.stride(0),
                                       ctypes.c_void_p(out.data_ptr()), rows, F, _stream()))
    return out


_workspaces: dict = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    key = (device.type, device.index)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() * 4 < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20) // 4 + 1, dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos, *, batch0: int = 0,
                scale: Optional[float] = None, out: Optional[torch.Tensor] = None, splits: int = 0,
                len_bound: int = 0) -> torch.Tensor:
    """One decode step of grouped-query attention: ``q`` is [B, heads, 128], the cache is
    [batch, kv_heads, max_len, 128] and keys ``0 .. pos`` of sequences ``batch0 .. batch0 + B - 1`` are attended
    (``pos``: int or one-element device ``int64`` tensor, the index of the newest key).  Returns [B, heads * 128].

    ``splits`` CTAs share the keys of one (sequence, KV head); 0 picks the count from ``B * kv_heads`` and
    ``len_bound`` (an upper bound of the context length of this and any replayed launch; default ``max_len``)."""
    if q.dim() != 3 or q.shape[2] != 128 or not q.is_contiguous():
        raise ValueError("q must be a contiguous [B, heads, 128] tensor")
    B, H, hd = q.shape
    if k_cache.dim() != 4 or k_cache.shape[3] != hd or k_cache.shape != v_cache.shape or k_cache.dtype != q.dtype:
        raise ValueError("cache must be [batch, kv_heads, max_len, 128] of the query's dtype")
    KV, max_len = k_cache.shape[1], k_cache.shape[2]
    if k_cache.stride(3) != 1 or k_cache.stride(2) != hd or k_cache.stride(1) != max_len * hd \
            or v_cache.stride() != k_cache.stride():
        raise ValueError("cache must have contiguous (kv_heads, max_len, hd)")
    if H % KV or H // KV > 16 or batch0 + B > k_cache.shape[0]:
        raise ValueError("bad head counts or sequences outside the cache")
    if out is None:
        out = torch.empty((B, H * hd), dtype=q.dtype, device=q.device)
    lib = _lib.lib()
    bound = len_bound or max_len
    if splits == 0:
        splits = lib.oob_attn_decode_auto_splits(B, KV, bound)
    a = _lib.AttnDecodeArgs()
    a.dtype, a.B, a.H, a.KV = dtype_code(q.dtype), B, H, KV
    a.q, a.k_cache, a.v_cache, a.out = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
    a.cache_batch_stride, a.max_len, a.batch0 = k_cache.stride(0), max_len, batch0
    if isinstance(pos, torch.Tensor):
        if pos.dtype != torch.int64 or pos.numel() != 1 or not pos.is_cuda:
            raise ValueError("pos must be a one-element int64 CUDA tensor")
        a.pos_dev, a.len = pos.data_ptr(), 0
    else:
        a.pos_dev, a.len = None, int(pos) + 1
    a.scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    a.splits, a.len_bound = splits, bound
    if splits > 1:
        ws = _workspace(q.device, lib.oob_attn_decode_workspace_bytes(B, H, splits))
        a.workspace = ws.data_ptr()
    else:
        a.workspace = None
    _lib.check(lib.oob_attn_decode(ctypes.byref(a), _stream()))
    return out


def attn_decode_reference(q, k_cache, v_cache, pos: int, *, batch0: int = 0, scale: Optional[float] = None):
    """fp32 PyTorch oracle of :func:`attn_decode`."""
    B, H, hd = q.shape
    KV = k_cache.shape[1]
    G = H // KV
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    k = k_cache[batch0:batch0 + B, :, :pos + 1].float().repeat_interleave(G, dim=1)  # [B, H, L, hd]
    v = v_cache[batch0:batch0 + B, :, :pos + 1].float().repeat_interleave(G, dim=1)
    s = torch.einsum("bhd,bhld->bhl", q.float(), k) * scale
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhl,bhld->bhd", p, v).reshape(B, H * hd)
