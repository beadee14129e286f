"""Tensor-parallel linear layers on this library's kernels.

* :class:`ColumnParallelLinear` — weight rows sharded over ranks, no communication (optionally preceded by
  an AllGather->GEMM when the input is sequence-sharded).
* :class:`RowParallelLinear` — weight columns sharded; the partial products are summed over ranks.  Small token
  counts (decode) use GEMM-into-slot + all-reduce (optionally fused with residual + RMSNorm); large ones (prefill)
  use the fused GEMM->AllReduce kernel.

Capability parity: the reference patches vLLM's Qwen2 ``o_proj`` / ``down_proj`` (row-parallel, bias-free,
unquantised) to run GEMM-into-slot + all-reduce
(patches/vllm/v0.25.0/vllm/model_executor/models/qwen2.py:84-120,153-156,274).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import GemmAllReduce, fused_allreduce_rmsnorm, gemm


class ColumnParallelLinear:
    def __init__(self, weight_shard: torch.Tensor):
        """``weight_shard``: [out_features / tp, in_features]."""
        self.weight = weight_shard

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return gemm(x, self.weight, out=out)


class RowParallelLinear:
    FUSED_MIN_TOKENS = 1024  # from here on the GEMM has several waves of tiles to overlap with

    def __init__(self, comm, weight_shard: torch.Tensor):
        """``weight_shard``: [out_features, in_features / tp]."""
        self.comm = comm
        self.weight = weight_shard
        self._fused = {}

    def partial_into_slot(self, x: torch.Tensor) -> torch.Tensor:
        """Local partial product written into the next all-reduce slot (not yet reduced)."""
        slot = self.comm.acquire_all_reduce_slot((x.shape[0], self.weight.shape[0]))
        gemm(x, self.weight, out=slot)
        return slot

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """``all_reduce(x @ W_shard^T)``; the result lives in registered memory."""
        if self.comm is None or self.comm.world == 1:
            return gemm(x, self.weight)
        M = x.shape[0]
        if M >= self.FUSED_MIN_TOKENS:
            op = self._fused.get(M)
            if op is None:
                op = self._fused[M] = GemmAllReduce(self.comm, M, self.weight.shape[0], x.dtype)
            return op(x, self.weight)
        slot = self.partial_into_slot(x)
        return self.comm.all_reduce_preloaded_slot(slot)

    def forward_norm(self, x: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float):
        """``h = residual + all_reduce(x @ W^T); y = rmsnorm(h) * norm_weight`` with the reduction, the residual
        add and the normalisation in one kernel.  Returns ``(y, h)``."""
        if self.comm is None or self.comm.world == 1:
            from ..ops import rmsnorm
            return rmsnorm(gemm(x, self.weight), norm_weight, eps, residual)
        slot = self.comm.commit_all_reduce_slot(self.partial_into_slot(x))
        return fused_allreduce_rmsnorm(self.comm, slot, norm_weight, eps, residual)
