"""Tensor-parallel building blocks and the vLLM backend hook."""
from .layers import ColumnParallelLinear, RowParallelLinear  # noqa: F401
from .vllm_adapter import OoverlapAllReduce, forced_backend, install, short_broker_key  # noqa: F401
