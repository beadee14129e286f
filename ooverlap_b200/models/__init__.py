"""Model families run on this library's kernels."""
from .llama import LLAMA3_8B, LLAMA3_70B, TINY, LlamaConfig, LlamaTP  # noqa: F401
