"""Model families run on this library's kernels."""
from .llama import LLAMA3_8B, LLAMA3_70B, TINY, TINY128, LlamaConfig, LlamaTP  # noqa: F401
