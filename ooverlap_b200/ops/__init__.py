"""Hot ops: hand-written sm_100a kernels behind small Python entry points."""
from . import solutions  # noqa: F401
from .decode import (attn_decode, attn_decode_reference, gemm_rope_kv_write, rope_kv_write, rope_tables,  # noqa: F401
                     silu_mul)
from .gemm import (gemm, gemm_plan_splits, gemm_swiglu, order_buffer, reserve_workspace, splitk_workspace_bytes,  # noqa: F401
                   stable_tile_waves, tile_order)
from .norm import (fused_allreduce_rmsnorm, fused_reduce_scatter_rmsnorm, rmsnorm,  # noqa: F401
                   rmsnorm_reference)
from .overlap import AllGatherGemm, GemmAllReduce, GemmReduceScatterNorm, gemm_all_reduce_unfused  # noqa: F401
