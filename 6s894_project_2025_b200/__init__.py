"""B200-native Walsh-Hadamard transform and fused W . H(X).

The directory name starts with a digit, so import it with
``importlib.import_module("6s894_project_2025_b200")``.
"""
from .ops import (  # noqa: F401
    HostPipeline,
    device_status,
    fused_gemm_workspace_bytes,
    fused_ht_gemm,
    fused_ht_gemv,
    hadamard_transform,
)
from .partition import (  # noqa: F401
    RowShardedGemv,
    gather_result,
    gather_rows,
    row_range,
    shard_rows,
    shard_tokens,
    token_range,
)
from . import torchlib  # noqa: F401  (registers torch.ops.b200ht.*)

__all__ = [
    "HostPipeline",
    "hadamard_transform",
    "fused_ht_gemm",
    "fused_ht_gemv",
    "fused_gemm_workspace_bytes",
    "device_status",
    "token_range",
    "shard_tokens",
    "gather_result",
    "row_range",
    "shard_rows",
    "gather_rows",
    "RowShardedGemv",
]
