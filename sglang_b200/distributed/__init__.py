from .ep_moe import ExpertParallelBlockFp8MoE
from .tp_linear import (ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear, shard_block_fp8_weight)

__all__ = ["ExpertParallelBlockFp8MoE", "ColumnParallelBlockFp8Linear", "RowParallelBlockFp8Linear", "shard_block_fp8_weight"]
