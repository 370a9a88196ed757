from .tp_linear import (ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear, shard_block_fp8_weight)

__all__ = ["ColumnParallelBlockFp8Linear", "RowParallelBlockFp8Linear", "shard_block_fp8_weight"]
