"""Tensor-parallel block-FP8 linears, following the reference's sharding rules:

* column-parallel (python/sglang/srt/layers/linear.py:242-413): weight rows N split p ways, every
  rank sees the full activation, no collective (gather_output=False);
* row-parallel (linear.py:1123-1304): weight columns K split p ways, each rank holds x[:, K/p],
  partial outputs are summed with one bf16 all-reduce (linear.py:1294-1300,
  python/sglang/srt/distributed/communication_op.py:11-13); bias only on rank 0 (linear.py:1293).
* block-quant divisibility (python/sglang/srt/layers/quantization/fp8.py:239-262): every shard
  boundary must fall on a 128-block boundary.

The local linear is injectable so the sharding/collective logic can be exercised with CPU
ranks (gloo); the default is the CUDA path and there is no CPU fallback in the product.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

BLOCK = 128


def shard_block_fp8_weight(weight: torch.Tensor, weight_scale: torch.Tensor, dim: int, rank: int,
                           world: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Slice weight [N,K] (e4m3) and its [N/128,K/128] block scales for `rank` along dim 0 (N,
    column-parallel) or dim 1 (K, row-parallel)."""
    size = weight.shape[dim]
    if size % world != 0:
        raise ValueError(f"dimension {dim} of size {size} is not divisible by tp size {world}")
    part = size // world
    if part % BLOCK != 0:
        # fp8.py:245-262: "Weight input/output_size_per_partition ... is not divisible by weight quantization block"
        raise ValueError(f"partition size {part} is not divisible by the weight quantization block {BLOCK}")
    lo = rank * part
    w = weight.narrow(dim, lo, part).contiguous()
    s = weight_scale.narrow(dim, lo // BLOCK, part // BLOCK).contiguous()
    return w, s


def _default_linear(x, w, ws, bias, out=None):
    from ..layers.quantization.fp8_utils import w8a8_block_fp8_linear
    return w8a8_block_fp8_linear(x, w, [BLOCK, BLOCK], ws, bias=bias, out=out)


class ColumnParallelBlockFp8Linear:
    def __init__(self, weight, weight_scale, bias: Optional[torch.Tensor] = None, group=None,
                 linear_fn: Callable = _default_linear, already_sharded: bool = False):
        self.group = group
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        if already_sharded or world == 1:
            self.weight, self.weight_scale, self.bias = weight, weight_scale, bias
        else:
            self.weight, self.weight_scale = shard_block_fp8_weight(weight, weight_scale, 0, rank, world)
            part = weight.shape[0] // world
            self.bias = None if bias is None else bias.narrow(0, rank * part, part).contiguous()
        self._linear = linear_fn

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._linear(x, self.weight, self.weight_scale, self.bias)

    __call__ = forward


class RowParallelBlockFp8Linear:
    """all_reduce: a SymmetricAllReduce (custom_all_reduce.py) to sum the partial outputs with this
    library's NVLink kernels; the GEMM then writes straight into the symmetric buffer.  None = NCCL
    (`dist.all_reduce`), as the reference does.

    overlap_chunks > 1: the rows are processed in that many chunks and the all-reduce of chunk i runs on
    a side stream while chunk i+1 is quantised and multiplied (CUDA only).  The sum per element is the
    same collective on the same values, so results equal the unchunked form.
    reserve_sms > 0 (with overlap_chunks > 1 and a SymmetricAllReduce that has a multicast address): the GEMMs of
    the chunks leave that many SMs free and the all-reduce runs in its multicast form on that many blocks -- the
    form whose speed does not depend on the block count -- so the two really run side by side; without it a
    persistent GEMM holds every SM and the collective waits for its last wave."""

    def __init__(self, weight, weight_scale, bias: Optional[torch.Tensor] = None, group=None,
                 linear_fn: Callable = _default_linear, reduce_results: bool = True, already_sharded: bool = False,
                 overlap_chunks: int = 1, all_reduce=None, reserve_sms: int = 0):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if already_sharded or self.world == 1:
            self.weight, self.weight_scale = weight, weight_scale
        else:
            self.weight, self.weight_scale = shard_block_fp8_weight(weight, weight_scale, 1, self.rank, self.world)
        self.bias = bias
        self.reduce_results = reduce_results
        self._linear = linear_fn
        self.overlap_chunks = max(1, int(overlap_chunks))
        self._comm_stream = None
        self.all_reduce = all_reduce
        self.reserve_sms = max(0, int(reserve_sms))

    def _reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.all_reduce is not None:
            return self.all_reduce.all_reduce(t)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def _out_buffer(self, M: int, x: torch.Tensor) -> torch.Tensor:
        N = self.weight.shape[0]
        if self.all_reduce is not None:
            return self.all_reduce.buffer((M, N), x.dtype)
        return torch.empty((M, N), dtype=x.dtype, device=x.device)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        bias = self.bias if self.rank == 0 else None   # added once, before the sum
        reduce = self.reduce_results and self.world > 1
        M = x_shard.shape[0] if x_shard.dim() == 2 else 0
        if not reduce:
            return self._linear(x_shard, self.weight, self.weight_scale, bias)
        if not (self.overlap_chunks > 1 and x_shard.is_cuda and M >= 256 * self.overlap_chunks):
            if self.all_reduce is not None and x_shard.dim() == 2:
                out = self._linear(x_shard, self.weight, self.weight_scale, bias, out=self._out_buffer(M, x_shard))
            else:
                out = self._linear(x_shard, self.weight, self.weight_scale, bias)
            return self._reduce(out)
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=x_shard.device)
        main = torch.cuda.current_stream(x_shard.device)
        out = self._out_buffer(M, x_shard)
        rows = (M + self.overlap_chunks - 1) // self.overlap_chunks
        rows = (rows + 127) // 128 * 128
        ar = self.all_reduce
        split = self.reserve_sms > 0 and ar is not None and getattr(ar, "has_multicast", False)
        if split:
            from ..sgl_kernel.gemm import set_sm_limit
            sms = torch.cuda.get_device_properties(x_shard.device).multi_processor_count
            old_limit = set_sm_limit(max(1, sms - self.reserve_sms))
            old_form, old_blocks = ("multicast" if ar.multicast else "peer"), ar.num_blocks
            ar.set_form("multicast")
            ar.num_blocks = self.reserve_sms
        try:
            for lo in range(0, M, rows):
                hi = min(M, lo + rows)
                self._linear(x_shard[lo:hi], self.weight, self.weight_scale, bias, out=out[lo:hi])
                ready = torch.cuda.Event()
                ready.record(main)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ready)
                    if ar is not None:
                        ar.all_reduce_(out[lo:hi])
                    else:
                        dist.all_reduce(out[lo:hi], op=dist.ReduceOp.SUM, group=self.group)
        finally:
            if split:
                set_sm_limit(old_limit)
                ar.set_form(old_form)
                ar.num_blocks = old_blocks
        main.wait_stream(self._comm_stream)
        return out

    __call__ = forward
