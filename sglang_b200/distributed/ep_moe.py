"""Expert-parallel block-FP8 MoE over NCCL all-to-all.

Sharding follows the reference: experts are split contiguously, E/p per rank
(python/sglang/srt/layers/moe/fused_moe_triton/layer.py:165-185); tokens stay sharded across ranks.
The reference moves tokens with DeepEP (python/sglang/srt/layers/moe/token_dispatcher/deepep.py:314-480,
which dispatches ALREADY-QUANTISED fp8 rows + scales, :328-336) or replicates tokens and all-reduces
(layer.py:813-818,850-851); it has no NCCL all-to-all dispatcher.  Here: one exchange each way with
`all_to_all_single`:

  dispatch  e4m3 rows [*, H] + fp32 scales [*, H/128] + local expert id per row
  combine   bf16 rows [*, H] back in the order they were sent

followed by the routing-weighted sum at the source rank (fp32 accumulate, j ascending) -- the same
arithmetic, in the same order, as the single-GPU path, so the result is bitwise the single-GPU result.
Split sizes come from an all-to-all of per-rank counts; NCCL needs them on the host, which costs one
small device->host copy per layer call.

The quantiser, the local expert computation and the weighted sum are injectable so the exchange
logic runs on CPU ranks (gloo) in the tests; the defaults are the CUDA kernels (no CPU fallback).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def _default_quant(x):
    from ..layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    return sglang_per_token_group_quant_fp8(x, 128)


def _default_local(a_q, a_s, ids, w13, w2, w13_s, w2_s, out_dtype):
    from ..layers.moe.cutlass_moe import grouped_experts_prequantized
    return grouped_experts_prequantized(a_q, a_s, ids, w13, w2, w13_s, w2_s, out_dtype)


def _default_weighted_sum(rows, perm, weights, m):
    from ..sgl_kernel import apply_shuffle_mul_sum
    out = torch.empty((m, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    apply_shuffle_mul_sum(rows, out, perm, weights)
    return out


class ExpertParallelBlockFp8MoE:
    """w13 [E_local, 2n, H], w2 [E_local, H, n] e4m3 and their block scales: this rank's experts
    (global ids [rank*E_local, (rank+1)*E_local))."""

    def __init__(self, w13, w2, w13_scale, w2_scale, group=None, quant_fn: Callable = _default_quant,
                 local_fn: Callable = _default_local, weighted_sum_fn: Callable = _default_weighted_sum):
        self.w13, self.w2, self.w13_scale, self.w2_scale = w13, w2, w13_scale, w2_scale
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.e_local = w13.shape[0]
        self._quant, self._local, self._wsum = quant_fn, local_fn, weighted_sum_fn

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        m, H = x.shape
        topk = topk_ids.shape[1]
        p, dev = self.world, x.device
        q, s = self._quant(x)                                            # quantise once per token
        flat_ids = topk_ids.reshape(-1).to(torch.int64)
        dest = torch.div(flat_ids, self.e_local, rounding_mode="floor")
        order = torch.argsort(dest, stable=True)                          # send order: by destination rank
        send_counts = torch.bincount(dest, minlength=p).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        if p > 1:
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        else:
            recv_counts.copy_(send_counts)
        send_split, recv_split = send_counts.tolist(), recv_counts.tolist()   # the one host sync
        n_recv = int(sum(recv_split))
        tok = torch.div(order, topk, rounding_mode="floor")
        send_q = q.view(torch.uint8)[tok].contiguous()
        send_s = s.contiguous()[tok].contiguous()
        send_e = (flat_ids[order] - dest[order] * self.e_local).to(torch.int32).contiguous()
        recv_q = torch.empty((n_recv, H), dtype=torch.uint8, device=dev)
        recv_s = torch.empty((n_recv, s.shape[1]), dtype=torch.float32, device=dev)
        recv_e = torch.empty((n_recv,), dtype=torch.int32, device=dev)
        if p > 1:
            dist.all_to_all_single(recv_q, send_q, recv_split, send_split, group=self.group)
            dist.all_to_all_single(recv_s, send_s, recv_split, send_split, group=self.group)
            dist.all_to_all_single(recv_e, send_e, recv_split, send_split, group=self.group)
        else:
            recv_q, recv_s, recv_e = send_q, send_s, send_e
        y = self._local(recv_q.view(torch.float8_e4m3fn), recv_s, recv_e, self.w13, self.w2, self.w13_scale,
                        self.w2_scale, x.dtype)
        back = torch.empty((order.numel(), H), dtype=x.dtype, device=dev)
        if p > 1:
            dist.all_to_all_single(back, y.contiguous(), send_split, recv_split, group=self.group)
        else:
            back = y
        # back[i] belongs to flat slot order[i]; the weighted sum reads slot f at row inv[f]
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=dev)
        return self._wsum(back, inv.to(torch.int32), topk_weights.to(x.dtype).contiguous(), m)

    __call__ = forward
