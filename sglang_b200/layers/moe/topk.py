"""Plain softmax top-k routing, the `fused_topk` of the reference
(python/sglang/srt/layers/moe/topk.py:337-363): allocate the two outputs, run the router kernel.
(Expert-location remapping and the padded-region mask of the reference belong to its serving runtime and are
not part of this path.)"""
from __future__ import annotations

import torch

from ...sgl_kernel import topk_softmax


def fused_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, topk: int, renormalize: bool):
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    M = hidden_states.shape[0]
    topk_weights = torch.empty(M, topk, dtype=torch.float32, device=hidden_states.device)
    topk_ids = torch.empty(M, topk, dtype=torch.int32, device=hidden_states.device)
    if M > 0:
        topk_softmax(topk_weights, topk_ids, gating_output, renormalize)
    return topk_weights, topk_ids
