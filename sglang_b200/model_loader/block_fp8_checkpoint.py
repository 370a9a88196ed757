"""Loading block-quantised FP8 checkpoints (Hugging Face layout) into the parameter owners of this package.

What the reference does across `Fp8Config.from_config` (python/sglang/srt/layers/quantization/fp8.py:155-167),
the weight loaders of its parallel linears (python/sglang/srt/layers/linear.py:333-399 column / merged-column,
:1207-1278 row; block scales are sharded in units of the 128-block, parameter.py:299-305) and of the fused MoE
layer (python/sglang/srt/layers/moe/fused_moe_triton/layer.py:465-720: gate_proj and up_proj of an expert are
stacked into w13, down_proj is w2, experts are split contiguously across expert-parallel ranks), reduced to the
block-FP8 path: read `weight` (e4m3 [N, K]) and `weight_scale_inv` (fp32 [N/128, K/128]) tensors from safetensors
shards, slice them for a tensor- or expert-parallel rank, and copy them into the parameters that
`Fp8LinearMethod.create_weights` / `Fp8MoEMethod.create_weights` registered.

Only host-side tensor plumbing lives here; nothing is computed.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch

from ..distributed.tp_linear import BLOCK, shard_block_fp8_weight
from ..layers.quantization.fp8 import Fp8Config

FP8 = torch.float8_e4m3fn


def read_quantization_config(model_dir: str) -> Fp8Config:
    """`quantization_config` of the checkpoint's config.json -> Fp8Config (fp8.py:155-167)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    q = cfg.get("quantization_config")
    if q is None:
        raise ValueError(f"{model_dir}/config.json has no quantization_config")
    return Fp8Config.from_config(q)


class SafetensorsIndex:
    """Name -> tensor access over the safetensors shards of a checkpoint directory, through
    `model.safetensors.index.json` when present, else over every `*.safetensors` file.  Files are opened lazily
    and tensors are read one at a time (a DeepSeek-V3 checkpoint is ~700 GB)."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open
        self._open = safe_open
        self.model_dir = model_dir
        self._files: Dict[str, object] = {}
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index) as f:
                self.weight_map: Dict[str, str] = dict(json.load(f)["weight_map"])
        else:
            self.weight_map = {}
            for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
                with safe_open(path, framework="pt", device="cpu") as f:
                    for k in f.keys():
                        self.weight_map[k] = os.path.basename(path)
        if not self.weight_map:
            raise FileNotFoundError(f"no safetensors weights under {model_dir}")

    def __contains__(self, name: str) -> bool:
        return name in self.weight_map

    def names(self) -> Iterator[str]:
        return iter(self.weight_map)

    def get(self, name: str) -> torch.Tensor:
        if name not in self.weight_map:
            raise KeyError(f"{name} is not in the checkpoint")
        fname = self.weight_map[name]
        f = self._files.get(fname)
        if f is None:
            f = self._files[fname] = self._open(os.path.join(self.model_dir, fname), framework="pt", device="cpu")
        return f.get_tensor(name)


def _check_block_pair(name: str, w: torch.Tensor, s: torch.Tensor) -> None:
    if w.dtype != FP8:
        raise ValueError(f"{name}.weight is {w.dtype}, expected float8_e4m3fn (is the checkpoint fp8-serialised?)")
    if s.dtype != torch.float32:
        raise ValueError(f"{name}.weight_scale_inv is {s.dtype}, expected float32")
    n, k = w.shape
    want = ((n + BLOCK - 1) // BLOCK, (k + BLOCK - 1) // BLOCK)
    if tuple(s.shape) != want:
        raise ValueError(f"{name}.weight_scale_inv has shape {tuple(s.shape)}, expected {want} for weight {tuple(w.shape)}")


def load_linear_shard(ckpt: SafetensorsIndex, names: Sequence[str], parallel: str, tp_rank: int = 0,
                      tp_size: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Weight and block scales of one (possibly merged) linear for one tensor-parallel rank.

    names     checkpoint prefixes whose outputs are stacked, e.g. ["…mlp.gate_proj", "…mlp.up_proj"] for the
              merged gate_up projection or one name for a plain projection
    parallel  "column" (output rows split; each stacked projection is split separately, as the merged-column
              loader does, linear.py:484-640), "row" (input columns split) or "replicated"
    Shard boundaries must fall on 128-block boundaries (fp8.py:239-262)."""
    if parallel not in ("column", "row", "replicated"):
        raise ValueError(f"parallel = {parallel!r}")
    ws, ss = [], []
    for name in names:
        w = ckpt.get(name + ".weight")
        s = ckpt.get(name + ".weight_scale_inv")
        _check_block_pair(name, w, s)
        if len(names) > 1 and w.shape[0] % BLOCK != 0:
            raise ValueError(f"Weight output_partition_size = {w.shape[0]} is not divisible by weight quantization "
                             f"block_n = {BLOCK}.")
        if parallel != "replicated" and tp_size > 1:
            w, s = shard_block_fp8_weight(w, s, 0 if parallel == "column" else 1, tp_rank, tp_size)
        ws.append(w)
        ss.append(s)
    if len(ws) == 1:
        return ws[0].contiguous(), ss[0].contiguous()
    return torch.cat(ws, dim=0).contiguous(), torch.cat(ss, dim=0).contiguous()


def load_linear(method, layer: torch.nn.Module, ckpt: SafetensorsIndex, names: Sequence[str], parallel: str,
                tp_rank: int = 0, tp_size: int = 1) -> None:
    """Fill `layer.weight` / `layer.weight_scale_inv` (registered by Fp8LinearMethod.create_weights) from the
    checkpoint and run process_weights_after_loading."""
    w, s = load_linear_shard(ckpt, names, parallel, tp_rank, tp_size)
    if tuple(layer.weight.shape) != tuple(w.shape) or tuple(layer.weight_scale_inv.shape) != tuple(s.shape):
        raise ValueError(f"{list(names)}: checkpoint shard {tuple(w.shape)} / {tuple(s.shape)} does not match the "
                         f"layer's {tuple(layer.weight.shape)} / {tuple(layer.weight_scale_inv.shape)}")
    layer.weight.data.copy_(w)
    layer.weight_scale_inv.data.copy_(s)
    method.process_weights_after_loading(layer)


def expert_range(num_experts: int, ep_rank: int, ep_size: int) -> range:
    """Experts held by an expert-parallel rank: contiguous blocks of num_experts / ep_size
    (python/sglang/srt/layers/moe/ep_moe/layer.py:170-185)."""
    if num_experts % ep_size != 0:
        raise ValueError(f"{num_experts} experts are not divisible by ep size {ep_size}")
    per = num_experts // ep_size
    return range(ep_rank * per, (ep_rank + 1) * per)


def load_experts(method, layer: torch.nn.Module, ckpt: SafetensorsIndex, prefix: str, experts: Iterable[int],
                 gate: str = "gate_proj", up: str = "up_proj", down: str = "down_proj") -> None:
    """Fill w13_weight [E_local, 2I, H] (gate rows then up rows), w2_weight [E_local, H, I] and their
    `_scale_inv` tensors from `{prefix}.{expert}.{gate|up|down}.(weight|weight_scale_inv)`
    (the stacking of fused_moe_triton/layer.py:465-720: shard ids w1 -> first half of w13, w3 -> second half,
    w2 -> down)."""
    experts = list(experts)
    if len(experts) != layer.w13_weight.shape[0]:
        raise ValueError(f"{len(experts)} experts for a layer that holds {layer.w13_weight.shape[0]}")
    inter = layer.w13_weight.shape[1] // 2
    for slot, e in enumerate(experts):
        parts = {}
        for key in (gate, up, down):
            name = f"{prefix}.{e}.{key}"
            w, s = ckpt.get(name + ".weight"), ckpt.get(name + ".weight_scale_inv")
            _check_block_pair(name, w, s)
            parts[key] = (w, s)
        gw, gs = parts[gate]
        uw, us = parts[up]
        dw, ds = parts[down]
        if gw.shape != uw.shape or gw.shape[0] != inter or tuple(dw.shape) != (gw.shape[1], inter):
            raise ValueError(f"{prefix}.{e}: expert shapes {tuple(gw.shape)}, {tuple(uw.shape)}, {tuple(dw.shape)} do not "
                             f"match the layer (intermediate {inter}, hidden {layer.w2_weight.shape[1]})")
        layer.w13_weight.data[slot, :inter].copy_(gw)
        layer.w13_weight.data[slot, inter:].copy_(uw)
        layer.w2_weight.data[slot].copy_(dw)
        sb = gs.shape[0]
        layer.w13_weight_scale_inv.data[slot, :sb].copy_(gs)
        layer.w13_weight_scale_inv.data[slot, sb:].copy_(us)
        layer.w2_weight_scale_inv.data[slot].copy_(ds)
    method.process_weights_after_loading(layer)
