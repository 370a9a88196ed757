"""CPU: a synthetic block-FP8 checkpoint in the Hugging Face layout (config.json with quantization_config,
two safetensors shards and their index) is read back into the parameter owners for tensor- and expert-parallel
ranks with the slicing rules of the reference's loaders (python/sglang/srt/layers/linear.py:333-399,1207-1278;
python/sglang/srt/layers/moe/fused_moe_triton/layer.py:465-720)."""
import json
import os

import pytest
import torch

from oracle import block_fp8_oracle as O
from sglang_b200.layers.quantization.fp8 import Fp8LinearMethod, Fp8MoEMethod
from sglang_b200.model_loader.block_fp8_checkpoint import (SafetensorsIndex, expert_range, load_experts, load_linear,
                                                           load_linear_shard, read_quantization_config)

H, I, E = 512, 256, 4   # hidden, intermediate, experts


@pytest.fixture(scope="module")
def ckpt_dir(tmp_path_factory):
    from safetensors.torch import save_file
    d = str(tmp_path_factory.mktemp("ckpt"))
    g = torch.Generator().manual_seed(0)
    tensors = {}

    def add(name, n, k):
        q, s = O.per_block_cast_to_fp8(torch.randn(n, k, generator=g) * 0.05)
        tensors[name + ".weight"], tensors[name + ".weight_scale_inv"] = q, s.contiguous()

    add("model.layers.0.mlp.gate_proj", I * 2, H)
    add("model.layers.0.mlp.up_proj", I * 2, H)
    add("model.layers.0.mlp.down_proj", H, I * 2)
    for e in range(E):
        add(f"model.layers.1.mlp.experts.{e}.gate_proj", I, H)
        add(f"model.layers.1.mlp.experts.{e}.up_proj", I, H)
        add(f"model.layers.1.mlp.experts.{e}.down_proj", H, I)
    names = sorted(tensors)
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    weight_map = {}
    for fname, keys in shards.items():
        save_file({k: tensors[k] for k in keys}, os.path.join(d, fname))
        weight_map.update({k: fname for k in keys})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"hidden_size": H, "quantization_config": {"quant_method": "fp8", "fmt": "e4m3",
                                                              "activation_scheme": "dynamic",
                                                              "weight_block_size": [128, 128]}}, f)
    return d, tensors


def _same(a, b):
    return a.dtype == b.dtype and a.shape == b.shape and torch.equal(a.view(torch.uint8) if a.dtype == torch.float8_e4m3fn else a,
                                                                      b.view(torch.uint8) if b.dtype == torch.float8_e4m3fn else b)


def test_config_and_index(ckpt_dir):
    d, tensors = ckpt_dir
    cfg = read_quantization_config(d)
    assert cfg.weight_block_size == [128, 128] and cfg.is_checkpoint_fp8_serialized
    idx = SafetensorsIndex(d)
    assert set(idx.names()) == set(tensors)
    assert _same(idx.get("model.layers.0.mlp.up_proj.weight"), tensors["model.layers.0.mlp.up_proj.weight"])
    with pytest.raises(KeyError):
        idx.get("model.layers.9.nothing.weight")
    os.rename(os.path.join(d, "model.safetensors.index.json"), os.path.join(d, "index.bak"))
    try:
        assert set(SafetensorsIndex(d).names()) == set(tensors)       # no index file: the shards are scanned
    finally:
        os.rename(os.path.join(d, "index.bak"), os.path.join(d, "model.safetensors.index.json"))


@pytest.mark.parametrize("tp_size", [1, 2])
def test_merged_column_and_row_parallel(ckpt_dir, tp_size):
    d, tensors = ckpt_dir
    idx = SafetensorsIndex(d)
    method = Fp8LinearMethod(read_quantization_config(d))
    gate, up = "model.layers.0.mlp.gate_proj", "model.layers.0.mlp.up_proj"
    down = "model.layers.0.mlp.down_proj"
    for rank in range(tp_size):
        part = 2 * I // tp_size
        layer = torch.nn.Module()
        method.create_weights(layer, H, [part, part], H, 4 * I, torch.bfloat16, tp_size=tp_size)
        load_linear(method, layer, idx, [gate, up], "column", rank, tp_size)
        lo = rank * part
        want_w = torch.cat([tensors[gate + ".weight"][lo:lo + part], tensors[up + ".weight"][lo:lo + part]])
        want_s = torch.cat([tensors[gate + ".weight_scale_inv"][lo // 128:(lo + part) // 128],
                            tensors[up + ".weight_scale_inv"][lo // 128:(lo + part) // 128]])
        assert _same(layer.weight.data, want_w) and _same(layer.weight_scale_inv.data, want_s)
        kpart = 2 * I // tp_size
        layer2 = torch.nn.Module()
        method.create_weights(layer2, kpart, [H], 2 * I, H, torch.bfloat16, tp_size=tp_size)
        load_linear(method, layer2, idx, [down], "row", rank, tp_size)
        klo = rank * kpart
        assert _same(layer2.weight.data, tensors[down + ".weight"][:, klo:klo + kpart].contiguous())
        assert _same(layer2.weight_scale_inv.data,
                     tensors[down + ".weight_scale_inv"][:, klo // 128:(klo + kpart) // 128].contiguous())


def test_shard_errors(ckpt_dir):
    d, _ = ckpt_dir
    idx = SafetensorsIndex(d)
    with pytest.raises(ValueError, match="not divisible"):      # 512 / 8 = 64 rows per rank: not a 128-block multiple
        load_linear_shard(idx, ["model.layers.0.mlp.gate_proj"], "column", 0, 8)
    with pytest.raises(ValueError):
        load_linear_shard(idx, ["model.layers.0.mlp.gate_proj"], "diagonal")
    method = Fp8LinearMethod(read_quantization_config(d))
    layer = torch.nn.Module()
    method.create_weights(layer, H, [128], H, 128, torch.bfloat16)
    with pytest.raises(ValueError, match="does not match"):
        load_linear(method, layer, idx, ["model.layers.0.mlp.gate_proj"], "replicated")


@pytest.mark.parametrize("ep_size", [1, 2])
def test_expert_parallel_loading(ckpt_dir, ep_size):
    d, tensors = ckpt_dir
    idx = SafetensorsIndex(d)
    method = Fp8MoEMethod(read_quantization_config(d))
    for rank in range(ep_size):
        ex = expert_range(E, rank, ep_size)
        layer = torch.nn.Module()
        method.create_weights(layer, len(ex), H, I, torch.bfloat16)
        load_experts(method, layer, idx, "model.layers.1.mlp.experts", ex)
        for slot, e in enumerate(ex):
            p = f"model.layers.1.mlp.experts.{e}."
            assert _same(layer.w13_weight.data[slot, :I], tensors[p + "gate_proj.weight"])
            assert _same(layer.w13_weight.data[slot, I:], tensors[p + "up_proj.weight"])
            assert _same(layer.w2_weight.data[slot], tensors[p + "down_proj.weight"])
            assert _same(layer.w13_weight_scale_inv.data[slot, :I // 128], tensors[p + "gate_proj.weight_scale_inv"])
            assert _same(layer.w13_weight_scale_inv.data[slot, I // 128:], tensors[p + "up_proj.weight_scale_inv"])
            assert _same(layer.w2_weight_scale_inv.data[slot], tensors[p + "down_proj.weight_scale_inv"])
    with pytest.raises(ValueError):
        expert_range(E, 0, 3)
