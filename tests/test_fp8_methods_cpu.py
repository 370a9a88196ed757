"""CPU: the parameter owners of the block-FP8 path (configuration errors, parameter shapes and the
tensor-parallel divisibility errors) behave as python/sglang/srt/layers/quantization/fp8.py:105-262,
526-671 do.  No kernel runs here."""
import pytest
import torch

from sglang_b200.layers.quantization.fp8 import Fp8Config, Fp8LinearMethod, Fp8MoEMethod

DEEPSEEK_QCFG = {"quant_method": "fp8", "activation_scheme": "dynamic", "fmt": "e4m3",
                 "weight_block_size": [128, 128]}


def test_config_from_hf_dictionary():
    cfg = Fp8Config.from_config(DEEPSEEK_QCFG)
    assert cfg.is_checkpoint_fp8_serialized and cfg.activation_scheme == "dynamic"
    assert cfg.weight_block_size == [128, 128] and cfg.ignored_layers == []
    assert Fp8Config.get_name() == "fp8"
    assert torch.bfloat16 in Fp8Config.get_supported_act_dtypes()
    with pytest.raises(ValueError):
        Fp8Config.from_config({"quant_method": "fp8"})          # activation_scheme is required


@pytest.mark.parametrize("kwargs,fragment", [
    (dict(activation_scheme="sometimes"), "Unsupported activation scheme"),
    (dict(is_checkpoint_fp8_serialized=False, weight_block_size=[128, 128]), "fp8-serialized"),
    (dict(is_checkpoint_fp8_serialized=True, weight_block_size=[128]), "2 dimensions"),
    (dict(is_checkpoint_fp8_serialized=True, activation_scheme="static", weight_block_size=[128, 128]),
     "dynamic activation scheme"),
])
def test_config_errors(kwargs, fragment):
    with pytest.raises(ValueError, match=fragment):
        Fp8Config(**kwargs)


def test_only_block_quant_is_built():
    with pytest.raises(NotImplementedError):
        Fp8LinearMethod(Fp8Config(is_checkpoint_fp8_serialized=True))
    with pytest.raises(NotImplementedError):
        Fp8MoEMethod(Fp8Config(is_checkpoint_fp8_serialized=True, weight_block_size=[64, 64]))


def test_linear_weights_shapes_and_sentinel():
    m = Fp8LinearMethod(Fp8Config.from_config(DEEPSEEK_QCFG))
    layer = torch.nn.Module()
    # merged gate_up of a tensor-parallel rank: two logical outputs of 2304 rows, K = 7168
    m.create_weights(layer, 7168, [2304, 2304], 7168, 36864, torch.bfloat16, tp_size=8)
    assert layer.weight.shape == (4608, 7168) and layer.weight.dtype == torch.float8_e4m3fn
    assert layer.weight_scale_inv.shape == (36, 56) and layer.weight_scale_inv.dtype == torch.float32
    assert bool((layer.weight_scale_inv == torch.finfo(torch.float32).min).all())   # "not loaded yet"
    assert layer.input_scale is None and layer.logical_widths == [2304, 2304]
    assert not layer.weight.requires_grad
    m.process_weights_after_loading(layer)
    assert layer.weight.shape == (4608, 7168)


def test_linear_tp_divisibility_errors():
    m = Fp8LinearMethod(Fp8Config.from_config(DEEPSEEK_QCFG))
    with pytest.raises(ValueError, match="block_k"):            # row parallel: K/p = 2304/8 = 288
        m.create_weights(torch.nn.Module(), 288, [7168], 2304, 7168, torch.bfloat16, tp_size=8)
    with pytest.raises(ValueError, match="block_n"):            # column parallel: N/p = 1600/8 = 200
        m.create_weights(torch.nn.Module(), 7168, [200], 7168, 1600, torch.bfloat16, tp_size=8)
    with pytest.raises(ValueError, match="block_n"):            # merged weights must align even at p = 1
        m.create_weights(torch.nn.Module(), 7168, [192, 192], 7168, 384, torch.bfloat16, tp_size=1)
    # a ragged single output at p = 1 is allowed (the scale grid is rounded up)
    layer = torch.nn.Module()
    m.create_weights(layer, 7168, [576], 7168, 576, torch.bfloat16, tp_size=1)
    assert layer.weight_scale_inv.shape == (5, 56)


def test_moe_weights_shapes_and_errors():
    m = Fp8MoEMethod(Fp8Config.from_config(DEEPSEEK_QCFG))
    layer = torch.nn.Module()
    m.create_weights(layer, 8, 7168, 2048, torch.bfloat16)
    assert layer.w13_weight.shape == (8, 4096, 7168) and layer.w2_weight.shape == (8, 7168, 2048)
    assert layer.w13_weight_scale_inv.shape == (8, 32, 56) and layer.w2_weight_scale_inv.shape == (8, 56, 16)
    assert m.expert_offsets.shape == (9,) and m.problem_sizes1.shape == (8, 3)
    with pytest.raises(ValueError, match="block_n"):
        m.create_weights(torch.nn.Module(), 8, 7168, 2000, torch.bfloat16)
