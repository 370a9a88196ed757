"""Owners of the block-FP8 parameters: the block-quantised part of the reference's
python/sglang/srt/layers/quantization/fp8.py.

  Fp8Config         :105-184   checkpoint description (`quant_method`, `activation_scheme`,
                               `weight_block_size`, `ignored_layers`) and its argument errors
  Fp8LinearMethod   :187-488   `weight [N_part, K_part]` e4m3 + `weight_scale_inv
                               [ceil(N_part/128), ceil(K_part/128)]` fp32, the tensor-parallel
                               divisibility errors (:239-262), `apply` -> the linear glue (:459-478)
  Fp8MoEMethod      :491-1065  `w13_weight [E, 2I, H]`, `w2_weight [E, H, I]`, their `_scale_inv`
                               tensors and the routing scratch (:551-671); `apply` ->
                               cutlass_fused_experts_fp8 with transposed views (:1030-1065)

Only the block-quantised, dynamic-activation, fp8-serialised form exists here; the per-tensor,
Marlin, ROCm and CPU branches of the reference belong to other paths and raise
NotImplementedError.  The reference reads the tensor-parallel world size from its global parallel
state; here it is an argument (`tp_size`), the only difference in the signatures.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .fp8_utils import (deepgemm_w8a8_block_fp8_linear_with_fallback, dispatch_w8a8_block_fp8_linear,
                        requant_weight_ue8m0_inplace)

ACTIVATION_SCHEMES = ["static", "dynamic"]
FP8 = torch.float8_e4m3fn


class Fp8Config:
    """Config class for FP8 (fp8.py:105-184)."""

    def __init__(self, is_checkpoint_fp8_serialized: bool = False, activation_scheme: str = "dynamic",
                 ignored_layers: Optional[List[str]] = None, weight_block_size: Optional[List[int]] = None) -> None:
        self.is_checkpoint_fp8_serialized = is_checkpoint_fp8_serialized
        if activation_scheme not in ACTIVATION_SCHEMES:
            raise ValueError(f"Unsupported activation scheme {activation_scheme}")
        self.activation_scheme = activation_scheme
        self.ignored_layers = ignored_layers or []
        if weight_block_size is not None:
            if not is_checkpoint_fp8_serialized:
                raise ValueError("The block-wise quantization only supports fp8-serialized checkpoint for now.")
            if len(weight_block_size) != 2:
                raise ValueError("The quantization block size of weight must have 2 dimensions, but got "
                                 f"{len(weight_block_size)} dimensions.")
            if activation_scheme != "dynamic":
                raise ValueError("The block-wise quantization only supports dynamic activation scheme for now, "
                                 f"but got {activation_scheme} activation scheme.")
        self.weight_block_size = weight_block_size

    @classmethod
    def get_name(cls) -> str:
        return "fp8"

    @classmethod
    def get_supported_act_dtypes(cls) -> List[torch.dtype]:
        return [torch.bfloat16, torch.half]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100      # this build runs on sm_100a only (the reference says 80)

    @classmethod
    def get_config_filenames(cls) -> List[str]:
        return []

    @staticmethod
    def _get(config: Dict[str, Any], key: str, default: Any = ...):
        if key in config:
            return config[key]
        if default is ...:
            raise ValueError(f"Cannot find any of ['{key}'] in the model's quantization config.")
        return default

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "Fp8Config":
        """`config` is the `quantization_config` dictionary of a Hugging Face `config.json`."""
        quant_method = cls._get(config, "quant_method")
        return cls(is_checkpoint_fp8_serialized="fp8" in quant_method,
                   activation_scheme=cls._get(config, "activation_scheme"),
                   ignored_layers=cls._get(config, "ignored_layers", None),
                   weight_block_size=cls._get(config, "weight_block_size", None))

    def get_scaled_act_names(self) -> List[str]:
        return []


def _require_block_quant(cfg: Fp8Config) -> None:
    if cfg.weight_block_size is None:
        raise NotImplementedError("only block-quantised FP8 (weight_block_size = [128, 128]) is built")
    if list(cfg.weight_block_size) != [128, 128]:
        raise NotImplementedError(f"weight_block_size {cfg.weight_block_size}: the kernels are built for [128, 128]")


class Fp8LinearMethod:
    """Linear method for block-quantised FP8 (fp8.py:187-488)."""

    def __init__(self, quant_config: Fp8Config, scale_ue8m0: bool = False):
        """scale_ue8m0: the reference's DeepGEMM mode with power-of-two scales, its default on Blackwell
        (DEEPGEMM_SCALE_UE8M0; fp8.py:345-357 re-quantises the weights after loading, fp8_utils.py:215-258 is the
        linear): weights get power-of-two block scales, activations are quantised with packed UE8M0 scales, and
        the product runs on the tensor core's block-scaling path."""
        _require_block_quant(quant_config)
        self.quant_config = quant_config
        self.block_quant = True
        self.scale_ue8m0 = bool(scale_ue8m0)
        self.w8a8_block_fp8_linear = dispatch_w8a8_block_fp8_linear()

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: List[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, tp_size: int = 1,
                       device: Optional[torch.device] = None, **extra_weight_attrs) -> None:
        output_size_per_partition = sum(output_partition_sizes)
        block_n, block_k = self.quant_config.weight_block_size
        # required by row parallel (fp8.py:245-251)
        if tp_size > 1 and input_size // input_size_per_partition == tp_size:
            if input_size_per_partition % block_k != 0:
                raise ValueError(f"Weight input_size_per_partition = {input_size_per_partition} is not divisible by "
                                 f"weight quantization block_k = {block_k}.")
        # required by column parallel or merged weights (fp8.py:252-262)
        if (tp_size > 1 and output_size // output_size_per_partition == tp_size) or len(output_partition_sizes) > 1:
            for output_partition_size in output_partition_sizes:
                if output_partition_size % block_n != 0:
                    raise ValueError(f"Weight output_partition_size = {output_partition_size} is not divisible by "
                                     f"weight quantization block_n = {block_n}.")
        layer.logical_widths = output_partition_sizes
        layer.input_size_per_partition = input_size_per_partition
        layer.output_size_per_partition = output_size_per_partition
        layer.orig_dtype = params_dtype
        assert self.quant_config.activation_scheme == "dynamic"
        weight = torch.nn.Parameter(
            torch.empty(output_size_per_partition, input_size_per_partition, dtype=FP8, device=device),
            requires_grad=False)
        scale = torch.nn.Parameter(
            torch.full(((output_size_per_partition + block_n - 1) // block_n,
                        (input_size_per_partition + block_k - 1) // block_k),
                       torch.finfo(torch.float32).min, dtype=torch.float32, device=device),
            requires_grad=False)
        layer.register_parameter("weight", weight)
        layer.register_parameter("weight_scale_inv", scale)
        layer.register_parameter("input_scale", None)

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        """Block-quantised weights are used as loaded (fp8.py:334-358); only the wrappers are renewed."""
        layer.weight = torch.nn.Parameter(layer.weight.data, requires_grad=False)
        layer.weight_scale_inv = torch.nn.Parameter(layer.weight_scale_inv.data, requires_grad=False)
        if self.scale_ue8m0 and layer.weight.shape[0] % 128 == 0 and layer.weight.shape[1] % 128 == 0:
            requant_weight_ue8m0_inplace(layer.weight, layer.weight_scale_inv, self.quant_config.weight_block_size)
            layer.weight_scale_is_ue8m0 = True

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        if getattr(layer, "weight_scale_is_ue8m0", False):
            return deepgemm_w8a8_block_fp8_linear_with_fallback(
                input=x, weight=layer.weight, block_size=self.quant_config.weight_block_size,
                weight_scale=layer.weight_scale_inv, input_scale=None, bias=bias, scale_ue8m0=True,
                weight_scale_ue8m0=True)
        return self.w8a8_block_fp8_linear(input=x, weight=layer.weight, block_size=self.quant_config.weight_block_size,
                                          weight_scale=layer.weight_scale_inv, input_scale=None, bias=bias)


class Fp8MoEMethod:
    """MoE method for block-quantised FP8 experts (fp8.py:491-1065, the SGLANG_CUTLASS_MOE branch)."""

    def __init__(self, quant_config: Fp8Config):
        _require_block_quant(quant_config)
        self.quant_config = quant_config
        self.block_quant = True

    def create_weights(self, layer: torch.nn.Module, num_experts: int, hidden_size: int, intermediate_size: int,
                       params_dtype: torch.dtype, tp_size: int = 1, device: Optional[torch.device] = None,
                       **extra_weight_attrs) -> None:
        block_n, block_k = self.quant_config.weight_block_size
        if intermediate_size % block_n != 0:
            raise ValueError(f"The output_size of gate's and up's weight = {intermediate_size} is not divisible by "
                             f"weight quantization block_n = {block_n}.")
        if tp_size > 1 and intermediate_size % block_k != 0:
            raise ValueError(f"The input_size of down's weight = {intermediate_size} is not divisible by "
                             f"weight quantization block_k = {block_k}.")
        assert self.quant_config.activation_scheme == "dynamic"

        def param(*shape, dtype, fill=None):
            t = torch.empty(*shape, dtype=dtype, device=device) if fill is None else \
                torch.full(shape, fill, dtype=dtype, device=device)
            return torch.nn.Parameter(t, requires_grad=False)

        layer.register_parameter("w13_weight", param(num_experts, 2 * intermediate_size, hidden_size, dtype=FP8))
        layer.register_parameter("w2_weight", param(num_experts, hidden_size, intermediate_size, dtype=FP8))
        layer.register_parameter("w13_weight_scale_inv", param(
            num_experts, 2 * ((intermediate_size + block_n - 1) // block_n), (hidden_size + block_k - 1) // block_k,
            dtype=torch.float32, fill=1.0))
        layer.register_parameter("w2_weight_scale_inv", param(
            num_experts, (hidden_size + block_n - 1) // block_n, (intermediate_size + block_k - 1) // block_k,
            dtype=torch.float32, fill=1.0))
        # routing tables, written on the device by every forward (fp8.py:661-671); the stride, pointer
        # and workspace tensors of the reference's CUTLASS launcher have no use here
        self.expert_offsets = torch.empty(num_experts + 1, device=device, dtype=torch.int32)
        self.problem_sizes1 = torch.empty(num_experts, 3, device=device, dtype=torch.int32)
        self.problem_sizes2 = torch.empty(num_experts, 3, device=device, dtype=torch.int32)

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        return

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, topk_output, *, activation: str = "silu",
              routed_scaling_factor: Optional[float] = None) -> torch.Tensor:
        from ..moe.cutlass_moe import cutlass_fused_experts_fp8
        assert activation == "silu", "only SiLU gating is built"
        topk_weights, topk_ids = topk_output[0], topk_output[1]
        output = cutlass_fused_experts_fp8(
            x, layer.w13_weight.transpose(1, 2), layer.w2_weight.transpose(1, 2),
            layer.w13_weight_scale_inv.transpose(1, 2), layer.w2_weight_scale_inv.transpose(1, 2),
            topk_weights, topk_ids, expert_offsets=self.expert_offsets, problem_sizes1=self.problem_sizes1,
            problem_sizes2=self.problem_sizes2, use_fp8_blockscale=True)
        if routed_scaling_factor is not None:
            output *= routed_scaling_factor
        return output
