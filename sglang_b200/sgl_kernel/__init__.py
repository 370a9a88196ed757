"""Drop-in for the block-FP8 subset of the reference's `sgl_kernel` package.

Importing this module registers the operators under torch.ops.sgl_kernel with the reference's
schemas verbatim (sgl-kernel/csrc/common_extension.cc:111-119,192-207), implemented for the
CUDA dispatch key by the B200 C-ABI library, and exposes the same-named Python wrappers
(sgl-kernel/python/sgl_kernel/{gemm,moe}.py).
"""
import torch

from .gemm import fp8_blockwise_scaled_mm, sgl_per_token_group_quant_fp8

_SCHEMAS = {
    "fp8_blockwise_scaled_mm":
        "(Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype) -> Tensor",
    "sgl_per_token_group_quant_fp8":
        "(Tensor input, Tensor output_q, Tensor output_s, int group_size, float eps, float fp8_min, "
        "float fp8_max, bool scale_ue8m0) -> ()",
}
_IMPLS = {
    "fp8_blockwise_scaled_mm": fp8_blockwise_scaled_mm,
    "sgl_per_token_group_quant_fp8": sgl_per_token_group_quant_fp8,
}

_library = None


def register_torch_ops() -> None:
    """Idempotent; skipped for operators another package (the real sgl_kernel) already defined."""
    global _library
    if _library is not None:
        return
    _library = torch.library.Library("sgl_kernel", "FRAGMENT")
    for name, schema in _SCHEMAS.items():
        try:
            _library.define(name + schema)
        except RuntimeError:
            continue  # already defined elsewhere: leave that definition alone
        _library.impl(name, _IMPLS[name], "CUDA")


register_torch_ops()

__all__ = ["fp8_blockwise_scaled_mm", "sgl_per_token_group_quant_fp8", "register_torch_ops"]
