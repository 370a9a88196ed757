"""Shared helpers for the tests: golden-vector loading and dtype views."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FP8 = torch.float8_e4m3fn


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def as_fp8(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(FP8)


def as_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def as_f16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float16)


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def same_bits(x, y):
    """Bitwise equality for fp8/bf16/fp32 tensors."""
    x, y = x.detach().cpu().contiguous(), y.detach().cpu().contiguous()
    assert x.dtype == y.dtype and x.shape == y.shape, (x.dtype, y.dtype, x.shape, y.shape)
    iv = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[x.element_size()]
    return bool(torch.equal(x.view(iv), y.view(iv)))


def count_diff_bits(x, y):
    x, y = x.detach().cpu().contiguous(), y.detach().cpu().contiguous()
    iv = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[x.element_size()]
    return int((x.view(iv) != y.view(iv)).sum())
