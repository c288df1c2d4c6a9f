"""Test helpers with the reference's names and argument meaning
(``torch_supa/testing/common_utils.py:64-168``): a CPU tensor and its ``supa`` twin from one random
draw, and a comparison whose golden is always the CPU result."""
from __future__ import annotations

import enum

import numpy as np
import torch

supa_device = "supa"

# Per-element tolerances repeated across the reference's test files (test/test_add.py:23-24).
RTOL = {torch.float32: 1.3e-6, torch.bfloat16: 1.6e-2, torch.float16: 1e-3, torch.float64: 1e-7}
ATOL = {torch.float32: 1e-5, torch.bfloat16: 1e-5, torch.float16: 1e-5, torch.float64: 1e-7}


class RandomMode(enum.Enum):
    uniform = 0
    norm = 1
    range = 2


def create_random_tensor(shape, dtype, format=None, min_value=-5, max_value=5, requires_grad=False,
                         mode: RandomMode = RandomMode.norm, seed=None):
    """Returns ``(cpu_tensor, supa_tensor)`` holding the same values.  Unlike the reference the draw can be
    seeded (its tests are unseeded)."""
    g = torch.Generator()
    if seed is not None:
        g.manual_seed(seed)
    else:
        g.seed()
    shape = tuple(shape)
    if dtype == torch.bool:
        x = torch.randint(0, 2, shape, generator=g).bool()
    elif dtype.is_floating_point:
        if mode is RandomMode.uniform:
            x = (torch.rand(shape, generator=g, dtype=torch.float64) * (max_value - min_value) + min_value).to(dtype)
        else:
            x = torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)
    else:
        x = torch.randint(int(min_value), int(max_value) + 1, shape, generator=g).to(dtype)
    cpu = x.clone().requires_grad_(requires_grad) if requires_grad else x.clone()
    dev = x.to(supa_device)
    if requires_grad:
        dev.requires_grad_(True)
    return cpu, dev


def assert_allclose(tensor_golden, tensor_compare, rtol, atol, equal_nan=False):
    """Golden first, as in the reference.  bf16 goes through ``torch.testing.assert_close``, everything
    else through numpy."""
    golden = tensor_golden.detach().cpu()
    compare = tensor_compare.detach().cpu()
    if golden.dtype == compare.dtype and compare.dtype == torch.bfloat16:
        torch.testing.assert_close(compare, golden, rtol=rtol, atol=atol, equal_nan=equal_nan)
        return
    if golden.dtype == torch.bfloat16:
        golden = golden.float()
    if compare.dtype == torch.bfloat16:
        compare = compare.float()
    np.testing.assert_allclose(golden.numpy(), compare.numpy(), rtol, atol, equal_nan)
