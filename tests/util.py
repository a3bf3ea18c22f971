"""Helpers shared by the GPU parity tests."""
import os

import numpy as np
import torch

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MAX_ABS_TOL = 2e-2   # acceptance: bf16 attention outputs vs an fp32 recomputation
MEAN_ABS_TOL = 2e-3


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def assert_close_attn(out: torch.Tensor, ref_fp32: torch.Tensor, what: str = ""):
    diff = (out.float().cpu() - ref_fp32.float().cpu()).abs()
    assert torch.isfinite(out.float()).all(), f"{what}: non-finite output"
    assert diff.max().item() <= MAX_ABS_TOL, f"{what}: max-abs {diff.max().item():.4g} > {MAX_ABS_TOL}"
    assert diff.mean().item() <= MEAN_ABS_TOL, f"{what}: mean-abs {diff.mean().item():.4g} > {MEAN_ABS_TOL}"


def no_device_error():
    from hyprstream_b200 import ffi

    flags = ffi.take_device_error()
    assert flags == 0, f"device error flags {flags}"
