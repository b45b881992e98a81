"""Helpers shared by the GPU parity tests: seeded inputs, layout conversion through the library, comparison."""
from __future__ import annotations

import torch

from oracle import dense as odense

DT = {"bf16": torch.bfloat16, "fp16": torch.float16}


def require_gpu():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def randn(shape, seed, scale=1.0, dtype=torch.bfloat16):
    """Seeded on the CPU so that the oracle and the device see the same bytes."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def rand_e4m3(shape, seed, scale=0.5):
    w = randn(shape, seed, scale, torch.float32).to(torch.float8_e4m3fn)
    raw = w.view(torch.uint8)
    assert not bool(((raw & 0x7F) == 0x7F).any()), "NaN encoding in generated e4m3 weights"
    return w


def assert_close(got, want, what="", atol=1e-2, rtol=1e-2, scale_atol=False):
    rep = odense.error_report(got.detach().cpu(), want, atol=atol, rtol=rtol, scale_atol=scale_atol)
    assert rep["ok"], f"{what}: {rep}"
    return rep
