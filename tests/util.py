"""Seeded synthetic inputs for the GEMM tests: bf16 bit patterns in numpy uint16 arrays.

Distributions follow the benchmark configurations: uniform[-1,1], N(0,1) activations, N(0,0.02)
weights, and the reference harness's integer-valued fill (values in [-5,4], common.h:283-289)
for which fp32 accumulation is exact and results must match bit for bit.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def uniform_bits(shape, seed: int) -> np.ndarray:
    return oracle.f32_to_bf16_bits(_rng(seed).uniform(-1.0, 1.0, size=shape).astype(np.float32))


def normal_bits(shape, seed: int, sigma: float = 1.0) -> np.ndarray:
    return oracle.f32_to_bf16_bits((_rng(seed).standard_normal(size=shape) * sigma).astype(np.float32))


def integer_bits(shape, seed: int) -> np.ndarray:
    return oracle.f32_to_bf16_bits(_rng(seed).integers(-5, 5, size=shape).astype(np.float32))


def f16_uniform_bits(shape, seed: int) -> np.ndarray:
    return oracle.f32_to_f16_bits(_rng(seed).uniform(-1.0, 1.0, size=shape).astype(np.float32))


def f16_integer_bits(shape, seed: int) -> np.ndarray:
    return oracle.f32_to_f16_bits(_rng(seed).integers(-5, 5, size=shape).astype(np.float32))


def to_device_f16(bits: np.ndarray):
    import torch
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.float16)


def to_device(bits: np.ndarray):
    """numpy uint16 bit patterns -> torch bfloat16 CUDA tensor (same bits)."""
    import torch
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def to_bits(t) -> np.ndarray:
    """torch bfloat16 tensor (any device) -> numpy uint16 bit patterns."""
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
