"""Seeded synthetic inputs shared by the CPU and GPU tests."""
import numpy as np
import torch


def bf16_from_bits(arr: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)


def gaussian(shape, seed=0, std=1.0, outlier_frac=0.0, outlier_mul=1.0):
    """CPU-generated so that CPU and GPU runs see identical bits."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * std
    if outlier_frac > 0:
        mask = torch.rand(shape, generator=g) < outlier_frac
        x = torch.where(mask, x * outlier_mul, x)
    return x.bfloat16()


def bf16_ulp(ref: torch.Tensor) -> torch.Tensor:
    """Size of one bf16 ulp at |ref| (fp32 tensor), 2^(floor(log2|ref|) - 7); bf16 min normal floor."""
    a = ref.abs().float().clamp(min=2.0 ** -126)
    e = torch.frexp(a)[1] - 1
    return torch.ldexp(torch.ones_like(a), e - 7)
