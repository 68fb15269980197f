"""Seeded inputs shared by the tests: made on the CPU so that the oracle and
the GPU see identical bits."""
from __future__ import annotations

import torch


def gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def weights(seed: int, n: int, k: int, std: float = 0.02, outliers: bool = False) -> torch.Tensor:
    g = gen(seed)
    w = torch.randn(n, k, generator=g) * std
    if outliers:
        mask = torch.rand(n, k, generator=g) < 0.001
        w = torch.where(mask, w * 50.0, w)
    return w


def acts(seed: int, m: int, k: int, dtype=torch.bfloat16) -> torch.Tensor:
    return torch.randn(m, k, generator=gen(seed)).to(dtype)


def u8(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.uint8).cpu()


def bits(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().contiguous().view(torch.int32)


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp(min=1e-30))
