"""Seeds and shapes of the golden cases (shared by the generator and the tests)."""
from __future__ import annotations

import torch

CAST_CASES = {
    "f32_small": (11, (48, 80), torch.float32),
    "bf16": (12, (64, 128), torch.bfloat16),
    "f32_wide": (13, (16, 512), torch.float32),
}

LAYER_CASES = {
    "ef": dict(seed=101, M=32, K=64, N=48, bias=True),
    "ef_3d_nobias": dict(seed=102, M=64, K=128, N=32, bias=False, batch=4),
    "srr": dict(seed=103, M=32, K=64, N=48, bias=True, srr=True),
    "abd": dict(seed=104, M=32, K=64, N=48, bias=False, abd=True),
    "delayed": dict(seed=105, M=32, K=64, N=48, bias=True, delayed=True),
    "hp_grad": dict(seed=106, M=32, K=64, N=48, bias=True, hp=True),
}


def cast_input(seed, shape, dtype):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * 1.7).to(dtype)


def layer_inputs(cfg):
    g = torch.Generator().manual_seed(cfg["seed"])
    M, K, N = cfg["M"], cfg["K"], cfg["N"]
    x = torch.randn(M, K, generator=g)
    if "batch" in cfg:
        x = x.reshape(cfg["batch"], M // cfg["batch"], K)
    w = torch.randn(N, K, generator=g) * 0.05
    b = torch.randn(N, generator=g) * 0.1 if cfg["bias"] else None
    target = torch.randn(*x.shape[:-1], N, generator=g)
    return x, w, b, target
