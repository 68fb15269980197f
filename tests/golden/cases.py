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
    "nf_aware": dict(seed=107, M=32, K=64, N=48, bias=True, nf=True),
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


# block-scaled path: weight (N, K), activation (M, K), gradient (M, N); N and K multiples of the block
BLOCK_CASES = {
    "bs32_ef": dict(seed=201, M=64, N=64, K=128, bs=32, ef=True),
    "bs64_ef": dict(seed=202, M=64, N=128, K=128, bs=64, ef=True),
    "bs128_noef": dict(seed=203, M=64, N=128, K=256, bs=128, ef=False),
    "bs32_zero_rows": dict(seed=204, M=32, N=64, K=64, bs=32, ef=True, zero_rows=True),
    "bs64_srr": dict(seed=205, M=32, N=64, K=128, bs=64, ef=False, srr_seed=1234567),
}


def block_inputs(cfg):
    g = torch.Generator().manual_seed(cfg["seed"])
    N, K, M = cfg["N"], cfg["K"], cfg["M"]
    w = torch.randn(N, K, generator=g) * 0.02
    mask = torch.rand(N, K, generator=g) < 0.01
    w = torch.where(mask, w * 50.0, w)
    if cfg.get("zero_rows"):
        w[0] = 0.0            # amax floor
        w[1] = 1.0            # exactly representable: zero residual -> sentinel
        w[2, :32] = 448.0 * 2.0**-9
    err = torch.randn(N, K, generator=g) * 1e-4 if cfg["ef"] else None
    if cfg.get("zero_rows") and err is not None:
        err[:3] = 0.0
    x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16)
    gr = torch.randn(M, N, generator=g) * 0.01
    return w, err, x, gr
