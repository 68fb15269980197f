"""Synthetic training workloads built from the TCFP-12 layers, for step timing
on 1/2/4/8 GPUs: the two MLP shapes and the 7B-shaped decoder stack named in
the benchmark configurations.  Random-init weights, random inputs; attention
and normalisation are plain torch ops -- only the Linear layers are the
subject here."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .tp import ColumnParallelLinear, ParallelMLP, RowParallelLinear, copy_to_parallel


def _world() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


class RMSNorm(nn.Module):
    def __init__(self, d: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight.to(x.dtype), self.eps)


class DecoderLayer(nn.Module):
    """Pre-norm Llama-style block, tensor-parallel: q/k/v/gate/up column-parallel
    (heads and FFN columns split on scale-block boundaries), o/down row-parallel
    with a bf16 all-reduce of the partial outputs."""

    def __init__(self, d_model: int, n_heads: int, ffn: int, *, granule: int = 64, **layer_kw):
        super().__init__()
        world = _world()
        assert n_heads % world == 0, "heads must divide over the tensor-parallel ranks"
        self.head_dim = d_model // n_heads
        self.heads_local = n_heads // world
        col = dict(bias=False, granule=max(granule, self.head_dim), reduce_input_grad=False, **layer_kw)
        self.norm1 = RMSNorm(d_model)
        self.q = ColumnParallelLinear(d_model, d_model, **col)
        self.k = ColumnParallelLinear(d_model, d_model, **col)
        self.v = ColumnParallelLinear(d_model, d_model, **col)
        self.o = RowParallelLinear(d_model, d_model, bias=False, granule=max(granule, self.head_dim),
                                   reduce_dtype=torch.bfloat16, **layer_kw)
        self.norm2 = RMSNorm(d_model)
        colf = dict(bias=False, granule=granule, reduce_input_grad=False, **layer_kw)
        self.gate = ColumnParallelLinear(d_model, ffn, **colf)
        self.up = ColumnParallelLinear(d_model, ffn, **colf)
        self.down = RowParallelLinear(ffn, d_model, bias=False, granule=granule, reduce_dtype=torch.bfloat16, **layer_kw)

    def forward(self, x):                      # x: (B, T, d) bf16
        B, T, _ = x.shape
        h = copy_to_parallel(self.norm1(x))
        shp = (B, T, self.heads_local, self.head_dim)
        q = self.q(h).view(shp).transpose(1, 2)
        k = self.k(h).view(shp).transpose(1, 2)
        v = self.v(h).view(shp).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        a = a.transpose(1, 2).reshape(B, T, self.heads_local * self.head_dim)
        x = x + self.o(a)
        h = copy_to_parallel(self.norm2(x))
        f = F.silu(self.gate(h)) * self.up(h)
        return x + self.down(f)


def build_decoder(n_layers=4, d_model=4096, n_heads=32, ffn=11008, block=64, **layer_kw) -> nn.Module:
    kw = dict(scale_block_size=block, out_dtype=torch.bfloat16, **layer_kw)
    m = nn.Sequential(*[DecoderLayer(d_model, n_heads, ffn, granule=block, **kw) for _ in range(n_layers)])
    _name_layers(m)
    _init_weights(m)
    return m


def build_mlp(d_model: int, d_hidden: int, **layer_kw) -> nn.Module:
    m = ParallelMLP(d_model, d_hidden, **layer_kw)
    _name_layers(m)
    _init_weights(m)
    return m


def _name_layers(model: nn.Module) -> None:
    from .nn import TCFPLinear

    for name, mod in model.named_modules():
        if isinstance(mod, TCFPLinear):
            mod._param_name = name


def _init_weights(model: nn.Module) -> None:
    from .nn import TCFPLinear

    rank = dist.get_rank() if dist.is_initialized() else 0
    g = torch.Generator().manual_seed(1005 + rank)
    with torch.no_grad():
        for mod in model.modules():
            if isinstance(mod, TCFPLinear):
                mod.weight.copy_(torch.randn(mod.weight.shape, generator=g) * 0.02)
