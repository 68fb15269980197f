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

from .tp import (ColumnParallelLinear, ParallelMLP, RowParallelLinear, copy_to_parallel,
                 gather_from_sequence_parallel, world_and_rank)


def _world() -> int:
    return world_and_rank()[0]


class RMSNorm(nn.Module):
    """``token_sharded=True``: every rank normalises its own tokens, so the
    gradient of the (replicated) weight is a partial sum and is all-reduced on
    the way back -- otherwise the ranks' copies of the weight drift apart."""

    def __init__(self, d: int, eps: float = 1e-5, token_sharded: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps
        self.token_sharded = token_sharded

    def forward(self, x):
        w = copy_to_parallel(self.weight) if self.token_sharded else self.weight
        return F.rms_norm(x, (x.shape[-1],), w.to(x.dtype), self.eps)


class DecoderLayer(nn.Module):
    """Pre-norm Llama-style block, tensor-parallel: q/k/v and gate/up are fused
    column-parallel layers (heads and FFN columns split on scale-block
    boundaries; one quantize + one GEMM per group), o/down row-parallel with a
    bf16 reduction of the partial outputs.

    ``sequence_parallel=False``: activations between the blocks are replicated,
    row-parallel outputs are all-reduced (chunked under the GEMM), the input
    gradients of the column-parallel groups are all-reduced under their
    weight-gradient GEMMs.  ``sequence_parallel=True``: activations between the
    blocks are sharded over tokens -- norms and residual adds touch tokens /
    world rows -- each column-parallel group all-gathers its input as FP8 codes
    after quantizing this rank's tokens and reduce-scatters its input gradient
    under the weight-gradient GEMM; each row-parallel layer reduce-scatters its
    output and all-gathers its output gradient."""

    def __init__(self, d_model: int, n_heads: int, ffn: int, *, granule: int = 64, sequence_parallel: bool = False,
                 overlap_chunks: int = 1, **layer_kw):
        super().__init__()
        world = _world()
        assert n_heads % world == 0, "heads must divide over the tensor-parallel ranks"
        self.sp = sequence_parallel and world > 1
        self.head_dim = d_model // n_heads
        self.heads_local = n_heads // world
        g_attn = max(granule, self.head_dim)
        self.norm1 = RMSNorm(d_model, token_sharded=self.sp)
        self.qkv = ColumnParallelLinear(d_model, (d_model, d_model, d_model), bias=False, granule=g_attn,
                                        sequence_parallel=self.sp, **layer_kw)
        self.o = RowParallelLinear(d_model, d_model, bias=False, granule=g_attn, reduce_dtype=torch.bfloat16,
                                   sequence_parallel=self.sp, overlap_chunks=overlap_chunks, **layer_kw)
        self.norm2 = RMSNorm(d_model, token_sharded=self.sp)
        self.gate_up = ColumnParallelLinear(d_model, (ffn, ffn), bias=False, granule=granule,
                                            sequence_parallel=self.sp, **layer_kw)
        self.down = RowParallelLinear(ffn, d_model, bias=False, granule=granule, reduce_dtype=torch.bfloat16,
                                      sequence_parallel=self.sp, overlap_chunks=overlap_chunks, **layer_kw)

    def forward(self, x):                      # x: (B, T, d) bf16; with sequence parallelism (B*T/world, d)
        B, T = self.batch_shape if self.sp else x.shape[:2]
        q, k, v = self.qkv(self.norm1(x))          # sequence parallel: the layer gathers its (quantized) input
        shp = (B, T, self.heads_local, self.head_dim)
        a = F.scaled_dot_product_attention(q.reshape(shp).transpose(1, 2), k.reshape(shp).transpose(1, 2),
                                           v.reshape(shp).transpose(1, 2), is_causal=True)
        a = a.transpose(1, 2).reshape(q.shape[:-1] + (self.heads_local * self.head_dim,))
        x = x + self.o(a)
        gate, up = self.gate_up(self.norm2(x))
        return x + self.down(F.silu(gate) * up)


class Decoder(nn.Module):
    """A stack of decoder blocks.  Input and output are ``(B, T, d)``; under
    sequence parallelism the stack works on this rank's token shard in between."""

    def __init__(self, layers: list[DecoderLayer]):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self.sp = bool(layers) and layers[0].sp

    def forward(self, x):
        if not self.sp:
            for layer in self.layers:
                x = layer(x)
            return x
        B, T, d = x.shape
        world, rank = dist.get_world_size(), dist.get_rank()
        tokens = x.reshape(B * T, d)
        rows = tokens.shape[0] // world
        h = tokens[rank * rows:(rank + 1) * rows]
        for layer in self.layers:
            layer.batch_shape = (B, T)
            h = layer(h)
        return gather_from_sequence_parallel(h).reshape(B, T, d)


def build_decoder(n_layers=4, d_model=4096, n_heads=32, ffn=11008, block=64, *, sequence_parallel=False,
                  overlap_chunks=1, **layer_kw) -> nn.Module:
    kw = dict(scale_block_size=block, out_dtype=torch.bfloat16, **layer_kw)
    m = Decoder([DecoderLayer(d_model, n_heads, ffn, granule=block, sequence_parallel=sequence_parallel,
                              overlap_chunks=overlap_chunks, **kw) for _ in range(n_layers)])
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
