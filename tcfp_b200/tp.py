"""Column- and row-parallel TCFP-12 linear layers for 1/2/4/8 GPUs of one node.

The reference has no distributed code; this follows the usual tensor-parallel
split of a transformer block.  Column-parallel layers shard the output
features (each rank quantizes and multiplies its own rows of W -- block scales
are per (row, K block), so every quantized byte equals the unsharded layer's);
row-parallel layers shard the input features on scale-block boundaries and sum
their partial outputs with an all-reduce over NCCL (NVLink / NVSwitch).

    y = RowParallel(act(ColumnParallel(x)))      # one all-reduce forward, one backward

One process per GPU, ``torch.distributed`` for the plumbing.  The layer class
is injectable so that the communication logic is testable on CPU with gloo.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
import torch.nn as nn


def shard_bounds(size: int, world: int, rank: int, granule: int = 1) -> tuple[int, int]:
    """[start, end) of ``rank``'s shard of ``size`` features, on multiples of
    ``granule`` (the scale block), as even as the granules allow: 11008
    features in blocks of 64 over 8 ranks gives four shards of 22 blocks and
    four of 21."""
    if size % granule != 0:
        raise ValueError(f"size ({size}) must be divisible by the shard granule ({granule})")
    units = size // granule
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    n = base + (1 if rank < extra else 0)
    if n == 0:
        raise ValueError(f"{size} features in granules of {granule} cannot be split over {world} ranks")
    return start * granule, (start + n) * granule


class _CopyToParallel(torch.autograd.Function):
    """Identity forward; all-reduce of the gradient backward (input of a
    column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _ReduceFromParallel(torch.autograd.Function):
    """All-reduce forward (output of a row-parallel layer); identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


# ---------------------------------------------------------------------------
# sequence parallelism: the token dimension (dim 0 of a (tokens, features)
# matrix) is sharded between the tensor-parallel regions, so norms, residual
# adds and dtype conversions run on tokens / world rows instead of replicated
# ---------------------------------------------------------------------------

def _all_gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    out = torch.empty((x.shape[0] * world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows = x.shape[0] // world
    if x.is_cuda:
        out = torch.empty((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), op=dist.ReduceOp.SUM, group=group)
        return out
    # gloo has no reduce-scatter: reduce everywhere, keep this rank's rows (CPU tests only)
    x = x.contiguous().clone()
    dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x[rank * rows:(rank + 1) * rows].clone()


class _GatherFromSequenceParallel(torch.autograd.Function):
    """All-gather the token shards forward (input of a column-parallel layer);
    reduce-scatter the gradient backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return x
        return _all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        if not dist.is_initialized() or dist.get_world_size(ctx.group) == 1:
            return g, None
        return _reduce_scatter_rows(g, ctx.group), None


class _ScatterToSequenceParallel(torch.autograd.Function):
    """Reduce-scatter the partial outputs of a row-parallel layer forward (sum
    over ranks, keep this rank's tokens); all-gather the gradient backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return x
        return _reduce_scatter_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        if not dist.is_initialized() or dist.get_world_size(ctx.group) == 1:
            return g, None
        return _all_gather_rows(g, ctx.group), None


def gather_from_sequence_parallel(x: torch.Tensor, group=None) -> torch.Tensor:
    return _GatherFromSequenceParallel.apply(x, group)


def scatter_to_sequence_parallel(x: torch.Tensor, group=None) -> torch.Tensor:
    return _ScatterToSequenceParallel.apply(x, group)


def _default_factory(in_features: int, out_features: int, bias: bool, **kw) -> nn.Module:
    from .nn import TCFPLinear

    return TCFPLinear(in_features, out_features, bias=bias, use_tensor_cores=True, **kw)


class ColumnParallelLinear(nn.Module):
    """``y_local = x @ W[rows of this rank].T``; output stays sharded."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, group=None, granule: int = 16,
                 layer_factory: Callable[..., nn.Module] = _default_factory, reduce_input_grad: bool = True,
                 **layer_kw):
        super().__init__()
        self.group = group
        # several column-parallel layers fed by one tensor (q/k/v, gate/up) share a single
        # gradient all-reduce: the caller applies copy_to_parallel once and turns this off
        self.reduce_input_grad = reduce_input_grad
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.out_start, self.out_end = shard_bounds(out_features, world, rank, granule)
        self.in_features, self.out_features = in_features, out_features
        self.inner = layer_factory(in_features, self.out_end - self.out_start, bias, **layer_kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.reduce_input_grad:
            x = _CopyToParallel.apply(x, self.group)
        return self.inner(x)


def copy_to_parallel(x: torch.Tensor, group=None) -> torch.Tensor:
    """Identity forward, gradient all-reduce backward."""
    return _CopyToParallel.apply(x, group)


class RowParallelLinear(nn.Module):
    """``y = sum_ranks x[..., cols of this rank] @ W[:, cols].T`` (+ bias once)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, group=None, granule: int = 16,
                 layer_factory: Callable[..., nn.Module] = _default_factory, reduce_dtype: torch.dtype | None = None,
                 sequence_parallel: bool = False, **layer_kw):
        super().__init__()
        self.group = group
        # with sequence parallelism the output is reduce-scattered over tokens instead of all-reduced
        self.sequence_parallel = sequence_parallel
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_start, self.in_end = shard_bounds(in_features, world, rank, granule)
        self.in_features, self.out_features = in_features, out_features
        self.reduce_dtype = reduce_dtype
        self.inner = layer_factory(self.in_end - self.in_start, out_features, False, **layer_kw)
        # the bias is added after the reduction, once
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        y = self.inner(x_shard)
        if self.reduce_dtype is not None and y.dtype != self.reduce_dtype:
            y = y.to(self.reduce_dtype)        # bf16 on the wire halves the NVLink bytes
        if self.sequence_parallel:
            y = _ScatterToSequenceParallel.apply(y, self.group)
        else:
            y = _ReduceFromParallel.apply(y, self.group)
        if self.bias is not None:
            # under sequence parallelism every rank adds the bias to its own tokens only, so the
            # bias gradient is a partial sum: all-reduce it on the way back
            b = _CopyToParallel.apply(self.bias, self.group) if self.sequence_parallel else self.bias
            y = y + b.to(y.dtype)
        return y


class ParallelMLP(nn.Module):
    """``down(act(up(x)))`` with ``up`` column-parallel and ``down``
    row-parallel: the hidden activation never leaves its rank.  With
    ``sequence_parallel`` the input and output are this rank's token shard
    (rows); the input is all-gathered before ``up`` and the output of ``down``
    reduce-scattered."""

    def __init__(self, d_model: int, d_hidden: int, *, group=None, granule: int = 16, bias: bool = True,
                 activation: Callable[[torch.Tensor], torch.Tensor] = torch.nn.functional.gelu,
                 layer_factory: Callable[..., nn.Module] = _default_factory, reduce_dtype=None,
                 sequence_parallel: bool = False, **layer_kw):
        super().__init__()
        self.group = group
        self.sequence_parallel = sequence_parallel
        self.up = ColumnParallelLinear(d_model, d_hidden, bias, group=group, granule=granule,
                                       layer_factory=layer_factory, reduce_input_grad=not sequence_parallel,
                                       **layer_kw)
        self.down = RowParallelLinear(d_hidden, d_model, bias, group=group, granule=granule,
                                      layer_factory=layer_factory, reduce_dtype=reduce_dtype,
                                      sequence_parallel=sequence_parallel, **layer_kw)
        self.activation = activation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            x = _GatherFromSequenceParallel.apply(x, self.group)
        return self.down(self.activation(self.up(x)))
