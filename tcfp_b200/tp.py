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

Overlap.  When the sharded layer is a ``TCFPLinear`` the collectives are
started from inside its autograd Function (``nn.LayerHooks``): a row-parallel
layer computes its output in row chunks and all-reduces chunk ``i`` on NCCL's
stream while the GEMM of chunk ``i + 1`` runs; a column-parallel layer starts
the all-reduce of its input gradient as soon as the dX GEMM is queued and
computes the weight gradient underneath it.

Scaling granularity.  With block scaling every shard's quantized bytes equal
the unsharded layer's.  With per-tensor scaling each shard scales by its OWN
amax (per-shard scaling, finer than the unsharded layer's single scale); the
reference has no distributed form to match, and reproducing the unsharded
scale would cost two dependent all-reduce(max) rounds per layer per step.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
import torch.nn as nn


_COLLECTIVES_ENABLED = True


class collectives_disabled:
    """Measurement aid: inside this context the data-path collectives of this
    module return at once, leaving the local partial results in place.  The
    numbers a model computes are then wrong; the time it takes is what the
    step costs without communication, and the difference from the normal step
    is the communication time that is not hidden behind compute."""

    def __enter__(self):
        global _COLLECTIVES_ENABLED
        self._prev = _COLLECTIVES_ENABLED
        _COLLECTIVES_ENABLED = False
        return self

    def __exit__(self, *exc):
        global _COLLECTIVES_ENABLED
        _COLLECTIVES_ENABLED = self._prev
        return False


_FORCE_SINGLE = False


class single_rank:
    """Measurement aid: layers constructed inside this context are built
    unsharded (world size 1) even under ``torch.distributed``, so that a
    multi-GPU run can time the single-GPU form of its own workload on the same
    box (run it under ``collectives_disabled()``: the hooks of such layers
    would otherwise still address the process group)."""

    def __enter__(self):
        global _FORCE_SINGLE
        self._prev = _FORCE_SINGLE
        _FORCE_SINGLE = True
        return self

    def __exit__(self, *exc):
        global _FORCE_SINGLE
        _FORCE_SINGLE = self._prev
        return False


def world_and_rank(group=None) -> tuple[int, int]:
    """(world size, rank) the tensor-parallel layers shard by."""
    if _FORCE_SINGLE or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def _active(group) -> bool:
    return _COLLECTIVES_ENABLED and dist.is_initialized() and dist.get_world_size(group) > 1


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
        if _active(ctx.group):
            # reduce a private copy: autograd may hand the same gradient tensor to other consumers
            g = g.clone(memory_format=torch.contiguous_format)
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _ReduceFromParallel(torch.autograd.Function):
    """All-reduce forward (output of a row-parallel layer); identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        if _active(group):
            # the partial output is this rank's own fresh GEMM result: reduce it in place and tell autograd
            if x.is_contiguous():
                dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
                ctx.mark_dirty(x)
            else:
                x = x.contiguous()
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
    if not _COLLECTIVES_ENABLED:
        # measurement aid: right shape, this rank's rows everywhere.  Real values matter: leaving the other
        # ranks' rows unfilled (zeros) made the same step 25 % faster, because GEMMs on zeros draw less power
        # and the clock rises -- a time that says nothing about the step.
        out.view(world, *x.shape).copy_(x.unsqueeze(0).expand(world, *x.shape))
        return out
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if x.shape[0] % world != 0:
        raise ValueError(f"sequence parallelism needs the token count ({x.shape[0]}) to be a multiple of the "
                         f"tensor-parallel world size ({world})")
    rows = x.shape[0] // world
    if not _COLLECTIVES_ENABLED:           # measurement aid: right shape, unreduced rows
        return x[rank * rows:(rank + 1) * rows].clone()
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


def _is_tcfp(layer: nn.Module) -> bool:
    from .nn import TCFPLinear

    return isinstance(layer, TCFPLinear)


class _Pending:
    """Handle of an asynchronous collective; ``wait()`` makes the current
    stream wait for it (no host synchronisation with NCCL)."""

    def __init__(self, work):
        self.work = work

    def wait(self):
        if self.work is not None:
            self.work.wait()


def _all_reduce_async(t: torch.Tensor, group):
    if not _active(group):
        return None
    return _Pending(dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group, async_op=True))


class _PendingWithInput(_Pending):
    """A pending collective that also keeps its input alive until waited for."""

    def __init__(self, work, keep):
        super().__init__(work)
        self.keep = keep

    def wait(self):
        super().wait()
        self.keep = None


class SequenceParallelIO:
    """The collectives of a layer whose input is this rank's token shard
    (``nn.LayerHooks.sp``): all-gather of row-sharded matrices -- FP8 codes go
    over the wire as bytes -- and of the ``(K / bs, rows)`` exponent planes,
    and the asynchronous reduce-scatter of the full input gradient."""

    def __init__(self, group=None):
        self.group = group

    def _world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def gather_rows(self, t: torch.Tensor) -> torch.Tensor:
        if self._world() == 1:
            return t
        t = t.contiguous()
        wire = t.view(torch.uint8) if t.element_size() == 1 else t        # NCCL has no FP8 type; bytes are bytes
        return _all_gather_rows(wire, self.group).view(t.dtype)

    def gather_rows_async(self, t: torch.Tensor):
        """Starts the all-gather of a row-sharded matrix; returns ``(handle
        or None, gathered matrix)``, valid once the handle has been waited for."""
        world = self._world()
        if world == 1:
            return None, t
        if not _COLLECTIVES_ENABLED or not t.is_cuda:
            return None, self.gather_rows(t)
        t = t.contiguous()
        out = torch.empty((t.shape[0] * world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        work = dist.all_gather_into_tensor(out, t, group=self.group, async_op=True)
        return _PendingWithInput(work, t), out

    def gather_planes(self, planes: torch.Tensor) -> torch.Tensor:
        """``(P, rows_local)`` -> ``(P, rows)``: the row index is the fast dimension of a plane."""
        world = self._world()
        if world == 1:
            return planes
        P, r = planes.shape
        g = _all_gather_rows(planes.contiguous(), self.group)             # (world * P, r), rank-major
        return g.view(world, P, r).permute(1, 0, 2).reshape(P, world * r)

    def scatter_rows_async(self, full: torch.Tensor):
        """Starts ``reduce_scatter(full)`` over the token dimension; returns
        ``(handle or None, this rank's rows)``.  The rows are valid once the
        handle has been waited for."""
        world = self._world()
        if world == 1:
            return None, full
        rank = dist.get_rank(self.group)
        if full.shape[0] % world != 0:
            raise ValueError(f"sequence parallelism needs the token count ({full.shape[0]}) to be a multiple of the "
                             f"tensor-parallel world size ({world})")
        rows = full.shape[0] // world
        if not _COLLECTIVES_ENABLED or not full.is_cuda:
            # measurement aid (unreduced rows), or gloo on CPU, which has no reduce-scatter
            return None, _reduce_scatter_rows(full, self.group)
        full = full.contiguous()
        out = torch.empty((rows,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
        work = dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        return _PendingWithInput(work, full), out


class ColumnParallelLinear(nn.Module):
    """``y_local = x @ W[rows of this rank].T``; output stays sharded.

    ``out_features`` may be a tuple: several projections fed by the same input
    (q/k/v, gate/up) fused into ONE layer whose local weight is the
    concatenation of this rank's shard of each part -- one weight quantizer
    launch, one activation quantizer launch and one GEMM instead of one per
    part, and a single input-gradient all-reduce.  ``forward`` then returns a
    tuple of the parts' local outputs.  Scale blocks are per weight row, so
    the fused layer's quantized bytes are those of the separate layers.

    ``sequence_parallel=True``: the input is this rank's token shard
    ``(tokens / world, in_features)`` and the output covers all tokens.  A
    ``TCFPLinear`` inside gathers the activation AFTER quantizing it (FP8
    codes and exponents on the wire, the quantizer runs on tokens / world
    rows) and reduce-scatters the input gradient under its weight-gradient
    GEMM; any other layer gets a plain all-gather in front.
    """

    def __init__(self, in_features: int, out_features, bias: bool = True, *, group=None, granule: int = 16,
                 layer_factory: Callable[..., nn.Module] = _default_factory, reduce_input_grad: bool = True,
                 comm_sms: int = 32, sequence_parallel: bool = False, **layer_kw):
        super().__init__()
        self.group = group
        self.sequence_parallel = sequence_parallel
        if sequence_parallel:
            reduce_input_grad = False      # the reduce-scatter of the token shards is the reduction
        # several column-parallel layers fed by one tensor may share a single gradient all-reduce:
        # the caller applies copy_to_parallel once and turns this off
        self.reduce_input_grad = reduce_input_grad
        world, rank = world_and_rank(group)
        self.fused = isinstance(out_features, (tuple, list))
        parts = tuple(out_features) if self.fused else (out_features,)
        self.bounds = [shard_bounds(n, world, rank, granule) for n in parts]
        self.local_sizes = [e - s for s, e in self.bounds]
        self.out_start, self.out_end = self.bounds[0]
        self.in_features, self.out_features = in_features, out_features
        self.inner = layer_factory(in_features, sum(self.local_sizes), bias, **layer_kw)
        # a TCFPLinear starts the gradient all-reduce itself, under its weight-gradient GEMM
        self._overlap = reduce_input_grad and _is_tcfp(self.inner)
        if self._overlap:
            from .nn import LayerHooks

            # the weight-gradient GEMM leaves `comm_sms` SMs to NCCL while the input gradient is being reduced
            self.inner._hooks = LayerHooks(dx_hook=lambda g: _all_reduce_async(g, self.group), reserve_sms=comm_sms)
        self._sp_fused = sequence_parallel and world > 1 and _is_tcfp(self.inner)
        if self._sp_fused:
            from .nn import LayerHooks

            self.inner._hooks = LayerHooks(sp=SequenceParallelIO(group), reserve_sms=comm_sms)

    def forward(self, x: torch.Tensor):
        if self.sequence_parallel and not self._sp_fused:
            x = _GatherFromSequenceParallel.apply(x, self.group)
        if self.reduce_input_grad and not self._overlap:
            x = _CopyToParallel.apply(x, self.group)
        y = self.inner(x)
        if self.fused:
            return torch.split(y, self.local_sizes, dim=-1)
        return y


def copy_to_parallel(x: torch.Tensor, group=None) -> torch.Tensor:
    """Identity forward, gradient all-reduce backward."""
    return _CopyToParallel.apply(x, group)


class RowParallelLinear(nn.Module):
    """``y = sum_ranks x[..., cols of this rank] @ W[:, cols].T`` (+ bias once).

    With a ``TCFPLinear`` inside, the reduction happens in place inside the
    layer's autograd Function (the gradient of an all-reduced sum is the
    identity).  ``overlap_chunks > 1`` produces the partial output in row
    chunks and starts each chunk's all-reduce while the next chunk's GEMM runs.
    Measured on 2 and 8 B200s this does not pay: the persistent GEMM occupies
    every SM, so NCCL's CTAs do not run beside it, and the smaller messages
    reduce less efficiently (8 GPUs, 32768 x 4096 bf16: GEMM 0.29 ms + one
    all-reduce 0.73 ms = 0.97 ms; in 4 chunks 1.27 ms) -- hence the default 1."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, group=None, granule: int = 16,
                 layer_factory: Callable[..., nn.Module] = _default_factory, reduce_dtype: torch.dtype | None = None,
                 sequence_parallel: bool = False, overlap_chunks: int = 1, comm_sms: int = 32, **layer_kw):
        super().__init__()
        self.group = group
        # with sequence parallelism the output is reduce-scattered over tokens instead of all-reduced
        self.sequence_parallel = sequence_parallel
        world, rank = world_and_rank(group)
        self.in_start, self.in_end = shard_bounds(in_features, world, rank, granule)
        self.in_features, self.out_features = in_features, out_features
        self.reduce_dtype = reduce_dtype
        if reduce_dtype == torch.bfloat16 and layer_factory is _default_factory:
            # let the GEMM epilogue write the wire format instead of an FP32 tensor plus a conversion pass
            layer_kw = dict(layer_kw, out_dtype=torch.bfloat16)
        self.inner = layer_factory(self.in_end - self.in_start, out_features, False, **layer_kw)
        # the bias is added after the reduction, once
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        inner_dtype = getattr(self.inner, "out_dtype", None)
        self._overlap = (_is_tcfp(self.inner) and not sequence_parallel and world > 1
                         and (reduce_dtype is None or reduce_dtype == inner_dtype))
        if self._overlap:
            from .nn import LayerHooks

            self.inner._hooks = LayerHooks(out_hook=lambda y: _all_reduce_async(y, self.group),
                                           row_chunks=overlap_chunks)
        # sequence parallel with a TCFPLinear inside: the reduce-scatter of the output and the gathers of the
        # output gradient (FP8 codes for dX, full precision under the dX GEMM for dW) happen inside the layer
        self._sp_fused = (_is_tcfp(self.inner) and sequence_parallel and world > 1
                          and (reduce_dtype is None or reduce_dtype == inner_dtype))
        if self._sp_fused:
            from .nn import LayerHooks

            self.inner._hooks = LayerHooks(sp_out=SequenceParallelIO(group), reserve_sms=comm_sms)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        y = self.inner(x_shard)
        if not self._overlap and not self._sp_fused:
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
                                       layer_factory=layer_factory, sequence_parallel=sequence_parallel,
                                       **layer_kw)
        self.down = RowParallelLinear(d_hidden, d_model, bias, group=group, granule=granule,
                                      layer_factory=layer_factory, reduce_dtype=reduce_dtype,
                                      sequence_parallel=sequence_parallel, **layer_kw)
        self.activation = activation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(self.activation(self.up(x)))
