"""CPU, world size 2 over gloo: the tensor-parallel plumbing (shard bounds,
gradient all-reduce of the column-parallel input, output all-reduce of the
row-parallel layer) against an unsharded ``nn.Linear`` MLP.  The layer class is
injected as plain ``nn.Linear`` so that no GPU is involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tcfp_b200.tp import ParallelMLP, shard_bounds


def test_shard_bounds_block_aligned_and_uneven():
    spans = [shard_bounds(11008, 8, r, 64) for r in range(8)]
    assert spans[0] == (0, 1408) and spans[-1][1] == 11008
    assert [e - s for s, e in spans] == [1408] * 4 + [1344] * 4
    assert all(s % 64 == 0 and e % 64 == 0 for s, e in spans)
    assert all(spans[i][1] == spans[i + 1][0] for i in range(7))
    assert shard_bounds(4096, 1, 0, 64) == (0, 4096)
    with pytest.raises(ValueError):
        shard_bounds(100, 2, 0, 64)
    with pytest.raises(ValueError):
        shard_bounds(64, 2, 1, 64)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        d, h, granule = 32, 96, 16
        ref_up = torch.nn.Linear(d, h)
        ref_down = torch.nn.Linear(h, d)
        x = torch.randn(8, d)
        target = torch.randn(8, d)

        factory = lambda i, o, b, **kw: torch.nn.Linear(i, o, bias=b)  # noqa: E731
        mlp = ParallelMLP(d, h, granule=granule, layer_factory=factory)
        s, e = mlp.up.out_start, mlp.up.out_end
        assert (mlp.down.in_start, mlp.down.in_end) == (s, e)
        with torch.no_grad():
            mlp.up.inner.weight.copy_(ref_up.weight[s:e])
            mlp.up.inner.bias.copy_(ref_up.bias[s:e])
            mlp.down.inner.weight.copy_(ref_down.weight[:, s:e])
            mlp.down.bias.copy_(ref_down.bias)

        xr = x.clone().requires_grad_(True)
        y_ref = ref_down(torch.nn.functional.gelu(ref_up(xr)))
        ((y_ref - target) ** 2).mean().backward()

        xp = x.clone().requires_grad_(True)
        y = mlp(xp)
        ((y - target) ** 2).mean().backward()

        ok = torch.allclose(y, y_ref, atol=1e-5)
        ok &= torch.allclose(xp.grad, xr.grad, atol=1e-5)                       # all-reduced dX
        ok &= torch.allclose(mlp.up.inner.weight.grad, ref_up.weight.grad[s:e], atol=1e-5)
        ok &= torch.allclose(mlp.down.inner.weight.grad, ref_down.weight.grad[:, s:e], atol=1e-5)
        ok &= torch.allclose(mlp.down.bias.grad, ref_down.bias.grad, atol=1e-5)
        # sequence-parallel form: token shards in, token shards out, same numbers
        sp = ParallelMLP(d, h, granule=granule, layer_factory=factory, sequence_parallel=True)
        sp.load_state_dict(mlp.state_dict())
        rows = x.shape[0] // world
        xs = x[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
        ys = sp(xs)
        ((ys - target[rank * rows:(rank + 1) * rows]) ** 2).sum().div(target.numel()).backward()
        ok &= ys.shape == (rows, d) and torch.allclose(ys, y_ref[rank * rows:(rank + 1) * rows], atol=1e-5)
        ok &= torch.allclose(xs.grad, xr.grad[rank * rows:(rank + 1) * rows], atol=1e-5)
        ok &= torch.allclose(sp.up.inner.weight.grad, ref_up.weight.grad[s:e], atol=1e-5)
        ok &= torch.allclose(sp.down.inner.weight.grad, ref_down.weight.grad[:, s:e], atol=1e-5)
        ok &= torch.allclose(sp.down.bias.grad, ref_down.bias.grad, atol=1e-5)
        # fused column-parallel group: one layer whose local weight is this rank's shard of each part
        from tcfp_b200.tp import ColumnParallelLinear

        ref_a, ref_b = torch.nn.Linear(d, 64), torch.nn.Linear(d, 96)
        fused = ColumnParallelLinear(d, (64, 96), granule=granule, layer_factory=factory)
        (a0, a1), (b0, b1) = fused.bounds
        with torch.no_grad():
            fused.inner.weight.copy_(torch.cat([ref_a.weight[a0:a1], ref_b.weight[b0:b1]]))
            fused.inner.bias.copy_(torch.cat([ref_a.bias[a0:a1], ref_b.bias[b0:b1]]))
        xf = x.clone().requires_grad_(True)
        ya, yb = fused(xf)
        (ya.square().sum() + yb.sum()).backward()
        xg = x.clone().requires_grad_(True)
        (ref_a(xg).square().sum() + ref_b(xg).sum()).backward()
        ok &= ya.shape == (8, a1 - a0) and torch.allclose(ya, ref_a(x)[:, a0:a1], atol=1e-5)
        ok &= torch.allclose(yb, ref_b(x)[:, b0:b1], atol=1e-5)
        ok &= torch.allclose(xf.grad, xg.grad, atol=1e-4)                       # one all-reduce for the whole group
        # the collectives of the fused sequence-parallel form (FP8 codes as bytes, exponent planes, reduce-scatter)
        from tcfp_b200.tp import SequenceParallelIO

        io = SequenceParallelIO()
        codes = [(torch.randn(4, 16, generator=torch.Generator().manual_seed(r))).to(torch.float8_e4m3fn) for r in range(world)]
        got = io.gather_rows(codes[rank])
        ok &= got.dtype == torch.float8_e4m3fn and torch.equal(got.view(torch.uint8), torch.cat(codes).view(torch.uint8))
        planes = [(torch.arange(6).reshape(2, 3) + 10 * r).to(torch.int8) for r in range(world)]
        ok &= torch.equal(io.gather_planes(planes[rank]), torch.cat(planes, dim=1))
        handle, mine = io.scatter_rows_async(torch.full((4, 3), float(rank + 1)))
        if handle is not None:
            handle.wait()
        ok &= mine.shape == (2, 3) and torch.equal(mine, torch.full((2, 3), 3.0))
        # measurement aid: layers built under single_rank() are unsharded and, with the collectives off, compute
        # the single-GPU form of the model inside a multi-rank job
        from tcfp_b200 import tp as tpmod

        with tpmod.single_rank():
            whole = ParallelMLP(d, h, granule=granule, layer_factory=factory)
        ok &= whole.up.inner.weight.shape == (h, d) and whole.down.inner.weight.shape == (d, h)
        with torch.no_grad():
            whole.up.inner.weight.copy_(ref_up.weight)
            whole.up.inner.bias.copy_(ref_up.bias)
            whole.down.inner.weight.copy_(ref_down.weight)
            whole.down.bias.copy_(ref_down.bias)
        with tpmod.collectives_disabled():
            ok &= torch.allclose(whole(x), y_ref, atol=1e-5)
        ok &= tpmod.world_and_rank() == (world, rank)
        # a norm applied to token shards: the replicated weight's gradient is summed over the ranks
        from tcfp_b200.workloads import RMSNorm

        whole_norm, shard_norm = RMSNorm(d), RMSNorm(d, token_sharded=True)
        (whole_norm(x) * target).sum().backward()
        (shard_norm(x[rank * rows:(rank + 1) * rows]) * target[rank * rows:(rank + 1) * rows]).sum().backward()
        ok &= torch.allclose(shard_norm.weight.grad, whole_norm.weight.grad, atol=1e-5)
        # a token count the world size does not divide is refused, not truncated
        try:
            sp.down(torch.randn(3, e - s))
            ok = False
        except ValueError as e:
            ok &= "multiple of the tensor-parallel world size" in str(e)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_parallel_mlp_matches_unsharded_world2():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_block_aligned_shards_reproduce_the_unsharded_quantized_bytes():
    """Column-parallel shards (rows of W) and row-parallel shards (K blocks of W
    and of the activation) quantize to exactly the bytes of the unsharded
    layer: block scales are per (row, K block).  Checked with the oracle."""
    from oracle import tcfp_oracle as O
    from tests.util import acts, weights

    bs, world = 64, 4
    N, K, M = 256, 704, 48                     # K = 11 blocks: uneven row-parallel shards (3,3,3,2)
    w = weights(700, N, K, outliers=True)
    err = weights(701, N, K, std=1e-4)
    x = acts(702, M, K, torch.bfloat16)
    hi, lo, eh, el, new_err = O.dual_quantize_block(w, bs, err)
    a, ea = O.block_quantize(x, bs)
    full = O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, bs)
    partial_sum = torch.zeros(M, N)
    for r in range(world):
        s, e = shard_bounds(N, world, r, bs)                       # column parallel: rows of W
        h2, l2, eh2, el2, ne2 = O.dual_quantize_block(w[s:e].contiguous(), bs, err[s:e].contiguous())
        assert torch.equal(h2.view(torch.uint8), hi[s:e].view(torch.uint8)) and torch.equal(l2.view(torch.uint8), lo[s:e].view(torch.uint8))
        assert torch.equal(eh2, eh[:, s:e]) and torch.equal(el2, el[:, s:e]) and torch.equal(ne2, new_err[s:e])
        ks, ke = shard_bounds(K, world, r, bs)                     # row parallel: K blocks
        h3, l3, eh3, el3, ne3 = O.dual_quantize_block(w[:, ks:ke].contiguous(), bs, err[:, ks:ke].contiguous())
        assert torch.equal(h3.view(torch.uint8), hi[:, ks:ke].view(torch.uint8))
        assert torch.equal(l3.view(torch.uint8), lo[:, ks:ke].view(torch.uint8))
        assert torch.equal(eh3, eh[ks // bs:ke // bs]) and torch.equal(ne3, new_err[:, ks:ke])
        a3, ea3 = O.block_quantize(x[:, ks:ke].contiguous(), bs)
        assert torch.equal(a3.view(torch.uint8), a[:, ks:ke].view(torch.uint8)) and torch.equal(ea3, ea[ks // bs:ke // bs])
        partial_sum += O.block_dual_gemm_nt(a3, ea3, h3, eh3, l3, el3, bs)
    assert float((partial_sum - full).norm() / full.norm()) <= 1e-6    # only the summation order differs
