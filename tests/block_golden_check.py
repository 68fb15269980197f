"""Comparison of a full block-scaled quantization result (from the oracle on
CPU or from the CUDA kernels) with the outputs of the reference's Triton
kernels recorded in ``tests/golden/block_path.npz``.

The recorded kernels ran under the Triton interpreter, whose FP8 cast is wrong
on a known set of elements (exponent carry across a power of two, exact ties,
subnormals, probes above 448); W_hi codes are compared outside that set, and
W_lo planes/codes only in scale blocks whose W_hi codes agree entirely --
W_lo is a function of the whole block's W_hi."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from tests.golden.cases import BLOCK_CASES, block_inputs

GOLD = np.load(Path(__file__).parent / "golden" / "block_path.npz")
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def codes(a, dt):
    return torch.from_numpy(a.copy()).view(dt)


def blocked(t, bs):
    R, C = t.shape
    return t.reshape(R, C // bs, bs)


def cast_defect(scaled, q):
    v = q.float().abs()
    mant, _ = torch.frexp(v)
    crosses = (v > 0) & (mant == 0.5) & (scaled.abs() < v)
    up = torch.nextafter(scaled, torch.full_like(scaled, float("inf"))).to(q.dtype)
    down = torch.nextafter(scaled, torch.full_like(scaled, float("-inf"))).to(q.dtype)
    tie = up.view(torch.uint8) != down.view(torch.uint8)
    subnormal = scaled.abs() < (2.0**-6 if q.dtype == E4 else 2.0**-14)
    return crosses | tie | subnormal


def check_dual_quantize(name, hi, lo, exp_hi, exp_lo):
    """hi/lo: (N,K) float8_e4m3fn CPU tensors, exp_*: (K/bs, N) int8 CPU tensors."""
    cfg = BLOCK_CASES[name]
    w, err, _, _ = block_inputs(cfg)
    bs, N, K = cfg["bs"], cfg["N"], cfg["K"]
    k_hi, k_lo = codes(GOLD[f"{name}/w_hi"], E4), codes(GOLD[f"{name}/w_lo"], E4)
    k_eh, k_el = torch.from_numpy(GOLD[f"{name}/exp_hi"]), torch.from_numpy(GOLD[f"{name}/exp_lo"])
    assert torch.equal(exp_hi, k_eh), "W_hi exponent plane differs from the reference kernel"
    wc = w + err if err is not None else w
    inv_hi = torch.exp2(k_eh.float()).t().unsqueeze(-1)
    scaled = (blocked(wc, bs) / inv_hi).reshape(N, K)
    differ = hi.view(torch.uint8) != k_hi.view(torch.uint8)
    assert not bool((differ & ~cast_defect(scaled, hi)).any()), "W_hi codes differ outside the interpreter's defects"
    # blocks whose W_hi agrees everywhere: W_lo must agree as well
    same_block = ~blocked(differ, bs).any(-1)                        # (N, K/bs); few at block 128
    plane_ok = same_block.t()
    assert torch.equal(exp_lo[plane_ok], k_el[plane_ok]), "W_lo exponent plane differs"
    residual = blocked(wc, bs) - blocked(k_hi.float(), bs) * inv_hi
    zero = k_el.t() == -128
    inv_lo = torch.where(zero, torch.ones(()), torch.exp2(k_el.t().float())).unsqueeze(-1)
    s_lo = (residual / inv_lo).clamp(-448, 448).reshape(N, K)
    skip = cast_defect(s_lo, lo)
    if "srr_seed" in cfg:
        rtn = s_lo.to(E4)
        rtn_f = rtn.float()
        direction = torch.where(s_lo - rtn_f >= 0, 1.0, -1.0)
        probe = rtn_f + direction * rtn_f.abs().clamp(min=1e-12) * 0.25
        skip = cast_defect(s_lo, rtn) | cast_defect(probe, probe.clamp(-448, 448).to(E4)) | (probe.abs() > 448)
    differ_lo = lo.view(torch.uint8) != k_lo.view(torch.uint8)
    in_scope = same_block.unsqueeze(-1).expand(N, K // bs, bs).reshape(N, K) & ~skip
    assert not bool((differ_lo & in_scope).any()), "W_lo codes differ outside the interpreter's defects"


def check_block_quantize(name, tag, q, e):
    cfg = BLOCK_CASES[name]
    _, _, x, g = block_inputs(cfg)
    t = x if tag == "act" else g
    dt = E4 if tag == "act" else E5
    bs = cfg["bs"]
    k_q, k_e = codes(GOLD[f"{name}/{tag}"], dt), torch.from_numpy(GOLD[f"{name}/{tag}_exp"])
    assert torch.equal(e, k_e), f"{tag} exponent plane differs from the reference kernel"
    R, C = t.shape
    scaled = (blocked(t.float(), bs) / torch.exp2(k_e.float()).t().unsqueeze(-1)).reshape(R, C)
    differ = q.view(torch.uint8) != k_q.view(torch.uint8)
    assert not bool((differ & ~cast_defect(scaled, q)).any()), f"{tag} codes differ outside the interpreter's defects"


def golden_operands(name):
    """The reference kernels' own quantized operands and GEMM outputs."""
    g = lambda k, dt: codes(GOLD[f"{name}/{k}"], dt)  # noqa: E731
    e = lambda k: torch.from_numpy(GOLD[f"{name}/{k}"])  # noqa: E731
    return dict(hi=g("w_hi", E4), lo=g("w_lo", E4), eh=e("exp_hi"), el=e("exp_lo"), a=g("act", E4), ea=e("act_exp"),
                g=g("grad", E5), eg=e("grad_exp"), y=e("y"), dx=e("dx"))
