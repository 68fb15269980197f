"""CPU: the oracle's block-scaled functions against the outputs of the
REFERENCE's own Triton kernels, executed by the Triton interpreter
(tests/golden/make_golden_block.py).  The interpreter's float32 -> FP8 cast
has two defects the hardware cast does not share: it drops the exponent carry
when rounding crosses a power of two (31.8 -> 16) and it rounds exact ties
away from zero instead of to even (25 -> 26), and it truncates in the
subnormal range.  Codes are compared everywhere
except on those elements, and each later stage is checked starting from the
kernel's own earlier outputs."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import tcfp_oracle as O
from tests.golden.cases import BLOCK_CASES, block_inputs

GOLD = np.load(Path(__file__).parent / "golden" / "block_path.npz")
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def codes(a, dt):
    return torch.from_numpy(a.copy()).view(dt)


def carry(scaled, q):
    """Elements the interpreter's cast gets wrong: round-to-nearest lands on a
    power of two from below, the value is an exact tie between two codes, or
    the result is subnormal."""
    v = q.float().abs()
    mant, _ = torch.frexp(v)
    crosses = (v > 0) & (mant == 0.5) & (scaled.abs() < v)
    up = torch.nextafter(scaled, torch.full_like(scaled, float("inf"))).to(q.dtype)
    down = torch.nextafter(scaled, torch.full_like(scaled, float("-inf"))).to(q.dtype)
    tie = up.view(torch.uint8) != down.view(torch.uint8)
    subnormal = scaled.abs() < (2.0**-6 if q.dtype == E4 else 2.0**-14)
    return crosses | tie | subnormal


def _blocked(t, bs):
    R, C = t.shape
    return t.reshape(R, C // bs, bs)


@pytest.mark.parametrize("name", list(BLOCK_CASES))
def test_dual_quantize_stages_match_reference_kernel(name):
    cfg = BLOCK_CASES[name]
    w, err, _, _ = block_inputs(cfg)
    bs, N, K = cfg["bs"], cfg["N"], cfg["K"]
    k_hi, k_lo = codes(GOLD[f"{name}/w_hi"], E4), codes(GOLD[f"{name}/w_lo"], E4)
    k_eh, k_el = torch.from_numpy(GOLD[f"{name}/exp_hi"]), torch.from_numpy(GOLD[f"{name}/exp_lo"])
    o_hi, _, o_eh, _, _ = O.dual_quantize_block(w, bs, err)
    # 1. W_hi exponent plane: bit exact (independent of any cast)
    assert torch.equal(o_eh, k_eh)
    # 2. W_hi codes: equal except where the interpreter loses the carry
    wc = w + err if err is not None else w
    inv_hi = torch.exp2(k_eh.float()).t().unsqueeze(-1)
    scaled = (_blocked(wc, bs) / inv_hi).reshape(N, K)
    differ = o_hi.view(torch.uint8) != k_hi.view(torch.uint8)
    assert not bool((differ & ~carry(scaled, o_hi)).any())
    assert int(differ.sum()) < 0.05 * N * K
    # 3. from the kernel's own W_hi: residual -> W_lo exponents incl. the -128 sentinel, bit exact
    residual = _blocked(wc, bs) - _blocked(k_hi.float(), bs) * inv_hi
    amax = residual.abs().amax(-1)
    zero = amax < 1e-12
    e_lo = O._block_exponent(amax, 448.0)
    plane = torch.where(zero, torch.full_like(e_lo, -128.0), e_lo).to(torch.int8).t().contiguous()
    assert torch.equal(plane, k_el)
    # 4. W_lo codes from that residual
    inv_lo = torch.where(zero, torch.ones_like(e_lo), torch.exp2(e_lo)).unsqueeze(-1)
    s_lo = (residual / inv_lo).clamp(-448, 448).reshape(N, K)
    if "srr_seed" in cfg:
        # stochastic residual: same uniforms (tl.rand(seed, n*K + k)), same neighbour search.  Besides the
        # cast defects on either probe, the interpreter does not saturate a probe beyond 448 the way the
        # hardware cast does.
        rand = O.philox_uniform(cfg["srr_seed"], 0, N * K).reshape(N, K)
        o_lo = O._sr_block(s_lo, rand)
        rtn = s_lo.to(E4)
        rtn_f = rtn.float()
        direction = torch.where(s_lo - rtn_f >= 0, 1.0, -1.0)
        probe = rtn_f + direction * rtn_f.abs().clamp(min=1e-12) * 0.25
        skip = carry(s_lo, rtn) | carry(probe, probe.clamp(-448, 448).to(E4)) | (probe.abs() > 448)
        differ = o_lo.view(torch.uint8) != k_lo.view(torch.uint8)
        assert not bool((differ & ~skip).any())
        assert float(skip.float().mean()) < 0.5
        assert int((k_lo.view(torch.uint8) != rtn.view(torch.uint8)).sum()) > 100      # it did round stochastically
        return
    o_lo = s_lo.to(E4)
    differ = o_lo.view(torch.uint8) != k_lo.view(torch.uint8)
    assert not bool((differ & ~carry(s_lo, o_lo)).any())
    if cfg.get("zero_rows"):
        assert bool((k_el[:, 1] == -128).all()) and bool((k_lo[1].float() == 0).all())


@pytest.mark.parametrize("name", list(BLOCK_CASES))
def test_block_quantize_matches_reference_kernel(name):
    cfg = BLOCK_CASES[name]
    _, _, x, g = block_inputs(cfg)
    bs = cfg["bs"]
    for tag, t, dt in (("act", x, E4), ("grad", g, E5)):
        q, e = O.block_quantize(t, bs, dt)
        k_q, k_e = codes(GOLD[f"{name}/{tag}"], dt), torch.from_numpy(GOLD[f"{name}/{tag}_exp"])
        assert torch.equal(e, k_e)
        R, C = t.shape
        scaled = (_blocked(t.float(), bs) / torch.exp2(e.float()).t().unsqueeze(-1)).reshape(R, C)
        differ = q.view(torch.uint8) != k_q.view(torch.uint8)
        assert not bool((differ & ~carry(scaled, q)).any())


@pytest.mark.parametrize("name", list(BLOCK_CASES))
def test_block_gemms_match_reference_kernels(name):
    """Forward and dX kernels of the reference on ITS quantized operands vs the
    oracle's dequantize-then-matmul (scale-plane layout, sentinel handling)."""
    cfg = BLOCK_CASES[name]
    bs = cfg["bs"]
    hi, lo = codes(GOLD[f"{name}/w_hi"], E4), codes(GOLD[f"{name}/w_lo"], E4)
    eh, el = torch.from_numpy(GOLD[f"{name}/exp_hi"]), torch.from_numpy(GOLD[f"{name}/exp_lo"])
    a, ea = codes(GOLD[f"{name}/act"], E4), torch.from_numpy(GOLD[f"{name}/act_exp"])
    g, eg = codes(GOLD[f"{name}/grad"], E5), torch.from_numpy(GOLD[f"{name}/grad_exp"])
    y = torch.from_numpy(GOLD[f"{name}/y"])
    dx = torch.from_numpy(GOLD[f"{name}/dx"])
    y_o = O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, bs)
    dx_o = O.block_backward_dx(g, eg, hi, eh, lo, el, bs)
    assert float((y - y_o).norm() / y_o.norm()) <= 1e-5
    assert float((dx - dx_o).norm() / dx_o.norm()) <= 1e-5


@pytest.mark.parametrize("name", list(BLOCK_CASES))
def test_full_oracle_pipeline_through_the_shared_checker(name):
    """The same checker the GPU test uses, fed with the oracle's end-to-end
    outputs (W_lo computed from the oracle's own W_hi)."""
    from tests.block_golden_check import check_block_quantize, check_dual_quantize

    cfg = BLOCK_CASES[name]
    w, err, x, g = block_inputs(cfg)
    hi, lo, eh, el, _ = O.dual_quantize_block(w, cfg["bs"], err, srr="srr_seed" in cfg, seed=cfg.get("srr_seed", 0))
    check_dual_quantize(name, hi, lo, eh, el)
    check_block_quantize(name, "act", *O.block_quantize(x, cfg["bs"], E4))
    check_block_quantize(name, "grad", *O.block_quantize(g, cfg["bs"], E5))
