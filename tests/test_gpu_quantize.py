"""GPU parity of the quantize kernels against the CPU oracle: code bytes,
scales and error buffers must match bit for bit."""
import pytest
import torch

from oracle import tcfp_oracle as O
from tests.util import acts, bits, u8, weights

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _adversarial_weight(n, k):
    """Blocks whose amax/448 sits on and next to powers of two, zeros, tiny
    and huge values -- the cases where the exponent rule can slip."""
    w = weights(7, n, k, std=0.02)
    w[0, :] = 0.0                                  # zero row -> amax floor, sentinel
    w[1, :32] = 448.0 * 2.0**-7                     # q exactly 2^-7
    w[1, 32:64] = torch.nextafter(torch.tensor(448.0 * 2.0**-7), torch.tensor(1.0))
    w[1, 64:96] = torch.nextafter(torch.tensor(448.0 * 2.0**-7), torch.tensor(0.0))
    for j in range(1, 24):
        base = torch.tensor(448.0 * 2.0**-(j % 12 + 3), dtype=torch.float32)
        w[2, 32 * (j % (k // 32))] = (base.view(torch.int32) + j).view(torch.float32)
    w[3, :] = 1e-20                                 # below the amax floor
    w[4, 5] = 3.0e4                                 # large outlier
    w[5, :] = 1.0                                   # exact codes -> zero residual
    return w


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("mode", ["none", "ef"])
def test_dual_quantize_block_bit_exact(bs, mode):
    from tcfp_b200.kernels import fused_dual_quantize_fp8

    for n, k, adv in [(64, 256, True), (100, 384, False), (256, 1024, False), (33, 128, False)]:
        w = _adversarial_weight(n, k) if adv else weights(11 + n, n, k, outliers=True)
        err = (weights(5, n, k, std=1e-4) if mode == "ef" else None)
        hi, lo, sh, sl, new_err = O.dual_quantize_block(w, bs, err)
        err_d = err.to(DEV).clone() if err is not None else None
        ghi, glo, gsh, gsl = fused_dual_quantize_fp8(w.to(DEV), bs, err_d)
        assert torch.equal(gsh.cpu(), sh), f"hi exponents differ n={n} k={k}"
        assert torch.equal(u8(ghi), u8(hi)), f"hi codes differ n={n} k={k}"
        assert torch.equal(gsl.cpu(), sl), f"lo exponents differ n={n} k={k}"
        assert torch.equal(u8(glo), u8(lo)), f"lo codes differ n={n} k={k}"
        if err is not None:
            assert torch.equal(bits(err_d), bits(new_err)), "error buffer differs"


@pytest.mark.parametrize("bs", [32, 128])
def test_dual_quantize_block_readonly_and_bf16(bs):
    from tcfp_b200.kernels import fused_dual_quantize_fp8

    w = weights(3, 64, 512).to(torch.bfloat16)
    err = weights(4, 64, 512, std=1e-4)
    hi, lo, sh, sl, _ = O.dual_quantize_block(w, bs, err)
    err_d = err.to(DEV).clone()
    ghi, glo, gsh, gsl = fused_dual_quantize_fp8(w.to(DEV), bs, err_d, update_error=False)
    assert torch.equal(u8(ghi), u8(hi)) and torch.equal(u8(glo), u8(lo))
    assert torch.equal(gsh.cpu(), sh) and torch.equal(gsl.cpu(), sl)
    assert torch.equal(bits(err_d), bits(err)), "read-only mode must not touch the buffer"


@pytest.mark.parametrize("bs", [32, 64, 128])
def test_dual_quantize_block_srr_bit_exact(bs):
    from tcfp_b200.kernels import fused_dual_quantize_fp8

    w = weights(21, 96, 256, outliers=True)
    seed, offset = 0x5EED, 12345
    hi, lo, sh, sl, _ = O.dual_quantize_block(w, bs, None, srr=True, seed=seed, offset=offset)
    ghi, glo, gsh, gsl = fused_dual_quantize_fp8(w.to(DEV), bs, None, True, seed=seed, offset=offset)
    assert torch.equal(u8(ghi), u8(hi)) and torch.equal(gsh.cpu(), sh) and torch.equal(gsl.cpu(), sl)
    assert torch.equal(u8(glo), u8(lo))
    # stochastic: differs from round-to-nearest somewhere, hi untouched
    _, lo_rtn, _, _, _ = O.dual_quantize_block(w, bs, None)
    assert not torch.equal(u8(lo_rtn), u8(lo))


def test_dual_quantize_block_srr_unbiased():
    """tests/test_fused_dual_quant.py:494-526 of the reference: mean of many
    draws approaches the RTN-free reconstruction."""
    from tcfp_b200.kernels import block_dequantize_fp8, fused_dual_quantize_fp8

    w = weights(8, 32, 128).to(DEV)
    acc = torch.zeros_like(w)
    draws = 200
    for i in range(draws):
        hi, lo, sh, sl = fused_dual_quantize_fp8(w, 32, None, True, seed=1000 + i)
        acc += block_dequantize_fp8(hi, sh, 32) + block_dequantize_fp8(lo, sl, 32)
    bias = (acc / draws - w).abs().mean() / w.abs().mean()
    assert bias < 1e-3


def test_dual_quantize_input_checks():
    from tcfp_b200.kernels import fused_dual_quantize_fp8

    w = weights(1, 32, 128).to(DEV)
    with pytest.raises(AssertionError, match="divisible"):
        fused_dual_quantize_fp8(w, 48)
    with pytest.raises(AssertionError, match="float32"):
        fused_dual_quantize_fp8(w, 32, torch.zeros(32, 128, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(AssertionError, match="shape"):
        fused_dual_quantize_fp8(w, 32, torch.zeros(16, 128, device=DEV))
    with pytest.raises(AssertionError, match="contiguous"):
        fused_dual_quantize_fp8(w.t(), 32)
    with pytest.raises(ValueError, match="mutually exclusive"):
        fused_dual_quantize_fp8(w, 32, torch.zeros_like(w), True)


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("fmt", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_quantize_bit_exact(bs, fmt, dtype):
    from tcfp_b200.kernels import block_quantize_fp8

    for m, k in [(100, 256), (257, 1024)]:
        x = acts(31 + m, m, k, dtype) * 3.0
        x[0, :] = 0
        q, e = O.block_quantize(x, bs, fmt)
        gq, ge, gdeq = block_quantize_fp8(x.to(DEV), bs, fmt, want_bf16=True)
        assert ge.shape == (k // bs, m) and ge.dtype == torch.int8
        assert torch.equal(ge.cpu(), e)
        assert torch.equal(u8(gq), u8(q))
        assert torch.equal(gdeq.float().cpu(), O.block_dequantize(q, e, bs))


def test_fused_dual_equals_two_sequential_block_quantizes():
    """tests/test_fused_dual_quant.py:80-155 of the reference."""
    from tcfp_b200.kernels import block_dequantize_fp8, block_quantize_fp8, fused_dual_quantize_fp8

    w = weights(77, 128, 512, outliers=True).to(DEV)
    hi, lo, sh, sl = fused_dual_quantize_fp8(w, 64)
    hi2, sh2 = block_quantize_fp8(w, 64)
    res = w - block_dequantize_fp8(hi2, sh2, 64)
    lo2, sl2 = block_quantize_fp8(res, 64)
    assert torch.equal(u8(hi), u8(hi2)) and torch.equal(sh, sh2)
    assert torch.equal(u8(lo), u8(lo2))
    keep = sl != -128
    assert torch.equal(sl[keep], sl2[keep])


@pytest.mark.parametrize("mode", ["none", "ef", "srr"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dual_quantize_per_tensor_bit_exact(mode, dtype):
    from tcfp_b200.core import dual_quantize_per_tensor

    for n, k in [(64, 128), (300, 512), (1024, 1024)]:
        w = weights(41 + n, n, k).to(dtype)
        err = weights(42, n, k, std=1e-4) if mode == "ef" else None
        srr = mode == "srr"
        hi, lo, ihi, ilo, new_err, ahi, alo = O.dual_quantize_per_tensor(w, err, srr=srr, seed=99, offset=7)
        err_d = err.to(DEV).clone() if err is not None else None
        ghi, glo, gihi, gilo, gam = dual_quantize_per_tensor(w.to(DEV), err_d, srr=srr, seed=99, offset=7,
                                                            want_amax=True)
        assert torch.equal(bits(gihi), bits(ihi)) and torch.equal(bits(gilo), bits(ilo))
        assert torch.equal(u8(ghi), u8(hi))
        assert torch.equal(u8(glo), u8(lo))
        assert torch.equal(bits(gam), bits(torch.stack([ahi, alo])))
        if err is not None:
            assert torch.equal(bits(err_d), bits(new_err))


def test_dual_quantize_per_tensor_given_amax():
    """Delayed scaling: caller-provided amax for W_hi and a predicted one for
    W_lo (tcfp/nn/__init__.py:250-309) -- the single-pass kernel."""
    from tcfp_b200.core import dual_quantize_per_tensor

    w = weights(51, 256, 512)
    err = weights(52, 256, 512, std=1e-4)
    a_hi = torch.tensor(0.11)
    a_lo = torch.tensor(0.11 / 8)
    for al in (None, a_lo):
        hi, lo, ihi, ilo, new_err, _, alo = O.dual_quantize_per_tensor(w, err, amax_hi=a_hi, amax_lo=al)
        err_d = err.to(DEV).clone()
        ghi, glo, gihi, gilo, gam = dual_quantize_per_tensor(w.to(DEV), err_d, amax_hi=a_hi.to(DEV),
                                                            amax_lo=None if al is None else al.to(DEV),
                                                            want_amax=True)
        assert torch.equal(u8(ghi), u8(hi)) and torch.equal(u8(glo), u8(lo))
        assert torch.equal(bits(gihi), bits(ihi)) and torch.equal(bits(gilo), bits(ilo))
        assert torch.equal(bits(err_d), bits(new_err))
        assert torch.equal(bits(gam[1:]), bits(alo.reshape(1)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_to_fp8_casts_bit_exact(dtype):
    from tcfp_b200.core import absmax, to_fp8_e4m3, to_fp8_e4m3_sr, to_fp8_e5m2

    x = acts(61, 200, 384, dtype)
    q, inv = O.to_fp8_e4m3(x)
    gq, ginv = to_fp8_e4m3(x.to(DEV))
    assert ginv.shape == (1,) and torch.equal(bits(ginv), bits(inv)) and torch.equal(u8(gq), u8(q))
    q, inv = O.to_fp8_e5m2(x)
    gq, ginv = to_fp8_e5m2(x.to(DEV))
    assert torch.equal(bits(ginv), bits(inv)) and torch.equal(u8(gq), u8(q))
    scale = torch.tensor(37.5)
    q, inv = O.to_fp8_e4m3(x, scale=scale)
    gq, ginv = to_fp8_e4m3(x.to(DEV), scale=scale.to(DEV))
    assert torch.equal(bits(ginv), bits(inv)) and torch.equal(u8(gq), u8(q))
    rand = O.philox_uniform_packed(5, 3, x.numel()).reshape(x.shape)
    q, inv = O.to_fp8_e4m3_sr(x, rand)
    gq, ginv = to_fp8_e4m3_sr(x.to(DEV), seed=5, offset=3)
    assert torch.equal(bits(ginv), bits(inv)) and torch.equal(u8(gq), u8(q))
    assert torch.equal(bits(absmax(x.to(DEV)).reshape(1)), bits(x.float().abs().max().reshape(1)))


def test_pack_scales_layout(lib):
    from tcfp_b200.kernels import pack_block_scales

    rows, num_kb, bs = 200, 6, 32
    g = torch.Generator().manual_seed(3)
    exps = torch.randint(-20, 10, (num_kb, rows), generator=g, dtype=torch.int8)
    exps[2, 5] = -128
    sf = pack_block_scales(exps.to(DEV), bs).cpu()
    k_groups = (num_kb + 3) // 4
    assert sf.numel() == ((rows + 127) // 128) * k_groups * 512
    for row in (0, 5, 31, 32, 127, 128, 199):
        for kb in range(num_kb):
            off = ((row // 128) * k_groups + kb // 4) * 512 + (row % 32) * 16 + ((row // 32) % 4) * 4 + kb % 4
            e = int(exps[kb, row])
            assert int(sf[off]) == (0 if e == -128 else e + 127)
    # tail blocks of the last K group hold a neutral scale
    assert int(sf[(0 * k_groups + 1) * 512 + 0 * 16 + 0 * 4 + 2]) == 127


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,C", [(1000, 384), (4096, 1024), (257, 2048), (31, 128)])
def test_gradient_quantizers_with_fused_bias_gradient(R, C, dtype):
    """The column sums (bias gradient, tcfp/nn/__init__.py:558, 753) come out
    of the gradient quantizers' own passes: same codes and scales as the plain
    quantizers bit for bit, sums within 1e-5 of a float64 sum, and identical
    bits on a repeated call (fixed summation order)."""
    from tcfp_b200.core import to_fp8_e5m2, to_fp8_e5m2_with_colsum
    from tcfp_b200.kernels import block_quantize_fp8

    g = (acts(90, R, C, torch.float32) * 3.0 + 0.25).to(dtype).to(DEV)
    want = g.double().sum(dim=0)
    scale = g.double().abs().sum(dim=0).clamp(min=1e-30)
    q, inv = to_fp8_e5m2(g)
    q2, inv2, cs = to_fp8_e5m2_with_colsum(g)
    assert torch.equal(u8(q2), u8(q)) and torch.equal(bits(inv2), bits(inv))
    assert float(((cs.double() - want).abs() / scale).max()) <= 1e-5
    assert torch.equal(bits(to_fp8_e5m2_with_colsum(g)[2]), bits(cs))
    for bs in (32, 128):
        q, e = block_quantize_fp8(g, bs, torch.float8_e5m2)
        q2, e2, cs = block_quantize_fp8(g, bs, torch.float8_e5m2, want_colsum=True)
        assert torch.equal(u8(q2), u8(q)) and torch.equal(e2, e)
        assert float(((cs.double() - want).abs() / scale).max()) <= 1e-5
        assert torch.equal(bits(block_quantize_fp8(g, bs, torch.float8_e5m2, want_colsum=True)[2]), bits(cs))
