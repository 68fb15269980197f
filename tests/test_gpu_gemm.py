"""GPU parity of the tcgen05 dual-GEMM kernels against the FP32 dequantized
dual matmul of the oracle.  Tolerance: relative Frobenius error <= 1e-3 (the
FP8 products are exact in FP32; only the accumulation order differs), plus
the reference's own absolute pins (tests/test_fused_kernels.py:120-134 uses
atol=rtol=1e-2; tests/test_block_scaling_kernels.py:147-169 uses 1e-3)."""
import pytest
import torch

from oracle import tcfp_oracle as O
from tests.util import acts, rel_fro, weights

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-3

SHAPES = [(128, 128, 128), (256, 384, 512), (48, 80, 112), (100, 128, 256), (1024, 1024, 1024), (130, 272, 144),
          (300, 272, 144), (1000, 528, 400), (257, 16, 16), (640, 2048, 96)]


def _per_tensor_operands(seed, M, N, K, grad=False):
    x = acts(seed, M, K, torch.float32)
    w = weights(seed + 1, N, K, std=1.0)
    a, ia = (O.to_fp8_e5m2 if grad else O.to_fp8_e4m3)(x)
    hi, lo, ihi, ilo, _, _, _ = O.dual_quantize_per_tensor(w)
    return a, ia, hi, ihi, lo, ilo


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_dual_gemm_forward(M, N, K):
    from tcfp_b200.kernels import fused_dual_gemm_forward

    a, ia, hi, ihi, lo, ilo = _per_tensor_operands(100, M, N, K)
    ref = O.dual_gemm_nt(a, ia, hi, ihi, lo, ilo)
    out = fused_dual_gemm_forward(a.to(DEV), hi.to(DEV), lo.to(DEV), ia.to(DEV), ihi.to(DEV), ilo.to(DEV))
    assert out.shape == (M, N) and out.dtype == torch.float32
    assert rel_fro(out, ref) <= TOL
    torch.testing.assert_close(out.cpu(), ref, atol=1e-2, rtol=1e-2)


def test_dual_gemm_forward_variants():
    from tcfp_b200.kernels import fused_dual_gemm_forward

    M, N, K = 256, 256, 256
    a, ia, hi, ihi, lo, ilo = _per_tensor_operands(101, M, N, K)
    d = lambda t: t.to(DEV)
    # zero W_lo equals the single GEMM (tests/test_fused_kernels.py:152-176)
    zero = torch.zeros_like(lo)
    single = fused_dual_gemm_forward(d(a), d(hi), None, d(ia), d(ihi), None)
    with_zero = fused_dual_gemm_forward(d(a), d(hi), d(zero), d(ia), d(ihi), d(ilo))
    torch.testing.assert_close(single, with_zero, atol=1e-4, rtol=1e-4)
    assert rel_fro(single, O.dual_gemm_nt(a, ia, hi, ihi, None, None)) <= TOL
    # scale linearity (tests/test_fused_kernels.py:178-204)
    o1 = fused_dual_gemm_forward(d(a), d(hi), d(lo), d(ia), d(ihi), d(ilo))
    o2 = fused_dual_gemm_forward(d(a), d(hi), d(lo), d(ia * 2), d(ihi), d(ilo))
    torch.testing.assert_close(o2, o1 * 2, atol=1e-5, rtol=1e-5)
    # bias + bf16 output
    bias = torch.randn(N)
    ob = fused_dual_gemm_forward(d(a), d(hi), d(lo), d(ia), d(ihi), d(ilo), bias=d(bias), out_dtype=torch.bfloat16)
    ref = O.dual_gemm_nt(a, ia, hi, ihi, lo, ilo) + bias
    assert ob.dtype == torch.bfloat16 and rel_fro(ob.float(), ref) <= 5e-3
    # deterministic run to run
    assert torch.equal(o1, fused_dual_gemm_forward(d(a), d(hi), d(lo), d(ia), d(ihi), d(ilo)))


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_dual_gemm_backward_dx(M, N, K):
    """dX = g . W with W in its native (D_out, D_in) layout: here K = D_out is
    the contraction and N = D_in."""
    from tcfp_b200.kernels import fused_dual_gemm_backward_dx

    g = acts(200, M, K, torch.float32)
    w = weights(201, K, N, std=1.0)
    gq, ig = O.to_fp8_e5m2(g)
    hi, lo, ihi, ilo, _, _, _ = O.dual_quantize_per_tensor(w)
    ref = O.dual_gemm_nn(gq, ig, hi, ihi, lo, ilo)
    out = fused_dual_gemm_backward_dx(gq.to(DEV), hi.to(DEV), lo.to(DEV), ig.to(DEV), ihi.to(DEV), ilo.to(DEV))
    assert out.shape == (M, N)
    assert rel_fro(out, ref) <= TOL
    torch.testing.assert_close(out.cpu(), ref, atol=1e-2, rtol=1e-2)


def _block_operands(seed, M, N, K, bs):
    x = acts(seed, M, K, torch.bfloat16)
    w = weights(seed + 1, N, K, outliers=True)
    a, ea = O.block_quantize(x, bs)
    hi, lo, eh, el, _ = O.dual_quantize_block(w, bs)
    return a, ea, hi, eh, lo, el


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (100, 100, 256), (512, 640, 1024), (64, 192, 384),
                                   (300, 272, 384), (1000, 528, 640), (257, 16, 128)])
def test_block_dual_gemm_forward(M, N, K, bs):
    from tcfp_b200.kernels import fused_block_scaled_dual_gemm_forward

    a, ea, hi, eh, lo, el = _block_operands(300, M, N, K, bs)
    ref = O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, bs)
    d = lambda t: t.to(DEV)
    out = fused_block_scaled_dual_gemm_forward(d(a), d(hi), d(lo), d(ea), d(eh), d(el), bs)
    assert rel_fro(out, ref) <= TOL
    torch.testing.assert_close(out.cpu(), ref, atol=1e-3, rtol=1e-3)


def test_block_gemm_single_and_sentinel():
    from tcfp_b200.kernels import block_scaled_gemm, fused_block_scaled_dual_gemm_forward

    M, N, K, bs = 128, 256, 512, 64
    a, ea, hi, eh, lo, el = _block_operands(301, M, N, K, bs)
    d = lambda t: t.to(DEV)
    single = block_scaled_gemm(d(a), d(hi), d(ea), d(eh), bs)
    assert rel_fro(single, O.block_dual_gemm_nt(a, ea, hi, eh, None, None, bs)) <= TOL
    # all-sentinel residual scales -> hi-only result
    # (tests/test_block_scaling_kernels.py:366-387, compared at atol=1e-2)
    sent = torch.full_like(el, -128)
    out = fused_block_scaled_dual_gemm_forward(d(a), d(hi), d(lo), d(ea), d(eh), d(sent), bs)
    torch.testing.assert_close(out, single, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (100, 256, 128), (512, 1024, 640), (300, 384, 256),
                                   (1000, 640, 384)])
def test_block_backward_dx(M, N, K, bs):
    """K = D_out (contraction), N = D_in."""
    from tcfp_b200.kernels import fused_block_scaled_dual_gemm_backward_dx

    g = acts(400, M, K, torch.float32)
    w = weights(401, K, N, outliers=True)
    gq, eg = O.block_quantize(g, bs, torch.float8_e5m2)
    hi, lo, eh, el, _ = O.dual_quantize_block(w, bs)
    ref = O.block_backward_dx(gq, eg, hi, eh, lo, el, bs)
    d = lambda t: t.to(DEV)
    out = fused_block_scaled_dual_gemm_backward_dx(d(gq), d(hi), d(lo), d(eg), d(eh), d(el), bs)
    assert rel_fro(out, ref) <= TOL
    torch.testing.assert_close(out.cpu(), ref, atol=1e-2, rtol=1e-2)


def test_gemm_rejects_bad_arguments(lib):
    from tcfp_b200 import _C
    from tcfp_b200.kernels import fused_dual_gemm_forward

    a = torch.zeros(16, 24, device=DEV, dtype=torch.float8_e4m3fn)   # K = 24: row pitch not 16-byte aligned
    w = torch.zeros(16, 24, device=DEV, dtype=torch.float8_e4m3fn)
    s = torch.ones(1, device=DEV)
    with pytest.raises(RuntimeError, match="16-byte"):
        fused_dual_gemm_forward(a, w, w, s, s, s)
    with pytest.raises(AssertionError, match="Shape mismatch"):
        fused_dual_gemm_forward(a, torch.zeros(16, 32, device=DEV, dtype=torch.float8_e4m3fn), w, s, s, s)
    assert lib.tcfp_dual_gemm(None, 0, None, None, None, None, None, None, None, 0, 16, 16, 16, 0, None) == -1
    assert "NULL" in _C.last_error()


def test_fp8_matmul_wrappers():
    """tests/test_core.py:129-145 of the reference: relative error of the FP8 product vs the FP32 product < 0.15."""
    from tcfp_b200.core import fp8_matmul, fp8_matmul_nn, to_fp8_e4m3

    a = acts(600, 256, 512, torch.float32).to(DEV)
    b = acts(601, 512, 384, torch.float32).to(DEV)
    aq, sa = to_fp8_e4m3(a)
    bq, sb = to_fp8_e4m3(b)
    ref = a @ b
    out = fp8_matmul(aq, bq, sa, sb)
    assert float((out - ref).norm() / ref.norm()) < 0.15
    deq = (aq.float() * sa) @ (bq.float() * sb)
    assert rel_fro(out, deq) <= TOL
    btq, sbt = to_fp8_e4m3(b.t().contiguous())
    assert rel_fro(fp8_matmul_nn(aq, btq, sa, sbt), (aq.float() * sa) @ (btq.float() * sbt).t()) <= TOL


def test_bf16_output_and_bias_on_pair_kernel():
    from tcfp_b200.kernels import fused_block_scaled_dual_gemm_forward, fused_dual_gemm_backward_dx

    M, N, K, bs = 512, 384, 256, 64
    a, ea, hi, eh, lo, el = _block_operands(302, M, N, K, bs)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(1))
    d = lambda t: t.to(DEV)
    out = fused_block_scaled_dual_gemm_forward(d(a), d(hi), d(lo), d(ea), d(eh), d(el), bs, bias=d(bias),
                                               out_dtype=torch.bfloat16)
    ref = O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, bs) + bias
    assert out.dtype == torch.bfloat16 and rel_fro(out.float(), ref) <= 5e-3
    g = acts(303, M, K, torch.float32)
    gq, ig = O.to_fp8_e5m2(g)
    w = weights(304, K, N, std=1.0)
    whi, wlo, ihi, ilo, _, _, _ = O.dual_quantize_per_tensor(w)
    out = fused_dual_gemm_backward_dx(d(gq), d(whi), d(wlo), d(ig), d(ihi), d(ilo), out_dtype=torch.bfloat16)
    assert rel_fro(out.float(), O.dual_gemm_nn(gq, ig, whi, ihi, wlo, ilo)) <= 5e-3
    single = fused_dual_gemm_backward_dx(d(gq), d(whi), None, d(ig), d(ihi), None)
    assert rel_fro(single, O.dual_gemm_nn(gq, ig, whi, ihi, None, None)) <= TOL


def test_bounded_wait_gives_up_and_reports(lib):
    """A wait that nothing satisfies ends after its limit, the status word
    records it, the host reads it as TCFP_ERR_DEVICE, and the context keeps
    working."""
    from tcfp_b200 import _C
    from tcfp_b200.kernels import fused_dual_gemm_forward

    _C.check_device_status()                                    # clean before
    _C.check(lib.tcfp_selftest_bounded_wait(1_000_000, _C.stream()))     # 1 ms
    with pytest.raises(RuntimeError, match="bounded wait"):
        _C.check_device_status()
    _C.check_device_status()                                    # the record was cleared
    a, ia, hi, ihi, lo, ilo = _per_tensor_operands(102, 128, 128, 128)
    d = lambda t: t.to(DEV)
    out = fused_dual_gemm_forward(d(a), d(hi), d(lo), d(ia), d(ihi), d(ilo))
    assert rel_fro(out, O.dual_gemm_nt(a, ia, hi, ihi, lo, ilo)) <= TOL
    assert lib.tcfp_selftest_bounded_wait(0, None) == -1


@pytest.mark.parametrize("bs,D_out,D_in", [(32, 384, 640), (64, 384, 640), (128, 384, 640), (32, 160, 96), (64, 192, 320)])
def test_block_retarget_is_exact_up_to_e4m3_underflow(bs, D_out, D_in):
    """The weight re-targeted for the dX contraction dequantizes to the same
    values as the quantized weight it came from: bit-equal wherever the
    exponent shift keeps the value on E4M3's grid, and within 2^-10 * 2^t of
    it where the shift runs into the subnormal step."""
    from tcfp_b200.kernels import block_retarget

    w = weights(410, D_out, D_in, outliers=True)
    w[5] = 0.0                                      # zero rows: -128 sentinel in the residual plane
    w[:, 64:96] *= 1e-3                             # a column block of small rows next to large ones
    hi, lo, eh, el, _ = O.dual_quantize_block(w, bs)
    d = lambda t: t.to(DEV)  # noqa: E731
    hi_t, lo_t, t_hi, t_lo = block_retarget(d(hi), d(lo), d(eh), d(el), bs)
    assert hi_t.shape == (D_in, D_out) and t_hi.shape == (D_out // bs, D_in)
    for codes, exps, codes_t, t, sentinel in ((hi, eh, hi_t, t_hi, False), (lo, el, lo_t, t_lo, True)):
        ref = (O._deq_lo(codes, exps, bs) if sentinel else O.block_dequantize(codes, exps, bs)).double()   # (D_out, D_in)
        scale_t = torch.exp2(t.cpu().double()).repeat_interleave(bs, dim=0)                 # (D_out, D_in)
        got = codes_t.cpu().float().double().t() * scale_t
        bound = 2.0 ** -10 * scale_t
        assert bool(((got - ref).abs() <= bound).all())
        exact = (got == ref).double().mean().item()
        assert exact > 0.85, f"only {exact:.3f} of the values survived the re-encoding bit for bit"
        # t is the largest live exponent of each (row block, column) -- nothing overflows
        assert int(codes_t.view(torch.uint8).cpu().bitwise_and(0x7F).max()) <= 0x7E
    # residual left out (asymmetric backward)
    hi_t2, lo_t2, t_hi2, t_lo2 = block_retarget(d(hi), None, d(eh), None, bs)
    assert lo_t2 is None and t_lo2 is None and torch.equal(hi_t2.view(torch.uint8), hi_t.view(torch.uint8))


@pytest.mark.parametrize("bs,M,D_out,D_in", [(32, 512, 256, 384), (128, 512, 256, 384), (32, 300, 160, 96),
                                             (64, 1000, 192, 320)])
def test_block_backward_dx_routes_agree_and_reuse_the_retargeted_weight(bs, M, D_out, D_in):
    from tcfp_b200.kernels import fused_block_scaled_backward_dx

    g = acts(420, M, D_out, torch.float32)
    w = weights(421, D_out, D_in, outliers=True)
    gq, eg = O.block_quantize(g, bs, torch.float8_e5m2)
    hi, lo, eh, el, _ = O.dual_quantize_block(w, bs)
    ref = O.block_backward_dx(gq, eg, hi, eh, lo, el, bs)
    d = lambda t: t.to(DEV)  # noqa: E731
    dhi, dlo, deh, del_ = d(hi), d(lo), d(eh), d(el)
    fp8 = fused_block_scaled_backward_dx(d(gq), dhi, dlo, d(eg), deh, del_, bs)
    cached = dhi._tcfp_dx
    again = fused_block_scaled_backward_dx(d(gq), dhi, dlo, d(eg), deh, del_, bs)
    assert dhi._tcfp_dx is cached and torch.equal(again, fp8)
    exact = fused_block_scaled_backward_dx(d(gq), dhi, dlo, d(eg), deh, del_, bs, exact_bf16=True)
    assert rel_fro(fp8, ref) <= TOL and rel_fro(exact, ref) <= TOL and rel_fro(fp8, exact) <= 1e-4
    hi_only = fused_block_scaled_backward_dx(d(gq), dhi, None, d(eg), deh, None, bs, out_dtype=torch.bfloat16)
    assert hi_only.dtype == torch.bfloat16
    assert rel_fro(hi_only.float(), O.block_backward_dx(gq, eg, hi, eh, None, None, bs)) <= 5e-3


def test_sm_reserve_shrinks_the_grid_not_the_result(lib):
    """GEMMs launched while SMs are reserved (for a collective beside them)
    walk the same tiles with fewer CTAs: identical bits; the setting is
    per host thread, validated, and restored by the context manager."""
    from tcfp_b200 import _C
    from tcfp_b200.kernels import fused_block_scaled_dual_gemm_forward, fused_dual_gemm_forward

    a, ea, hi, eh, lo, el = _block_operands(305, 1024, 768, 512, 64)
    d = lambda t: t.to(DEV)  # noqa: E731
    ops = [d(t) for t in (a, hi, lo, ea, eh, el)]
    full = fused_block_scaled_dual_gemm_forward(*ops, 64)
    with _C.sm_reserve(32):
        assert lib.tcfp_set_sm_reserve(32) == 32          # reads back what the context manager set
        part = fused_block_scaled_dual_gemm_forward(*ops, 64)
    assert lib.tcfp_set_sm_reserve(0) == 0                # restored on exit
    assert torch.equal(part, full)
    pa, ia, phi, ihi, plo, ilo = [d(t) for t in _per_tensor_operands(306, 200, 256, 384)]   # small M: one-SM kernel
    full = fused_dual_gemm_forward(pa, phi, plo, ia, ihi, ilo)
    with _C.sm_reserve(100):
        assert torch.equal(fused_dual_gemm_forward(pa, phi, plo, ia, ihi, ilo), full)
    assert lib.tcfp_set_sm_reserve(-1) == -1 and "sm_reserve" in _C.last_error()
    assert lib.tcfp_set_sm_reserve(500) == -1


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("M,N,K", [(512, 128, 512), (384, 256, 1024), (300, 384, 256), (1000, 96, 640), (128, 512, 128)])
def test_prologue_fused_activation_quantize_matches_the_two_kernel_route(M, N, K, bs):
    """One kernel that block-quantizes the bf16 activation inside the GEMM's K
    loop: its side outputs are the bytes ``block_quantize_fp8`` produces, its
    output is the separate route's to rounding (a different kernel form sums
    in a different order) and the oracle's within 1e-3; ragged M, N and a K
    that ends inside a 128-wide stage included."""
    from tcfp_b200.kernels import block_quantize_fp8, fused_act_quant_dual_gemm_forward

    x = acts(500 + M, M, K, torch.bfloat16)
    w = weights(501 + N, N, K, outliers=True)
    hi, lo, eh, el, _ = O.dual_quantize_block(w, bs)
    d = lambda t: t.to(DEV)  # noqa: E731
    xd, dhi, dlo, deh, del_ = d(x), d(hi), d(lo), d(eh), d(el)
    y_f, a_f, s_f = fused_act_quant_dual_gemm_forward(xd, dhi, dlo, deh, del_, bs, fuse=True)
    y_s, a_s, s_s = fused_act_quant_dual_gemm_forward(xd, dhi, dlo, deh, del_, bs, fuse=False)
    q, e = block_quantize_fp8(xd, bs)
    assert torch.equal(a_f.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s_f, e)
    assert torch.equal(a_s.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s_s, e)
    assert rel_fro(y_f, y_s) <= 1e-5
    a, ea = O.block_quantize(x, bs)
    assert rel_fro(y_f, O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, bs)) <= TOL
    y2, a2, s2 = fused_act_quant_dual_gemm_forward(xd, dhi, dlo, deh, del_, bs, save_side_outputs=False, fuse=True)
    assert a2 is None and s2 is None and torch.equal(y2, y_f)
    bias = torch.randn(N, device=DEV)
    y3, _, _ = fused_act_quant_dual_gemm_forward(xd, dhi, dlo, deh, del_, bs, bias=bias, out_dtype=torch.bfloat16, fuse=True)
    assert y3.dtype == torch.bfloat16 and rel_fro(y3.float(), y_f + bias) <= 5e-3
