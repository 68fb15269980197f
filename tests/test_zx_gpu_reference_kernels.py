"""GPU: this library's kernels beside the REFERENCE'S OWN kernels on the same
device -- its Triton quantizers and GEMMs (tcfp/kernels.py) and its cuBLASLt
extension (tcfp/csrc/fused_dual_gemm.cu) -- imported unmodified from
``oracle/_ref`` (built by ``python -m oracle.build_ref``; the tests skip when
it is absent).

Quantizers: every code byte, both exponent planes and the error buffer must be
``torch.equal``.  GEMMs: relative Frobenius error <= 1e-3 (the reference's dX
runs a TF32 dot, so it is the less exact side there).

The last test is the drop-in proof: the reference's ``tcfp.nn`` layers and
autograd Functions are re-imported with ``tcfp.kernels`` / ``tcfp.cuda_ext``
replaced by ``tcfp_b200.kernels`` / ``tcfp_b200.cuda_ext`` and must train to
the same numbers as on their own kernels.
"""
import contextlib
import warnings

import pytest
import torch

from oracle import ref_loader
from tests.util import acts, bits, rel_fro, u8, weights

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_loader.available(), reason="oracle/_ref not built (python -m oracle.build_ref)")]
DEV = "cuda"
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
SRR_SEED = 0x5EED


@pytest.fixture(scope="module")
def ref():
    pkg = ref_loader.load_reference()
    import tcfp.cuda_ext as rc
    import tcfp.kernels as rk

    if not rk.is_triton_available():
        pytest.skip("Triton cannot run the reference kernels on this device")
    yield pkg, rk, rc
    ref_loader.unload()


@contextlib.contextmanager
def fixed_srr_seed(seed: int):
    """The reference draws its stochastic-rounding seed with ``torch.randint``
    inside the wrapper (tcfp/kernels.py:1828-1831); pin it for the call."""
    orig = torch.randint

    def fake(*a, **k):
        return torch.tensor([seed], device=k.get("device", "cpu"))

    torch.randint = fake
    try:
        yield
    finally:
        torch.randint = orig


def _ulp_sweep_weight(n: int, k: int, fmax: float) -> torch.Tensor:
    """Every 32-wide block's amax sits a few ulps around ``fmax * 2^e`` -- the
    inputs on which ``ceil(log2(amax / fmax))`` is decided by the last bits of
    the device's division and log2."""
    w = weights(7, n, k, std=0.02) * 1e-3
    blocks = k // 32
    for r in range(n):
        for b in range(blocks):
            base = torch.tensor(fmax * 2.0 ** (-(r % 40) + 8), dtype=torch.float32)
            off = (b + 3 * r) % 80 - 8
            w[r, 32 * b] = (base.view(torch.int32) + off).view(torch.float32)
            w[r, 32 * b + 1:32 * b + 32] *= 1e-4 * float(base)
    w[0, :] = 0.0
    w[1, :] = 1e-20
    w[2, :] = 1.0
    w[3, 5] = 3.0e4
    return w


def _cases():
    return [("ulp_sweep", _ulp_sweep_weight(128, 512, 448.0)),
            ("outliers", weights(11, 256, 1024, outliers=True)),
            ("config3_slice", weights(1003, 1024, 2048, outliers=True))]


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("mode", ["none", "ef", "srr"])
def test_dual_quantize_bytes_equal_the_reference_triton_kernel(ref, bs, mode):
    """tcfp/kernels.py:288-459 + the error update of its wrapper (:1867-1873)."""
    from tcfp_b200.kernels import fused_dual_quantize_fp8

    _, rk, _ = ref
    for tag, w in _cases():
        wd = w.to(DEV)
        err = weights(5, *w.shape, std=1e-4).to(DEV) if mode == "ef" else None
        e_ref = err.clone() if err is not None else None
        e_own = err.clone() if err is not None else None
        with fixed_srr_seed(SRR_SEED):
            rh, rl, rsh, rsl = rk.fused_dual_quantize_fp8(wd, bs, e_ref, mode == "srr")
        oh, ol, osh, osl = fused_dual_quantize_fp8(wd, bs, e_own, mode == "srr", seed=SRR_SEED, offset=0)
        assert torch.equal(osh, rsh), f"{tag}: W_hi exponents differ in {(osh != rsh).sum().item()} blocks"
        assert torch.equal(u8(oh), u8(rh)), f"{tag}: W_hi codes differ"
        assert torch.equal(osl, rsl), f"{tag}: W_lo exponents differ in {(osl != rsl).sum().item()} blocks"
        assert torch.equal(u8(ol), u8(rl)), f"{tag}: W_lo codes differ"
        if err is not None:
            assert torch.equal(bits(e_own), bits(e_ref)), f"{tag}: error buffer differs"


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("fmt", [E4, E5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_quantize_bytes_equal_the_reference_triton_kernel(ref, bs, fmt, dtype):
    """tcfp/kernels.py:205-275."""
    from tcfp_b200.kernels import block_quantize_fp8

    _, rk, _ = ref
    fmax = 448.0 if fmt == E4 else 57344.0
    for tag, x in [("ulp_sweep", _ulp_sweep_weight(128, 512, fmax)), ("acts", acts(3, 300, 1024, torch.float32)),
                   ("grads", acts(4, 256, 768, torch.float32) * 37.0)]:
        xd = x.to(dtype).to(DEV)
        rq, rs = rk.block_quantize_fp8(xd, bs, fmt)
        oq, os_ = block_quantize_fp8(xd, bs, fmt)
        assert torch.equal(os_, rs), f"{tag}: exponents differ in {(os_ != rs).sum().item()} blocks"
        assert torch.equal(u8(oq), u8(rq)), f"{tag}: codes differ"


def _block_operands(bs, M=768, N=640, K=1024):
    from tcfp_b200.kernels import block_quantize_fp8, fused_dual_quantize_fp8

    x = acts(1, M, K).to(DEV)
    w = weights(2, N, K, outliers=True).to(DEV)
    hi, lo, sh, sl = fused_dual_quantize_fp8(w, bs)
    a, sa = block_quantize_fp8(x, bs, E4)
    return x, a, sa, hi, lo, sh, sl


@pytest.mark.parametrize("bs", [32, 64, 128])
def test_block_gemms_match_the_reference_triton_kernels(ref, bs):
    """Forward tcfp/kernels.py:628-796, dX :1051-1205, single GEMM :491-600."""
    from tcfp_b200.kernels import (block_quantize_fp8, block_scaled_gemm, fused_block_scaled_dual_gemm_backward_dx,
                                   fused_block_scaled_dual_gemm_forward)

    _, rk, _ = ref
    x, a, sa, hi, lo, sh, sl = _block_operands(bs)
    y_ref = rk.fused_block_scaled_dual_gemm_forward(a, hi, lo, sa, sh, sl, bs)
    y = fused_block_scaled_dual_gemm_forward(a, hi, lo, sa, sh, sl, bs)
    assert y.dtype == y_ref.dtype and rel_fro(y, y_ref) <= 1e-3
    assert rel_fro(block_scaled_gemm(a, hi, sa, sh, bs), rk.block_scaled_gemm(a, hi, sa, sh, bs)) <= 1e-3
    g = acts(3, a.shape[0], hi.shape[0], torch.float32).to(DEV)
    gq, sg = block_quantize_fp8(g, bs, E5)
    dx_ref = rk.fused_block_scaled_dual_gemm_backward_dx(gq, hi, lo, sg, sh, sl, bs)
    dx = fused_block_scaled_dual_gemm_backward_dx(gq, hi, lo, sg, sh, sl, bs)
    assert rel_fro(dx, dx_ref) <= 1e-3                  # the reference side is a TF32 dot


@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("n_out", [128, 384, 512])
def test_fused_act_quant_forward_and_side_outputs(ref, bs, n_out):
    """tcfp/kernels.py:2031-2149; the reference's own pins are
    tests/test_fused_act_quant_gemm.py:116-144 (side outputs bit-equal to
    ``block_quantize_fp8``) and :513-547 (``None`` when not saved)."""
    from tcfp_b200.kernels import block_quantize_fp8, fused_act_quant_dual_gemm_forward

    _, rk, _ = ref
    x, a, sa, hi, lo, sh, sl = _block_operands(bs, M=512, N=n_out, K=512)
    y_ref, a_ref, sa_ref = rk.fused_act_quant_dual_gemm_forward(x, hi, lo, sh, sl, bs)
    y, a_own, sa_own = fused_act_quant_dual_gemm_forward(x, hi, lo, sh, sl, bs)
    assert rel_fro(y, y_ref) <= 1e-3
    assert torch.equal(u8(a_own), u8(a_ref)) and torch.equal(sa_own, sa_ref)
    for fuse in (True, False):          # the prologue-fused kernel and the two-kernel route, whichever the default took
        yk, ak, sk = fused_act_quant_dual_gemm_forward(x, hi, lo, sh, sl, bs, fuse=fuse)
        assert rel_fro(yk, y_ref) <= 1e-3 and torch.equal(u8(ak), u8(a_ref)) and torch.equal(sk, sa_ref)
    q, s = block_quantize_fp8(x, bs, E4)
    assert torch.equal(u8(a_own), u8(q)) and torch.equal(sa_own, s)
    y2, a2, s2 = fused_act_quant_dual_gemm_forward(x, hi, lo, sh, sl, bs, save_side_outputs=False)
    assert a2 is None and s2 is None and torch.equal(y2, y)


def test_per_tensor_dual_gemm_against_triton_and_the_cublaslt_extension(ref):
    """tcfp/kernels.py:1545-1666 and tcfp/cuda_ext.py:241-282 (two cuBLASLt
    GEMMs, tcfp/csrc/fused_dual_gemm.cu:119-274) -- through the shim names of
    ``tcfp_b200.cuda_ext`` as well."""
    from tcfp_b200 import cuda_ext as own_ext
    from tcfp_b200.core import dual_quantize_per_tensor, to_fp8_e4m3, to_fp8_e5m2
    from tcfp_b200.kernels import fused_dual_gemm_backward_dx, fused_dual_gemm_forward, is_triton_available

    pkg, rk, rc = ref
    assert own_ext.is_cuda_ext_available() and is_triton_available()
    M, N, K = 512, 384, 768
    x = acts(1, M, K).to(DEV)
    w = weights(2, N, K, std=1.0).to(DEV)
    hi, lo, ih, il, _ = dual_quantize_per_tensor(w)
    a, ia = to_fp8_e4m3(x)
    # the activation cast itself against the reference's torch chain on the same device (tcfp/core.py:85-106)
    ra, ria = pkg.core.to_fp8_e4m3(x)
    assert torch.equal(u8(ra), u8(a)) and torch.equal(bits(ria.reshape(1)), bits(ia.reshape(1)))
    y = fused_dual_gemm_forward(a, hi, lo, ia, ih, il)
    assert torch.equal(own_ext.cuda_ext_dual_gemm_forward(a, hi, lo, ia, ih, il), y)
    assert rel_fro(y, rk.fused_dual_gemm_forward(a, hi, lo, ia, ih, il)) <= 1e-3
    g = acts(3, M, N, torch.float32).to(DEV)
    gq, ig = to_fp8_e5m2(g)
    dx = fused_dual_gemm_backward_dx(gq, hi, lo, ig, ih, il)
    assert torch.equal(own_ext.cuda_ext_dual_gemm_backward_dx(gq, hi, lo, ig, ih, il), dx)
    assert rel_fro(dx, rk.fused_dual_gemm_backward_dx(gq, hi, lo, ig, ih, il)) <= 1e-3
    if rc.is_cuda_ext_available():
        assert rel_fro(y, rc.cuda_ext_dual_gemm_forward(a, hi, lo, ia, ih, il)) <= 1e-3
        assert rel_fro(dx, rc.cuda_ext_dual_gemm_backward_dx(gq, hi, lo, ig, ih, il)) <= 1e-3


def _train_two_steps(pkg, layer_kw, x, target, w0, b0):
    layer = pkg.nn.TCFPLinear(w0.shape[1], w0.shape[0], bias=True, use_tensor_cores=True, **layer_kw).to(DEV)
    with torch.no_grad():
        layer.weight.copy_(w0)
        layer.bias.copy_(b0)
    layer._param_name = "layer"
    opt = torch.optim.SGD(layer.parameters(), lr=1e-2)
    out = {}
    for step in range(2):
        opt.zero_grad()
        xin = x.clone().requires_grad_(True)
        y = layer(xin)
        ((y - target) ** 2).mean().backward()
        out[f"y{step}"] = y.detach().float().clone()
        out[f"dx{step}"] = xin.grad.float().clone()
        out[f"dw{step}"] = layer.weight.grad.float().clone()
        out[f"db{step}"] = layer.bias.grad.float().clone()
        st = layer._error_state
        if st is not None and "layer" in st._buffers:
            out[f"ef{step}"] = st._buffers["layer"].clone()
        opt.step()
    return out


@pytest.mark.parametrize("layer_kw", [dict(scale_block_size=64), dict(scale_block_size=32, hp_grad_weight=True),
                                      dict(), dict(delayed_scaling=True), dict(abd=True, scale_block_size=128)],
                         ids=["block64", "block32_hp", "per_tensor", "per_tensor_delayed", "block128_abd"])
def test_reference_nn_runs_unmodified_on_these_kernels(layer_kw):
    """Drop-in proof: ``tcfp.nn.TCFPLinear`` of the reference, two SGD steps,
    once on its own Triton / cuBLASLt kernels and once with ``tcfp.kernels`` and
    ``tcfp.cuda_ext`` swapped for this library's modules (the call sites at
    tcfp/nn/__init__.py:394-403, 509-515, 627-650, 724-741)."""
    M, K, N = 512, 256, 384
    x = acts(21, M, K, torch.float32).to(DEV)
    target = acts(22, M, N, torch.float32).to(DEV)
    w0 = weights(23, N, K, std=0.05).to(DEV)
    b0 = (weights(24, 1, N, std=0.1)[0]).to(DEV)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        native = _train_two_steps(ref_loader.load_reference(), layer_kw, x, target, w0, b0)
        import tcfp.nn as rnn_native

        assert rnn_native._HAS_FUSED_KERNELS
        swapped_pkg = ref_loader.load_reference_on_b200_kernels()
        import tcfp.nn as rnn

        assert rnn._HAS_FUSED_KERNELS and rnn._HAS_CUDA_EXT
        assert rnn.fused_dual_quantize_fp8.__module__ == "tcfp_b200.kernels"
        assert rnn.cuda_ext_dual_gemm_forward.__module__ == "tcfp_b200.cuda_ext"
        swapped = _train_two_steps(swapped_pkg, layer_kw, x, target, w0, b0)
    ref_loader.unload()
    assert native.keys() == swapped.keys()
    for key in native:
        if key == "ef0":
            # same weight, same buffer in: the quantizer must leave identical bits behind (the second step
            # quantizes an SGD-updated weight whose gradient differs in the last bits between the two runs)
            assert torch.equal(bits(swapped[key]), bits(native[key])), "error buffer after the first step differs"
            continue
        tol = 1e-2 if key.startswith("dx") else 2e-3     # reference dX is a TF32 dot
        assert rel_fro(swapped[key], native[key]) <= tol, f"{key}: {rel_fro(swapped[key], native[key]):.2e}"
