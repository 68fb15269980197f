"""GPU parity at the sizes of the benchmark configurations (the other GPU
tests use small shapes): the kernels run ONE full-size launch -- grid size,
64-bit indexing and tile tails as in the benchmark -- and are compared with
the CPU oracle, bit for bit for the quantizers, within 1e-3 relative
Frobenius error on a 512-row slice for the GEMMs.

configuration 1: 4096 x 4096 per-tensor error feedback + 4096^3 forward;
configuration 2: 8192 x 8192 with 0.1 % x50 outliers, block 32 / 64 / 128 error
                 feedback, 8192^3 forward and dX;
configuration 3: 16384 x 4096 per-tensor stochastic residual, seed 0x5EED;
configuration 4: the weight gradient of one decoder projection (32768 tokens,
                 4096 -> 12288) from a bf16 gradient and from an FP32 one.
"""
import pytest
import torch

from oracle import tcfp_oracle as O
from tests.util import acts, bits, rel_fro, u8, weights

pytestmark = pytest.mark.gpu
DEV = "cuda"
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def test_per_tensor_error_feedback_4096_and_forward():
    from tcfp_b200.core import dual_quantize_per_tensor, to_fp8_e4m3
    from tcfp_b200.kernels import fused_dual_gemm_forward

    n = 4096
    w = weights(1002, n, n, std=1.0)
    err = weights(6, n, n, std=1e-3)
    hi, lo, ihi, ilo, new_err, _, _ = O.dual_quantize_per_tensor(w, err)
    err_d = err.to(DEV)
    ghi, glo, gihi, gilo, _ = dual_quantize_per_tensor(w.to(DEV), err_d)
    assert torch.equal(u8(ghi), u8(hi)) and torch.equal(u8(glo), u8(lo))
    assert torch.equal(bits(gihi), bits(ihi)) and torch.equal(bits(gilo), bits(ilo))
    assert torch.equal(bits(err_d), bits(new_err))
    x = acts(1102, n, n)
    a, ia = O.to_fp8_e4m3(x)
    ga, gia = to_fp8_e4m3(x.to(DEV))
    assert torch.equal(u8(ga), u8(a)) and torch.equal(bits(gia), bits(ia))
    y = fused_dual_gemm_forward(ga, ghi, glo, gia, gihi, gilo)
    ref = O.dual_gemm_nt(a[:512], ia, hi, ihi, lo, ilo)
    assert rel_fro(y[:512], ref) <= 1e-3


@pytest.mark.parametrize("bs", [32, 64, 128])
def test_block_error_feedback_8192_with_outliers_forward_and_dx(bs):
    from tcfp_b200.kernels import (block_quantize_fp8, fused_block_scaled_dual_gemm_backward_dx,
                                   fused_block_scaled_dual_gemm_forward, fused_dual_quantize_fp8)

    n = 8192
    w = weights(1003, n, n, outliers=True)
    err = weights(7, n, n, std=1e-4)
    hi, lo, eh, el, new_err = O.dual_quantize_block(w, bs, err)
    err_d = err.to(DEV)
    ghi, glo, geh, gel = fused_dual_quantize_fp8(w.to(DEV), bs, err_d)
    assert torch.equal(geh.cpu(), eh) and torch.equal(gel.cpu(), el)
    assert torch.equal(u8(ghi), u8(hi)) and torch.equal(u8(glo), u8(lo))
    assert torch.equal(bits(err_d), bits(new_err))
    del err_d, new_err, err, w

    x = acts(1103, n, n)
    ga, gea = block_quantize_fp8(x.to(DEV), bs, E4)
    rows = 512
    a, ea = O.block_quantize(x[:rows], bs)
    assert torch.equal(u8(ga[:rows]), u8(a)) and torch.equal(gea[:, :rows].cpu(), ea)
    y = fused_block_scaled_dual_gemm_forward(ga, ghi, glo, gea, geh, gel, bs)
    ref = O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, bs)
    assert rel_fro(y[:rows], ref) <= 1e-3
    # rows from the far end too: the last tile row of the persistent schedule
    a2, ea2 = O.block_quantize(x[-rows:], bs)
    assert rel_fro(y[-rows:], O.block_dual_gemm_nt(a2, ea2, hi, eh, lo, el, bs)) <= 1e-3
    del y, ga, gea

    g = acts(1203, n, n, torch.float32)
    gq, geg = block_quantize_fp8(g.to(DEV), bs, E5)
    q, eg = O.block_quantize(g[:rows], bs, E5)
    assert torch.equal(u8(gq[:rows]), u8(q)) and torch.equal(geg[:, :rows].cpu(), eg)
    dx = fused_block_scaled_dual_gemm_backward_dx(gq, ghi, glo, geg, geh, gel, bs)
    assert rel_fro(dx[:rows], O.block_backward_dx(q, eg, hi, eh, lo, el, bs)) <= 1e-3


def test_per_tensor_stochastic_residual_16384x4096():
    """The stochastic residual of the large MLP's weight: W_hi and both inverse
    scales over the whole tensor, W_lo on three row slabs (first, middle,
    last) whose uniforms are the stream's elements ``offset + n*K + k``."""
    from tcfp_b200.core import dual_quantize_per_tensor

    N, K = 16384, 4096
    seed, offset = 0x5EED, 3 * N * K
    w = weights(1004, N, K)
    ghi, glo, gihi, gilo, _ = dual_quantize_per_tensor(w.to(DEV), None, srr=True, seed=seed, offset=offset)
    s_hi = (O.FP8_E4M3_MAX / w.abs().max().clamp(min=1e-12)).to(torch.float32)
    hi, ihi = O.to_fp8_e4m3(w, scale=s_hi)
    assert torch.equal(u8(ghi), u8(hi)) and torch.equal(bits(gihi), bits(ihi))
    residual = w - hi.float() * ihi
    s_lo = (O.FP8_E4M3_MAX / residual.abs().max().clamp(min=1e-12)).to(torch.float32)
    for r0 in (0, N // 2 - 64, N - 128):
        r1 = r0 + 128
        rand = O.philox_uniform_packed(seed, offset + r0 * K, (r1 - r0) * K).reshape(r1 - r0, K)
        lo, ilo = O.to_fp8_e4m3_sr(residual[r0:r1], rand, scale=s_lo)
        assert torch.equal(u8(glo[r0:r1]), u8(lo)), f"W_lo rows {r0}..{r1} differ"
        assert torch.equal(bits(gilo), bits(ilo))


def test_block_path_weight_gradient_at_decoder_size():
    """dW = g^T . x over 32768 tokens for the fused q/k/v projection (4096 ->
    12288): the single bf16 product (256 x 256 tiles) for a bf16 gradient and
    the head + tail dual product for an FP32 gradient, each checked on three
    128 x 256 windows (first, interior across tile borders, last) against a
    float64 product of the same operands.  Tolerance: the tensor core adds each
    product block into its FP32 accumulator with truncation, a bias of about
    2^-25 per accumulation step towards zero; 32768 tokens are 2048 steps for
    one product (measured below 5e-5) and 4096 for head + tail (measured 7.6e-5).
    Short contractions meet 2e-5 (tests/test_gpu_nn.py)."""
    from tcfp_b200.kernels import bf16_weight_grad

    tokens, d_out, d_in = 32768, 12288, 4096
    g = acts(1301, tokens, d_out, torch.float32) * 0.01
    x = acts(1302, tokens, d_in)
    xd = x.to(DEV)
    windows = [(0, 0), (6100, 1900), (d_out - 128, d_in - 256)]
    for grad, tol in ((g.to(torch.bfloat16), 1e-4), (g, 2e-4)):
        out = bf16_weight_grad(grad.to(DEV), xd)
        assert out.shape == (d_out, d_in)
        for r0, c0 in windows:
            ref = grad[:, r0:r0 + 128].double().t() @ x[:, c0:c0 + 256].double()
            assert rel_fro(out[r0:r0 + 128, c0:c0 + 256], ref) <= tol, (grad.dtype, r0, c0)
        del out
