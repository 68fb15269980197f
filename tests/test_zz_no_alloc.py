"""The allocation-free block-scaled GEMM entry point.

``tcfp_block_dual_gemm_static`` serves callers that own no allocator -- a
plugin handed nothing but input and output buffers, or code that must not
call cudaMalloc -- by keeping the re-packed scale factors in an array that
ships inside the library.  It must return exactly what the regular two-step
route (``tcfp_pack_scales`` into caller buffers, then
``tcfp_block_dual_gemm``) returns, call after call, even though every call
reuses the same scratch.  This file sorts last on purpose: a run that stops
at the first failure has then already run every other test.
"""
import pytest
import torch

from oracle import tcfp_oracle as O
from tests.util import acts, weights

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _operands(seed, M, N, K, bs):
    x = acts(seed, M, K, torch.bfloat16)
    w = weights(seed + 1, N, K, outliers=True)
    a, ea = O.block_quantize(x, bs)
    hi, lo, eh, el, _ = O.dual_quantize_block(w, bs)
    return [t.to(DEV) for t in (a, ea, hi, eh, lo, el)]


def _static(lib, a, ea, hi, eh, lo, el, bs, bias=None, dtype=torch.float32):
    from tcfp_b200 import _C

    M, K = a.shape
    N = hi.shape[0]
    out = torch.empty(M, N, device=DEV, dtype=dtype)
    _C.check(lib.tcfp_block_dual_gemm_static(
        a.data_ptr(), ea.data_ptr(), hi.data_ptr(), eh.data_ptr(), _C.ptr(lo), _C.ptr(el), _C.ptr(bias),
        out.data_ptr(), _C.F32 if dtype == torch.float32 else _C.BF16, M, N, K, bs, _C.stream()))
    return out


def test_static_scratch_gemm_matches_regular_entry_point_twice(lib):
    from tcfp_b200.kernels import fused_block_scaled_dual_gemm_forward

    # two calls in a row with different shapes and block sizes: the second
    # must not see anything the first left in the shared scratch
    for seed, (M, N, K, bs) in ((700, (256, 384, 512, 32)), (710, (100, 128, 1024, 128))):
        a, ea, hi, eh, lo, el = _operands(seed, M, N, K, bs)
        got = _static(lib, a, ea, hi, eh, lo, el, bs)
        want = fused_block_scaled_dual_gemm_forward(a, hi, lo, ea, eh, el, bs)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        ref = O.block_dual_gemm_nt(*(t.cpu() for t in (a, ea, hi, eh, lo, el)), bs)
        assert float((got.cpu() - ref).norm() / ref.norm()) <= 1e-3


def test_static_scratch_variants_match_the_two_step_route(lib):
    """Residual left out (the third scratch region stays unused), bias with a
    bf16 epilogue, and a K whose scale blocks do not fill a group of four --
    each bit for bit what the regular entry points return; a call refused for
    its output type launches nothing and the next call is unaffected."""
    from tcfp_b200 import _C
    from tcfp_b200.kernels import fused_block_scaled_dual_gemm_forward

    a, ea, hi, eh, lo, el = _operands(720, 256, 256, 512, 64)
    got = _static(lib, a, ea, hi, eh, None, None, 64)
    assert torch.equal(got, fused_block_scaled_dual_gemm_forward(a, hi, None, ea, eh, None, 64))
    bias = torch.randn(256, device=DEV)
    got = _static(lib, a, ea, hi, eh, lo, el, 64, bias=bias, dtype=torch.bfloat16)
    assert torch.equal(got, fused_block_scaled_dual_gemm_forward(a, hi, lo, ea, eh, el, 64, bias=bias,
                                                                 out_dtype=torch.bfloat16))
    a3, ea3, hi3, eh3, lo3, el3 = _operands(730, 128, 128, 192, 64)          # 3 scale blocks along K
    want3 = fused_block_scaled_dual_gemm_forward(a3, hi3, lo3, ea3, eh3, el3, 64)
    out = torch.empty(256, 256, device=DEV)
    rc = lib.tcfp_block_dual_gemm_static(a.data_ptr(), ea.data_ptr(), hi.data_ptr(), eh.data_ptr(), lo.data_ptr(),
                                         el.data_ptr(), None, out.data_ptr(), 7, 256, 256, 512, 64, _C.stream())
    assert rc == -1 and "float32 or bfloat16" in _C.last_error()
    assert torch.equal(_static(lib, a3, ea3, hi3, eh3, lo3, el3, 64), want3)


def test_static_scratch_rejects_oversized_operands(lib):
    from tcfp_b200 import _C

    limit = lib.tcfp_static_scratch_bytes_per_operand()
    assert limit == 2 << 20
    M, N, K, bs = 16384, 128, 8192, 32          # packed activation scales: 4 MiB > 2 MiB
    assert lib.tcfp_sf_packed_bytes(M, K, bs) > limit
    dummy = torch.zeros(16, device=DEV, dtype=torch.uint8)
    rc = lib.tcfp_block_dual_gemm_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                         dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), _C.F32,
                                         M, N, K, bs, _C.stream())
    assert rc == -2 and "built-in scratch" in _C.last_error()
