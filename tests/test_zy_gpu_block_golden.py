"""GPU: the CUDA block-scaled kernels against the outputs of the reference's
own Triton kernels (tests/golden/block_path.npz, recorded under the Triton
interpreter; see tests/block_golden_check.py for what is compared)."""
import pytest
import torch

from tests.block_golden_check import check_block_quantize, check_dual_quantize, golden_operands
from tests.golden.cases import BLOCK_CASES, block_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.mark.parametrize("name", list(BLOCK_CASES))
def test_quantizers_match_reference_triton_kernels(name):
    from tcfp_b200.kernels import block_quantize_fp8, fused_dual_quantize_fp8

    cfg = BLOCK_CASES[name]
    w, err, x, g = block_inputs(cfg)
    srr = "srr_seed" in cfg
    hi, lo, eh, el = fused_dual_quantize_fp8(w.to(DEV), cfg["bs"], None if err is None else err.to(DEV), srr,
                                             seed=cfg.get("srr_seed"), offset=0)
    check_dual_quantize(name, hi.cpu(), lo.cpu(), eh.cpu(), el.cpu())
    q, e = block_quantize_fp8(x.to(DEV), cfg["bs"], E4)
    check_block_quantize(name, "act", q.cpu(), e.cpu())
    q, e = block_quantize_fp8(g.to(DEV), cfg["bs"], E5)
    check_block_quantize(name, "grad", q.cpu(), e.cpu())


@pytest.mark.parametrize("name", list(BLOCK_CASES))
def test_gemms_match_reference_triton_kernels(name):
    """Forward and dX on the reference kernels' own quantized operands,
    against the reference kernels' FP32 outputs (tolerance: 1e-3 relative
    Frobenius error; measured ~1e-7)."""
    from tcfp_b200.kernels import fused_block_scaled_dual_gemm_backward_dx, fused_block_scaled_dual_gemm_forward

    bs = BLOCK_CASES[name]["bs"]
    o = golden_operands(name)
    d = lambda t: t.to(DEV)  # noqa: E731
    y = fused_block_scaled_dual_gemm_forward(d(o["a"]), d(o["hi"]), d(o["lo"]), d(o["ea"]), d(o["eh"]), d(o["el"]), bs)
    dx = fused_block_scaled_dual_gemm_backward_dx(d(o["g"]), d(o["hi"]), d(o["lo"]), d(o["eg"]), d(o["eh"]), d(o["el"]), bs)
    assert float((y.cpu() - o["y"]).norm() / o["y"].norm()) <= 1e-3
    assert float((dx.cpu() - o["dx"]).norm() / o["dx"].norm()) <= 1e-3
