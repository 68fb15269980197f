"""Same three names as the reference's ``tcfp/cuda_ext.py:236-282``, served by
the tcgen05 dual-GEMM kernel instead of two cuBLASLt calls
(tcfp/csrc/fused_dual_gemm.cu:119-274)."""
from __future__ import annotations

import torch

from . import _C
from .kernels import fused_dual_gemm_backward_dx, fused_dual_gemm_forward


def is_cuda_ext_available() -> bool:
    """True when ``libtcfp_b200.so`` loads on an sm_100 device."""
    return _C.is_available()


def cuda_ext_dual_gemm_forward(act_fp8, w_hi_fp8, w_lo_fp8, act_inv, w_hi_inv, w_lo_inv) -> torch.Tensor:
    """tcfp/cuda_ext.py:241-259 -> ``(M, N)`` FP32."""
    return fused_dual_gemm_forward(act_fp8, w_hi_fp8, w_lo_fp8, act_inv, w_hi_inv, w_lo_inv)


def cuda_ext_dual_gemm_backward_dx(grad_fp8, w_hi_fp8, w_lo_fp8, grad_inv, w_hi_inv, w_lo_inv) -> torch.Tensor:
    """tcfp/cuda_ext.py:262-282 -> ``(M, D_in)`` FP32."""
    return fused_dual_gemm_backward_dx(grad_fp8, w_hi_fp8, w_lo_fp8, grad_inv, w_hi_inv, w_lo_inv)
