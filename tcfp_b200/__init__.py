"""tcfp_b200: the TCFP-12 linear-layer hot path on B200 (sm_100a).

Host side is Python/PyTorch; the compute lives in ``libtcfp_b200.so`` (C ABI in
``include/tcfp_b200.h``), built in-tree by ``python -m tcfp_b200.build``.
Sub-modules: ``core`` (FP8 casts, error-feedback state), ``kernels`` and
``cuda_ext`` (launch wrappers under the reference's names), ``nn``
(``TCFPLinear``, ``convert_to_tcfp``), ``tp`` (tensor parallelism),
``checkpoint``, ``host_pipeline``, ``workloads``, ``microbench``.
"""
from . import core as _core

__version__ = "0.1.0"
__all__ = [
    "FP8_E4M3_MAX", "FP8_E5M2_MAX", "ErrorFeedbackState", "TCFPMode", "absmax", "dual_quantize_per_tensor",
    "ensure_column_major", "fp8_matmul", "fp8_matmul_nn", "to_fp8_e4m3", "to_fp8_e4m3_nf_aware", "to_fp8_e4m3_sr",
    "to_fp8_e5m2",
]
globals().update({name: getattr(_core, name) for name in __all__})
