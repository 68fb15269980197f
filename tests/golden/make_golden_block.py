"""Generates ``tests/golden/block_path.npz`` by executing the REFERENCE's own
Triton kernel bodies on CPU tensors with the Triton interpreter
(``TRITON_INTERPRET=1``; the autotuner is bypassed by calling ``kernel.fn``
with an explicit block size).

    python tests/golden/make_golden_block.py /path/to/reference

Recorded per case: the raw outputs of
  * ``_fused_dual_quantize_kernel``  (tcfp/kernels.py:288-459): W_hi / W_lo codes, both exponent planes
  * ``_block_quantize_kernel``       (tcfp/kernels.py:205-275): codes + exponent plane, E4M3 and E5M2
  * ``_fused_block_scaled_dual_gemm_kernel`` (tcfp/kernels.py:628-796) and
    ``_fused_block_scaled_backward_dx_kernel`` (tcfp/kernels.py:1051-1205): FP32 outputs

Known defect of the interpreter (not of the reference): its float32 -> FP8
cast drops the exponent carry when round-to-nearest crosses a power of two
(31.8 -> 16 instead of 32).  The tests therefore compare codes everywhere
except on those elements, and compare every stage that follows (residual,
W_lo exponents, W_lo codes) starting from the kernel's OWN W_hi codes.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 2:
    sys.exit("usage: make_golden_block.py <path to a checkout of the reference project>")
sys.path.append(sys.argv[1])

import tcfp.kernels as rk  # noqa: E402

from tests.golden.cases import BLOCK_CASES, block_inputs  # noqa: E402

out: dict[str, np.ndarray] = {}
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def u8(t):
    return t.contiguous().view(torch.uint8).numpy().copy()


def body(kernel):
    return kernel.fn if hasattr(kernel, "fn") and not callable(getattr(kernel, "run", None)) else kernel.fn


for name, cfg in BLOCK_CASES.items():
    w, err, x, g = block_inputs(cfg)
    N, K, M, bs = cfg["N"], cfg["K"], cfg["M"], cfg["bs"]
    nkb = K // bs
    # --- dual quantize
    hi = torch.empty(N, K, dtype=E4)
    lo = torch.empty(N, K, dtype=E4)
    sh = torch.empty(nkb, N, dtype=torch.int8)
    sl = torch.empty(nkb, N, dtype=torch.int8)
    has_err = err is not None
    eo = err if has_err else w
    BN = 32
    body(rk._fused_dual_quantize_kernel)[((N + BN - 1) // BN, nkb)](
        w, eo, hi, lo, sh, sl, N, K, w.stride(0), w.stride(1), eo.stride(0) if has_err else 0,
        eo.stride(1) if has_err else 0, hi.stride(0), hi.stride(1), lo.stride(0), lo.stride(1), sh.stride(1),
        sh.stride(0), sl.stride(1), sl.stride(0), cfg.get("srr_seed", 0), HAS_ERROR=has_err,
        STOCHASTIC_LO="srr_seed" in cfg, FP8_MAX=448.0, BLOCK_K=bs, BLOCK_N=BN)
    out[f"{name}/w_hi"], out[f"{name}/w_lo"] = u8(hi), u8(lo)
    out[f"{name}/exp_hi"], out[f"{name}/exp_lo"] = sh.numpy().copy(), sl.numpy().copy()
    # --- block quantize of activations (E4M3) and gradients (E5M2, blocks along N)
    for tag, t, dt, fmax in (("act", x, E4, 448.0), ("grad", g, E5, 57344.0)):
        R, C = t.shape
        q = torch.empty(R, C, dtype=dt)
        e = torch.empty(C // bs, R, dtype=torch.int8)
        BMq = 32
        body(rk._block_quantize_kernel)[((R + BMq - 1) // BMq, C // bs)](
            t, q, e, R, C, t.stride(0), t.stride(1), q.stride(0), q.stride(1), e.stride(1), e.stride(0),
            FP8_MAX=fmax, BLOCK_SIZE=bs, BLOCK_M=BMq)
        out[f"{name}/{tag}"], out[f"{name}/{tag}_exp"] = u8(q), e.numpy().copy()
        if tag == "act":
            a_q, a_e = q, e
        else:
            g_q, g_e = q, e
    # --- forward GEMM on the kernel's own quantized operands
    y = torch.empty(M, N, dtype=torch.float32)
    BMg, BNg = 64, 64
    tiles = ((M + BMg - 1) // BMg) * ((N + BNg - 1) // BNg)
    body(rk._fused_block_scaled_dual_gemm_kernel)[(tiles,)](
        a_q, hi, lo, y, a_e, sh, sl, M, N, K, nkb, a_q.stride(0), a_q.stride(1), hi.stride(1), hi.stride(0),
        lo.stride(1), lo.stride(0), y.stride(0), y.stride(1), a_e.stride(1), a_e.stride(0), sh.stride(1),
        sh.stride(0), sl.stride(1), sl.stride(0), BLOCK_M=BMg, BLOCK_N=BNg, BLOCK_K=bs, GROUP_M=8,
        SPARSE_THRESHOLD=0.0, num_sms_launch=1 << 30)
    out[f"{name}/y"] = y.numpy().copy()
    # --- backward dX: grad (M, N=D_out) blocks along D_out; W (D_out, D_in) scales (D_in/bs, D_out)
    dx = torch.empty(M, K, dtype=torch.float32)
    BMd = 64
    tiles = ((M + BMd - 1) // BMd) * (K // bs)
    body(rk._fused_block_scaled_backward_dx_kernel)[(tiles,)](
        g_q, hi, lo, dx, g_e, sh, sl, M, K, N, N // bs, g_q.stride(0), g_q.stride(1), hi.stride(0), hi.stride(1),
        lo.stride(0), lo.stride(1), dx.stride(0), dx.stride(1), g_e.stride(0), g_e.stride(1), sh.stride(0),
        sh.stride(1), BLOCK_M=BMd, BLOCK_K=bs, GROUP_M=8, num_sms_launch=1 << 30)
    out[f"{name}/dx"] = dx.numpy().copy()
    print(name, "done", flush=True)

np.savez_compressed(HERE / "block_path.npz", **out)
print("wrote", HERE / "block_path.npz", sum(v.nbytes for v in out.values()) // 1024, "KiB raw")
