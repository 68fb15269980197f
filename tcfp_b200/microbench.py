"""Kernel micro-benchmarks (CUDA events, inputs larger than L2 at the default
sizes).  Used to time single kernels and as the target of ncu captures:

    python -m tcfp_b200.microbench gemm   [N]   # per-tensor dual / single GEMM, N^3
    python -m tcfp_b200.microbench block  [N]   # block-scaled dual GEMM fwd + dX, N^3, block 32/64/128
    python -m tcfp_b200.microbench quant  [N]   # block and per-tensor quantizers on N x N
    python -m tcfp_b200.microbench lib    [N]   # library comparators: torch._scaled_mm, bf16 matmul
    python -m tcfp_b200.microbench qvar   [N]   # the ALU-heavy quantizer variants only (no error buffer, stochastic
                                                # residual, per-tensor stochastic), few launches: the ncu target
    python -m tcfp_b200.microbench dx     [N]   # block dX: re-targeting pass + FP8 GEMM, and the exact bf16 route
    python -m tcfp_b200.microbench actq   [M]   # narrow layers (N = 128..512, K = 4096): prologue-fused activation
                                                # quantize vs block quantizer + GEMM
"""
from __future__ import annotations

import sys

import torch

DEV = "cuda"


def timeit(fn, iters=20, warmup=3) -> float:
    for _ in range(warmup):
        fn()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _fp8(n, m, dtype=torch.float8_e4m3fn):
    return torch.randn(n, m, device=DEV).to(dtype)


def gemm(n: int) -> None:
    from .kernels import fp8_weight_grad, fused_dual_gemm_backward_dx, fused_dual_gemm_forward

    a, hi, lo = _fp8(n, n), _fp8(n, n), _fp8(n, n)
    g = _fp8(n, n, torch.float8_e5m2)
    s = torch.ones(1, device=DEV)
    ms = timeit(lambda: fused_dual_gemm_forward(a, hi, lo, s, s, s))
    print(f"dual GEMM fwd  {n}^3: {ms:.3f} ms  {4 * n**3 / ms / 1e9:.0f} TFLOP/s (both products)")
    ms = timeit(lambda: fused_dual_gemm_backward_dx(g, hi, lo, s, s, s))
    print(f"dual GEMM dX   {n}^3: {ms:.3f} ms  {4 * n**3 / ms / 1e9:.0f} TFLOP/s (both products)")
    ms = timeit(lambda: fused_dual_gemm_forward(a, hi, None, s, s, None))
    print(f"single GEMM    {n}^3: {ms:.3f} ms  {2 * n**3 / ms / 1e9:.0f} TFLOP/s")
    ms = timeit(lambda: fp8_weight_grad(g, a, s, s))
    print(f"dW GEMM (g^T x) {n}^3: {ms:.3f} ms  {2 * n**3 / ms / 1e9:.0f} TFLOP/s")


def block(n: int) -> None:
    from .kernels import (block_quantize_fp8, fused_block_scaled_backward_dx, fused_block_scaled_dual_gemm_forward,
                          fused_dual_quantize_fp8)

    x = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, n, device=DEV) * 0.02
    gy = torch.randn(n, n, device=DEV)
    for bs in (32, 64, 128):
        hi, lo, sh, sl = fused_dual_quantize_fp8(w, bs)
        a, sa = block_quantize_fp8(x, bs)
        ms = timeit(lambda: fused_block_scaled_dual_gemm_forward(a, hi, lo, sa, sh, sl, bs))
        print(f"block-{bs} dual GEMM fwd {n}^3: {ms:.3f} ms  {4 * n**3 / ms / 1e9:.0f} TFLOP/s (both products)")
        gq, sg = block_quantize_fp8(gy, bs, torch.float8_e5m2)
        ms = timeit(lambda: fused_block_scaled_backward_dx(gq, hi, lo, sg, sh, sl, bs))
        print(f"block-{bs} dX (FP8, weight re-targeted once) {n}^3: {ms:.3f} ms  {4 * n**3 / ms / 1e9:.0f} TFLOP/s (both products)")


def quant(n: int) -> None:
    from .core import dual_quantize_per_tensor, to_fp8_e4m3, to_fp8_e5m2
    from .kernels import block_quantize_fp8, fused_dual_quantize_fp8

    w = torch.randn(n, n, device=DEV) * 0.02
    err = torch.zeros(n, n, device=DEV)
    x = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
    gy = torch.randn(n, n, device=DEV)
    e = n * n

    def report(name, ms, bytes_per_elem):
        print(f"{name:<46s} {ms * 1e3:8.1f} us  {bytes_per_elem * e / ms / 1e6:7.0f} GB/s ({bytes_per_elem} B/elem algorithmic)")

    for bs in (32, 64, 128):
        report(f"dual_quantize block-{bs} EF", timeit(lambda: fused_dual_quantize_fp8(w, bs, err)), 14)
    report("dual_quantize block-64 no EF", timeit(lambda: fused_dual_quantize_fp8(w, 64, None)), 6)
    report("dual_quantize block-64 SRR", timeit(lambda: fused_dual_quantize_fp8(w, 64, None, True, seed=1)), 6)
    report("block_quantize bf16 -> E4M3 block-64", timeit(lambda: block_quantize_fp8(x, 64)), 3)
    report("block_quantize f32 -> E5M2 (+bf16 copy) block-64",
           timeit(lambda: block_quantize_fp8(gy, 64, torch.float8_e5m2, want_bf16=True)), 7)
    report("dual_quantize per-tensor EF (3 passes)", timeit(lambda: dual_quantize_per_tensor(w, err)), 14)
    a_hi = torch.tensor(0.1, device=DEV)
    a_lo = torch.tensor(0.0125, device=DEV)
    report("dual_quantize per-tensor EF, amax given (1 pass)",
           timeit(lambda: dual_quantize_per_tensor(w, err, amax_hi=a_hi, amax_lo=a_lo)), 14)
    report("dual_quantize per-tensor SRR", timeit(lambda: dual_quantize_per_tensor(w, None, srr=True)), 6)
    report("to_fp8_e4m3 bf16 (2 passes)", timeit(lambda: to_fp8_e4m3(x)), 3)
    report("to_fp8_e5m2 f32 (2 passes)", timeit(lambda: to_fp8_e5m2(gy)), 5)


def qvar(n: int) -> None:
    from .core import dual_quantize_per_tensor
    from .kernels import fused_dual_quantize_fp8

    w = torch.randn(n, n, device=DEV) * 0.02
    e = n * n
    for name, fn in (("dual_quantize block-64 no EF", lambda: fused_dual_quantize_fp8(w, 64, None)),
                     ("dual_quantize block-64 SRR", lambda: fused_dual_quantize_fp8(w, 64, None, True, seed=1)),
                     ("dual_quantize per-tensor SRR", lambda: dual_quantize_per_tensor(w, None, srr=True, seed=1))):
        ms = timeit(fn, iters=5, warmup=2)
        print(f"{name:<34s} {ms * 1e3:8.1f} us  {6 * e / ms / 1e6:7.0f} GB/s (6 B/elem algorithmic)")


def ptq(n: int) -> None:
    """Per-tensor dual quantizer with fresh scales (three dependent passes) on an
    n x n/2 weight with its error buffer: the case to capture under ncu for the
    DRAM bytes each pass really moves."""
    from .core import dual_quantize_per_tensor

    w = torch.randn(n, n // 2, device=DEV) * 0.02
    err = torch.zeros_like(w)
    e = w.numel()
    ms = timeit(lambda: dual_quantize_per_tensor(w, err), iters=5, warmup=2)
    print(f"dual_quantize per-tensor EF fresh scales {n}x{n // 2}: {ms * 1e3:.1f} us  {14 * e / ms / 1e6:.0f} GB/s "
          f"(14 B/elem algorithmic; W + e = {8 * e / 1e6:.0f} MB)")


def aux(n: int) -> None:
    """The small HBM-bound kernels around the block-path backward at n x n:
    FP32 -> bf16 head + tail, saved FP8 activation -> bf16, weight re-targeting."""
    from .kernels import block_dequantize_bf16, block_quantize_fp8, block_retarget, fused_dual_quantize_fp8, split_bf16

    e = n * n
    g = torch.randn(n, n, device=DEV)
    x = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
    a, sa = block_quantize_fp8(x, 64)
    hi, lo, sh, sl = fused_dual_quantize_fp8(torch.randn(n, n, device=DEV) * 0.02, 64)
    for name, fn, bpe in (("split_bf16 (f32 -> bf16 head + tail)", lambda: split_bf16(g), 8),
                          ("block_dequantize_bf16 (E4M3 block-64 -> bf16)", lambda: block_dequantize_bf16(a, sa, 64), 3),
                          ("block_retarget block-64 (both planes)", lambda: block_retarget(hi, lo, sh, sl, 64), 4)):
        ms = timeit(fn, iters=10, warmup=3)
        print(f"{name:<48s} {ms * 1e3:7.1f} us  {bpe * e / ms / 1e6:6.0f} GB/s ({bpe} B/elem algorithmic)")


def dx(n: int) -> None:
    from .kernels import block_quantize_fp8, block_retarget, fused_block_scaled_backward_dx, fused_dual_quantize_fp8

    w = torch.randn(n, n, device=DEV) * 0.02
    gy = torch.randn(n, n, device=DEV)
    for bs in (32, 64, 128):
        hi, lo, sh, sl = fused_dual_quantize_fp8(w, bs)
        gq, sg = block_quantize_fp8(gy, bs, torch.float8_e5m2)
        ms_r = timeit(lambda: block_retarget(hi, lo, sh, sl, bs), iters=10)
        fused_block_scaled_backward_dx(gq, hi, lo, sg, sh, sl, bs)
        ms_g = timeit(lambda: fused_block_scaled_backward_dx(gq, hi, lo, sg, sh, sl, bs), iters=10)
        ms_b = timeit(lambda: fused_block_scaled_backward_dx(gq, hi, lo, sg, sh, sl, bs, exact_bf16=True), iters=10)
        print(f"block-{bs} dX {n}^3: retarget {ms_r * 1e3:.1f} us ({4 * n * n / ms_r / 1e6:.0f} GB/s) + FP8 GEMM {ms_g:.3f} ms "
              f"({4 * n**3 / ms_g / 1e9:.0f} TFLOP/s); exact bf16 route {ms_b:.3f} ms")


def actq(m: int) -> None:
    from .kernels import fused_act_quant_dual_gemm_forward, fused_dual_quantize_fp8

    k = 4096
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    for bs in (32, 64, 128):
        for n in (128, 256, 384, 512):
            w = torch.randn(n, k, device=DEV) * 0.02
            hi, lo, sh, sl = fused_dual_quantize_fp8(w, bs)
            fused = timeit(lambda: fused_act_quant_dual_gemm_forward(x, hi, lo, sh, sl, bs, fuse=True), iters=10)
            split = timeit(lambda: fused_act_quant_dual_gemm_forward(x, hi, lo, sh, sl, bs, fuse=False), iters=10)
            print(f"block-{bs} M={m} N={n} K={k}: fused prologue {fused * 1e3:7.1f} us   quantize + GEMM {split * 1e3:7.1f} us")


def dw(tokens: int) -> None:
    """Weight gradient of a bf16 output gradient (one bf16 product, both operands
    read in their forward layouts) at the decoder layer's four shapes."""
    from .kernels import bf16_weight_grad

    for d_out, d_in in ((12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008), (8192, 8192)):
        g = torch.randn(tokens, d_out, device=DEV, dtype=torch.bfloat16)
        x = torch.randn(tokens, d_in, device=DEV, dtype=torch.bfloat16)
        ms = timeit(lambda: bf16_weight_grad(g, x), iters=10)
        ms_lib = timeit(lambda: g.t() @ x, iters=10)
        fl = 2.0 * tokens * d_out * d_in
        print(f"dW bf16 tokens={tokens} {d_out}x{d_in}: {ms:.3f} ms {fl / ms / 1e9:.0f} TFLOP/s   "
              f"(torch bf16 matmul, bf16 output: {ms_lib:.3f} ms {fl / ms_lib / 1e9:.0f} TFLOP/s)")


def lib(n: int) -> None:
    a, hi, lo = _fp8(n, n), _fp8(n, n), _fp8(n, n)
    s = torch.ones(1, device=DEV)
    mm = lambda w, dt: torch._scaled_mm(a, w.t(), scale_a=s, scale_b=s, out_dtype=dt)  # noqa: E731
    ms = timeit(lambda: mm(hi, torch.float32))
    print(f"torch._scaled_mm fp8->f32  {n}^3: {ms:.3f} ms  {2 * n**3 / ms / 1e9:.0f} TFLOP/s")
    ms = timeit(lambda: mm(hi, torch.bfloat16))
    print(f"torch._scaled_mm fp8->bf16 {n}^3: {ms:.3f} ms  {2 * n**3 / ms / 1e9:.0f} TFLOP/s")
    ms = timeit(lambda: mm(hi, torch.float32) + mm(lo, torch.float32))
    print(f"2 x _scaled_mm + add (the reference's fallback, tcfp/nn/__init__.py:405-421) {n}^3: {ms:.3f} ms  "
          f"{4 * n**3 / ms / 1e9:.0f} TFLOP/s (both products)")
    x = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
    y = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
    ms = timeit(lambda: x @ y)
    print(f"bf16 matmul {n}^3: {ms:.3f} ms  {2 * n**3 / ms / 1e9:.0f} TFLOP/s")


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    size = int(sys.argv[2]) if len(sys.argv) > 2 else 8192
    {"gemm": gemm, "block": block, "quant": quant, "lib": lib, "qvar": qvar, "dx": dx, "actq": actq, "dw": dw, "ptq": ptq, "aux": aux}[what](size)
