"""Launch wrappers with the names and return conventions of the reference's
``tcfp/kernels.py`` (:1537-2469), backed by ``libtcfp_b200.so``.

Every wrapper allocates its outputs with torch (as the reference's do,
tcfp/kernels.py:1572, 1699-1700, 1806-1813), hands raw pointers and the current
stream to the C ABI, and raises on failure -- there is no Triton and no CPU
path behind these names.

Additions the reference does not have, all keyword-only and optional:
``seed`` / ``offset`` for the stochastic residual (the reference draws a fresh
seed per launch, tcfp/kernels.py:1828-1831), ``update_error`` (read the error
buffer without writing it, replacing the clone at tcfp/nn/__init__.py:607-608)
and ``out_dtype``.
"""
from __future__ import annotations

import torch

from . import _C

_FP8_E4M3_MAX = 448.0
_FP8_E5M2_MAX = 57344.0
_FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)


def is_triton_available() -> bool:
    """Capability probe kept under its reference name (tcfp/kernels.py:1537):
    True when the fused kernels can run, i.e. the library loads on sm_100."""
    return _C.is_available()


def _fmt(t: torch.Tensor) -> int:
    if t.dtype == torch.float8_e4m3fn:
        return _C.E4M3
    if t.dtype == torch.float8_e5m2:
        return _C.E5M2
    raise TypeError(f"expected an FP8 tensor, got {t.dtype}")


def _out_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _C.F32
    if dtype == torch.bfloat16:
        return _C.BF16
    raise TypeError(f"out_dtype must be float32 or bfloat16, got {dtype}")


def _scalar(t: torch.Tensor) -> torch.Tensor:
    assert t.numel() == 1 and t.dtype == torch.float32, "scales must be 1-element float32 tensors"
    return t


# ---------------------------------------------------------------------------
# packed scale factors ride along with the reference-layout exponent planes
# ---------------------------------------------------------------------------

def _alloc_sf(rows: int, K: int, bs: int, device) -> torch.Tensor:
    n = _C.load().tcfp_sf_packed_bytes(rows, K, bs)
    return torch.empty(n, dtype=torch.uint8, device=device)


def packed_scale_rows(sf: torch.Tensor, r0: int, r1: int, K: int, block_size: int) -> torch.Tensor:
    """The part of a packed scale-factor array that covers rows ``[r0, r1)``
    of its operand (``r0`` a multiple of 128: chunks hold 128 rows each)."""
    assert r0 % 128 == 0, "row slices of packed scale factors start on multiples of 128"
    per_row_block = ((K // block_size + 3) // 4) * 512
    return sf[(r0 // 128) * per_row_block:((r1 + 127) // 128) * per_row_block]


def _attach_sf(exps: torch.Tensor, sf: torch.Tensor, block_size: int) -> None:
    # the packed copy is only valid for the bytes it was packed from: remember the plane's
    # version counter and address so that an in-place edit or a re-bound storage repacks
    exps._tcfp_sf = (sf, exps._version, exps.data_ptr(), block_size)


def pack_block_scales(exps: torch.Tensor, block_size: int) -> torch.Tensor:
    """int8 exponent plane ``(K // bs, rows)`` -> packed E8M0 chunk array.
    A quantizer of this module attaches the packed copy it wrote in the same
    pass; it is reused only while the plane is unmodified."""
    cached = getattr(exps, "_tcfp_sf", None)
    if cached is not None:
        sf, version, addr, bs = cached
        if version == exps._version and addr == exps.data_ptr() and bs == block_size:
            return sf
    assert exps.dtype == torch.int8 and exps.ndim == 2 and exps.is_contiguous()
    num_kb, rows = exps.shape
    K = num_kb * block_size
    sf = _alloc_sf(rows, K, block_size, exps.device)
    _C.check(_C.load().tcfp_pack_scales(_C.ptr(exps), _C.ptr(sf), rows, K, block_size, _C.stream()))
    return sf


# ---------------------------------------------------------------------------
# per-tensor dual GEMM (tcfp/kernels.py:1545-1666)
# ---------------------------------------------------------------------------

def fused_dual_gemm_forward(act_fp8, w_hi_fp8, w_lo_fp8, act_inv, w_hi_inv, w_lo_inv, *,
                            bias=None, out_dtype=torch.float32, out=None):
    """``(act @ W_hi.T) * s + (act @ W_lo.T) * s`` -> ``(M, N)``
    (tcfp/kernels.py:1545-1601).  ``w_lo_fp8`` / ``w_lo_inv`` may be ``None``."""
    M, K = act_fp8.shape
    N, K2 = w_hi_fp8.shape
    assert K == K2 and (w_lo_fp8 is None or w_lo_fp8.shape == (N, K)), (
        f"Shape mismatch: act({M},{K}), w_hi({N},{K2}), w_lo{None if w_lo_fp8 is None else tuple(w_lo_fp8.shape)}"
    )
    assert act_fp8.is_contiguous() and w_hi_fp8.is_contiguous(), "operands must be contiguous"
    if out is None:
        out = torch.empty((M, N), device=act_fp8.device, dtype=out_dtype)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.is_contiguous(), "bad out buffer"
    _C.check(_C.load().tcfp_dual_gemm(
        _C.ptr(act_fp8), _fmt(act_fp8), _C.ptr(w_hi_fp8), _C.ptr(w_lo_fp8),
        _C.ptr(_scalar(act_inv)), _C.ptr(_scalar(w_hi_inv)), _C.ptr(None if w_lo_inv is None else _scalar(w_lo_inv)),
        _C.ptr(bias), _C.ptr(out), _out_code(out_dtype), M, N, K, 0, _C.stream()))
    return out


def fused_dual_gemm_backward_dx(grad_fp8, w_hi_fp8, w_lo_fp8, grad_inv, w_hi_inv, w_lo_inv, *,
                                out_dtype=torch.float32):
    """``(grad @ W_hi) * s + (grad @ W_lo) * s`` -> ``(M, D_in)``
    (tcfp/kernels.py:1604-1666); the weights stay in their ``(D_out, D_in)``
    layout."""
    M, D_out = grad_fp8.shape
    D_out2, D_in = w_hi_fp8.shape
    assert D_out == D_out2 and (w_lo_fp8 is None or w_lo_fp8.shape == (D_out, D_in)), (
        f"Shape mismatch: grad({M},{D_out}), w_hi({D_out2},{D_in})"
    )
    assert grad_fp8.is_contiguous() and w_hi_fp8.is_contiguous(), "operands must be contiguous"
    out = torch.empty((M, D_in), device=grad_fp8.device, dtype=out_dtype)
    _C.check(_C.load().tcfp_dual_gemm(
        _C.ptr(grad_fp8), _fmt(grad_fp8), _C.ptr(w_hi_fp8), _C.ptr(w_lo_fp8),
        _C.ptr(_scalar(grad_inv)), _C.ptr(_scalar(w_hi_inv)), _C.ptr(None if w_lo_inv is None else _scalar(w_lo_inv)),
        None, _C.ptr(out), _out_code(out_dtype), M, D_in, D_out, 1, _C.stream()))
    return out


def fp8_weight_grad(grad_fp8, act_fp8, grad_inv, act_inv, *, out_dtype=torch.float32):
    """``dW = (grad^T @ act) * (s_g * s_a)`` -> ``(D_out, D_in)`` from the
    gradient ``(M, D_out)`` and the saved activation codes ``(M, D_in)`` as
    they are (tcfp/nn/__init__.py:546-555 without the transposed copies)."""
    M, D_out = grad_fp8.shape
    M2, D_in = act_fp8.shape
    assert M == M2, f"Shape mismatch: grad({M},{D_out}), act({M2},{D_in})"
    assert grad_fp8.is_contiguous() and act_fp8.is_contiguous(), "operands must be contiguous"
    out = torch.empty((D_out, D_in), device=grad_fp8.device, dtype=out_dtype)
    _C.check(_C.load().tcfp_dw_gemm(
        _C.ptr(grad_fp8), _fmt(grad_fp8), _C.ptr(act_fp8), _C.ptr(_scalar(grad_inv)), _C.ptr(_scalar(act_inv)),
        _C.ptr(out), _out_code(out_dtype), M, D_out, D_in, _C.stream()))
    return out


def split_bf16(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """FP32 tensor -> ``(head, tail)`` bf16 with ``head = bf16(x)`` and
    ``tail = bf16(x - head)``: ``head + tail`` carries 16 significant bits of
    ``x``.  One pass (the three torch operations it replaces move 22 B/elem)."""
    assert x.dtype == torch.float32 and x.is_cuda
    x = x.contiguous()
    if x.numel() % 4 != 0:
        head = x.to(torch.bfloat16)
        return head, (x - head.float()).to(torch.bfloat16)
    head = torch.empty_like(x, dtype=torch.bfloat16)
    tail = torch.empty_like(head)
    _C.check(_C.load().tcfp_split_bf16(_C.ptr(x), _C.ptr(head), _C.ptr(tail), x.numel(), _C.stream()))
    return head, tail


def bf16_weight_grad(grad: torch.Tensor, act_bf16: torch.Tensor) -> torch.Tensor:
    """``dW = grad^T @ act`` -> ``(D_out, D_in)`` FP32 for an FP32 (or bf16)
    gradient ``(M, D_out)`` and a bf16 activation ``(M, D_in)``: the gradient
    is split into a bf16 head and tail (16 significant bits) and both ride one
    bf16 tensor-core GEMM -- the FP32 matmul of tcfp/nn/__init__.py:744-750 at
    about a tenth of its time.  Returns a transposed view (the kernel produces
    dW^T)."""
    M, D_out = grad.shape
    M2, D_in = act_bf16.shape
    assert M == M2 and act_bf16.dtype == torch.bfloat16
    if grad.dtype == torch.bfloat16:
        # nothing to split: compute dW = grad^T @ act directly (grad is the transposed operand)
        out = torch.empty((D_out, D_in), device=grad.device, dtype=torch.float32)
        _C.check(_C.load().tcfp_bf16_dw_gemm(_C.ptr(grad.contiguous()), _C.ptr(act_bf16.contiguous()), None, _C.ptr(out),
                                             _C.F32, M, D_out, D_in, _C.stream()))
        return out
    g_lo = None
    if grad.dtype == torch.float32:
        g_hi, g_lo = split_bf16(grad)
    else:
        g_hi = grad.to(torch.bfloat16)
    out = torch.empty((D_in, D_out), device=grad.device, dtype=torch.float32)
    _C.check(_C.load().tcfp_bf16_dw_gemm(_C.ptr(act_bf16.contiguous()), _C.ptr(g_hi), _C.ptr(g_lo), _C.ptr(out),
                                         _C.F32, M, D_in, D_out, _C.stream()))
    return out.t()


# ---------------------------------------------------------------------------
# block quantizers (tcfp/kernels.py:1675-1875)
# ---------------------------------------------------------------------------

def _colsum_workspace(R: int, C: int, device) -> torch.Tensor:
    return torch.empty(_C.load().tcfp_colsum_workspace_bytes(R, C), dtype=torch.uint8, device=device)


def block_quantize_fp8(tensor, block_size=128, fp8_dtype=torch.float8_e4m3fn, *, want_bf16=False, want_colsum=False):
    """Per-block FP8 quantization (tcfp/kernels.py:1675-1722).  Returns
    ``(fp8 (M,K), int8 exponents (K // bs, M))``; with ``want_bf16`` a third
    tensor holds the dequantized values as bf16; with ``want_colsum`` a third
    tensor holds the FP32 column sums of the input (the bias gradient when the
    input is an output gradient), accumulated in the same pass."""
    M, K = tensor.shape
    assert K % block_size == 0, f"K ({K}) must be divisible by block_size ({block_size})"
    assert tensor.is_contiguous(), "input must be contiguous"
    num_kb = K // block_size
    out = torch.empty((M, K), device=tensor.device, dtype=fp8_dtype)
    scales = torch.empty((num_kb, M), device=tensor.device, dtype=torch.int8)
    sf = _alloc_sf(M, K, block_size, tensor.device)
    if want_colsum:
        assert not want_bf16, "want_colsum and want_bf16 are separate variants"
        colsum = torch.empty(K, device=tensor.device, dtype=torch.float32)
        _C.check(_C.load().tcfp_quantize_colsum(
            _C.ptr(tensor), _C.dtype_code(tensor), _C.ptr(out), _C.ptr(scales), _C.ptr(sf), M, K, block_size, _fmt(out),
            _C.ptr(colsum), _C.ptr(_colsum_workspace(M, K, tensor.device)), _C.stream()))
        _attach_sf(scales, sf, block_size)
        return out, scales, colsum
    deq = torch.empty((M, K), device=tensor.device, dtype=torch.bfloat16) if want_bf16 else None
    _C.check(_C.load().tcfp_quantize(
        _C.ptr(tensor), _C.dtype_code(tensor), _C.ptr(out), _C.ptr(scales), _C.ptr(sf), _C.ptr(deq),
        M, K, block_size, _fmt(out), None, None, 0, 0, 0, None, _C.stream()))
    _attach_sf(scales, sf, block_size)
    if want_bf16:
        return out, scales, deq
    return out, scales


def block_dequantize_fp8(fp8_tensor, block_scales, block_size):
    """``(M, K)`` FP32 from codes and int8 exponents (tcfp/kernels.py:1725-1746);
    torch ops, exactly as in the reference."""
    M, K = fp8_tensor.shape
    blocked = fp8_tensor.float().reshape(M, K // block_size, block_size)
    float_scales = torch.exp2(block_scales.float())
    return (blocked * float_scales.t().unsqueeze(-1)).reshape(M, K)


def block_dequantize_bf16(fp8_tensor, block_scales, block_size, *, sentinel_zero=False):
    """Codes + exponents -> bf16 values (exact: at most 4 significant bits)."""
    M, K = fp8_tensor.shape
    out = torch.empty((M, K), device=fp8_tensor.device, dtype=torch.bfloat16)
    _C.check(_C.load().tcfp_block_dequantize_bf16(
        _C.ptr(fp8_tensor), _C.ptr(block_scales), _C.ptr(out), M, K, block_size, _fmt(fp8_tensor),
        1 if sentinel_zero else 0, _C.stream()))
    return out


_srr_seed_gen: torch.Generator | None = None


def _fresh_seed() -> int:
    # one 31-bit seed per launch, drawn on the host (the reference draws it on
    # the device and synchronises to fetch it, tcfp/kernels.py:1828-1831)
    global _srr_seed_gen
    if _srr_seed_gen is None:
        _srr_seed_gen = torch.Generator(device="cpu")
        _srr_seed_gen.manual_seed(torch.initial_seed() & 0x7FFFFFFF)
    return int(torch.randint(0, 2**31, (1,), generator=_srr_seed_gen).item())


def fused_dual_quantize_fp8(weight, block_size=128, error_buf=None, stochastic_lo=False, *,
                            seed=None, offset=0, update_error=True):
    """W -> ``(w_hi, w_lo, scales_hi, scales_lo)`` in one kernel
    (tcfp/kernels.py:1749-1875).  ``error_buf`` is read and, unless
    ``update_error=False``, overwritten in place with
    ``W - deq(W_hi) - deq(W_lo)``."""
    assert weight.is_contiguous(), "Weight must be contiguous (N, K) row-major"
    N, K = weight.shape
    assert K % block_size == 0, f"K ({K}) must be divisible by block_size ({block_size})"
    if stochastic_lo and error_buf is not None:
        raise ValueError(
            "stochastic_lo and error_buf are mutually exclusive: "
            "SRR eliminates the need for error feedback buffers."
        )
    if error_buf is not None:
        assert error_buf.dtype == torch.float32, "error_buf must be float32"
        assert error_buf.shape == (N, K), f"error_buf shape {tuple(error_buf.shape)} != weight shape {(N, K)}"
        assert error_buf.is_contiguous(), "error_buf must be contiguous"
    num_kb = K // block_size
    dev = weight.device
    w_hi = torch.empty((N, K), device=dev, dtype=torch.float8_e4m3fn)
    w_lo = torch.empty((N, K), device=dev, dtype=torch.float8_e4m3fn)
    scales_hi = torch.empty((num_kb, N), device=dev, dtype=torch.int8)
    scales_lo = torch.empty((num_kb, N), device=dev, dtype=torch.int8)
    sf_hi = _alloc_sf(N, K, block_size, dev)
    sf_lo = _alloc_sf(N, K, block_size, dev)
    if stochastic_lo:
        mode = _C.Q_SRR
        if seed is None:
            seed = _fresh_seed()
    elif error_buf is not None:
        mode = _C.Q_EF if update_error else _C.Q_EF_READONLY
    else:
        mode = _C.Q_NONE
    _C.check(_C.load().tcfp_dual_quantize(
        _C.ptr(weight), _C.dtype_code(weight), _C.ptr(error_buf), _C.ptr(w_hi), _C.ptr(w_lo),
        _C.ptr(scales_hi), _C.ptr(scales_lo), _C.ptr(sf_hi), _C.ptr(sf_lo), N, K, block_size, mode,
        int(seed or 0), int(offset), None, None, None, None, _C.stream()))
    _attach_sf(scales_hi, sf_hi, block_size)
    _attach_sf(scales_lo, sf_lo, block_size)
    return w_hi, w_lo, scales_hi, scales_lo


# ---------------------------------------------------------------------------
# block-scaled GEMMs (tcfp/kernels.py:1878-2149, 2326-2469)
# ---------------------------------------------------------------------------

def fused_block_scaled_dual_gemm_forward(act_fp8, w_hi_fp8, w_lo_fp8, act_scales, w_hi_scales, w_lo_scales,
                                         block_size, sparse_threshold=0.0, persistent=True, launch_mult=1, *,
                                         bias=None, out_dtype=torch.float32, out=None, act_sf=None):
    """Block-scaled 2-GEMM forward (tcfp/kernels.py:1939-2028).  The tuning
    arguments of the reference are accepted and ignored: the kernel is always
    persistent with one CTA per SM.  ``act_sf`` passes the packed activation
    scale factors explicitly (a row slice of a larger operand's array);
    ``act_scales`` is then not consulted."""
    M, K = act_fp8.shape
    N, K2 = w_hi_fp8.shape
    assert K == K2 and (w_lo_fp8 is None or w_lo_fp8.shape == (N, K)), (
        f"Shape mismatch: act({M},{K}), w_hi({N},{K2})"
    )
    assert K % block_size == 0, f"K ({K}) must be divisible by block_size ({block_size})"
    sf_a = act_sf if act_sf is not None else pack_block_scales(act_scales, block_size)
    sf_hi = pack_block_scales(w_hi_scales, block_size)
    sf_lo = pack_block_scales(w_lo_scales, block_size) if w_lo_fp8 is not None else None
    if out is None:
        out = torch.empty((M, N), device=act_fp8.device, dtype=out_dtype)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.is_contiguous(), "bad out buffer"
    _C.check(_C.load().tcfp_block_dual_gemm(
        _C.ptr(act_fp8), _C.ptr(sf_a), _C.ptr(w_hi_fp8), _C.ptr(sf_hi), _C.ptr(w_lo_fp8), _C.ptr(sf_lo),
        _C.ptr(bias), _C.ptr(out), _out_code(out_dtype), M, N, K, block_size, _C.stream()))
    return out


def block_scaled_gemm(a_fp8, b_fp8, scales_a, scales_b, block_size=128):
    """Single block-scaled GEMM (tcfp/kernels.py:1878-1936): the dual kernel
    with the residual operand left out."""
    M, K = a_fp8.shape
    N, K2 = b_fp8.shape
    assert K == K2, f"K mismatch: A ({K}) vs B ({K2})"
    assert K % block_size == 0, f"K ({K}) not divisible by block_size ({block_size})"
    return fused_block_scaled_dual_gemm_forward(a_fp8, b_fp8, None, scales_a, scales_b, None, block_size)


# Widest layer (output features) for which the prologue-fused kernel is dispatched by default.  Measured on a
# B200 at M = 32768, K = 4096, block 64: fused 166 / 270 / 392 / 402 us against 105 / 124 / 146 / 164 us for the
# block quantizer followed by the GEMM at N = 128 / 256 / 384 / 512 -- the converters re-quantize the activation
# tile for every 128-column tile and set the pace of the K loop -- so the separate route wins at every width and
# the default never fuses; ``fuse=True`` selects the fused kernel explicitly.
FUSED_ACT_MAX_N = 0


def fused_act_quant_dual_gemm_forward(act, w_hi_fp8, w_lo_fp8, w_hi_scales, w_lo_scales, block_size,
                                      sparse_threshold=0.0, persistent=True, launch_mult=1,
                                      save_side_outputs=True, *, bias=None, out_dtype=torch.float32, fuse=None):
    """Activation quantize + block-scaled 2-GEMM (tcfp/kernels.py:2031-2149).
    Returns ``(output, act_fp8, act_scales)``; the side outputs are ``None``
    when ``save_side_outputs`` is False.

    ``fuse=True`` runs ONE kernel that quantizes the bf16 activation tiles in
    the GEMM prologue (``tcfp_block_dual_gemm_fused_act``); ``fuse=False``
    runs the block quantizer and then the GEMM.  The default picks the fused
    kernel for bf16 activations and ``N <= FUSED_ACT_MAX_N`` (0: the two-kernel
    route measured faster at every width).  Both produce the same side-output
    bytes."""
    M, K = act.shape
    N, K2 = w_hi_fp8.shape
    assert K == K2 and w_lo_fp8.shape == (N, K), f"Shape mismatch: act({M},{K}), w_hi({N},{K2})"
    assert K % block_size == 0, f"K ({K}) must be divisible by block_size ({block_size})"
    fusable = act.dtype == torch.bfloat16 and act.is_contiguous()
    if fuse is None:
        fuse = fusable and N <= FUSED_ACT_MAX_N
    if fuse:
        assert fusable, "the fused kernel takes a contiguous bfloat16 activation"
        out = torch.empty((M, N), device=act.device, dtype=out_dtype)
        act_fp8 = act_scales = None
        if save_side_outputs:
            act_fp8 = torch.empty((M, K), device=act.device, dtype=torch.float8_e4m3fn)
            act_scales = torch.empty((K // block_size, M), device=act.device, dtype=torch.int8)
        # keep the packed scale arrays alive in locals until the launch is queued: a temporary freed between the
        # two pack launches would hand its block to the second one
        sf_hi = pack_block_scales(w_hi_scales, block_size)
        sf_lo = pack_block_scales(w_lo_scales, block_size)
        _C.check(_C.load().tcfp_block_dual_gemm_fused_act(
            _C.ptr(act), _C.ptr(w_hi_fp8), _C.ptr(sf_hi), _C.ptr(w_lo_fp8), _C.ptr(sf_lo), _C.ptr(bias), _C.ptr(out),
            _out_code(out_dtype), _C.ptr(act_fp8), _C.ptr(act_scales), M, N, K, block_size, _C.stream()))
        return out, act_fp8, act_scales
    act_fp8, act_scales = block_quantize_fp8(act, block_size, torch.float8_e4m3fn)
    out = fused_block_scaled_dual_gemm_forward(act_fp8, w_hi_fp8, w_lo_fp8, act_scales, w_hi_scales, w_lo_scales,
                                               block_size, bias=bias, out_dtype=out_dtype)
    if save_side_outputs:
        return out, act_fp8, act_scales
    return out, None, None


def block_retarget(w_hi_fp8, w_lo_fp8, w_hi_scales, w_lo_scales, block_size):
    """One launch of ``tcfp_block_retarget``: ``(hi_t, lo_t, t_hi, t_lo)`` with
    the codes transposed to ``(D_in, D_out)`` and int8 exponent planes
    ``(D_out // bs, D_in)``; ``lo`` entries ``None`` without ``w_lo_fp8``."""
    D_out, D_in = w_hi_fp8.shape
    assert w_hi_fp8.is_contiguous() and w_hi_scales.is_contiguous(), "operands must be contiguous"
    assert w_hi_scales.shape == (D_in // block_size, D_out), "scales must be (D_in // block_size, D_out)"
    dev = w_hi_fp8.device
    hi_t = torch.empty((D_in, D_out), device=dev, dtype=torch.float8_e4m3fn)
    t_hi = torch.empty((D_out // block_size, D_in), device=dev, dtype=torch.int8)
    lo_t = t_lo = None
    if w_lo_fp8 is not None:
        assert w_lo_fp8.is_contiguous() and w_lo_scales.is_contiguous(), "operands must be contiguous"
        lo_t = torch.empty((D_in, D_out), device=dev, dtype=torch.float8_e4m3fn)
        t_lo = torch.empty((D_out // block_size, D_in), device=dev, dtype=torch.int8)
    _C.check(_C.load().tcfp_block_retarget(
        _C.ptr(w_hi_fp8), _C.ptr(w_lo_fp8), _C.ptr(w_hi_scales), _C.ptr(w_lo_scales), _C.ptr(hi_t), _C.ptr(lo_t),
        _C.ptr(t_hi), _C.ptr(t_lo), D_out, D_in, block_size, _C.stream()))
    return hi_t, lo_t, t_hi, t_lo


def retarget_block_weights(w_hi_fp8, w_lo_fp8, w_hi_scales, w_lo_scales, block_size):
    """Quantized weight ``(D_out, D_in)`` with scales along ``D_in`` -> the
    operands of the input-gradient GEMM: codes transposed to ``(D_in, D_out)``
    and scale factors along ``D_out`` (``tcfp_block_retarget``).  Returns
    ``(hi_t, lo_t, sf_hi_t, sf_lo_t)`` (``lo`` entries ``None`` without
    ``w_lo_fp8``).  The result depends only on the quantized weight; it is
    kept on ``w_hi_fp8`` and reused while none of the four inputs changes, so
    gradient-accumulation micro-batches pay for it once."""
    D_out, D_in = w_hi_fp8.shape
    key = (w_hi_fp8._version, w_hi_scales._version, w_hi_scales.data_ptr(), block_size,
           None if w_lo_fp8 is None else (w_lo_fp8.data_ptr(), w_lo_fp8._version, w_lo_scales._version))
    cached = getattr(w_hi_fp8, "_tcfp_dx", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    hi_t, lo_t, t_hi, t_lo = block_retarget(w_hi_fp8, w_lo_fp8, w_hi_scales, w_lo_scales, block_size)
    out = (hi_t, lo_t, pack_block_scales(t_hi, block_size), None if t_lo is None else pack_block_scales(t_lo, block_size))
    w_hi_fp8._tcfp_dx = (key, out)
    return out


def fused_block_scaled_backward_dx(grad_fp8, w_hi_fp8, w_lo_fp8, grad_scales, w_hi_scales, w_lo_scales, block_size,
                                   persistent=True, launch_mult=1, *, out_dtype=torch.float32, exact_bf16=False,
                                   grad_bf16=None):
    """Block-scaled dX ``(M, D_in)`` (tcfp/kernels.py:2326-2425).  The weight
    scales run along ``D_in`` but dX contracts over ``D_out``: the quantized
    weight is re-targeted once per weight version (:func:`retarget_block_weights`)
    and the product runs on the FP8 block-scaled tensor-core path, like the
    forward.  ``exact_bf16=True`` takes the other route: every operand is
    dequantized to bf16 (exact) and multiplied on the bf16 tensor-core path at
    half the rate."""
    M, D_out = grad_fp8.shape
    D_out2, D_in = w_hi_fp8.shape
    assert D_out == D_out2 and (w_lo_fp8 is None or w_lo_fp8.shape == (D_out, D_in)), (
        f"Shape mismatch: grad({M},{D_out}), w_hi({D_out2},{D_in})"
    )
    assert D_out % block_size == 0, f"D_out={D_out} must be divisible by block_size={block_size}"
    assert D_in % block_size == 0, f"D_in={D_in} must be divisible by block_size={block_size}"
    out = torch.empty((M, D_in), device=grad_fp8.device, dtype=out_dtype)
    if exact_bf16:
        if grad_bf16 is None:
            grad_bf16 = block_dequantize_bf16(grad_fp8, grad_scales, block_size)
        hi = block_dequantize_bf16(w_hi_fp8, w_hi_scales, block_size)
        lo = None
        if w_lo_fp8 is not None:
            lo = block_dequantize_bf16(w_lo_fp8, w_lo_scales, block_size, sentinel_zero=True)
        _C.check(_C.load().tcfp_bf16_dual_gemm(
            _C.ptr(grad_bf16), _C.ptr(hi), _C.ptr(lo), None, _C.ptr(out), _out_code(out_dtype),
            M, D_in, D_out, 1, _C.stream()))
        return out
    assert grad_fp8.dtype == torch.float8_e5m2 and grad_fp8.is_contiguous(), "gradient codes must be contiguous E5M2"
    hi_t, lo_t, sf_hi_t, sf_lo_t = retarget_block_weights(w_hi_fp8, w_lo_fp8, w_hi_scales, w_lo_scales, block_size)
    sf_g = pack_block_scales(grad_scales, block_size)
    _C.check(_C.load().tcfp_block_dx_gemm(
        _C.ptr(grad_fp8), _C.ptr(sf_g), _C.ptr(hi_t), _C.ptr(sf_hi_t), _C.ptr(lo_t), _C.ptr(sf_lo_t), _C.ptr(out),
        _out_code(out_dtype), M, D_in, D_out, block_size, _C.stream()))
    return out


def fused_block_scaled_dual_gemm_backward_dx(grad_fp8, w_hi_fp8, w_lo_fp8, grad_scales, w_hi_scales, w_lo_scales,
                                             block_size):
    """Reference name of the dX dispatch (tcfp/kernels.py:2428-2469)."""
    return fused_block_scaled_backward_dx(grad_fp8, w_hi_fp8, w_lo_fp8, grad_scales, w_hi_scales, w_lo_scales,
                                          block_size=block_size)
