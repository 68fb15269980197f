"""CPU restatement (torch CPU ops + numpy) of the reference TCFP-12 hot path.

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.

Every function cites the reference file:line it follows (paths are relative
to the reference project root).  The per-tensor functions are pinned
bit-for-bit against the reference itself, imported on CPU, by the golden
fixtures in ``tests/golden`` (generator: ``tests/golden/make_golden.py``).
The block-scaled functions restate Triton kernels; they are pinned against
the reference's own kernel bodies executed on CPU by the Triton interpreter
(``tests/golden/make_golden_block.py`` -> ``tests/golden/block_path.npz``):
exponent planes, the zero-residual sentinel, the stochastic-rounding stream
and the two GEMM formulas bit-for-bit / to 1e-5, FP8 codes everywhere except
on the elements the interpreter's (not the hardware's) FP8 cast gets wrong --
see ``tests/test_oracle_block_golden.py``.

Conventions: weights ``(N, K)`` row-major, activations ``(M, K)``, block
exponent planes ``(K // bs, rows)`` int8 with ``-128`` as the zero-residual
sentinel, per-tensor inverse scales of shape ``(1,)`` float32.
"""
from __future__ import annotations

import numpy as np
import torch

FP8_E4M3_MAX = 448.0          # tcfp/core.py:29
FP8_E5M2_MAX = 57344.0        # tcfp/core.py:35
E4M3 = torch.float8_e4m3fn
E5M2 = torch.float8_e5m2


# ---------------------------------------------------------------------------
# Philox4x32-10 uniforms: the seed/offset contract of the stochastic paths
# ---------------------------------------------------------------------------

_PHILOX_KEY_A = np.uint32(0x9E3779B9)
_PHILOX_KEY_B = np.uint32(0xBB67AE85)
_PHILOX_ROUND_A = np.uint64(0xD2511F53)
_PHILOX_ROUND_B = np.uint64(0xCD9E8D57)


def philox4x32_10(seed: int, counter: np.ndarray, all_words: bool = False) -> np.ndarray:
    """First 32-bit output word of Philox4x32-10 (all four, stacked on axis 0,
    with ``all_words``).

    key = (seed & 2^32-1, seed >> 32); counter words = (ctr & 2^32-1,
    ctr >> 32, 0, 0).  This is the published Philox algorithm (Salmon et al.,
    SC'11) with the word order used by ``tl.rand`` (the generator the
    reference's block kernel draws from, tcfp/kernels.py:415-417).
    """
    ctr = np.asarray(counter, dtype=np.uint64)
    c0 = (ctr & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    c1 = (ctr >> np.uint64(32)).astype(np.uint32)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0 = np.uint32(seed & 0xFFFFFFFF)
    k1 = np.uint32((seed >> 32) & 0xFFFFFFFF)
    with np.errstate(over="ignore"):
        for _ in range(10):
            pb = _PHILOX_ROUND_B * c2.astype(np.uint64)
            pa = _PHILOX_ROUND_A * c0.astype(np.uint64)
            n0 = (pb >> np.uint64(32)).astype(np.uint32) ^ c1 ^ k0
            n2 = (pa >> np.uint64(32)).astype(np.uint32) ^ c3 ^ k1
            n1 = (pb & np.uint64(0xFFFFFFFF)).astype(np.uint32)
            n3 = (pa & np.uint64(0xFFFFFFFF)).astype(np.uint32)
            c0, c1, c2, c3 = n0, n1, n2, n3
            k0 = np.uint32((int(k0) + int(_PHILOX_KEY_A)) & 0xFFFFFFFF)
            k1 = np.uint32((int(k1) + int(_PHILOX_KEY_B)) & 0xFFFFFFFF)
    if all_words:
        return np.stack([c0, c1, c2, c3])
    return c0


def _word_to_uniform(w: np.ndarray) -> np.ndarray:
    w = w.view(np.int32).astype(np.int64)
    w = np.where(w < 0, -w - 1, w)
    return w.astype(np.float32) * np.float32(4.6566127342e-10)


def philox_uniform(seed: int, offset: int, numel: int) -> torch.Tensor:
    """Uniforms ``u[i] in [0,1)`` for linear element index ``i``.

    ``u[i] = f(philox4x32_10(seed, offset + i))`` where ``f`` reinterprets the
    word as int32, maps negatives ``x -> -x-1`` and multiplies the
    int->float32 conversion by 4.6566127342e-10 (the ``tl.rand`` mapping).
    With ``offset = 0`` and a 31-bit seed these are the numbers the
    reference's ``_fused_dual_quantize_kernel`` draws for element
    ``n*K + k`` (tcfp/kernels.py:415-417).
    """
    idx = np.arange(numel, dtype=np.uint64) + np.uint64(offset)
    return torch.from_numpy(_word_to_uniform(philox4x32_10(seed, idx)))


def philox_uniform_packed(seed: int, offset: int, numel: int) -> torch.Tensor:
    """Uniforms of the PER-TENSOR stochastic paths, whose stream is this
    build's own definition (the reference draws ``torch.rand_like`` there,
    tcfp/core.py:462, which no other implementation can reproduce): element
    ``j = offset + i`` takes output word ``j & 3`` of
    ``philox4x32_10(seed, j >> 2)`` -- all four words of every generator call
    are used -- through the same word -> float mapping as above."""
    idx = np.arange(numel, dtype=np.uint64) + np.uint64(offset)
    first = int(offset) >> 2
    last = (int(offset) + max(numel, 1) - 1) >> 2
    words = philox4x32_10(seed, np.arange(first, last + 1, dtype=np.uint64), all_words=True)   # (4, calls)
    call = (idx >> np.uint64(2)).astype(np.int64) - first
    lane = (idx & np.uint64(3)).astype(np.int64)
    return torch.from_numpy(_word_to_uniform(np.ascontiguousarray(words[lane, call])))


# ---------------------------------------------------------------------------
# Per-tensor casts (tcfp/core.py)
# ---------------------------------------------------------------------------

def _per_tensor_scale(t: torch.Tensor, fmax: float) -> torch.Tensor:
    # tcfp/core.py:100-101 (and :128-129, :152-153)
    amax = t.abs().max().clamp(min=1e-12)
    return (fmax / amax).to(torch.float32)


def to_fp8_e4m3(t: torch.Tensor, scale: torch.Tensor | None = None):
    """tcfp/core.py:85-106."""
    if scale is None:
        scale = _per_tensor_scale(t, FP8_E4M3_MAX)
    scaled = (t.float() * scale).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX)
    inv = torch.ones(1, dtype=torch.float32) / scale
    return scaled.to(E4M3), inv


def to_fp8_e5m2(t: torch.Tensor, scale: torch.Tensor | None = None):
    """tcfp/core.py:137-158."""
    if scale is None:
        scale = _per_tensor_scale(t, FP8_E5M2_MAX)
    scaled = (t.float() * scale).clamp(-FP8_E5M2_MAX, FP8_E5M2_MAX)
    inv = torch.ones(1, dtype=torch.float32) / scale
    return scaled.to(E5M2), inv


def stochastic_round_to_fp8_e4m3(t: torch.Tensor, rand: torch.Tensor) -> torch.Tensor:
    """tcfp/core.py:418-464 with the uniforms passed in instead of drawn."""
    lo = t.to(E4M3)
    lo_f = lo.float()
    direction = torch.sign(t - lo_f)
    exact = t == lo_f
    nudge = direction * (2.0 ** -6) * 0.5
    hi = (lo_f + nudge).to(E4M3)
    same = (hi.float() == lo_f) & ~exact
    abs_lo = lo_f.abs().clamp(min=2.0 ** -6)
    hi_retry = (lo_f + direction * abs_lo * 0.25).to(E4M3)
    hi = torch.where(same, hi_retry, hi)
    hi_f = hi.float()
    gap = (hi_f - lo_f).abs().clamp(min=1e-45)
    frac = ((t - lo_f).abs() / gap).clamp(0.0, 1.0)
    return torch.where(exact, lo, torch.where(rand < frac, hi, lo))


def to_fp8_e4m3_sr(t: torch.Tensor, rand: torch.Tensor, scale: torch.Tensor | None = None):
    """tcfp/core.py:109-134."""
    if scale is None:
        scale = _per_tensor_scale(t, FP8_E4M3_MAX)
    scaled = (t.float() * scale).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX)
    inv = torch.ones(1, dtype=torch.float32) / scale
    return stochastic_round_to_fp8_e4m3(scaled, rand), inv


def nf_aware_target_max(t: torch.Tensor, sigma_factor: float = 3.0) -> torch.Tensor:
    """tcfp/core.py:182-185."""
    t = t.float()
    std = t.std().clamp(min=1e-12)
    return t.abs().max().clamp(min=1e-12) if std < 1e-6 else sigma_factor * std


def to_fp8_e4m3_nf_aware(t: torch.Tensor, sigma_factor: float = 3.0):
    """tcfp/core.py:161-193 (round-to-nearest form)."""
    scale = (FP8_E4M3_MAX / nf_aware_target_max(t, sigma_factor)).to(torch.float32)
    return to_fp8_e4m3(t, scale=scale)


def dual_quantize_per_tensor(
    weight: torch.Tensor,
    error: torch.Tensor | None = None,
    *,
    srr: bool = False,
    seed: int = 0,
    offset: int = 0,
    amax_hi: torch.Tensor | None = None,
    amax_lo: torch.Tensor | None = None,
):
    """Steps 1-4 of ``_TCFP12TensorCoreFunction.forward``
    (tcfp/nn/__init__.py:343-383).

    Returns ``(w_hi, w_lo, inv_hi, inv_lo, new_error, cur_amax_hi,
    cur_amax_lo)``.  ``amax_hi`` / ``amax_lo`` override the fresh amax the way
    delayed scaling does (tcfp/nn/__init__.py:282-285, 302-309); the current
    (pre-clamp) amaxes are returned for the caller's EMA bookkeeping.
    ``new_error`` is ``None`` without an error buffer.
    """
    w = weight.float()
    if error is not None:
        w = w + error
    cur_hi = w.abs().max()
    s_hi = (FP8_E4M3_MAX / (cur_hi.clamp(min=1e-12) if amax_hi is None else amax_hi)).to(torch.float32)
    w_hi, inv_hi = to_fp8_e4m3(w, scale=s_hi)
    residual = w - w_hi.float() * inv_hi
    cur_lo = residual.abs().max()
    s_lo = (FP8_E4M3_MAX / (cur_lo.clamp(min=1e-12) if amax_lo is None else amax_lo)).to(torch.float32)
    if srr:
        rand = philox_uniform_packed(seed, offset, w.numel()).reshape(w.shape)
        w_lo, inv_lo = to_fp8_e4m3_sr(residual, rand, scale=s_lo)
    else:
        w_lo, inv_lo = to_fp8_e4m3(residual, scale=s_lo)
    new_error = None
    if error is not None:
        recon = w_hi.float() * inv_hi + w_lo.float() * inv_lo
        new_error = weight.float() - recon
    return w_hi, w_lo, inv_hi, inv_lo, new_error, cur_hi, cur_lo


# ---------------------------------------------------------------------------
# Block-scaled quantizers (tcfp/kernels.py)
# ---------------------------------------------------------------------------

def _block_exponent(amax: torch.Tensor, fmax: float) -> torch.Tensor:
    """``max(ceil(log2(max(amax, 1e-12) / FP8_MAX)), -126)`` (tcfp/kernels.py:
    250-256, 367-370, 387-390) as the reference's kernels evaluate it on the
    GPU.  Triton compiles ``/`` on float32 to the PTX instruction
    ``div.full.f32`` (not an IEEE division) and ``tl.log2`` to a float32 log2
    accurate to the last bit.  Measured against the reference's own kernel on
    a B200 over every amax within -6..+320 ulps of ``1.75 * 2^a`` for
    a = -34..23 and 200 000 random amax values, for both FP8 maxima: the
    quotient equals ``amax * float32(1 / FP8_MAX)`` (one rounding of the
    product with the rounded reciprocal), and the exponent then follows from a
    correctly rounded float32 log2.  An IEEE division differs from it on amax
    values 1-20 ulps above ``1.75 * 2^a``, where it moves the exponent by one."""
    recip = (torch.ones((), dtype=torch.float32) / torch.tensor(fmax, dtype=torch.float32))
    q = amax.clamp(min=1e-12).float() * recip
    raw = torch.ceil(torch.log2(q.double()).float())
    return raw.clamp(min=-126.0)


def block_quantize(x: torch.Tensor, bs: int, fp8_dtype: torch.dtype = E4M3):
    """``block_quantize_fp8`` / ``_block_quantize_kernel``
    (tcfp/kernels.py:205-275, 1675-1722).  Returns codes ``(M, K)`` and int8
    exponents ``(K // bs, M)``."""
    M, K = x.shape
    assert K % bs == 0
    fmax = FP8_E5M2_MAX if fp8_dtype == E5M2 else FP8_E4M3_MAX
    xb = x.float().reshape(M, K // bs, bs)
    e = _block_exponent(xb.abs().amax(dim=-1), fmax)
    q = (xb / torch.exp2(e).unsqueeze(-1)).clamp(-fmax, fmax).to(fp8_dtype)
    return q.reshape(M, K), e.to(torch.int8).t().contiguous()


def block_dequantize(codes: torch.Tensor, exps: torch.Tensor, bs: int) -> torch.Tensor:
    """``block_dequantize_fp8`` (tcfp/kernels.py:1725-1746)."""
    M, K = codes.shape
    scales = torch.exp2(exps.float())
    return (codes.float().reshape(M, K // bs, bs) * scales.t().unsqueeze(-1)).reshape(M, K)


def _sr_block(x: torch.Tensor, rand: torch.Tensor) -> torch.Tensor:
    """Stochastic rounding of the block kernel (tcfp/kernels.py:398-423)."""
    # values are clamped to +-448 before the cast; the nudged probe can reach
    # 560, which the hardware cast saturates to 448 -- clamp to mirror that.
    rtn = x.to(E4M3)
    rtn_f = rtn.float()
    diff = x - rtn_f
    direction = torch.where(diff >= 0, 1.0, -1.0)
    abs_rtn = rtn_f.abs().clamp(min=1e-12)
    nudge = direction * abs_rtn * 0.25
    other = (rtn_f + nudge).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX).to(E4M3)
    other_f = other.float()
    gap = (other_f - rtn_f).abs().clamp(min=1e-45)
    frac = (diff.abs() / gap).clamp(max=1.0)
    boundary = (other_f - rtn_f).abs() < 1e-45
    exact = (diff.abs() < 1e-45) | boundary
    return torch.where(exact, rtn, torch.where(rand < frac, other, rtn))


def dual_quantize_block(
    weight: torch.Tensor,
    bs: int,
    error: torch.Tensor | None = None,
    *,
    srr: bool = False,
    seed: int = 0,
    offset: int = 0,
):
    """``fused_dual_quantize_fp8`` / ``_fused_dual_quantize_kernel``
    (tcfp/kernels.py:288-459, 1749-1875).

    Returns ``(w_hi, w_lo, exp_hi, exp_lo, new_error)``; the reference writes
    ``new_error`` into ``error`` in place, this restatement returns it.
    """
    N, K = weight.shape
    assert K % bs == 0
    w = weight.float()
    wc = w + error if error is not None else w
    wb = wc.reshape(N, K // bs, bs)
    e_hi = _block_exponent(wb.abs().amax(dim=-1), FP8_E4M3_MAX)
    inv_hi = torch.exp2(e_hi).unsqueeze(-1)
    hi = (wb / inv_hi).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX).to(E4M3)
    residual = wb - hi.float() * inv_hi
    amax_lo = residual.abs().amax(dim=-1)
    zero = amax_lo < 1e-12
    e_lo = _block_exponent(amax_lo, FP8_E4M3_MAX)
    inv_lo = torch.where(zero, torch.ones_like(e_lo), torch.exp2(e_lo)).unsqueeze(-1)
    lo_in = (residual / inv_lo).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX)
    if srr:
        rand = philox_uniform(seed, offset, N * K).reshape(N, K // bs, bs)
        lo = _sr_block(lo_in, rand)
    else:
        lo = lo_in.to(E4M3)
    exp_hi = e_hi.to(torch.int8).t().contiguous()
    exp_lo = torch.where(zero, torch.full_like(e_lo, -128.0), e_lo).to(torch.int8).t().contiguous()
    hi = hi.reshape(N, K)
    lo = lo.reshape(N, K)
    new_error = None
    if error is not None:
        # tcfp/kernels.py:1870-1873: from the STORED codes, against the
        # ORIGINAL weight
        new_error = w - block_dequantize(hi, exp_hi, bs) - block_dequantize(lo, exp_lo, bs)
    return hi, lo, exp_hi, exp_lo, new_error


# ---------------------------------------------------------------------------
# GEMMs: FP32 dequantized dual matmuls
# ---------------------------------------------------------------------------

def dual_gemm_nt(a, inv_a, w_hi, inv_hi, w_lo, inv_lo):
    """``out = (A.W_hi^T).(s_a s_hi) + (A.W_lo^T).(s_a s_lo)``
    (tcfp/kernels.py:108-119, 183-184; tcfp/csrc/fused_dual_gemm.h:8)."""
    af = a.float()
    out = (af @ w_hi.float().t()) * (inv_a * inv_hi)
    if w_lo is not None:
        out = out + (af @ w_lo.float().t()) * (inv_a * inv_lo)
    return out


def dual_gemm_nn(g, inv_g, w_hi, inv_hi, w_lo, inv_lo):
    """``dX = (g.W_hi).(s_g s_hi) + (g.W_lo).(s_g s_lo)``
    (tcfp/kernels.py:1604-1666; tcfp/csrc/fused_dual_gemm.h:9)."""
    gf = g.float()
    out = (gf @ w_hi.float()) * (inv_g * inv_hi)
    if w_lo is not None:
        out = out + (gf @ w_lo.float()) * (inv_g * inv_lo)
    return out


def _deq_lo(codes, exps, bs):
    # sentinel -128 -> scale 0 (tcfp/kernels.py:762-764)
    M, K = codes.shape
    scales = torch.where(exps == -128, torch.zeros((), dtype=torch.float32), torch.exp2(exps.float()))
    return (codes.float().reshape(M, K // bs, bs) * scales.t().unsqueeze(-1)).reshape(M, K)


def block_dual_gemm_nt(a, exp_a, w_hi, exp_hi, w_lo, exp_lo, bs):
    """Block-scaled forward (tcfp/kernels.py:687-692, 738-778): dequantize,
    then FP32 matmul -- the comparison the reference's own tests use
    (tests/test_block_scaling_kernels.py:147-169)."""
    af = block_dequantize(a, exp_a, bs)
    out = af @ block_dequantize(w_hi, exp_hi, bs).t()
    if w_lo is not None:
        out = out + af @ _deq_lo(w_lo, exp_lo, bs).t()
    return out


def block_backward_dx(g, exp_g, w_hi, exp_hi, w_lo, exp_lo, bs):
    """Block-scaled dX (tcfp/kernels.py:1146-1189, 2464-2469): g blocks run
    along D_out, weight blocks along D_in."""
    gf = block_dequantize(g, exp_g, bs)
    w = block_dequantize(w_hi, exp_hi, bs)
    if w_lo is not None:
        w = w + _deq_lo(w_lo, exp_lo, bs)
    return gf @ w


# ---------------------------------------------------------------------------
# Layer level: TCFPLinear forward / backward on the tensor-core path
# ---------------------------------------------------------------------------

class LayerState:
    """The pieces of ``ErrorFeedbackState`` the per-tensor layer touches
    (tcfp/core.py:298-410), plus the SRR stream position."""

    def __init__(self, ema_decay: float = 0.999, interval: int = 100):
        self.error: torch.Tensor | None = None
        self.delayed_amax: torch.Tensor | None = None
        self.ratio: torch.Tensor | None = None
        self.steps = 0
        self.ema_decay = ema_decay
        self.interval = interval
        self.srr_offset = 0

    def get_delayed_amax(self, current):           # tcfp/core.py:341-358
        if self.delayed_amax is None:
            self.delayed_amax = current.clone()
            return current
        self.delayed_amax = self.ema_decay * self.delayed_amax + (1 - self.ema_decay) * current
        return self.delayed_amax

    def should_validate(self):                     # tcfp/core.py:393-403
        self.steps += 1
        return self.steps == 1 or self.steps % self.interval == 0

    def predict(self, main_amax):                  # tcfp/core.py:360-372
        if self.ratio is None:
            return (main_amax / 8.0).clamp(min=1e-12)
        return (main_amax * self.ratio).clamp(min=1e-12)

    def update_ratio(self, main_amax, actual):     # tcfp/core.py:374-391
        r = actual / main_amax.clamp(min=1e-12)
        self.ratio = r if self.ratio is None else self.ema_decay * self.ratio + (1 - self.ema_decay) * r


def linear_forward(x, weight, bias, state: LayerState | None, *, srr=False, abd=False, delayed=False,
                   hp_grad_weight=False, update_ef=True, seed=0, nf_sigma=None):
    """``_TCFP12TensorCoreFunction.forward`` (tcfp/nn/__init__.py:324-459) with
    the GEMMs as FP32 dequantized matmuls.  ``state`` is None for SRR / no-EF
    layers except that SRR uses ``state.srr_offset`` when a state is given.
    Returns ``(output, ctx)``."""
    use_ef = state is not None and not srr
    w = weight.float()
    if use_ef:
        if state.error is None or state.error.shape != w.shape:
            state.error = torch.zeros_like(w)
        w = w + state.error
    if delayed and use_ef:
        current = w.abs().max().clamp(min=1e-12)                       # :282
        d = state.get_delayed_amax(current)
        w_hi, inv_hi = to_fp8_e4m3(w, scale=(FP8_E4M3_MAX / d).to(torch.float32))
        residual = w - w_hi.float() * inv_hi
        if state.should_validate():                                   # :302-305
            actual = residual.abs().max().clamp(min=1e-12)
            state.update_ratio(d, actual)
            s_lo = (FP8_E4M3_MAX / actual).to(torch.float32)
        else:
            s_lo = (FP8_E4M3_MAX / state.predict(d)).to(torch.float32)
        w_lo, inv_lo = to_fp8_e4m3(residual, scale=s_lo)
    else:
        # sigma-based scale for W_hi when nf_aware_scaling is set (:356-359)
        w_hi, inv_hi = to_fp8_e4m3(w) if nf_sigma is None else to_fp8_e4m3_nf_aware(w, nf_sigma)
        residual = w - w_hi.float() * inv_hi
        if srr:
            off = state.srr_offset if state is not None else 0
            rand = philox_uniform_packed(seed, off, w.numel()).reshape(w.shape)
            if state is not None:
                state.srr_offset += w.numel()
            w_lo, inv_lo = to_fp8_e4m3_sr(residual, rand)
        else:
            w_lo, inv_lo = to_fp8_e4m3(residual)
    if use_ef and update_ef:                                           # :378-383
        state.error = weight.float() - (w_hi.float() * inv_hi + w_lo.float() * inv_lo)
    x2d = x.reshape(-1, x.shape[-1])
    a, inv_a = to_fp8_e4m3(x2d)
    out = dual_gemm_nt(a, inv_a, w_hi, inv_hi, w_lo, inv_lo)
    if bias is not None:
        out = out + bias
    ctx = dict(x2d=x2d, a=a, inv_a=inv_a, w_hi=w_hi, w_lo=None if abd else w_lo, inv_hi=inv_hi,
               inv_lo=None if abd else inv_lo, hp=hp_grad_weight, has_bias=bias is not None, shape=x.shape)
    return out.reshape(*x.shape[:-1], out.shape[-1]), ctx


def linear_backward(ctx, grad_out):
    """``_TCFP12TensorCoreFunction.backward`` (tcfp/nn/__init__.py:461-566)."""
    g2d = grad_out.reshape(-1, grad_out.shape[-1])
    gq, inv_g = to_fp8_e5m2(g2d)
    dx = dual_gemm_nn(gq, inv_g, ctx["w_hi"], ctx["inv_hi"], ctx["w_lo"], ctx["inv_lo"]).reshape(ctx["shape"])
    if ctx["hp"]:
        dw = g2d.t() @ ctx["x2d"]
    elif g2d.shape[0] % 16 != 0:
        dw = g2d.t() @ (ctx["a"].float() * ctx["inv_a"])
    else:
        dw = ((gq.float().t() @ ctx["a"].float()) * (inv_g * ctx["inv_a"]))
    db = g2d.sum(dim=0) if ctx["has_bias"] else None
    return dx, dw, db
