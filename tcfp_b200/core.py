"""FP8 primitives and error-feedback state with the names and semantics of the
reference's ``tcfp/core.py``, computed by the CUDA kernels of
``libtcfp_b200.so``.  CUDA tensors only: there is no CPU implementation here.
"""
from __future__ import annotations

from enum import Enum, auto

import torch

from . import _C

# tcfp/core.py:27-43 -- part of the numeric contract
FP8_E4M3_MAX: float = 448.0
FP8_E4M3_MIN: float = -448.0
FP8_E4M3_SMALLEST_NORMAL: float = 2**-6
FP8_E5M2_MAX: float = 57344.0
FP8_E5M2_MIN: float = -57344.0
DEFAULT_BLOCK_SIZE: int = 32
VALID_BLOCK_SIZES: tuple[int, ...] = (16, 32, 64, 128)


class TCFPMode(Enum):
    """tcfp/core.py:46-49."""

    TCFP12 = auto()


def _require_cuda(t: torch.Tensor, who: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{who}: tcfp_b200 runs on CUDA (sm_100) tensors only, got a {t.device} tensor")


def _flat2d(t: torch.Tensor) -> tuple[torch.Tensor, int, int]:
    t = t.contiguous()
    n = t.numel()
    if n % 4 != 0:
        raise RuntimeError(f"tensor size ({n}) must be a multiple of 4 elements")
    return t, 1, n


def _cast(tensor: torch.Tensor, scale: torch.Tensor | None, fp8_dtype: torch.dtype, fmt: int, who: str,
          stochastic: bool = False, seed: int = 0, offset: int = 0):
    _require_cuda(tensor, who)
    src = tensor if tensor.dtype in (torch.float32, torch.bfloat16) else tensor.float()
    src, R, C = _flat2d(src)
    out = torch.empty(tensor.shape, device=tensor.device, dtype=fp8_dtype)
    inv = torch.empty(1, device=tensor.device, dtype=torch.float32)
    scale_t = None
    if scale is not None:
        scale_t = scale.to(device=tensor.device, dtype=torch.float32).reshape(1).contiguous()
    _C.check(_C.load().tcfp_quantize(
        _C.ptr(src), _C.dtype_code(src), _C.ptr(out), _C.ptr(inv), None, None, R, C, 0, fmt,
        None, _C.ptr(scale_t), 1 if stochastic else 0, int(seed), int(offset),
        _C.ptr(_C.workspace(tensor.device)), _C.stream()))
    return out, inv


def to_fp8_e4m3(tensor: torch.Tensor, scale: torch.Tensor | None = None):
    """tcfp/core.py:85-106: ``(fp8, inv_scale (1,))`` with
    ``scale = 448 / max(|t|, 1e-12)`` unless given."""
    return _cast(tensor, scale, torch.float8_e4m3fn, _C.E4M3, "to_fp8_e4m3")


def to_fp8_e5m2(tensor: torch.Tensor, scale: torch.Tensor | None = None):
    """tcfp/core.py:137-158."""
    return _cast(tensor, scale, torch.float8_e5m2, _C.E5M2, "to_fp8_e5m2")


def to_fp8_e5m2_with_colsum(grad2d: torch.Tensor):
    """``to_fp8_e5m2`` of a 2-D gradient plus its FP32 column sums (the bias
    gradient, tcfp/nn/__init__.py:558): the pass that finds the amax also
    accumulates the sums, instead of a separate ``sum(dim=0)`` read.  Returns
    ``(fp8, inv_scale (1,), colsum (C,))``."""
    _require_cuda(grad2d, "to_fp8_e5m2_with_colsum")
    assert grad2d.ndim == 2 and grad2d.is_contiguous() and grad2d.dtype in (torch.float32, torch.bfloat16)
    R, C = grad2d.shape
    lib = _C.load()
    out = torch.empty((R, C), device=grad2d.device, dtype=torch.float8_e5m2)
    inv = torch.empty(1, device=grad2d.device, dtype=torch.float32)
    colsum = torch.empty(C, device=grad2d.device, dtype=torch.float32)
    ws = torch.empty(lib.tcfp_colsum_workspace_bytes(R, C), dtype=torch.uint8, device=grad2d.device)
    _C.check(lib.tcfp_quantize_colsum(_C.ptr(grad2d), _C.dtype_code(grad2d), _C.ptr(out), _C.ptr(inv), None, R, C, 0,
                                      _C.E5M2, _C.ptr(colsum), _C.ptr(ws), _C.stream()))
    return out, inv, colsum


def nf_aware_target_max(tensor: torch.Tensor, sigma_factor: float = 3.0) -> torch.Tensor:
    """The effective maximum of tcfp/core.py:182-185: ``sigma_factor * std``,
    or the amax for near-constant tensors (std < 1e-6).  The standard
    deviation is torch's own reduction, as in the reference."""
    t = tensor.float()
    std = t.std().clamp(min=1e-12)
    return torch.where(std < 1e-6, t.abs().max().clamp(min=1e-12), sigma_factor * std)


def to_fp8_e4m3_nf_aware(tensor: torch.Tensor, sigma_factor: float = 3.0, stochastic: bool = False, *,
                         seed: int = 0, offset: int = 0):
    """tcfp/core.py:161-193: scale to ``sigma_factor`` standard deviations
    instead of the maximum; values beyond are clipped to +-448."""
    scale = (FP8_E4M3_MAX / nf_aware_target_max(tensor, sigma_factor)).to(torch.float32)
    if stochastic:
        return to_fp8_e4m3_sr(tensor, scale, seed=seed, offset=offset)
    return to_fp8_e4m3(tensor, scale)


def absmax(tensor: torch.Tensor, error: torch.Tensor | None = None) -> torch.Tensor:
    """``max |tensor (+ error)|`` as a 0-dim float32 device tensor
    (the reduction of tcfp/core.py:100, tcfp/nn/__init__.py:282)."""
    _require_cuda(tensor, "absmax")
    src = tensor if tensor.dtype in (torch.float32, torch.bfloat16) else tensor.float()
    src = src.contiguous()
    out = torch.empty(1, device=tensor.device, dtype=torch.float32)
    _C.check(_C.load().tcfp_absmax(_C.ptr(src), _C.dtype_code(src), _C.ptr(error), src.numel(), _C.ptr(out),
                                   _C.stream()))
    return out.reshape(())


def dual_quantize_per_tensor(weight: torch.Tensor, error: torch.Tensor | None = None, *, srr: bool = False,
                             update_error: bool = True, seed: int = 0, offset: int = 0,
                             amax_hi: torch.Tensor | None = None, amax_lo: torch.Tensor | None = None,
                             want_amax: bool = False):
    """Steps 1-4 of the reference's per-tensor forward
    (tcfp/nn/__init__.py:343-383) as fused kernels.

    Returns ``(w_hi, w_lo, inv_hi (1,), inv_lo (1,), amax (2,) | None)``.
    ``error`` is updated IN PLACE (mode EF) unless ``update_error`` is False.
    """
    _require_cuda(weight, "dual_quantize_per_tensor")
    assert weight.is_contiguous(), "Weight must be contiguous (N, K) row-major"
    N, K = weight.shape
    if srr and error is not None:
        raise ValueError("srr and an error buffer are mutually exclusive")
    dev = weight.device
    w_hi = torch.empty((N, K), device=dev, dtype=torch.float8_e4m3fn)
    w_lo = torch.empty((N, K), device=dev, dtype=torch.float8_e4m3fn)
    inv_hi = torch.empty(1, device=dev, dtype=torch.float32)
    inv_lo = torch.empty(1, device=dev, dtype=torch.float32)
    amax = torch.empty(2, device=dev, dtype=torch.float32) if want_amax else None
    if srr:
        mode = _C.Q_SRR
    elif error is not None:
        mode = _C.Q_EF if update_error else _C.Q_EF_READONLY
    else:
        mode = _C.Q_NONE
    a_hi = None if amax_hi is None else amax_hi.to(torch.float32).reshape(1).contiguous()
    a_lo = None if amax_lo is None else amax_lo.to(torch.float32).reshape(1).contiguous()
    _C.check(_C.load().tcfp_dual_quantize(
        _C.ptr(weight), _C.dtype_code(weight), _C.ptr(error), _C.ptr(w_hi), _C.ptr(w_lo), _C.ptr(inv_hi),
        _C.ptr(inv_lo), None, None, N, K, 0, mode, int(seed), int(offset), _C.ptr(a_hi), _C.ptr(a_lo),
        _C.ptr(amax), _C.ptr(_C.workspace(dev)), _C.stream()))
    return w_hi, w_lo, inv_hi, inv_lo, amax


def to_fp8_e4m3_sr(tensor: torch.Tensor, scale: torch.Tensor | None = None, *, seed: int = 0, offset: int = 0):
    """tcfp/core.py:109-134 with a seeded Philox stream in place of
    ``torch.rand_like``: element ``i`` draws word ``(offset + i) & 3`` of
    ``philox4x32-10(seed, (offset + i) >> 2)`` (all four words of a call are used)."""
    return _cast(tensor, scale, torch.float8_e4m3fn, _C.E4M3, "to_fp8_e4m3_sr", stochastic=True, seed=seed,
                 offset=offset)


def ensure_column_major(t: torch.Tensor) -> torch.Tensor:
    """tcfp/core.py:196-213 (layout helper for ``torch._scaled_mm`` callers)."""
    assert t.ndim == 2, f"ensure_column_major requires 2-D tensor, got {t.ndim}-D"
    if t.stride(0) == 1 and t.stride(1) == t.shape[0]:
        return t
    return t.t().contiguous().t()


def fp8_matmul(a_fp8: torch.Tensor, b_fp8: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
               out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``(a * scale_a) @ (b * scale_b)`` for ``a (M,K)``, ``b (K,N)`` FP8 with
    scalar inverse scales (tcfp/core.py:519-553) -- the single-operand form of
    the dual GEMM, reading ``b`` in place."""
    from .kernels import fused_dual_gemm_backward_dx

    return fused_dual_gemm_backward_dx(a_fp8.contiguous(), b_fp8.contiguous(), None, scale_a.reshape(1),
                                       scale_b.reshape(1), None, out_dtype=out_dtype)


def fp8_matmul_nn(a_fp8: torch.Tensor, b_fp8_t: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                  out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Same with ``b`` given transposed, ``(N, K)`` (tcfp/core.py:556-578)."""
    from .kernels import fused_dual_gemm_forward

    return fused_dual_gemm_forward(a_fp8.contiguous(), b_fp8_t.contiguous(), None, scale_a.reshape(1),
                                   scale_b.reshape(1), None, out_dtype=out_dtype)


class ErrorFeedbackState:
    """Per-parameter state of the tensor-core path.

    Five dictionaries with the reference's names and key scheme
    (tcfp/core.py:298-410) -- ``_buffers[name]`` the FP32 error buffer,
    ``_amax_ema``, ``_delayed_amax[name + ".w_hi"]``, ``_residual_ratio[name +
    ".ratio"]`` and ``_step_count[name + ".steps"]`` -- so that ``ef_state.pt``
    files written by either implementation load in the other
    (tcfp/training/checkpointing.py:200-271).  All moving averages are
    ``decay * previous + (1 - decay) * new`` evaluated in that order on device
    tensors; nothing here synchronises with the host except the step counter,
    which is a host integer by design."""

    def __init__(self, ema_decay: float = 0.999, residual_validation_interval: int = 100) -> None:
        self._buffers: dict[str, torch.Tensor] = {}
        self._amax_ema: dict[str, torch.Tensor] = {}
        self._delayed_amax: dict[str, torch.Tensor] = {}
        self._residual_ratio: dict[str, torch.Tensor] = {}
        self._step_count: dict[str, int] = {}
        self._ema_decay: float = ema_decay
        self._residual_validation_interval: int = residual_validation_interval

    # -- shared moving-average step ---------------------------------------
    def _blend(self, table: dict[str, torch.Tensor], key: str, value: torch.Tensor) -> tuple[torch.Tensor, bool]:
        """Folds ``value`` into ``table[key]``; returns (stored value, was_first)."""
        value = value.detach()
        if key not in table:
            return value, True
        d = self._ema_decay
        table[key] = d * table[key] + (1 - d) * value
        return table[key], False

    # -- error buffer -------------------------------------------------------
    def get_error(self, name: str, like: torch.Tensor) -> torch.Tensor:
        """The buffer for ``name``: FP32, zero on first use or after a shape change."""
        buf = self._buffers.get(name)
        if buf is None or buf.shape != like.shape:
            buf = torch.zeros_like(like, dtype=torch.float32)
            self._buffers[name] = buf
        return buf

    def update_error(self, name: str, error: torch.Tensor) -> None:
        self._buffers[name] = error.detach()

    # -- amax tracking --------------------------------------------------------
    def get_amax_ema(self, name: str, current_amax: torch.Tensor) -> torch.Tensor:
        stored, first = self._blend(self._amax_ema, name, current_amax)
        if first:
            self._amax_ema[name] = stored.clone()
        return self._amax_ema[name]

    def get_delayed_amax(self, name: str, current_amax: torch.Tensor) -> torch.Tensor:
        """Delayed-scaling amax: the very first call stores and returns the
        current value unchanged (no delay on step 0), later calls return the
        moving average that already includes the current value."""
        stored, first = self._blend(self._delayed_amax, name, current_amax)
        if first:
            self._delayed_amax[name] = stored.clone()
            return current_amax
        return stored

    def predict_residual_amax(self, name: str, main_amax: torch.Tensor) -> torch.Tensor:
        """Residual amax predicted from the main one: tracked ratio, or 1/8
        (three mantissa bits) before any ratio was observed."""
        ratio = self._residual_ratio.get(f"{name}.ratio")
        predicted = main_amax / 8.0 if ratio is None else main_amax * ratio
        return predicted.clamp(min=1e-12)

    def update_residual_ratio(self, name: str, main_amax: torch.Tensor, actual_residual_amax: torch.Tensor) -> None:
        key = f"{name}.ratio"
        ratio = actual_residual_amax / main_amax.clamp(min=1e-12)
        stored, first = self._blend(self._residual_ratio, key, ratio)
        if first:
            self._residual_ratio[key] = stored

    def should_validate_residual(self, name: str) -> bool:
        """True on the first call and on every ``residual_validation_interval``-th."""
        key = f"{name}.steps"
        n = self._step_count.get(key, 0) + 1
        self._step_count[key] = n
        return n == 1 or n % self._residual_validation_interval == 0

    def reset(self) -> None:
        for table in (self._buffers, self._amax_ema, self._delayed_amax, self._residual_ratio, self._step_count):
            table.clear()
