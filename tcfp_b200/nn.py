"""``TCFPLinear`` on the tensor-core path, with the reference's class name,
constructor flags, state and autograd behaviour (tcfp/nn/__init__.py:250-1077),
computed by the sm_100a kernels of ``libtcfp_b200.so``.

Scope: the tensor-core path only (``use_tensor_cores=True``), per-tensor or
block-32/64/128 scaling, error feedback or stochastic residual rounding,
delayed scaling, ABD, high-precision weight gradients.  The fake-quantize
format of the reference (``use_tensor_cores=False``) is a different numeric
format and is not provided.
"""
from __future__ import annotations

import warnings

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _C
from .core import (
    DEFAULT_BLOCK_SIZE,
    ErrorFeedbackState,
    TCFPMode,
    absmax,
    dual_quantize_per_tensor,
    nf_aware_target_max,
    to_fp8_e4m3,
    to_fp8_e5m2,
    to_fp8_e5m2_with_colsum,
)
from .kernels import (
    bf16_weight_grad,
    block_dequantize_bf16,
    block_quantize_fp8,
    fp8_weight_grad,
    fused_block_scaled_backward_dx,
    fused_block_scaled_dual_gemm_forward,
    fused_dual_gemm_backward_dx,
    fused_dual_gemm_forward,
    fused_dual_quantize_fp8,
    pack_block_scales,
    packed_scale_rows,
)


def _flat2d(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1, t.shape[-1]).contiguous()


def _dx_dtype(input: torch.Tensor) -> torch.dtype:
    # autograd casts the input gradient to the input's dtype anyway; a bf16 input gets its gradient
    # written as bf16 by the GEMM epilogue instead of an FP32 tensor plus a conversion pass
    return torch.bfloat16 if input.dtype == torch.bfloat16 else torch.float32


def _master(weight: torch.Tensor) -> torch.Tensor:
    w = weight.detach()
    if w.dtype not in (torch.float32, torch.bfloat16):
        w = w.float()
    return w.contiguous()


class LayerHooks:
    """Communication hooks a tensor-parallel wrapper installs on a layer
    (``TCFPLinear._hooks``); the autograd Functions call them at the points
    where a collective can overlap the layer's own GEMMs.

    ``out_hook(chunk)`` is called with each finished row chunk of the forward
    output (``row_chunks`` of them, on 128-row boundaries) and may start an
    asynchronous in-place reduction of it; ``dx_hook(grad_input)`` is called
    with the input gradient before the weight gradient is computed.  Both
    return ``None`` or an object whose ``wait()`` makes the current stream
    wait for the collective.

    ``sp`` (sequence parallelism) turns the layer's input into this rank's
    TOKEN SHARD, a 2-D ``(tokens / world, K)`` matrix: the Function quantizes
    the shard, calls ``sp.gather_rows`` on the FP8 codes (one byte per element
    on the wire instead of two) and ``sp.gather_planes`` on the exponent planes
    -- the per-tensor Function, whose scale needs the global amax, gathers the
    input itself -- and the output covers all tokens.  Backward,
    ``sp.scatter_rows_async(dX)`` starts the reduce-scatter of the full input
    gradient and returns ``(handle, this rank's rows)``; the weight gradient is
    computed while it runs.

    ``sp_out`` is the mirror image for a layer whose OUTPUT is reduced over
    ranks and sharded over tokens: the forward output goes through
    ``sp_out.scatter_rows_async`` and the layer returns this rank's rows.
    Backward it receives the gradient of those rows; with block scaling it
    quantizes them, gathers the E5M2 codes and exponents for the dX GEMM, and
    gathers the full-precision gradient the weight gradient needs with
    ``sp_out.gather_rows_async`` while the dX GEMM runs."""

    def __init__(self, out_hook=None, row_chunks: int = 1, dx_hook=None, reserve_sms: int = 0, sp=None, sp_out=None):
        self.sp = sp
        self.sp_out = sp_out
        self.out_hook = out_hook
        self.row_chunks = max(1, int(row_chunks))
        self.dx_hook = dx_hook
        # SMs the weight-gradient GEMM leaves free while the collective started by dx_hook is in flight
        # (the GEMMs are persistent, one CTA per SM: without free SMs the collective's kernel cannot start)
        self.reserve_sms = int(reserve_sms)


def _row_chunks(M: int, hooks) -> list[tuple[int, int]]:
    if hooks is None or hooks.out_hook is None:
        return [(0, M)]
    rows = -(-M // hooks.row_chunks)
    rows = max(128, -(-rows // 128) * 128)
    return [(r0, min(M, r0 + rows)) for r0 in range(0, M, rows)]


def _wait_all(pending) -> None:
    for h in pending:
        if h is not None:
            h.wait()


def _cached_quantize(cache: dict | None, w: torch.Tensor, error_buf, update_ef: bool, srr: bool, tag, quantize):
    """Weight quantization reused across forwards that must produce the same
    bytes.  The reference re-quantizes on every forward (tcfp/nn/__init__.py:
    344-372, 627-632); between two optimizer steps -- gradient-accumulation
    micro-batches, checkpoint recomputation -- the weight and the error buffer
    do not change, so every forward after the one that updated the buffer
    quantizes the same ``W + e`` to the same codes.  Those are kept on the
    layer, keyed on the weight's and the buffer's version counters and
    addresses.  Not used for the stochastic residual (fresh randoms per
    forward), for a forward that updates the error buffer, or while a CUDA
    graph is being captured (a replayed step must quantize the weight it finds)."""
    reusable = (cache is not None and not srr and (error_buf is None or not update_ef)
                and not torch.cuda.is_current_stream_capturing())
    if not reusable:
        if cache is not None:
            cache.clear()
        return quantize()
    key = (tag, w.data_ptr(), w._version, tuple(w.shape), w.dtype,
           None if error_buf is None else (error_buf.data_ptr(), error_buf._version))
    if cache.get("key") == key:
        return cache["value"]
    value = quantize()
    cache["key"], cache["value"] = key, value
    return value


# ---------------------------------------------------------------------------
# per-tensor scaling (tcfp/nn/__init__.py:312-566)
# ---------------------------------------------------------------------------

class _TCFP12TensorCoreFunction(torch.autograd.Function):
    """Two FP8 GEMMs sharing one quantized activation, per-tensor scales."""

    @staticmethod
    def forward(ctx, input, weight, bias, hp_grad_weight, error_state, param_name, delayed_scaling, abd, srr,
                update_ef, srr_seed, srr_offset, out_dtype=torch.float32, nf_sigma=None, wq_cache=None, hooks=None):
        w = _master(weight)
        error_buf = None
        if error_state is not None:
            # lazily zero-initialised FP32 buffer, updated in place by the kernel
            error_buf = error_state.get_error(param_name, w)

        if nf_sigma is not None:
            # sigma-based scale for W_hi (tcfp/nn/__init__.py:356-359, tcfp/core.py:161-193); with delayed
            # scaling the sigma target feeds the EMA instead of the amax (:263-280)
            target = nf_aware_target_max(w.float() + error_buf if error_buf is not None else w, nf_sigma)
            if delayed_scaling and error_state is not None:
                target = error_state.get_delayed_amax(param_name + ".w_hi", target)
                if error_state.should_validate_residual(param_name):
                    w_hi, w_lo, inv_hi, inv_lo, amax = dual_quantize_per_tensor(
                        w, error_buf, update_error=update_ef, amax_hi=target, want_amax=True)
                    error_state.update_residual_ratio(param_name, target, amax[1].clamp(min=1e-12))
                else:
                    w_hi, w_lo, inv_hi, inv_lo, _ = dual_quantize_per_tensor(
                        w, error_buf, update_error=update_ef, amax_hi=target,
                        amax_lo=error_state.predict_residual_amax(param_name, target))
            else:
                w_hi, w_lo, inv_hi, inv_lo, _ = dual_quantize_per_tensor(
                    w, error_buf, srr=srr, update_error=update_ef, seed=srr_seed, offset=srr_offset, amax_hi=target)
        elif delayed_scaling and error_state is not None:
            # predictive dual-track delayed scaling (tcfp/nn/__init__.py:250-309)
            current = absmax(w, error_buf).clamp(min=1e-12)
            delayed = error_state.get_delayed_amax(param_name + ".w_hi", current)
            if error_state.should_validate_residual(param_name):
                w_hi, w_lo, inv_hi, inv_lo, amax = dual_quantize_per_tensor(
                    w, error_buf, update_error=update_ef, amax_hi=delayed, want_amax=True)
                error_state.update_residual_ratio(param_name, delayed, amax[1].clamp(min=1e-12))
            else:
                predicted = error_state.predict_residual_amax(param_name, delayed)
                w_hi, w_lo, inv_hi, inv_lo, _ = dual_quantize_per_tensor(
                    w, error_buf, update_error=update_ef, amax_hi=delayed, amax_lo=predicted)
        else:
            w_hi, w_lo, inv_hi, inv_lo, _ = _cached_quantize(
                wq_cache, w, error_buf, update_ef, srr, "per_tensor",
                lambda: dual_quantize_per_tensor(w, error_buf, srr=srr, update_error=update_ef, seed=srr_seed,
                                                 offset=srr_offset))
        if wq_cache is not None and (nf_sigma is not None or (delayed_scaling and error_state is not None)):
            wq_cache.clear()       # these modes advance scaling state on every forward: nothing to reuse

        input_shape = input.shape
        x2d = _flat2d(input)
        sp = None if hooks is None else hooks.sp
        if sp is not None:
            x2d = sp.gather_rows(x2d.contiguous())               # the scale below is the amax over all tokens
        act_fp8, act_inv = to_fp8_e4m3(x2d)                      # always fresh (:390)
        bias_f = None if bias is None else bias.detach().float().contiguous()
        out2d = torch.empty((x2d.shape[0], w_hi.shape[0]), device=x2d.device, dtype=out_dtype)
        pending = []
        for r0, r1 in _row_chunks(x2d.shape[0], hooks):
            fused_dual_gemm_forward(act_fp8[r0:r1], w_hi, w_lo, act_inv, inv_hi, inv_lo, bias=bias_f,
                                    out_dtype=out_dtype, out=out2d[r0:r1])
            if hooks is not None and hooks.out_hook is not None:
                pending.append(hooks.out_hook(out2d[r0:r1]))
        _wait_all(pending)
        sp_out = None if hooks is None else hooks.sp_out
        if sp_out is not None:
            handle, out2d = sp_out.scatter_rows_async(out2d)
            _wait_all([handle])
        ctx.dx_hook = None if hooks is None else hooks.dx_hook
        ctx.sp, ctx.sp_out = sp, sp_out
        ctx.reserve_sms = 0 if hooks is None else hooks.reserve_sms
        ctx.dx_dtype = _dx_dtype(input)
        ctx.hp_grad_weight = hp_grad_weight
        ctx.input_shape = input_shape
        ctx.has_bias = bias is not None
        ctx.abd = abd
        saved = [x2d if hp_grad_weight else act_fp8, w_hi]
        if not abd:
            saved += [w_lo, inv_lo]
        saved += [inv_hi, act_inv]
        ctx.save_for_backward(*saved)
        if sp is not None or sp_out is not None:
            return out2d
        return out2d.reshape(*input_shape[:-1], out2d.shape[-1])

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors
        if ctx.abd:
            saved_act, w_hi, inv_hi, act_inv = saved
            w_lo = inv_lo = None
        else:
            saved_act, w_hi, w_lo, inv_lo, inv_hi, act_inv = saved
        g2d = _flat2d(grad_output)
        if g2d.dtype not in (torch.float32, torch.bfloat16):
            g2d = g2d.float()
        if ctx.sp_out is not None:
            g2d = ctx.sp_out.gather_rows(g2d)          # the gradient's scale is the amax over all tokens
        # always fresh (:494); with a bias its gradient (the column sums, :558) comes out of the same passes
        grad_bias = None
        if ctx.has_bias and g2d.shape[1] % 8 == 0:
            grad_fp8, grad_inv, grad_bias = to_fp8_e5m2_with_colsum(g2d)
        else:
            grad_fp8, grad_inv = to_fp8_e5m2(g2d)
            if ctx.has_bias:
                grad_bias = g2d.float().sum(dim=0)
        grad_input = fused_dual_gemm_backward_dx(grad_fp8, w_hi, w_lo, grad_inv, inv_hi, inv_lo,
                                                 out_dtype=ctx.dx_dtype)
        # either collective overlaps the dW GEMM below
        if ctx.sp is not None:
            dx_pending, grad_input = ctx.sp.scatter_rows_async(grad_input)
        else:
            dx_pending = ctx.dx_hook(grad_input) if ctx.dx_hook is not None else None
        grad_input = grad_input.reshape(ctx.input_shape)
        with _C.sm_reserve(ctx.reserve_sms if dx_pending is not None else 0):
            if ctx.hp_grad_weight:
                if saved_act.dtype == torch.bfloat16 and g2d.shape[1] % 16 == 0 and saved_act.shape[1] % 16 == 0:
                    grad_weight = bf16_weight_grad(g2d, saved_act)
                else:
                    grad_weight = g2d.float().t() @ saved_act.float()    # (:541-542)
            else:
                grad_weight = fp8_weight_grad(grad_fp8, saved_act, grad_inv, act_inv)   # (:546-555)
        _wait_all([dx_pending])
        return (grad_input, grad_weight, grad_bias) + (None,) * 13


# ---------------------------------------------------------------------------
# block scaling (tcfp/nn/__init__.py:574-761)
# ---------------------------------------------------------------------------

class _TCFP12BlockScaledFunction(torch.autograd.Function):
    """Per-block power-of-two scales along K; the tensor core applies them."""

    @staticmethod
    def forward(ctx, input, weight, bias, scale_block_size, hp_grad_weight, error_state, param_name, abd, srr,
                update_ef, srr_seed, srr_offset, out_dtype=torch.float32, wq_cache=None, hooks=None):
        w = _master(weight)
        error_buf = None
        if error_state is not None:
            error_buf = error_state.get_error(param_name, w)
        bs = scale_block_size
        # update_ef False (gradient accumulation, checkpoint recomputation):
        # the kernel reads the buffer and leaves it alone -- the reference
        # clones it for the same effect (:607-608)
        w_hi, w_lo, s_hi, s_lo = _cached_quantize(
            wq_cache, w, error_buf, update_ef, srr, ("block", bs),
            lambda: fused_dual_quantize_fp8(w, bs, error_buf, srr, seed=srr_seed, offset=srr_offset,
                                            update_error=update_ef))
        input_shape = input.shape
        x2d = _flat2d(input)
        if x2d.dtype not in (torch.float32, torch.bfloat16):
            x2d = x2d.float()
        act_fp8, act_scales = block_quantize_fp8(x2d, bs, torch.float8_e4m3fn)
        sp = None if hooks is None else hooks.sp
        if sp is not None:
            # block scales are local to a row: quantize this rank's tokens, gather codes and exponents
            act_fp8 = sp.gather_rows(act_fp8)
            act_scales = sp.gather_planes(act_scales)
            if hp_grad_weight:
                x2d = sp.gather_rows(x2d.contiguous())
        bias_f = None if bias is None else bias.detach().float().contiguous()
        M, K = act_fp8.shape
        out2d = torch.empty((M, w_hi.shape[0]), device=x2d.device, dtype=out_dtype)
        act_sf = pack_block_scales(act_scales, bs)
        pending = []
        for r0, r1 in _row_chunks(M, hooks):
            fused_block_scaled_dual_gemm_forward(
                act_fp8[r0:r1], w_hi, w_lo, act_scales, s_hi, s_lo, bs, bias=bias_f, out_dtype=out_dtype,
                out=out2d[r0:r1], act_sf=packed_scale_rows(act_sf, r0, r1, K, bs))
            if hooks is not None and hooks.out_hook is not None:
                pending.append(hooks.out_hook(out2d[r0:r1]))
        _wait_all(pending)
        sp_out = None if hooks is None else hooks.sp_out
        if sp_out is not None:
            handle, out2d = sp_out.scatter_rows_async(out2d)
            _wait_all([handle])
        ctx.dx_hook = None if hooks is None else hooks.dx_hook
        ctx.sp, ctx.sp_out = sp, sp_out
        ctx.reserve_sms = 0 if hooks is None else hooks.reserve_sms
        ctx.dx_dtype = _dx_dtype(input)
        ctx.hp_grad_weight = hp_grad_weight
        ctx.input_shape = input_shape
        ctx.has_bias = bias is not None
        ctx.bs = bs
        ctx.abd = abd
        if hp_grad_weight:
            saved = [x2d, w_hi, s_hi]
        else:
            saved = [act_fp8, w_hi, s_hi, act_scales]
        if not abd:
            saved += [w_lo, s_lo]
        ctx.save_for_backward(*saved)
        if sp is not None or sp_out is not None:
            return out2d
        return out2d.reshape(*input_shape[:-1], out2d.shape[-1])

    @staticmethod
    def backward(ctx, grad_output):
        saved = list(ctx.saved_tensors)
        bs = ctx.bs
        if ctx.hp_grad_weight:
            saved_act, w_hi, s_hi = saved[:3]
            act_scales = None
            rest = saved[3:]
        else:
            saved_act, w_hi, s_hi, act_scales = saved[:4]
            rest = saved[4:]
        w_lo, s_lo = (None, None) if ctx.abd else rest
        g2d = _flat2d(grad_output)
        if g2d.dtype not in (torch.float32, torch.bfloat16):
            g2d = g2d.float()
        # E5M2 block quantize of the gradient along D_out (:724-726); dX on the FP8 block-scaled MMA against
        # the weight re-targeted for this contraction (once per weight version, kept on w_hi)
        g_pending = None
        if ctx.sp_out is not None:
            # g2d holds this rank's tokens: quantize them, gather codes and exponents for dX, and fetch the
            # full-precision rows of the other ranks (dW needs them) while the dX GEMM runs
            grad_fp8, grad_scales = block_quantize_fp8(g2d, bs, torch.float8_e5m2)
            grad_fp8 = ctx.sp_out.gather_rows(grad_fp8)
            grad_scales = ctx.sp_out.gather_planes(grad_scales)
            g_pending, g2d = ctx.sp_out.gather_rows_async(g2d)
            grad_bias = None
        elif ctx.has_bias:      # the bias gradient (column sums, :753) rides the quantizer's pass
            grad_fp8, grad_scales, grad_bias = block_quantize_fp8(g2d, bs, torch.float8_e5m2, want_colsum=True)
        else:
            grad_fp8, grad_scales = block_quantize_fp8(g2d, bs, torch.float8_e5m2)
            grad_bias = None
        with _C.sm_reserve(ctx.reserve_sms if g_pending is not None else 0):
            grad_input = fused_block_scaled_backward_dx(grad_fp8, w_hi, w_lo, grad_scales, s_hi, s_lo, bs,
                                                        out_dtype=ctx.dx_dtype)
        if ctx.sp_out is not None:
            _wait_all([g_pending])
            if ctx.has_bias:
                grad_bias = g2d.float().sum(dim=0)
        # either collective overlaps the dW GEMM below
        if ctx.sp is not None:
            dx_pending, grad_input = ctx.sp.scatter_rows_async(grad_input)
        else:
            dx_pending = ctx.dx_hook(grad_input) if ctx.dx_hook is not None else None
        grad_input = grad_input.reshape(ctx.input_shape)
        # dW in full precision, as in the reference (:744-750)
        with _C.sm_reserve(ctx.reserve_sms if dx_pending is not None else 0):
            if ctx.hp_grad_weight:
                if saved_act.dtype == torch.bfloat16:
                    grad_weight = bf16_weight_grad(g2d, saved_act)
                else:
                    grad_weight = g2d.float().t() @ saved_act.float()
            else:
                # the saved codes dequantize exactly to bf16; the FP32 gradient goes in as bf16 head + tail
                grad_weight = bf16_weight_grad(g2d, block_dequantize_bf16(saved_act, act_scales, bs))
        _wait_all([dx_pending])
        return (grad_input, grad_weight, grad_bias) + (None,) * 12


# ---------------------------------------------------------------------------
# TCFPLinear (tcfp/nn/__init__.py:769-1077)
# ---------------------------------------------------------------------------

class TCFPLinear(nn.Module):
    """Drop-in ``nn.Linear`` on the TCFP-12 tensor-core path.

    Constructor arguments, attribute names, warnings and validation follow
    tcfp/nn/__init__.py:810-946; flags are re-read on every forward because
    training policies mutate them live.  ``use_fused_kernel`` and
    ``use_cuda_ext`` are accepted for compatibility: there is exactly one
    backend here.  Additional keywords: ``srr_seed`` seeds the stochastic
    residual stream (element ``n*K+k`` of forward call ``i`` is stream position
    ``j = i*N*K + n*K + k``: ``philox(seed, j)[0]`` with block scaling -- the
    reference kernel's ``tl.rand`` stream -- and word ``j & 3`` of
    ``philox(seed, j >> 2)`` with per-tensor scaling); ``out_dtype=torch.bfloat16`` makes the
    GEMM epilogue write bf16 (the reference always returns FP32).
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, mode: TCFPMode = TCFPMode.TCFP12,
                 block_size: int = DEFAULT_BLOCK_SIZE, *, nf4_residual: bool = False, nf_aware_scaling: bool = False,
                 sigma_factor: float = 3.0, stochastic_rounding: bool = False, warmup_steps: int = 0,
                 use_tensor_cores: bool = False, hp_grad_weight: bool = False, error_feedback: bool = True,
                 delayed_scaling: bool = False, use_fused_kernel: bool = True, use_cuda_ext: bool = True,
                 scale_block_size: int | None = None, abd: bool = False, srr: bool = False,
                 srr_seed: int | None = None, out_dtype: torch.dtype = torch.float32, device=None, dtype=None) -> None:
        super().__init__()
        if nf4_residual and use_tensor_cores and mode == TCFPMode.TCFP12:
            warnings.warn("nf4_residual is ignored in tensor core mode — NF4 cannot run on tensor cores. "
                          "The residual uses FP8 E4M3 instead.", stacklevel=2)
        if delayed_scaling and not use_tensor_cores:
            warnings.warn("delayed_scaling requires use_tensor_cores=True and is ignored without it.", stacklevel=2)
        if nf_aware_scaling and stochastic_rounding and use_tensor_cores:
            raise ValueError("nf_aware_scaling with stochastic_rounding of W_hi is not provided on the tensor-core path")
        self.in_features = in_features
        self.out_features = out_features
        self.mode = mode
        self.block_size = block_size
        self.nf4_residual = nf4_residual
        self.nf_aware_scaling = nf_aware_scaling
        self.sigma_factor = sigma_factor
        self.stochastic_rounding = stochastic_rounding
        self._warmup_steps = warmup_steps
        self._warmup_remaining = warmup_steps
        self.use_tensor_cores = use_tensor_cores
        self.hp_grad_weight = hp_grad_weight
        self.use_fused_kernel = use_fused_kernel
        self.use_cuda_ext = use_cuda_ext
        if scale_block_size is not None:
            if scale_block_size not in (32, 64, 128):
                raise ValueError(f"scale_block_size must be 32, 64, or 128, got {scale_block_size}")
            if in_features % scale_block_size != 0:
                raise ValueError(f"in_features ({in_features}) must be divisible by "
                                 f"scale_block_size ({scale_block_size})")
            if out_features % scale_block_size != 0:
                raise ValueError(f"out_features ({out_features}) must be divisible by "
                                 f"scale_block_size ({scale_block_size}). Backward pass "
                                 f"block-quantizes gradients along the output dimension.")
            if not use_tensor_cores:
                warnings.warn("scale_block_size requires use_tensor_cores=True and is ignored without it.",
                              stacklevel=2)
                scale_block_size = None
            if delayed_scaling and scale_block_size is not None:
                warnings.warn("Per-block scaling (scale_block_size) and delayed_scaling are mutually exclusive. "
                              "Ignoring delayed_scaling.", stacklevel=2)
                delayed_scaling = False
        self.scale_block_size = scale_block_size
        self.delayed_scaling = delayed_scaling
        if abd and not use_tensor_cores:
            warnings.warn("abd=True requires use_tensor_cores=True and is ignored without it.", stacklevel=2)
            abd = False
        self.abd = abd
        if srr and not use_tensor_cores:
            warnings.warn("srr=True requires use_tensor_cores=True and is ignored without it.", stacklevel=2)
            srr = False
        if srr and delayed_scaling:
            warnings.warn("srr=True is mutually exclusive with delayed_scaling=True. Disabling delayed_scaling.",
                          stacklevel=2)
            delayed_scaling = False
            self.delayed_scaling = False
        self.srr = srr
        if out_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("out_dtype must be torch.float32 (the reference's output type) or torch.bfloat16")
        self.out_dtype = out_dtype
        self.srr_seed = int(srr_seed if srr_seed is not None else (torch.initial_seed() & 0x7FFFFFFF))
        self._srr_offset = 0

        self._error_state: ErrorFeedbackState | None = None
        if use_tensor_cores and error_feedback and not srr:
            self._error_state = ErrorFeedbackState()
        self._param_name: str = ""
        self._last_weight_version: int = -1
        self._bf16_fallback: bool = False
        # quantized weight of the last forward that did not update the error buffer (see _cached_quantize)
        self._wq_cache: dict = {}
        # communication hooks installed by the tensor-parallel wrappers (LayerHooks) or None
        self._hooks = None

        kw = {"device": device, "dtype": dtype}
        self.weight = nn.Parameter(torch.empty(out_features, in_features, **kw))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, **kw))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=5**0.5)
        if self.bias is not None:
            bound = 1 / self.weight.shape[1] ** 0.5
            nn.init.uniform_(self.bias, -bound, bound)

    def fallback_to_bf16(self) -> None:
        """Switch this layer to plain ``F.linear`` (tcfp/nn/__init__.py:962-964)."""
        self._bf16_fallback = True

    def restore_tcfp(self) -> None:
        self._bf16_fallback = False

    @torch.compiler.disable
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._bf16_fallback:
            return F.linear(x, self.weight, self.bias)
        if self._warmup_remaining > 0:
            self._warmup_remaining -= 1
            return F.linear(x, self.weight, self.bias)
        if not self.use_tensor_cores:
            raise NotImplementedError(
                "tcfp_b200 provides the tensor-core path only: construct TCFPLinear with use_tensor_cores=True"
            )
        if not x.is_cuda:
            raise RuntimeError("TCFPLinear (tcfp_b200) runs on CUDA sm_100 devices only; there is no CPU path")
        _C.load()
        # skip the EF update when the weight has not changed (gradient
        # accumulation) or under no_grad (checkpoint recomputation), :989-994
        ver = self.weight._version
        update_ef = ver != self._last_weight_version and torch.is_grad_enabled()
        if update_ef:
            self._last_weight_version = ver
        srr = self.srr and self._error_state is None
        srr_offset = self._srr_offset
        if srr:
            self._srr_offset += self.weight.numel()
        if self.mode == TCFPMode.TCFP12 and self.scale_block_size is not None:
            return _TCFP12BlockScaledFunction.apply(
                x, self.weight, self.bias, self.scale_block_size, self.hp_grad_weight, self._error_state,
                self._param_name, self.abd, srr, update_ef, self.srr_seed, srr_offset, self.out_dtype, self._wq_cache, self._hooks)
        return _TCFP12TensorCoreFunction.apply(
            x, self.weight, self.bias, self.hp_grad_weight, self._error_state, self._param_name,
            self.delayed_scaling, self.abd, srr, update_ef, self.srr_seed, srr_offset, self.out_dtype,
            self.sigma_factor if self.nf_aware_scaling else None, self._wq_cache, self._hooks)

    def extra_repr(self) -> str:
        parts = [f"in_features={self.in_features}", f"out_features={self.out_features}",
                 f"bias={self.bias is not None}", f"mode={self.mode.name}", f"block_size={self.block_size}"]
        if self.use_tensor_cores:
            parts.append("use_tensor_cores=True")
        if self.hp_grad_weight:
            parts.append("hp_grad_weight=True")
        if self.nf_aware_scaling:
            parts.append("nf_aware_scaling=True")
        if self.delayed_scaling:
            parts.append("delayed_scaling=True")
        if self.use_fused_kernel:
            parts.append("use_fused_kernel=True")
        if self.use_cuda_ext:
            parts.append("use_cuda_ext=True")
        if self.scale_block_size is not None:
            parts.append(f"scale_block_size={self.scale_block_size}")
        if self.abd:
            parts.append("abd=True")
        if self.srr:
            parts.append("srr=True")
        if self._warmup_steps > 0:
            parts.append(f"warmup_steps={self._warmup_steps}")
        if self._bf16_fallback:
            parts.append("bf16_fallback=True")
        return ", ".join(parts)


def convert_to_tcfp(model: nn.Module, mode: TCFPMode = TCFPMode.TCFP12, block_size: int = DEFAULT_BLOCK_SIZE,
                    skip_patterns: tuple[str, ...] = ("head",), *, nf4_residual: bool = False,
                    nf_aware_scaling: bool = False, stochastic_rounding: bool = False, warmup_steps: int = 0,
                    use_tensor_cores: bool = False, hp_grad_weight: bool = False, error_feedback: bool = True,
                    delayed_scaling: bool = False, use_fused_kernel: bool = True, use_cuda_ext: bool = True,
                    scale_block_size: int | None = None, abd: bool = False, srr: bool = False,
                    _parent_path: str = "") -> nn.Module:
    """Swaps ``nn.Linear`` children for ``TCFPLinear`` in place, with the
    signature, defaults and traversal of tcfp/nn/__init__.py:1190-1308:

    * every child is recursed into FIRST; ``skip_patterns`` is matched against
      the child's own name only, so a ``Linear`` inside a container called
      ``head`` is still converted while a ``Linear`` named ``head`` is not;
    * a ``Linear`` whose ``in_features`` the format block size does not divide
      is left alone (:1276-1277);
    * block scaling falls back to per-tensor scaling for layers whose
      dimensions ``scale_block_size`` does not divide (:1285-1290);
    * the new layer shares the old ``Parameter`` objects and ``_param_name``
      is the dotted module path (the key of the error-feedback state and of
      ``ef_state.pt``).

    One difference, by scope: only the tensor-core path exists here.  Where
    the reference would build a fake-quantize ``TCFPLinear`` -- when
    ``use_tensor_cores`` is False (its default) or a dimension is not a
    multiple of 16 (:1279-1282) -- the ``nn.Linear`` stays as it is.
    ``nn.LayerNorm`` / ``nn.Embedding`` conversion (fake-quantize formats) is
    likewise not provided.
    """
    for name, module in list(model.named_children()):
        full_path = f"{_parent_path}.{name}" if _parent_path else name
        convert_to_tcfp(module, mode, block_size, skip_patterns, nf4_residual=nf4_residual,
                        nf_aware_scaling=nf_aware_scaling, stochastic_rounding=stochastic_rounding,
                        warmup_steps=warmup_steps, use_tensor_cores=use_tensor_cores, hp_grad_weight=hp_grad_weight,
                        error_feedback=error_feedback, delayed_scaling=delayed_scaling,
                        use_fused_kernel=use_fused_kernel, use_cuda_ext=use_cuda_ext,
                        scale_block_size=scale_block_size, abd=abd, srr=srr, _parent_path=full_path)
        if any(pat in name for pat in skip_patterns):
            continue
        if not isinstance(module, nn.Linear) or isinstance(module, TCFPLinear):
            continue
        if module.in_features % block_size != 0:
            continue
        layer_tc = use_tensor_cores and module.in_features % 16 == 0 and module.out_features % 16 == 0
        if not layer_tc:
            continue
        layer_sbs = scale_block_size
        if layer_sbs is not None and (module.in_features % layer_sbs != 0 or module.out_features % layer_sbs != 0):
            layer_sbs = None
        new = TCFPLinear(module.in_features, module.out_features, bias=module.bias is not None, mode=mode,
                         block_size=block_size, nf4_residual=nf4_residual, nf_aware_scaling=nf_aware_scaling,
                         stochastic_rounding=stochastic_rounding, warmup_steps=warmup_steps, use_tensor_cores=True,
                         hp_grad_weight=hp_grad_weight, error_feedback=error_feedback, delayed_scaling=delayed_scaling,
                         use_fused_kernel=use_fused_kernel, use_cuda_ext=use_cuda_ext, scale_block_size=layer_sbs,
                         abd=abd, srr=srr, device=module.weight.device, dtype=module.weight.dtype)
        new._param_name = full_path
        new.weight = module.weight
        if module.bias is not None:
            new.bias = module.bias
        setattr(model, name, new)
    return model
