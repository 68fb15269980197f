"""ctypes binding of ``libtcfp_b200.so`` (the C ABI in ``include/tcfp_b200.h``).

Takes the place of the reference's JIT loader ``tcfp/cuda_ext.py:155-238``:
the library is prebuilt in-tree by :mod:`tcfp_b200.build`; loading never
compiles.  There is no fallback: if the library is missing or a call fails,
the caller gets a ``RuntimeError``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int32, c_int64, c_size_t, c_uint64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libtcfp_b200.so"

F32, BF16 = 0, 1
E4M3, E5M2 = 0, 1
Q_NONE, Q_EF, Q_EF_READONLY, Q_SRR = 0, 1, 2, 3

_SIGNATURES = {
    "tcfp_version": (c_int32, []),
    "tcfp_last_error": (c_int32, [c_char_p, c_size_t]),
    "tcfp_set_sm_reserve": (c_int32, [c_int32]),
    "tcfp_check_device_status": (c_int32, [c_void_p]),
    "tcfp_selftest_bounded_wait": (c_int32, [c_uint64, c_void_p]),
    "tcfp_dual_quantize": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_uint64, c_uint64,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "tcfp_dual_quantize_workspace_bytes": (c_size_t, []),
    "tcfp_absmax": (c_int32, [c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_void_p]),
    "tcfp_quantize": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                c_int32, c_int32, c_void_p, c_void_p, c_int32, c_uint64, c_uint64, c_void_p,
                                c_void_p]),
    "tcfp_colsum_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "tcfp_quantize_colsum": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32,
                                       c_int32, c_void_p, c_void_p, c_void_p]),
    "tcfp_sf_packed_bytes": (c_size_t, [c_int64, c_int64, c_int32]),
    "tcfp_pack_scales": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p]),
    "tcfp_block_dequantize_bf16": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32,
                                             c_int32, c_void_p]),
    "tcfp_split_bf16": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "tcfp_dual_gemm": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_void_p]),
    "tcfp_dw_gemm": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64,
                               c_int64, c_void_p]),
    "tcfp_block_dual_gemm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_void_p]),
    "tcfp_block_dual_gemm_fused_act": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32,
                                                 c_void_p]),
    "tcfp_block_retarget": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int64, c_int64, c_int32, c_void_p]),
    "tcfp_block_dx_gemm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                     c_int64, c_int64, c_int64, c_int32, c_void_p]),
    "tcfp_block_dual_gemm_static": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_void_p]),
    "tcfp_static_scratch_bytes_per_operand": (c_size_t, []),
    "tcfp_bf16_dw_gemm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int64, c_void_p]),
    "tcfp_bf16_dual_gemm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64,
                                      c_int64, c_int32, c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises ``RuntimeError`` when absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tcfp_b200.build` "
                "(there is no CPU or Triton fallback)"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def is_available() -> bool:
    """True when the library loads and the current CUDA device is sm_100."""
    if not torch.cuda.is_available():
        return False
    try:
        load()
    except (RuntimeError, OSError):
        return False
    return torch.cuda.get_device_capability()[0] == 10


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    load().tcfp_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"tcfp_b200 call failed ({rc}): {last_error()}")


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


class sm_reserve:
    """Context manager: the GEMMs launched inside leave ``n`` SMs free (for a
    collective running beside them); see ``tcfp_set_sm_reserve``."""

    def __init__(self, n: int):
        self.n = int(n)

    def __enter__(self):
        self.prev = load().tcfp_set_sm_reserve(self.n) if self.n > 0 else None
        return self

    def __exit__(self, *exc):
        if self.prev is not None:
            load().tcfp_set_sm_reserve(max(self.prev, 0))
        return False


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"expected float32 or bfloat16, got {t.dtype}")


def check_device_status() -> None:
    """Synchronises and raises if a kernel gave up a bounded wait."""
    check(load().tcfp_check_device_status(stream()))


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def workspace(device: torch.device) -> torch.Tensor:
    """Small per-(device, stream) scratch for the per-tensor amax words."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream())
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(64, dtype=torch.int32, device=device)
        _workspaces[key] = ws
    return ws
