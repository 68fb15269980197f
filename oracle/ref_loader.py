"""Imports the reference package installed by ``oracle.build_ref`` from
``oracle/_ref`` -- as it is, or with its two kernel modules swapped for this
library's drop-in modules.  Test infrastructure only (tests, the benchmark's
reference arm); the ``tcfp_b200`` package never imports it.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
from pathlib import Path

REF_OUT = Path(__file__).resolve().parent / "_ref"


def available() -> bool:
    return (REF_OUT / "tcfp" / "kernels.py").exists()


def _purge() -> None:
    for name in [n for n in sys.modules if n == "tcfp" or n.startswith("tcfp.")]:
        del sys.modules[name]


def _on_path() -> None:
    p = str(REF_OUT)
    if p not in sys.path:
        sys.path.insert(0, p)


def load_reference():
    """The reference's ``tcfp`` package, unmodified, with its own Triton
    kernels.  If the prebuilt cuBLASLt extension is present it is handed to
    the reference's loader (tcfp/cuda_ext.py:155-238 would JIT-compile the same
    two sources; the installed wheel does not carry them)."""
    if not available():
        raise RuntimeError("oracle/_ref is empty: run `python -m oracle.build_ref` where the reference checkout is")
    _purge()
    _on_path()
    os.environ.setdefault("CUDA_HOME", "/usr/local/cuda")
    import tcfp.cuda_ext as ce          # import the leaf first: tcfp/__init__ pulls in tcfp.nn, which probes it

    ext = load_reference_extension()
    if ext is not None:
        ce._cuda_ext = ext
        ce._load_attempted = True
    # tcfp.nn cached its availability flags at import time (tcfp/nn/__init__.py:53, 64)
    import tcfp.nn as rnn

    rnn._HAS_CUDA_EXT = ce.is_cuda_ext_available()
    return importlib.import_module("tcfp")


def load_reference_extension():
    """The reference's pybind11 module ``tcfp_fused_dual_gemm`` (``forward``,
    ``backward_dx``; tcfp/csrc/fused_dual_gemm_bind.cpp:6-16), or ``None``."""
    so = REF_OUT / "tcfp_fused_dual_gemm.so"
    if not so.exists():
        return None
    import torch  # noqa: F401  (the module links against libtorch)

    spec = importlib.util.spec_from_file_location("tcfp_fused_dual_gemm", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_reference_on_b200_kernels():
    """The reference's ``tcfp`` package with ``tcfp.kernels`` and
    ``tcfp.cuda_ext`` replaced by ``tcfp_b200.kernels`` / ``tcfp_b200.cuda_ext``
    before anything imports them: the reference's own ``tcfp.nn`` layers and
    autograd Functions then run on this library's kernels."""
    if not available():
        raise RuntimeError("oracle/_ref is empty: run `python -m oracle.build_ref` where the reference checkout is")
    import tcfp_b200.cuda_ext
    import tcfp_b200.kernels

    _purge()
    _on_path()
    sys.modules["tcfp.kernels"] = tcfp_b200.kernels
    sys.modules["tcfp.cuda_ext"] = tcfp_b200.cuda_ext
    return importlib.import_module("tcfp")


def unload() -> None:
    _purge()
