"""Installs the UNMODIFIED reference into ``oracle/_ref/`` (git-ignored) so that
GPU tests and the benchmark's reference arm can run the reference's own
kernels beside this library's on the same device.  Test infrastructure only:
nothing in the ``tcfp_b200`` package imports anything from ``oracle/``.

    python -m oracle.build_ref [--reference /path/to/tcfp-checkout] [--force]

Two artefacts, both built from the reference checkout where it lies:

* ``oracle/_ref/tcfp/`` -- ``pip install --no-deps --target`` of the reference
  package (its Triton kernels, ``tcfp.nn``, ``tcfp.core``), installed from a
  temporary copy because the checkout is read-only;
* ``oracle/_ref/tcfp_fused_dual_gemm.so`` -- the reference's cuBLASLt
  extension (tcfp/csrc/fused_dual_gemm.cu, fused_dual_gemm_bind.cpp) compiled
  for sm_100a with the flags of its own JIT loader (tcfp/cuda_ext.py:185-226).
  The loader itself looks for the sources beside the installed package, where
  the wheel does not put them, so ``oracle.ref_loader`` hands it this module.

Without a reference checkout the script leaves whatever is already in
``oracle/_ref/`` alone and returns; the consumers skip when it is empty.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref"
DEFAULT_REFERENCE = HERE.parent.parent / "reference"


def _install_package(reference: Path) -> None:
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "src"
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns(".git", "__pycache__"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--upgrade", "--target", str(REF_OUT), str(src)]
        wheelhouse = Path("/opt/wheelhouse")
        if wheelhouse.exists():
            cmd[5:5] = ["--find-links", str(wheelhouse)]
        subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def _build_extension(reference: Path) -> None:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load

    csrc = reference / "tcfp" / "csrc"
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    with tempfile.TemporaryDirectory() as tmp:
        load(name="tcfp_fused_dual_gemm",
             sources=[str(csrc / "fused_dual_gemm.cu"), str(csrc / "fused_dual_gemm_bind.cpp")],
             extra_cflags=["-O3"], extra_cuda_cflags=["-O3"], extra_ldflags=["-lcublasLt"],
             extra_include_paths=[str(csrc), str(Path(cuda_home) / "include")],
             build_directory=tmp, verbose=False, is_python_module=False)
        shutil.copy2(Path(tmp) / "tcfp_fused_dual_gemm.so", REF_OUT / "tcfp_fused_dual_gemm.so")


def build(reference: Path = DEFAULT_REFERENCE, force: bool = False) -> bool:
    """Returns True when ``oracle/_ref`` holds the reference afterwards."""
    have_pkg = (REF_OUT / "tcfp" / "kernels.py").exists()
    have_ext = (REF_OUT / "tcfp_fused_dual_gemm.so").exists()
    if not (reference / "tcfp" / "kernels.py").exists():
        return have_pkg
    REF_OUT.mkdir(exist_ok=True)
    if force or not have_pkg:
        _install_package(reference)
    if force or not have_ext:
        try:
            _build_extension(reference)
        except Exception as exc:  # the Triton kernels are still usable without the extension
            print(f"reference cuBLASLt extension not built: {exc!r}"[:400], file=sys.stderr)
    return (REF_OUT / "tcfp" / "kernels.py").exists()


if __name__ == "__main__":
    ref = DEFAULT_REFERENCE
    if "--reference" in sys.argv:
        ref = Path(sys.argv[sys.argv.index("--reference") + 1])
    ok = build(ref, force="--force" in sys.argv)
    print(f"{REF_OUT}: {'ready' if ok else 'absent'}")
