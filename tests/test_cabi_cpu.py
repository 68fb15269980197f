"""CPU: the C-ABI library loads and exports every symbol the header declares;
argument validation that needs no GPU returns the documented status codes."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from tcfp_b200 import _C, build

    build.build()
    return _C.load()


def test_every_declared_symbol_is_exported(lib):
    from tcfp_b200 import _C

    header = (ROOT / "include" / "tcfp_b200.h").read_text()
    declared = set(re.findall(r"\b(tcfp_[a-z0-9_]+)\s*\(", header))
    declared -= {"tcfp_dtype", "tcfp_fp8", "tcfp_qmode"}
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/tcfp_b200.h but not exported"
    assert declared == set(_C.EXPORTED_SYMBOLS), declared ^ set(_C.EXPORTED_SYMBOLS)


def test_version_and_error_text(lib):
    from tcfp_b200 import _C

    assert lib.tcfp_version() >= 100
    rc = lib.tcfp_dual_quantize(None, 0, None, None, None, None, None, None, None, 8, 8, 32, 0, 0, 0, None, None, None,
                                None, None)
    assert rc == -1 and "NULL" in _C.last_error()
    assert lib.tcfp_sf_packed_bytes(8192, 8192, 32) == 2 << 20
    assert lib.tcfp_sf_packed_bytes(100, 96, 32) == 512
    assert lib.tcfp_dual_quantize_workspace_bytes() == 256
    buf = ctypes.create_string_buffer(8)
    assert lib.tcfp_last_error(buf, 8) == 0 and len(buf.value) <= 7


def test_product_path_has_no_cpu_fallback():
    import torch

    from tcfp_b200.core import to_fp8_e4m3
    from tcfp_b200.nn import TCFPLinear

    with pytest.raises(RuntimeError, match="CUDA"):
        to_fp8_e4m3(torch.randn(4, 4))
    layer = TCFPLinear(16, 16, use_tensor_cores=True)
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(torch.randn(2, 16))
    with pytest.raises(NotImplementedError):
        TCFPLinear(16, 16)(torch.randn(2, 16))
