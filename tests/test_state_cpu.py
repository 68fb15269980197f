"""CPU: ``ErrorFeedbackState`` state machine (the reference's
tests/test_delayed_scaling.py:22-118 run on CPU tensors) and the ``ef_state.pt``
schema, including a file written by the reference's own checkpointer."""
from pathlib import Path

import numpy as np
import torch

from tcfp_b200.checkpoint import ef_state_dict, load_ef_state, save_ef_state
from tcfp_b200.core import ErrorFeedbackState
from tcfp_b200.nn import TCFPLinear, convert_to_tcfp

GOLD = Path(__file__).parent / "golden"


def test_delayed_amax_first_call_and_ema():
    st = ErrorFeedbackState()
    a = torch.tensor(3.14)
    assert torch.allclose(st.get_delayed_amax("w", a), a)
    st = ErrorFeedbackState()
    st.get_delayed_amax("w", torch.tensor(1.0))
    for _ in range(5000):
        r = st.get_delayed_amax("w", torch.tensor(2.0))
    assert abs(r.item() - 2.0) < 0.1
    st = ErrorFeedbackState()
    for _ in range(101):
        st.get_delayed_amax("w", torch.tensor(1.0))
    assert st.get_delayed_amax("w", torch.tensor(10.0)).item() < 2.0       # one spike is smoothed


def test_residual_prediction_and_validation_cadence():
    st = ErrorFeedbackState()
    main = torch.tensor(4.0)
    assert torch.allclose(st.predict_residual_amax("w", main), torch.tensor(0.5))     # amax / 8 fallback
    st.update_residual_ratio("w", main, torch.tensor(0.8))
    assert abs(st.predict_residual_amax("w", main).item() - 0.8) < 0.01
    st = ErrorFeedbackState(residual_validation_interval=10)
    res = [st.should_validate_residual("w") for _ in range(25)]
    assert res[0] and res[9] and res[19] and not res[1] and not res[5]
    st.get_delayed_amax("w", torch.tensor(1.0))
    st.reset()
    assert st.should_validate_residual("w") is True and not st._delayed_amax and not st._buffers


def test_error_buffer_is_lazy_fp32_and_rebinds():
    st = ErrorFeedbackState()
    like = torch.zeros(4, 8, dtype=torch.bfloat16)
    buf = st.get_error("p", like)
    assert buf.dtype == torch.float32 and buf.shape == (4, 8) and st.get_error("p", like) is buf
    assert st.get_error("p", torch.zeros(2, 8)).shape == (2, 8)          # shape change re-allocates
    new = torch.ones(2, 8)
    st.update_error("p", new)
    assert st._buffers["p"].data_ptr() == new.data_ptr()        # detached alias, no copy


def test_ef_state_schema_round_trip(tmp_path):
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32))
    convert_to_tcfp(model, skip_patterns=(), use_tensor_cores=True, delayed_scaling=True)
    l0 = model[0]
    assert isinstance(l0, TCFPLinear) and l0._param_name == "0"
    st = l0._error_state
    st._buffers["0"] = torch.randn(64, 32)
    st._delayed_amax["0.w_hi"] = torch.tensor(0.3)
    st._residual_ratio["0.ratio"] = torch.tensor(0.11)
    st._step_count["0.steps"] = 7
    snap = ef_state_dict(model)
    assert set(snap) == {"0", "2"}
    assert set(snap["0"]) == {"_buffers", "_amax_ema", "_delayed_amax", "_residual_ratio", "_step_count", "_ema_decay"}
    save_ef_state(model, tmp_path / "ef_state.pt")
    fresh = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32))
    convert_to_tcfp(fresh, skip_patterns=(), use_tensor_cores=True, delayed_scaling=True)
    load_ef_state(fresh, tmp_path / "ef_state.pt")
    f = fresh[0]._error_state
    assert torch.equal(f._buffers["0"], st._buffers["0"]) and f._step_count["0.steps"] == 7
    assert torch.equal(f._delayed_amax["0.w_hi"], torch.tensor(0.3))
    assert torch.equal(f._residual_ratio["0.ratio"], torch.tensor(0.11))


def test_loads_a_file_written_by_the_reference_checkpointer():
    """``ef_state_ref.pt`` was written by the reference's TCFPCheckpointer for
    the delayed-scaling golden layer after its two steps."""
    gold = np.load(GOLD / "per_tensor.npz")
    wrap = torch.nn.Sequential()
    layer = TCFPLinear(64, 48, use_tensor_cores=True, delayed_scaling=True)
    layer._param_name = "layer"
    wrap.add_module("layer", layer)
    load_ef_state(wrap, GOLD / "ef_state_ref.pt")
    st = layer._error_state
    bits = lambda t: t.float().contiguous().view(torch.int32).numpy()  # noqa: E731
    assert np.array_equal(bits(st._buffers["layer"]), gold["layer/delayed/step1/ef"])
    assert np.array_equal(bits(st._delayed_amax["layer.w_hi"].reshape(1)), gold["layer/delayed/step1/delayed/layer.w_hi"])
    assert np.array_equal(bits(st._residual_ratio["layer.ratio"].reshape(1)), gold["layer/delayed/step1/ratio/layer.ratio"])
    assert st._step_count["layer.steps"] == 2


def test_srr_stream_position_is_checkpointed(tmp_path):
    m = torch.nn.Sequential(TCFPLinear(32, 32, use_tensor_cores=True, srr=True, srr_seed=5))
    m[0]._srr_offset = 4096
    save_ef_state(m, tmp_path / "s.pt")
    n = torch.nn.Sequential(TCFPLinear(32, 32, use_tensor_cores=True, srr=True, srr_seed=9))
    load_ef_state(n, tmp_path / "s.pt")
    assert n[0].srr_seed == 5 and n[0]._srr_offset == 4096


def test_state_machine_is_bit_identical_to_the_reference_class():
    """Differential run against the reference's own ``ErrorFeedbackState``
    when its checkout is available (it is where the goldens are generated;
    it is not on the GPU box, where this test skips)."""
    import importlib.util
    import random
    import sys

    import pytest

    import os

    # a checkout named "reference" next to this repository, or wherever TCFP_REFERENCE_ROOT points
    ref_root = Path(os.environ.get("TCFP_REFERENCE_ROOT", Path(__file__).resolve().parents[2] / "reference"))
    if not (ref_root / "tcfp" / "core.py").exists():
        pytest.skip("reference checkout not present")
    spec = importlib.util.spec_from_file_location("_ref_tcfp_core", ref_root / "tcfp" / "core.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    r, o = mod.ErrorFeedbackState(residual_validation_interval=7), ErrorFeedbackState(residual_validation_interval=7)
    torch.manual_seed(0)
    random.seed(0)
    for i in range(200):
        a = torch.rand(()) * 3 + 0.01
        b = torch.rand(()) * 0.5 + 0.001
        for name in ("x", "y"):
            assert torch.equal(r.get_delayed_amax(name + ".w_hi", a), o.get_delayed_amax(name + ".w_hi", a))
            assert torch.equal(r.get_amax_ema(name, a), o.get_amax_ema(name, a))
            assert torch.equal(r.predict_residual_amax(name, a), o.predict_residual_amax(name, a))
            assert r.should_validate_residual(name) == o.should_validate_residual(name)
            if i % 3 == 0:
                r.update_residual_ratio(name, a, b)
                o.update_residual_ratio(name, a, b)
    for table in ("_amax_ema", "_delayed_amax", "_residual_ratio"):
        d1, d2 = getattr(r, table), getattr(o, table)
        assert d1.keys() == d2.keys() and all(torch.equal(d1[k], d2[k]) for k in d1)
    assert r._step_count == o._step_count


def _nested_model():
    nn = torch.nn

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = nn.Linear(64, 128)
            self.odd = nn.Linear(48, 64)            # 48 % 32 != 0 -> format block size skip
            self.tiny = nn.Linear(64, 24)           # out_features % 16 != 0 -> no tensor-core layer
            self.head = nn.Linear(64, 64)           # own name matches the skip pattern

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([Block(), Block()])
            self.head = nn.Sequential(nn.Linear(128, 64), nn.ReLU(), nn.Linear(64, 128, bias=False))
            self.out_head = nn.Linear(64, 64)
            self.narrow = nn.Linear(96, 64)          # 96 % 64 != 0 -> per-tensor fallback of block scaling

    return Net()


def test_convert_to_tcfp_signature_and_traversal_match_the_reference():
    """Same positional order, defaults and converted-module set as
    tcfp/nn/__init__.py:1190-1308, checked against the reference function
    itself when ``oracle/_ref`` holds it (differential), and against the
    written-down expectation otherwise."""
    import inspect
    import warnings

    from oracle import ref_loader

    sig = inspect.signature(convert_to_tcfp)
    names = list(sig.parameters)
    assert names[:4] == ["model", "mode", "block_size", "skip_patterns"]
    assert sig.parameters["skip_patterns"].kind is inspect.Parameter.POSITIONAL_OR_KEYWORD
    assert sig.parameters["use_tensor_cores"].default is False
    for kw in ("nf4_residual", "nf_aware_scaling", "stochastic_rounding", "use_fused_kernel", "use_cuda_ext",
               "_parent_path"):
        assert sig.parameters[kw].kind is inspect.Parameter.KEYWORD_ONLY

    from tcfp_b200.core import TCFPMode

    ours = _nested_model()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        convert_to_tcfp(ours, TCFPMode.TCFP12, 32, ("head",), use_tensor_cores=True, scale_block_size=64,
                        use_fused_kernel=True, use_cuda_ext=True, nf4_residual=False)
    mine = {n: (m.scale_block_size, m._param_name) for n, m in ours.named_modules() if isinstance(m, TCFPLinear)}
    # a Linear inside the container called "head" IS converted; Linears named "...head" are not
    assert set(mine) == {"blocks.0.proj", "blocks.1.proj", "head.0", "head.2", "narrow"}
    assert all(v[1] == k for k, v in mine.items())
    assert mine["narrow"][0] is None and mine["head.0"][0] == 64
    assert ours.head[2].bias is None and isinstance(ours.blocks[0].odd, torch.nn.Linear)

    # default call converts nothing here (use_tensor_cores defaults to False: fake-quantize is not provided)
    plain = _nested_model()
    convert_to_tcfp(plain)
    assert not any(isinstance(m, TCFPLinear) for m in plain.modules())

    if not ref_loader.available():
        return
    ref = ref_loader.load_reference()
    try:
        theirs = _nested_model()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            ref.nn.convert_to_tcfp(theirs, ref.core.TCFPMode.TCFP12, 32, ("head",), use_tensor_cores=True,
                                   scale_block_size=64)
        got = {n: (m.scale_block_size, m._param_name) for n, m in theirs.named_modules()
               if isinstance(m, ref.nn.TCFPLinear) and m.use_tensor_cores}
        assert got == mine
        ref_sig = inspect.signature(ref.nn.convert_to_tcfp)
        assert list(ref_sig.parameters) == names
        for n in names[1:]:
            assert ref_sig.parameters[n].default == sig.parameters[n].default or n == "mode"
            assert ref_sig.parameters[n].kind == sig.parameters[n].kind
    finally:
        ref_loader.unload()


def test_reference_checkpointer_loads_a_file_written_here(tmp_path):
    """The other direction of the schema check: ``ef_state.pt`` written by
    ``save_ef_state`` is restored by the reference's own
    ``TCFPCheckpointer._load_ef_state`` (tcfp/training/checkpointing.py:225-271)
    into the reference's own layers.  Needs ``oracle/_ref``; skips without it."""
    import pytest

    from oracle import ref_loader

    if not ref_loader.available():
        pytest.skip("oracle/_ref not built")
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32))
    convert_to_tcfp(model, skip_patterns=(), use_tensor_cores=True, delayed_scaling=True)
    for i, name in ((0, "0"), (2, "2")):
        st = model[i]._error_state
        st._buffers[name] = torch.randn(model[i].weight.shape)
        st._amax_ema[name] = torch.tensor(0.5 + i)
        st._delayed_amax[name + ".w_hi"] = torch.tensor(0.3 + i)
        st._residual_ratio[name + ".ratio"] = torch.tensor(0.11 + i)
        st._step_count[name + ".steps"] = 7 + i
    save_ef_state(model, tmp_path / "ef_state.pt")
    ref = ref_loader.load_reference()
    try:
        from tcfp.training.checkpointing import TCFPCheckpointer

        theirs = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32))
        ref.nn.convert_to_tcfp(theirs, skip_patterns=(), use_tensor_cores=True, delayed_scaling=True)
        TCFPCheckpointer(tmp_path / "ckpts")._load_ef_state(tmp_path, theirs)
        for i, name in ((0, "0"), (2, "2")):
            a, b = model[i]._error_state, theirs[i]._error_state
            for table in ("_buffers", "_amax_ema", "_delayed_amax", "_residual_ratio"):
                da, db = getattr(a, table), getattr(b, table)
                assert da.keys() == db.keys() and all(torch.equal(da[k], db[k]) for k in da)
            assert a._step_count == b._step_count and a._ema_decay == b._ema_decay
    finally:
        ref_loader.unload()
