"""Generates ``tests/golden/per_tensor.npz`` by running the REFERENCE itself
on CPU (``PYTHONPATH=<reference root>``) on small seeded inputs.

    python tests/golden/make_golden.py /path/to/reference

What is recorded (all as raw bits: uint8 codes, int32 views of float32):
  * to_fp8_e4m3 / to_fp8_e5m2 on float32 and bfloat16 inputs (tcfp/core.py:85-158)
  * stochastic_round_to_fp8_e4m3 with ``torch.rand_like`` patched to return
    the Philox contract uniforms (tcfp/core.py:418-464)
  * two consecutive training steps of TCFPLinear(use_tensor_cores=True,
    use_fused_kernel=False, use_cuda_ext=False) in the error-feedback,
    SRR and delayed-scaling configurations: outputs, input/weight gradients,
    and the error-feedback / delayed-amax state after each step
    (tcfp/nn/__init__.py:312-566, 769-1041)
The inputs are regenerated from the seeds by the tests; only outputs are
stored.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <path to a checkout of the reference project>")
ref_root = sys.argv[1]
sys.path.append(ref_root)  # after the repo root: both trees have a ``tests`` package

import tcfp.core as rcore  # noqa: E402
import tcfp.nn as rnn  # noqa: E402

from oracle import tcfp_oracle as O  # noqa: E402
from tests.golden.cases import CAST_CASES, LAYER_CASES, layer_inputs, cast_input  # noqa: E402

out: dict[str, np.ndarray] = {}


def u8(t):
    return t.detach().contiguous().view(torch.uint8).numpy().copy()


def i32(t):
    return t.detach().float().contiguous().view(torch.int32).numpy().copy()


for name, (seed, shape, dtype) in CAST_CASES.items():
    x = cast_input(seed, shape, dtype)
    q, inv = rcore.to_fp8_e4m3(x)
    out[f"cast/{name}/e4m3"], out[f"cast/{name}/e4m3_inv"] = u8(q), i32(inv)
    q, inv = rcore.to_fp8_e5m2(x)
    out[f"cast/{name}/e5m2"], out[f"cast/{name}/e5m2_inv"] = u8(q), i32(inv)
    q, inv = rcore.to_fp8_e4m3_nf_aware(x)
    out[f"cast/{name}/nf_aware"], out[f"cast/{name}/nf_aware_inv"] = u8(q), i32(inv)
    # stochastic rounding under the seed/offset contract
    scaled = (x.float() * (448.0 / x.float().abs().max())).clamp(-448, 448)
    rand = O.philox_uniform_packed(seed, 17, scaled.numel()).reshape(scaled.shape)
    orig = torch.rand_like
    rcore.torch.rand_like = lambda t, *a, **k: rand.to(t.dtype)
    try:
        out[f"cast/{name}/sr"] = u8(rcore.stochastic_round_to_fp8_e4m3(scaled))
    finally:
        rcore.torch.rand_like = orig


class _PatchedRand:
    """Feeds the reference's ``torch.rand_like`` the contract uniforms:
    call ``i`` of a step draws elements ``offset_i + element`` of the packed per-tensor stream."""

    def __init__(self, seed):
        self.seed = seed
        self.offset = 0

    def __call__(self, t, *a, **k):
        r = O.philox_uniform_packed(self.seed, self.offset, t.numel()).reshape(t.shape).to(t.dtype)
        self.offset += t.numel()
        return r


for name, cfg in LAYER_CASES.items():
    x, w, b, target = layer_inputs(cfg)
    layer = rnn.TCFPLinear(cfg["K"], cfg["N"], bias=cfg["bias"], use_tensor_cores=True, use_fused_kernel=False,
                           use_cuda_ext=False, srr=cfg.get("srr", False), abd=cfg.get("abd", False),
                           delayed_scaling=cfg.get("delayed", False), hp_grad_weight=cfg.get("hp", False),
                           nf_aware_scaling=cfg.get("nf", False))
    layer._param_name = "layer"
    with torch.no_grad():
        layer.weight.copy_(w)
        if b is not None:
            layer.bias.copy_(b)
    patched = _PatchedRand(cfg["seed"])
    orig = torch.rand_like
    rcore.torch.rand_like = patched
    try:
        for step in range(2):
            xin = x.clone().requires_grad_(True)
            y = layer(xin)
            loss = ((y - target) ** 2).mean()
            layer.zero_grad()
            loss.backward()
            out[f"layer/{name}/step{step}/y"] = i32(y)
            out[f"layer/{name}/step{step}/dx"] = i32(xin.grad)
            out[f"layer/{name}/step{step}/dw"] = i32(layer.weight.grad)
            if b is not None:
                out[f"layer/{name}/step{step}/db"] = i32(layer.bias.grad)
            st = layer._error_state
            if st is not None:
                out[f"layer/{name}/step{step}/ef"] = i32(st._buffers["layer"])
                for k, v in st._delayed_amax.items():
                    out[f"layer/{name}/step{step}/delayed/{k}"] = i32(v.reshape(1))
                for k, v in st._residual_ratio.items():
                    out[f"layer/{name}/step{step}/ratio/{k}"] = i32(v.reshape(1))
            with torch.no_grad():
                layer.weight -= 0.05 * layer.weight.grad      # plain SGD keeps the fixture self-contained
    finally:
        rcore.torch.rand_like = orig
    if name == "delayed":
        layer_for_ckpt = layer

# ef_state.pt as the reference's own checkpointer writes it, for the delayed-scaling layer after two steps
import tempfile  # noqa: E402

from tcfp.training.checkpointing import TCFPCheckpointer  # noqa: E402

wrap = torch.nn.Sequential()
wrap.add_module("layer", layer_for_ckpt)
with tempfile.TemporaryDirectory() as td:
    ck = TCFPCheckpointer(td)
    ck._save_ef_state(Path(td), wrap)
    (HERE / "ef_state_ref.pt").write_bytes((Path(td) / "ef_state.pt").read_bytes())

np.savez_compressed(HERE / "per_tensor.npz", **out)
print("wrote", HERE / "per_tensor.npz", len(out), "arrays",
      sum(v.nbytes for v in out.values()) // 1024, "KiB raw")
