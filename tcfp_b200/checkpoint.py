"""Error-feedback state I/O in the reference's ``ef_state.pt`` schema
(tcfp/training/checkpointing.py:200-271): a dict keyed by each layer's
``_param_name`` (or its module path when that is empty) holding the five
``ErrorFeedbackState`` dictionaries with tensors on CPU.  Files written by the
reference's ``TCFPCheckpointer`` load here and vice versa.  SRR layers carry no
error state; their stream position ``(srr_seed, _srr_offset)`` is stored under
the additional key ``"_srr"`` which the reference ignores."""
from __future__ import annotations

from pathlib import Path

import torch
import torch.nn as nn

from .nn import TCFPLinear


def _key(mod_name: str, module: TCFPLinear) -> str:
    return module._param_name if module._param_name else mod_name


def ef_state_dict(model: nn.Module) -> dict[str, object]:
    snap: dict[str, object] = {}
    for mod_name, module in model.named_modules():
        if not isinstance(module, TCFPLinear):
            continue
        ef = module._error_state
        if ef is None:
            if module.srr:
                snap[_key(mod_name, module)] = {"_srr": {"seed": module.srr_seed, "offset": module._srr_offset}}
            continue
        snap[_key(mod_name, module)] = {
            "_buffers": {k: v.cpu() for k, v in ef._buffers.items()},
            "_amax_ema": {k: v.cpu() for k, v in ef._amax_ema.items()},
            "_delayed_amax": {k: v.cpu() for k, v in ef._delayed_amax.items()},
            "_residual_ratio": {k: v.cpu() for k, v in ef._residual_ratio.items()},
            "_step_count": dict(ef._step_count),
            "_ema_decay": ef._ema_decay,
        }
    return snap


def save_ef_state(model: nn.Module, path: str | Path) -> None:
    torch.save(ef_state_dict(model), path)


def load_ef_state(model: nn.Module, path: str | Path) -> None:
    snap = torch.load(path, weights_only=False)
    layers = {_key(n, m): m for n, m in model.named_modules() if isinstance(m, TCFPLinear)}
    for outer, state in snap.items():
        module = layers.get(str(outer))
        if module is None or not isinstance(state, dict):
            continue
        if "_srr" in state and module.srr:
            module.srr_seed = int(state["_srr"]["seed"])
            module._srr_offset = int(state["_srr"]["offset"])
        ef = module._error_state
        if ef is None:
            continue
        dev = module.weight.device
        ef._buffers.update({k: v.to(dev) for k, v in state.get("_buffers", {}).items()})
        ef._amax_ema.update({k: v.to(dev) for k, v in state.get("_amax_ema", {}).items()})
        ef._delayed_amax.update({k: v.to(dev) for k, v in state.get("_delayed_amax", {}).items()})
        ef._residual_ratio.update({k: v.to(dev) for k, v in state.get("_residual_ratio", {}).items()})
        ef._step_count.update(state.get("_step_count", {}))
        if state.get("_ema_decay") is not None:
            ef._ema_decay = float(state["_ema_decay"])
