"""Error-feedback state I/O in the reference's ``ef_state.pt`` schema
(tcfp/training/checkpointing.py:200-271): a dict keyed by each layer's
``_param_name`` (or its module path when that is empty) holding the five
``ErrorFeedbackState`` dictionaries with tensors on CPU.  Files written by the
reference's ``TCFPCheckpointer`` load here and vice versa.  SRR layers carry no
error state; their stream position ``(srr_seed, _srr_offset)`` is stored under
the additional key ``"_srr"`` which the reference ignores.

The reference copies every tensor to the host with a blocking ``.cpu()``
(checkpointing.py:216-221): one synchronising pageable transfer per tensor,
with training stopped for all of them -- 3.2 GB of FP32 buffers for the
7B-shaped 4-layer stack.  Here a snapshot is taken in two steps that keep the
training stream moving: the device tensors are cloned on the device (a few
milliseconds; the next step's quantizer overwrites the buffers in place, so
the copy must not read them later), then the clones travel to pinned host
memory on a side stream while training continues.  ``snapshot_ef_state_async``
returns at once; ``save_ef_state_async`` also writes the file from a
background thread.  ``ef_state_dict`` / ``save_ef_state`` are the blocking
forms of the same path (one wait for everything instead of one per tensor)."""
from __future__ import annotations

import threading
from pathlib import Path

import torch
import torch.nn as nn

from .nn import TCFPLinear

_TENSOR_TABLES = ("_buffers", "_amax_ema", "_delayed_amax", "_residual_ratio")


def _key(mod_name: str, module: TCFPLinear) -> str:
    return module._param_name if module._param_name else mod_name


class EFSnapshot:
    """A snapshot in flight.  ``wait()`` blocks the calling host thread until
    the device-to-host copies have landed and returns the ``ef_state.pt``
    dict; the training stream is never made to wait."""

    def __init__(self, snap: dict[str, object], event):
        self._snap = snap
        self._event = event

    def done(self) -> bool:
        return self._event is None or self._event.query()

    def wait(self) -> dict[str, object]:
        if self._event is not None:
            self._event.synchronize()
            self._event = None
        return self._snap


def snapshot_ef_state_async(model: nn.Module, *, pin_memory: bool = True) -> EFSnapshot:
    """Starts a snapshot of every layer's error-feedback state as of the work
    queued so far on the current stream and returns without waiting."""
    snap: dict[str, object] = {}
    jobs: list[tuple[dict, str, torch.Tensor]] = []
    for mod_name, module in model.named_modules():
        if not isinstance(module, TCFPLinear):
            continue
        ef = module._error_state
        if ef is None:
            if module.srr:
                snap[_key(mod_name, module)] = {"_srr": {"seed": module.srr_seed, "offset": module._srr_offset}}
            continue
        entry: dict[str, object] = {t: {} for t in _TENSOR_TABLES}
        for table in _TENSOR_TABLES:
            for k, v in getattr(ef, table).items():
                if v.is_cuda:
                    jobs.append((entry[table], k, v))
                else:
                    entry[table][k] = v.detach().clone()
        entry["_step_count"] = dict(ef._step_count)
        entry["_ema_decay"] = ef._ema_decay
        snap[_key(mod_name, module)] = entry
    if not jobs:
        return EFSnapshot(snap, None)
    dev = jobs[0][2].device
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream()
        # 1. device-side clones on the training stream: consistent with everything queued before this call
        clones = [(dst, k, v.detach().clone()) for dst, k, v in jobs]
        ready = torch.cuda.Event()
        ready.record(main)
        # 2. clones -> pinned host memory on a side stream; training goes on underneath
        side = torch.cuda.Stream()
        side.wait_event(ready)
        with torch.cuda.stream(side):
            for dst, k, c in clones:
                host = torch.empty(c.shape, dtype=c.dtype, device="cpu", pin_memory=pin_memory)
                host.copy_(c, non_blocking=True)
                c.record_stream(side)
                dst[k] = host
            done = torch.cuda.Event()
            done.record(side)
    return EFSnapshot(snap, done)


def ef_state_dict(model: nn.Module) -> dict[str, object]:
    """The ``ef_state.pt`` dict with all tensors on the host (blocking)."""
    return snapshot_ef_state_async(model).wait()


def save_ef_state(model: nn.Module, path: str | Path) -> None:
    torch.save(ef_state_dict(model), path)


def save_ef_state_async(model: nn.Module, path: str | Path) -> threading.Thread:
    """Snapshot now, write ``path`` from a background thread once the copies
    have landed.  Returns the thread; ``join()`` it before relying on the file."""
    pending = snapshot_ef_state_async(model)

    def _write():
        torch.save(pending.wait(), path)

    t = threading.Thread(target=_write, name="tcfp-ef-save", daemon=False)
    t.start()
    return t


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
