"""Benchmark of the TCFP-12 hot path: block-scaled dual-FP8 GEMM at 8192^3.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gemm|mlp|mlp_large|decoder] [--sp] [--no-extras] [--kernel-table]

One "step" is one forward pass of the hot path over one batch: the fused
block-scaled dual GEMM  out = X_q . W_hi^T + X_q . W_lo^T  (both products
counted: 4*M*N*K FLOP) on operands already quantized and resident in HBM.
``e2e`` times the layer call a user makes, starting from a pinned HOST
activation buffer: H2D copy, weight dual-quantize (error feedback), activation
block-quantize, dual GEMM, D2H copy of the FP32 output.

Under torchrun (N > 1) ``value`` is N independent column shards of a layer
whose output width is N*8192 (no data-path collective: it shows that the GEMM
path itself does not degrade, nothing about tensor-parallel scaling).  The
tensor-parallel TRAINING steps, with their NCCL collectives inside the timed
region, are reported in every line under ``extra``: ``mlp_train_step``
(configuration 0), ``mlp_large_train_step`` (configuration 3) and
``decoder_train_step`` (configuration 4), each with the step time, the time
the same step takes with the collectives switched off, and the difference.

``--impl reference`` times the CPU form of the reference's block-scaled path
(its kernels are Triton and need a GPU) on all host cores, whole 8192-row
passes; when a GPU and ``oracle/_ref`` are present it also reports, under
``reference_gpu``, the reference's own GPU kernels on the same operands.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N = K = 8192
BS = 64
FLOP_PER_STEP = 4.0 * M * N * K
WORKLOAD = "block-scaled TCFP-12 dual GEMM forward, M=N=K=8192, block 64 (benchmark configuration 2)"
PROFILE = ROOT / "profiles" / "dual_gemm_pair_mxf8_8192_bench.md"
E2E_CHUNKS = 16     # row chunks of the host-streamed layer call: the first download starts after 1/16 of the work


def _config(world: int) -> dict:
    return {"workload": WORKLOAD,
            "l2": "operands + output = 448 MB per step, larger than the 126 MB L2",
            "parallelism": f"column-parallel shards x{world}, no collective" if world > 1 else "single GPU"}


def _peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm": float(d["hbm_gbs"]), "src": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "src": "fallback"}


def _profiled_traffic():
    """DRAM bytes per launch of the benchmark's kernel, from the kept ncu
    summary (rows ``| launch | duration | clock | tensor % | read MB | write MB |``)."""
    try:
        rows = re.findall(r"^\|\s*\d+\s*\|.*?\|\s*([\d.]+)\s*MB\s*\|\s*([\d.]+)\s*MB\s*\|\s*$", PROFILE.read_text(), re.M)
        if rows:
            return sum(float(r) + float(w) for r, w in rows) / len(rows) * 1e6, str(PROFILE.relative_to(ROOT))
    except OSError:
        pass
    return None, None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) in a
    background thread while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index = index
        self.period = period_s
        self.sm: list[int] = []
        self.reasons_seen = 0
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nv = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                if nv is not None:
                    self.sm.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                    self.reasons_seen |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                else:
                    out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits",
                                          "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                    a, b = (int(v) for v in out.strip().splitlines()[0].split(","))
                    self.sm.append(a)
                    self.sm_max = b
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm = sorted(self.sm)
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        reasons = [n for bit, n in names.items() if self.reasons_seen & bit]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_mhz_min": sm[0] if sm else None,
                "sm_max_mhz": self.sm_max, "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's block path
# ---------------------------------------------------------------------------

def _cpu_operands():
    import torch

    from oracle import tcfp_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1003)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g) * 0.02
    a, ea = O.block_quantize(x, BS)
    hi, lo, eh, el, _ = O.dual_quantize_block(w, BS)
    return O, cores, (a, ea, hi, eh, lo, el)


def _cpu_passes(passes: int, warmup: int):
    """Whole passes of the workload on the host: dequantize + FP32 dual matmul
    over all 8192 activation rows.  Returns (TFLOP/s from the mean pass,
    cores, list of pass seconds)."""
    O, cores, (a, ea, hi, eh, lo, el) = _cpu_operands()
    for _ in range(warmup):
        O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, BS)
    times = []
    for _ in range(passes):
        t0 = time.perf_counter()
        O.block_dual_gemm_nt(a, ea, hi, eh, lo, el, BS)
        times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return FLOP_PER_STEP / mean / 1e12, cores, times


# ---------------------------------------------------------------------------
# the reference's own GPU kernels, same box, same operands
# ---------------------------------------------------------------------------

def _reference_gpu(dev, a, s_a, w_hi, w_lo, s_hi, s_lo, x, w, ours_ms: float | None) -> dict:
    """Times the reference's GPU paths for this step on the operands the
    benchmark uses: its Triton block-scaled dual GEMM (tcfp/kernels.py:
    1939-2028), its per-tensor fallback of two ``torch._scaled_mm`` plus an
    add (tcfp/nn/__init__.py:405-421), its cuBLASLt extension
    (tcfp/csrc/fused_dual_gemm.cu) and its Triton per-tensor kernel."""
    import torch

    from oracle import ref_loader

    if not ref_loader.available():
        return {"unavailable": "oracle/_ref not built (python -m oracle.build_ref needs the reference checkout)"}
    out: dict = {"operands": "the benchmark's own quantized operands, 8192^3; CUDA events, 5 launches after warm-up"}

    def t(fn, n=5, warm=2):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    try:
        ref_loader.load_reference()
        import tcfp.cuda_ext as rc
        import tcfp.kernels as rk

        def entry(ms):
            return {"ms": ms, "tflops": FLOP_PER_STEP / ms / 1e9}

        if rk.is_triton_available():
            y = rk.fused_block_scaled_dual_gemm_forward(a, w_hi, w_lo, s_a, s_hi, s_lo, BS)   # autotunes on first call
            del y
            out["triton_block_scaled_dual_gemm_bs64"] = entry(t(lambda: rk.fused_block_scaled_dual_gemm_forward(
                a, w_hi, w_lo, s_a, s_hi, s_lo, BS)))
        # per-tensor comparators on per-tensor operands of the same tensors
        from tcfp_b200.core import dual_quantize_per_tensor, to_fp8_e4m3
        from tcfp_b200.kernels import fused_dual_gemm_forward

        p_hi, p_lo, i_hi, i_lo, _ = dual_quantize_per_tensor(w)
        p_a, i_a = to_fp8_e4m3(x)

        def two_scaled_mm():
            y = torch._scaled_mm(p_a, p_hi.t(), scale_a=i_a, scale_b=i_hi, out_dtype=torch.float32)
            y += torch._scaled_mm(p_a, p_lo.t(), scale_a=i_a, scale_b=i_lo, out_dtype=torch.float32)
            return y

        out["two_scaled_mm_plus_add_per_tensor"] = entry(t(two_scaled_mm))
        if rk.is_triton_available():
            rk.fused_dual_gemm_forward(p_a, p_hi, p_lo, i_a, i_hi, i_lo)
            out["triton_per_tensor_dual_gemm"] = entry(t(lambda: rk.fused_dual_gemm_forward(p_a, p_hi, p_lo, i_a, i_hi, i_lo)))
        if rc.is_cuda_ext_available():
            out["cublaslt_ext_per_tensor"] = entry(t(lambda: rc.cuda_ext_dual_gemm_forward(p_a, p_hi, p_lo, i_a, i_hi, i_lo)))
        out["ours_per_tensor_dual_gemm"] = entry(t(lambda: fused_dual_gemm_forward(p_a, p_hi, p_lo, i_a, i_hi, i_lo)))
        # the small-N case the reference fuses its activation quantizer into (tcfp/nn/__init__.py:620-640):
        # its fused Triton kernel against this library's quantize + GEMM pair, same inputs
        if rk.is_triton_available():
            from tcfp_b200.kernels import fused_act_quant_dual_gemm_forward, fused_dual_quantize_fp8

            small = {}
            m_tok, k_in = 32768, 4096
            xa = torch.randn(m_tok, k_in, device=dev, dtype=torch.bfloat16)
            for n_out in (128, 256, 512):
                ws = torch.randn(n_out, k_in, device=dev) * 0.02
                hi_s, lo_s, sh_s, sl_s = fused_dual_quantize_fp8(ws, BS)
                rk.fused_act_quant_dual_gemm_forward(xa, hi_s, lo_s, sh_s, sl_s, BS)
                ref_ms = t(lambda: rk.fused_act_quant_dual_gemm_forward(xa, hi_s, lo_s, sh_s, sl_s, BS), n=3, warm=1)
                own_ms = t(lambda: fused_act_quant_dual_gemm_forward(xa, hi_s, lo_s, sh_s, sl_s, BS), n=5, warm=2)
                small[f"N{n_out}"] = {"reference_fused_triton_ms": ref_ms, "ours_quantize_plus_gemm_ms": own_ms,
                                      "speedup": ref_ms / own_ms}
            out["act_quant_fused_small_n_M32768_K4096_bs64"] = small
            del xa
        if ours_ms is not None:
            out["ours_block_scaled_dual_gemm_bs64"] = entry(ours_ms)
            ref = out.get("triton_block_scaled_dual_gemm_bs64")
            if ref:
                out["speedup_vs_reference_block_kernel"] = ref["ms"] / ours_ms
    except Exception as e:
        out["error"] = repr(e)[:300]
    finally:
        ref_loader.unload()
    return out


# ---------------------------------------------------------------------------
# training-step workloads (tensor parallel over the launched ranks)
# ---------------------------------------------------------------------------

TRAIN_DESC = {
    "mlp": "MLP 1024->4096->1024 GELU, 64x128 tokens bf16, per-tensor EF, Adam, fwd+bwd+step (configuration 0)",
    "mlp_large": "MLP 4096->16384->4096 GELU, 16x2048 tokens bf16, bf16 layer outputs, per-tensor SRR, AdamW, fwd+bwd+step "
                 "(configuration 3)",
    "decoder": "4 decoder layers d=4096 h=32 ffn=11008, batch 8 x seq 4096 bf16, block-64 EF, AdamW, fwd+bwd+step "
               "(configuration 4)",
}


def _build_train_workload(name: str, dev, world: int, sp: bool):
    import torch

    from tcfp_b200.workloads import build_decoder, build_mlp

    if name == "mlp":
        d, h, tokens, seed = 1024, 4096, 64 * 128, 1001
        model = build_mlp(d, h).to(dev)
        opt_cls, lr = torch.optim.Adam, 1e-4
        shape = (tokens, d)
        flop = 2.0 * tokens * d * h * 2 * 5           # two layers x (2 fwd + 2 dX + 1 dW) products
    elif name == "mlp_large":
        d, h, tokens, seed = 4096, 16384, 16 * 2048, 1004
        # bf16 activations between the layers and bf16 partial sums on the wire (the GEMM epilogues write bf16)
        model = build_mlp(d, h, srr=True, out_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16).to(dev)
        opt_cls, lr = torch.optim.AdamW, 3e-4
        shape = (tokens, d)
        flop = 2.0 * tokens * d * h * 2 * 5
    else:
        d, seed = 4096, 1005
        model = build_decoder(sequence_parallel=sp).to(dev)
        opt_cls, lr = torch.optim.AdamW, 3e-4
        shape = (8, 4096, d)
        flop = 2.0 * 8 * 4096 * 4 * (4 * d * d + 3 * d * 11008) * 5
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g).to(torch.bfloat16).to(dev)
    target = torch.randn(shape, generator=g).to(torch.bfloat16).to(dev)
    opt = opt_cls(model.parameters(), lr=lr)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.mse_loss(model(x).float(), target.float())
        loss.backward()
        opt.step()
        return loss

    return step, flop


def _kernel_table(step, top: int = 30) -> dict:
    """Device time per kernel over two steps of a workload, as the torch
    profiler records it on this rank (``--kernel-table``)."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(2):
            step()
        torch.cuda.synchronize()
    rows = [(e.key, e.count, e.device_time_total) for e in prof.key_averages()
            if e.device_time_total > 0 and e.device_type.name == "CUDA"]
    rows.sort(key=lambda r: -r[2])
    total = sum(r[2] for r in rows)
    return {"kernel_ms_per_step": total / 2e3, "launches_per_step": sum(r[1] for r in rows) / 2,
            "rows": [{"kernel": k[:120], "launches_per_step": c / 2, "ms_per_step": t / 2e3, "share": t / total}
                     for k, c, t in rows[:top]]}


def _train_step_extra(name: str, dev, world: int, timed, steps: int, sp: bool = False, kernel_table: bool = False,
                      single_ms: float | None = None) -> dict:
    """One tensor-parallel training workload: ms per step with the NCCL
    collectives inside the timed region, the same step with the collectives
    switched off, and their difference (communication not hidden by compute)."""
    import torch

    from tcfp_b200 import tp

    step, flop = _build_train_workload(name, dev, world, sp)
    ms = timed(step, steps, 3) / steps
    res = {"config": TRAIN_DESC[name], "parallelism": (f"tp{world}" + (" sequence-parallel" if sp else "")) if world > 1
           else "single GPU", "ms_per_step": ms, "steps": steps,
           "linear_tflops_effective": flop / (ms * 1e-3) / 1e12, "loss": float(step().item())}
    if kernel_table:
        res["kernel_table"] = _kernel_table(step)
    if world > 1:
        with tp.collectives_disabled():
            ms_nocomm = timed(step, steps, 2) / steps
        res["ms_per_step_collectives_off"] = ms_nocomm
        res["comm_ms_per_step"] = max(0.0, ms - ms_nocomm)
        if sp:
            res["collectives_off_note"] = ("with the collectives off the gathered tensors are filled by copies of the local "
                                           "rows, which the real step does not pay: a lower bound on the exposed communication")
        res["collective"] = "NCCL all-reduce (bf16/fp32 partial outputs forward, input gradients backward)" if not sp \
            else "NCCL all-gather (FP8 codes forward, bf16 gradients backward) + reduce-scatter"
        # the single-GPU form of the same step, every rank running its own copy at the same time on this box
        # (``single_ms``: already measured in this run for the same workload)
        if single_ms is None:
            del step
            torch.cuda.empty_cache()
            with tp.single_rank():
                step, _ = _build_train_workload(name, dev, 1, False)
            with tp.collectives_disabled():
                single_ms = timed(step, steps, 2) / steps
        res["ms_per_step_single_gpu"] = single_ms
        res["efficiency_vs_n1"] = single_ms / (world * ms)
    res["peak_mem_gb"] = torch.cuda.max_memory_allocated() / 2**30
    del step
    torch.cuda.empty_cache()
    return res


def _kernel_extras(dev, timed) -> dict:
    """Driver-run figures for the other kernels of the path at 8192 x 8192
    (inputs 128-512 MB, larger than L2): quantizers in GB/s of ALGORITHMIC
    bytes, block 32 / 128 forward, dX (with and without the per-weight-version
    re-targeting pass), dW."""
    import torch

    from tcfp_b200.core import dual_quantize_per_tensor, to_fp8_e4m3, to_fp8_e5m2
    from tcfp_b200.kernels import (bf16_weight_grad, block_dequantize_bf16, block_quantize_fp8, block_retarget,
                                   fp8_weight_grad, fused_block_scaled_backward_dx,
                                   fused_block_scaled_dual_gemm_forward, fused_dual_quantize_fp8)

    n = 8192
    e = n * n
    g = torch.Generator().manual_seed(7)
    w = (torch.randn(n, n, generator=g) * 0.02).to(dev)
    err = torch.zeros(n, n, device=dev)
    x = torch.randn(n, n, generator=g).to(torch.bfloat16).to(dev)
    gy = torch.randn(n, n, generator=g).to(dev)
    hbm = _peaks()["hbm"]
    out: dict = {"shape": "8192 x 8192", "hbm_peak_gbs": hbm}
    iters = 10

    def q(name, fn, bytes_per_elem):
        ms = timed(fn, iters, 3) / iters
        gbs = bytes_per_elem * e / ms / 1e6
        out[name] = {"us": ms * 1e3, "algorithmic_bytes_per_elem": bytes_per_elem, "gbs": gbs, "frac_of_hbm": gbs / hbm}

    for bs in (32, 64, 128):
        q(f"dual_quantize_block{bs}_ef", lambda: fused_dual_quantize_fp8(w, bs, err), 14)
    q("dual_quantize_block64_no_ef", lambda: fused_dual_quantize_fp8(w, 64, None), 6)
    q("dual_quantize_block64_srr", lambda: fused_dual_quantize_fp8(w, 64, None, True, seed=1), 6)
    q("act_quantize_block64_bf16_e4m3", lambda: block_quantize_fp8(x, 64), 3)
    q("grad_quantize_block64_f32_e5m2", lambda: block_quantize_fp8(gy, 64, torch.float8_e5m2), 5)
    q("dual_quantize_per_tensor_ef_fresh", lambda: dual_quantize_per_tensor(w, err), 14)
    a_hi, a_lo = torch.tensor(0.1, device=dev), torch.tensor(0.0125, device=dev)
    q("dual_quantize_per_tensor_ef_delayed", lambda: dual_quantize_per_tensor(w, err, amax_hi=a_hi, amax_lo=a_lo), 14)
    q("dual_quantize_per_tensor_srr", lambda: dual_quantize_per_tensor(w, None, srr=True), 6)
    q("act_cast_per_tensor_bf16_e4m3", lambda: to_fp8_e4m3(x), 3)
    q("grad_cast_per_tensor_f32_e5m2", lambda: to_fp8_e5m2(gy), 5)

    flop = 4.0 * n**3

    def gemm(name, fn, fl=flop):
        ms = timed(fn, iters, 3) / iters
        out[name] = {"ms": ms, "tflops": fl / ms / 1e9}

    for bs in (32, 128):
        hi, lo, sh, sl = fused_dual_quantize_fp8(w, bs)
        a, sa = block_quantize_fp8(x, bs)
        gemm(f"block{bs}_forward", lambda: fused_block_scaled_dual_gemm_forward(a, hi, lo, sa, sh, sl, bs))
    hi, lo, sh, sl = fused_dual_quantize_fp8(w, 64)
    a, sa = block_quantize_fp8(x, 64)
    gq, sg = block_quantize_fp8(gy, 64, torch.float8_e5m2)
    fused_block_scaled_backward_dx(gq, hi, lo, sg, sh, sl, 64)                       # fills the re-targeting cache
    gemm("block64_dx_gemm_weight_retargeted", lambda: fused_block_scaled_backward_dx(gq, hi, lo, sg, sh, sl, 64))
    ms = timed(lambda: block_retarget(hi, lo, sh, sl, 64), iters, 3) / iters
    out["block64_retarget_pass"] = {"us": ms * 1e3, "gbs": 4.0 * e / ms / 1e6, "note": "once per weight version"}
    out["block64_dx_total_first_use"] = {"ms": out["block64_dx_gemm_weight_retargeted"]["ms"] + ms}
    gemm("block64_dx_exact_bf16_route", lambda: fused_block_scaled_backward_dx(gq, hi, lo, sg, sh, sl, 64, exact_bf16=True))
    xb = block_dequantize_bf16(a, sa, 64)
    gemm("block64_dw_f32_gradient_bf16_head_tail", lambda: bf16_weight_grad(gy, xb), 2.0 * n**3)
    gyb = gy.to(torch.bfloat16)
    gemm("block64_dw_bf16_gradient", lambda: bf16_weight_grad(gyb, xb), 2.0 * n**3)
    ms = timed(lambda: block_dequantize_bf16(a, sa, 64), iters, 3) / iters
    out["block64_dequantize_saved_activation"] = {"us": ms * 1e3, "algorithmic_bytes_per_elem": 3, "gbs": 3.0 * e / ms / 1e6,
                                                  "frac_of_hbm": 3.0 * e / ms / 1e6 / hbm}
    pa, ia = to_fp8_e4m3(x)
    pg, ig = to_fp8_e5m2(gy)
    gemm("per_tensor_dw_fp8", lambda: fp8_weight_grad(pg, pa, ig, ia), 2.0 * n**3)
    return out


def run_train_workload(args) -> None:
    """``--workload mlp|mlp_large|decoder``: one training workload alone, one JSON line."""
    import torch
    import torch.distributed as dist

    from tcfp_b200 import _C

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    _C.load()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    timed = _make_timed(dev, world)
    with ClockSampler(local) as clk:
        res = _train_step_extra(args.workload, dev, world, timed, args.steps, sp=args.sp, kernel_table=args.kernel_table)
    _C.check_device_status()
    if rank == 0:
        print(json.dumps({
            "metric": "train_step_ms", "value": res["ms_per_step"], "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": 3, "ms_per_step": res["ms_per_step"], "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": res["config"], "parallelism": res["parallelism"]}, "detail": res,
            "clocks": clk.summary()}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _make_timed(dev, world):
    import torch
    import torch.distributed as dist

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        """Total device milliseconds of ``steps`` calls after ``warmup`` calls;
        barrier + synchronize on both sides, maximum over the ranks."""
        for _ in range(warmup):
            fn()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    return timed


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    passes, warm = max(1, args.steps), max(0, min(args.warmup, 3))
    val, cores, times = _cpu_passes(passes, warm)
    mean_ms = sum(times) / len(times) * 1e3
    sample = (f"{passes} whole passes of the workload (all 8192 activation rows, an 8192x8192x8192 dual matmul each) "
              f"after {warm} warm-up passes; value from the mean pass")
    line = {
        "impl": "reference", "metric": "dual_fp8_gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": passes, "warmup": warm, "ms_per_step": mean_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": _config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "timing": "host wall clock around each pass, CPU",
        "note": "CPU restatement of the reference's block-scaled path (its Triton kernels need a GPU): "
                "dequantize + FP32 dual matmul on all host cores, operands quantized beforehand",
    }
    if not args.no_extras:
        try:
            import torch

            if torch.cuda.is_available():
                from tcfp_b200.kernels import block_quantize_fp8, fused_dual_quantize_fp8

                dev = torch.device("cuda", 0)
                g = torch.Generator().manual_seed(1003)
                x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
                w = (torch.randn(N, K, generator=g) * 0.02).to(dev)
                w_hi, w_lo, s_hi, s_lo = fused_dual_quantize_fp8(w, BS)
                a, s_a = block_quantize_fp8(x, BS)
                line["reference_gpu"] = _reference_gpu(dev, a, s_a, w_hi, w_lo, s_hi, s_lo, x, w, None)
        except Exception as e:
            line["reference_gpu"] = {"error": repr(e)[:200]}
    line["wall_s"] = time.perf_counter() - t0
    print(json.dumps(line), flush=True)


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def _bind_near_gpu(index: int):
    """Multi-rank runs: restrict this process to the CPUs of its GPU's NUMA
    node (sysfs ``local_cpulist`` of the GPU's PCI function) BEFORE the pinned
    host buffers are allocated, so that they land in the memory next to the
    GPU's PCIe root instead of wherever the launcher started the process.
    Returns the CPU list applied, or None when there is nothing to do."""
    try:
        import pynvml

        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(index)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()[-12:]
        text = Path(f"/sys/bus/pci/devices/{bus}/local_cpulist").read_text().strip()
        allowed = os.sched_getaffinity(0)
        want = _parse_cpulist(text) & allowed
        if want and want != allowed:
            os.sched_setaffinity(0, want)
            return text
    except Exception:
        pass
    return None


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from tcfp_b200 import _C
    from tcfp_b200.kernels import (block_dequantize_fp8, block_quantize_fp8, fused_block_scaled_dual_gemm_forward,
                                   fused_dual_quantize_fp8)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    _C.load()  # no library, no benchmark
    cpu_binding = _bind_near_gpu(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    g = torch.Generator().manual_seed(1003 + rank)
    x_host = torch.randn(M, K, generator=g).to(torch.bfloat16).pin_memory()
    w = (torch.randn(N, K, generator=g) * 0.02)
    mask = torch.rand(N, K, generator=g) < 0.001
    w = torch.where(mask, w * 50.0, w).to(dev)
    err = torch.zeros(N, K, device=dev)
    out_host = torch.empty(M, N, dtype=torch.float32).pin_memory()

    x = x_host.to(dev, non_blocking=True)
    w_hi, w_lo, s_hi, s_lo = fused_dual_quantize_fp8(w, BS, err)
    a, s_a = block_quantize_fp8(x, BS)
    launches_per_step = 1
    y_dev = torch.empty(M, N, device=dev, dtype=torch.float32)

    def step():
        return fused_block_scaled_dual_gemm_forward(a, w_hi, w_lo, s_a, s_hi, s_lo, BS, out=y_dev)

    from tcfp_b200.host_pipeline import HostStreamedLinear

    streamed = HostStreamedLinear(w, BS, chunks=E2E_CHUNKS)

    def e2e_step():
        streamed.forward_from_host(x_host, out_host)

    timed = _make_timed(dev, world)
    warmup = max(args.warmup, 3)
    with ClockSampler(local) as clk:
        total_ms = timed(step, args.steps, warmup)
    clocks = clk.summary()
    ms_per_step = total_ms / args.steps

    # the output that was just timed, checked on a row slice against a plain FP32 product of the dequantized operands
    rows = slice(0, 256)
    ref = block_dequantize_fp8(a[rows], s_a[:, rows].contiguous(), BS) @ (
        block_dequantize_fp8(w_hi, s_hi, BS) + block_dequantize_fp8(w_lo, s_lo, BS)).t()
    rel = float((y_dev[rows] - ref).norm() / ref.norm())
    del ref
    if not rel <= 1e-3:
        raise RuntimeError(f"the timed GEMM output is wrong: relative Frobenius error {rel:.3e} on rows 0..255")

    # sustained: the same launch back to back for at least two seconds, clocks sampled throughout
    sus_steps = max(args.steps, int(2200.0 / ms_per_step))
    with ClockSampler(local, period_s=0.01) as clk_s:
        sus_ms = timed(step, sus_steps, 1) / sus_steps
    sus_clk = clk_s.summary()

    e2e_steps = max(2, min(args.steps, 10))
    e2e_ms = timed(e2e_step, e2e_steps, 2)
    _C.check_device_status()

    value = world * FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12
    e2e_value = world * FLOP_PER_STEP / (e2e_ms / e2e_steps * 1e-3) / 1e12
    peaks = _peaks()
    fp8_peak = 2.0 * peaks["bf16"]
    per_gpu = value / world
    traffic, traffic_src = _profiled_traffic()
    line = {
        "metric": "dual_fp8_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": _config(world),
        "pct_of_nominal_fp8_peak": per_gpu / 4500.0,
        "output_check": {"rel_frobenius_vs_fp32_dequantized_product": rel, "rows": 256, "tolerance": 1e-3},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": fp8_peak, "unit": "TFLOP/s",
                     "frac": per_gpu / fp8_peak, "traffic": traffic,
                     "traffic_note": f"mean dram__bytes_read + dram__bytes_write per launch from {traffic_src} "
                                     "(ncu on this same command); algorithmic 448 MB",
                     "peak_source": f"2 x {peaks['src']} cuBLAS bf16 burst ({peaks['bf16']} TFLOP/s): no FP8 peak was measured; "
                                    "FP8 tensor rate is twice the bf16 rate",
                     "kernel": "dual_gemm_pair_kernel<KIND_MXF8>", "flop_per_launch": FLOP_PER_STEP},
        "sustained": {"seconds": sus_ms * sus_steps / 1e3, "launches": sus_steps, "ms_per_step": sus_ms,
                      "tflops": FLOP_PER_STEP / sus_ms / 1e9, "sm_mhz_median": sus_clk["sm_mhz"],
                      "sm_mhz_min": sus_clk["sm_mhz_min"], "reasons": sus_clk["reasons"], "samples": sus_clk["samples"],
                      "ms_times_mhz": (sus_ms * sus_clk["sm_mhz"]) if sus_clk["sm_mhz"] else None,
                      "frac_of_2x_bf16_sustained": FLOP_PER_STEP / sus_ms / 1e9 / (2.0 * peaks["bf16_sustained"])},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 4,
                "ms_per_step": e2e_ms / e2e_steps, "host_cpus": cpu_binding,
                "path": "HostStreamedLinear.forward_from_host: pinned host X -> H2D -> fused_dual_quantize_fp8(W, EF) -> "
                        f"block_quantize_fp8(X) -> dual GEMM -> D2H out, in {E2E_CHUNKS} row chunks on 3 streams"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    del streamed, x_host, out_host
    extra: dict = {}
    if not args.no_extras:
        if world == 1:
            try:
                extra["reference_gpu"] = _reference_gpu(dev, a, s_a, w_hi, w_lo, s_hi, s_lo, x, w, ms_per_step)
            except Exception as e:
                extra["reference_gpu"] = {"error": repr(e)[:200]}
        del a, s_a, w_hi, w_lo, s_hi, s_lo, x, w, err, y_dev
        torch.cuda.empty_cache()
        if world == 1:
            try:
                extra["kernels"] = _kernel_extras(dev, timed)
            except Exception as e:
                extra["kernels"] = {"error": repr(e)[:200]}
            torch.cuda.empty_cache()
        for key, name, steps in (("mlp_train_step", "mlp", 10), ("mlp_large_train_step", "mlp_large", 5),
                                 ("decoder_train_step", "decoder", 3)):
            try:  # the headline line must not depend on an extra measurement
                extra[key] = _train_step_extra(name, dev, world, timed, steps)
            except Exception as e:
                extra[key] = {"error": repr(e)[:200]}
            torch.cuda.empty_cache()
        if world > 1:
            try:
                extra["decoder_train_step_sequence_parallel"] = _train_step_extra(
                    "decoder", dev, world, timed, 3, sp=True,
                    single_ms=extra.get("decoder_train_step", {}).get("ms_per_step_single_gpu"))
            except Exception as e:
                extra["decoder_train_step_sequence_parallel"] = {"error": repr(e)[:200]}
            torch.cuda.empty_cache()
    line["extra"] = extra
    _C.check_device_status()
    if rank == 0 and world == 1:
        val, cores, times = _cpu_passes(3, 1)
        line["cpu_baseline"] = {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                "sample": "3 whole passes of the workload (8192x8192x8192 dequantize + FP32 dual matmul) "
                                          "after 1 warm-up pass; value from the mean pass"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm", choices=["gemm", "mlp", "mlp_large", "decoder"])
    ap.add_argument("--sp", action="store_true", help="decoder workload: sequence-parallel form")
    ap.add_argument("--no-extras", action="store_true", help="headline line only")
    ap.add_argument("--kernel-table", action="store_true",
                    help="with --workload: add the per-kernel device time of two steps (torch profiler) to the line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "gemm":
        run_train_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
