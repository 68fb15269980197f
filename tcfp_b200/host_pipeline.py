"""Block-scaled TCFP-12 forward for activations that live in HOST memory.

``HostStreamedLinear`` takes a pinned host activation matrix and a pinned host
output buffer and runs  H2D copy -> activation quantize -> fused dual GEMM ->
D2H copy  in row chunks on three CUDA streams, so that the upload of chunk
i+1, the GEMM of chunk i and the download of chunk i-1 overlap (PCIe is full
duplex).  The weight is dual-quantized once per call, with error feedback, as
``TCFPLinear`` does every forward.
"""
from __future__ import annotations

import torch

from .kernels import block_quantize_fp8, fused_block_scaled_dual_gemm_forward, fused_dual_quantize_fp8


class HostStreamedLinear:
    def __init__(self, weight: torch.Tensor, block_size: int = 64, *, chunks: int = 8, error_feedback: bool = True,
                 bias: torch.Tensor | None = None):
        assert weight.is_cuda and weight.ndim == 2
        self.weight = weight.contiguous()
        self.bias = bias
        self.bs = block_size
        self.chunks = chunks
        self.err = torch.zeros_like(self.weight, dtype=torch.float32) if error_feedback else None
        dev = weight.device
        self._s_up = torch.cuda.Stream(device=dev)
        self._s_down = torch.cuda.Stream(device=dev)
        self._x_dev = None
        self._y_dev = None
        self._ev_comp: list[torch.cuda.Event] = []
        self._ev_down: list[torch.cuda.Event] = []

    def _buffers(self, x_host: torch.Tensor):
        M, K = x_host.shape
        N = self.weight.shape[0]
        if self._x_dev is None or self._x_dev.shape != x_host.shape or self._x_dev.dtype != x_host.dtype:
            self._x_dev = torch.empty_like(x_host, device=self.weight.device)
            self._y_dev = torch.empty(M, N, device=self.weight.device, dtype=torch.float32)
            self._ev_comp = [torch.cuda.Event() for _ in range(self.chunks)]
            self._ev_down = [torch.cuda.Event() for _ in range(self.chunks)]
            for e in self._ev_comp + self._ev_down:
                e.record()
        return self._x_dev, self._y_dev

    def forward_from_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """``out_host[:] = x_host @ W_q^T`` (FP32), both pinned host tensors.
        Enqueues everything and returns; the current stream is made to wait for
        the last download, so a synchronize / event on it covers the call."""
        assert x_host.is_pinned() and out_host.is_pinned(), "host buffers must be pinned"
        M, K = x_host.shape
        assert K == self.weight.shape[1] and out_host.shape == (M, self.weight.shape[0])
        cur = torch.cuda.current_stream()
        x_dev, y_dev = self._buffers(x_host)
        # the uploads start with the call: they do not depend on the weight quantizer queued next
        start_ev = torch.cuda.Event()
        start_ev.record(cur)
        self._s_up.wait_event(start_ev)
        w_hi, w_lo, s_hi, s_lo = fused_dual_quantize_fp8(self.weight, self.bs, self.err)
        rows = -(-M // self.chunks)
        rows = -(-rows // 128) * 128
        for c in range(self.chunks):
            r0, r1 = c * rows, min(M, (c + 1) * rows)
            if r0 >= r1:
                break
            up_ev = torch.cuda.Event()
            with torch.cuda.stream(self._s_up):
                self._s_up.wait_event(self._ev_comp[c])          # previous call's readers of this slice are done
                x_dev[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                up_ev.record(self._s_up)
            cur.wait_event(up_ev)
            cur.wait_event(self._ev_down[c])                     # previous download of this output slice is done
            a, sa = block_quantize_fp8(x_dev[r0:r1], self.bs)
            fused_block_scaled_dual_gemm_forward(a, w_hi, w_lo, sa, s_hi, s_lo, self.bs, bias=self.bias,
                                                 out=y_dev[r0:r1])
            self._ev_comp[c].record(cur)
            with torch.cuda.stream(self._s_down):
                self._s_down.wait_event(self._ev_comp[c])
                out_host[r0:r1].copy_(y_dev[r0:r1], non_blocking=True)
                self._ev_down[c].record(self._s_down)
        done = torch.cuda.Event()
        done.record(self._s_down)
        cur.wait_event(done)
        return out_host
