"""Forgetting attention for callers whose tensors live in (pinned) host memory.

One fwd+bwd step from host buffers is three stages: host-to-device copies of q, k, v, log_fgate, dout;
the operator; device-to-host copies of out and the four gradients.  Run back to back they cost the sum of
the three (PCIe moves ~0.4 GB each way for the T=16k shape, more time than the kernels take).  This class
runs the stages of consecutive steps on three CUDA streams with two sets of device buffers, so that a
step's copies overlap its neighbours' compute and the step time tends to the slowest stage.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .ops import forgetting_attention

__all__ = ["HostStreamedAttention"]

_IN = ("q", "k", "v", "log_fgate", "dout")
_OUT = ("out", "dq", "dk", "dv", "dlog_fgate")


class HostStreamedAttention:
    """``submit(host_inputs)`` queues one fwd+bwd step on pinned host tensors (head-first layout) and
    returns the pinned host tensors its results will land in; ``finish()`` waits for everything queued.
    Results of a step are valid after ``finish()`` or after the returned event has completed."""

    def __init__(self, device: torch.device, seq_start: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None,
                 adaptive_threshold=None, attention=None, depth: int = 2):
        self.device = device
        self.seq_start = seq_start
        self.sm_scale = sm_scale
        self.adaptive_threshold = adaptive_threshold
        self.attention = attention  # callable(q, k, v, log_fgate) -> out, e.g. a context-parallel wrapper
        self.depth = depth
        self.s_in = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self.s_compute = torch.cuda.current_stream(device)
        self.dev_in: List[Optional[Dict[str, torch.Tensor]]] = [None] * depth
        self.host_out: List[Optional[Dict[str, torch.Tensor]]] = [None] * depth
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]       # inputs of the slot have landed
        self.ev_compute = [torch.cuda.Event() for _ in range(depth)]  # the slot's step has been computed
        self.ev_out = [torch.cuda.Event() for _ in range(depth)]      # the slot's results are on the host
        self.step = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def submit(self, host: Dict[str, torch.Tensor]):
        slot = self.step % self.depth
        first_use = self.dev_in[slot] is None
        if first_use:
            self.dev_in[slot] = {n: torch.empty(host[n].shape, dtype=host[n].dtype, device=self.device) for n in _IN}
        dev = self.dev_in[slot]
        # ---- stage 1: host -> device, once the step that last used this slot has been computed ----
        with torch.cuda.stream(self.s_in):
            if first_use:
                # the buffers were just allocated on the compute stream: a block the allocator recycled may
                # still be read by kernels queued there
                self.s_in.wait_stream(self.s_compute)
            else:
                self.s_in.wait_event(self.ev_compute[slot])
            for n in _IN:
                dev[n].copy_(host[n], non_blocking=True)
            self.ev_in[slot].record(self.s_in)
        self.h2d_bytes = sum(host[n].numel() * host[n].element_size() for n in _IN)
        # ---- stage 2: the operator ----
        self.s_compute.wait_event(self.ev_in[slot])
        q, k, v, lf = [dev[n].detach().requires_grad_() for n in ("q", "k", "v", "log_fgate")]
        if self.attention is not None:
            out = self.attention(q, k, v, lf)
        else:
            out = forgetting_attention(q, k, v, lf, head_first=True, seq_start=self.seq_start, sm_scale=self.sm_scale,
                                       adaptive_threshold=self.adaptive_threshold)
        out.backward(dev["dout"])
        res = dict(zip(_OUT, (out.detach(), q.grad, k.grad, v.grad, lf.grad)))
        self.ev_compute[slot].record(self.s_compute)
        # ---- stage 3: device -> host (the slot's host buffers are overwritten `depth` steps later) ----
        if self.host_out[slot] is None:
            self.host_out[slot] = {n: torch.empty(t.shape, dtype=t.dtype).pin_memory() for n, t in res.items()}
        hout = self.host_out[slot]
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_compute[slot])
            for n in _OUT:
                hout[n].copy_(res[n], non_blocking=True)
                res[n].record_stream(self.s_out)   # the allocator may reuse it only after the copy
            self.ev_out[slot].record(self.s_out)
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in hout.values())
        self.step += 1
        return hout, self.ev_out[slot]

    def finish(self):
        self.s_in.synchronize()
        self.s_compute.synchronize()
        self.s_out.synchronize()
