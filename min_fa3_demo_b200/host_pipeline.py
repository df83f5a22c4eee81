"""Attention forward + backward for callers whose tensors live in (pinned) host memory.

``forward`` / ``backward`` take device tensors, as the reference's operators do
(``min_fa3_op.py:25-52``, bindings.cpp:240).  A caller that starts from host buffers pays for
the host->device copy of q, k, v, dout and the device->host copy of out, dq, dk, dv; done one
after the other around the kernels, those copies take three times as long as the attention
itself on a PCIe link.  :class:`HostPipeline` overlaps the three legs: batch elements of a
BSHD problem are independent, so element ``b`` is uploaded on one stream while element
``b - 1`` is computed on a second and element ``b - 2`` is downloaded on a third (PCIe is full
duplex).  Results are bit-identical to one call over the whole batch up to the (order-dependent)
fp32 dQ accumulation, because each element runs the same kernels on the same data.
"""

from __future__ import annotations

from typing import Dict

import torch

from . import min_fa3_op as _op

_IN = ("q", "k", "v", "dout")
_OUT = ("out", "dq", "dk", "dv")


class HostPipeline:
    """Reusable streams, events and device staging buffers for one problem shape.

    ``run(host_in, host_out, is_causal)`` consumes pinned bf16 host tensors ``q, k, v, dout``
    of shape ``[B, S, H, 128]`` and fills pinned host tensors ``out, dq, dk, dv``; it returns
    after enqueueing and making the caller's current stream wait for the last download, so
    ``torch.cuda.current_stream().synchronize()`` (or any later work on that stream) sees the
    results.
    """

    def __init__(self, device: torch.device, seqlen: int, heads_q: int, heads_k: int, slots: int = 2,
                 seqlen_k: int | None = None):
        self.device = device
        self.slots = slots
        self.s_in = torch.cuda.Stream(device)
        self.s_compute = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        shape_q = (1, seqlen, heads_q, 128)
        shape_k = (1, seqlen if seqlen_k is None else seqlen_k, heads_k, 128)
        def buf(shape):
            return torch.empty(shape, dtype=torch.bfloat16, device=device)
        self.dev_in = [{"q": buf(shape_q), "k": buf(shape_k), "v": buf(shape_k), "dout": buf(shape_q)}
                       for _ in range(slots)]
        self.dev_out = [{"out": buf(shape_q), "dq": buf(shape_q), "dk": buf(shape_k), "dv": buf(shape_k)}
                        for _ in range(slots)]
        self.ev_uploaded = [torch.cuda.Event() for _ in range(slots)]
        self.ev_computed = [torch.cuda.Event() for _ in range(slots)]
        self.ev_downloaded = [torch.cuda.Event() for _ in range(slots)]

    def run(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor], is_causal: bool) -> None:
        for name in _IN:
            t = host_in[name]
            if t.device.type != "cpu" or not t.is_pinned() or t.dtype != torch.bfloat16 or t.dim() != 4:
                raise ValueError(f"{name} must be a pinned bf16 host tensor [B, S, H, 128]")
        for name in _OUT:
            t = host_out[name]
            if t.device.type != "cpu" or not t.is_pinned() or t.dtype != torch.bfloat16:
                raise ValueError(f"{name} must be a pinned bf16 host tensor")
        batch = host_in["q"].size(0)
        caller = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(caller)
        for s in (self.s_in, self.s_compute, self.s_out):
            s.wait_event(start)

        for b in range(batch):
            slot = b % self.slots
            reuse = b >= self.slots
            with torch.cuda.stream(self.s_in):
                if reuse:
                    self.s_in.wait_event(self.ev_computed[slot])     # inputs of element b - slots consumed
                for name in _IN:
                    self.dev_in[slot][name].copy_(host_in[name][b:b + 1], non_blocking=True)
                self.ev_uploaded[slot].record(self.s_in)
            with torch.cuda.stream(self.s_compute):
                self.s_compute.wait_event(self.ev_uploaded[slot])
                if reuse:
                    self.s_compute.wait_event(self.ev_downloaded[slot])   # outputs of element b - slots read
                i, o = self.dev_in[slot], self.dev_out[slot]
                out, lse = _op.forward(i["q"], i["k"], i["v"], is_causal, return_lse=True)
                o["out"].copy_(out)
                _op.backward(i["dout"], i["q"], i["k"], i["v"], out, lse, is_causal,
                             dq=o["dq"], dk=o["dk"], dv=o["dv"])
                self.ev_computed[slot].record(self.s_compute)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_computed[slot])
                for name in _OUT:
                    host_out[name][b:b + 1].copy_(self.dev_out[slot][name], non_blocking=True)
                self.ev_downloaded[slot].record(self.s_out)
        done = torch.cuda.Event()
        done.record(self.s_out)
        caller.wait_event(done)
        # Upload and compute streams finish before the last download by construction.


def forward_backward_host(host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor],
                          is_causal: bool, device: torch.device | None = None) -> None:
    """One-shot convenience wrapper around :class:`HostPipeline`."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    q, k = host_in["q"], host_in["k"]
    HostPipeline(device, q.size(1), q.size(2), k.size(2), seqlen_k=k.size(1)).run(host_in, host_out, is_causal)
