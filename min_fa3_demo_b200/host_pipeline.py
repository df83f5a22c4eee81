"""Attention forward + backward for callers whose tensors live in (pinned) host memory.

``forward`` / ``backward`` take device tensors, as the reference's operators do
(``min_fa3_op.py:25-52``, bindings.cpp:240).  A caller that starts from host buffers pays for
the host->device copy of q, k, v, dout and the device->host copy of out, dq, dk, dv; done one
after the other around the kernels, those copies take three times as long as the attention
itself on a PCIe link.  :class:`HostPipeline` overlaps the three legs.  A BSHD problem splits
into independent chunks — one batch element times one group of KV heads with their query
heads — so chunk ``c`` is uploaded on one stream while chunk ``c - 1`` is computed on a second
and chunk ``c - 2`` is downloaded on a third (PCIe is full duplex); within a chunk the forward
starts as soon as q, k, v have arrived (dout follows during the forward) and ``out`` goes back
while the backward runs.  The head subset of a ``[B, S, H, 128]`` host tensor is strided; it is
moved with the library's 2-D copy (``b2a_copy_2d``) straight between the pinned tensor and a
contiguous device buffer.  Results equal one call over the whole problem bit for bit except dq,
whose fp32 accumulation order is not fixed (every head sees the same kernels and data).
"""

from __future__ import annotations

import ctypes
from typing import Dict

import torch

from . import _cabi
from . import min_fa3_op as _op

_IN = ("q", "k", "v", "dout")
_OUT = ("out", "dq", "dk", "dv")
_H2D, _D2H = 1, 2


class HostPipeline:
    """Reusable streams, events and device staging buffers for one problem shape.

    ``run(host_in, host_out, is_causal)`` consumes pinned bf16 host tensors ``q, dout``
    ``[B, S, QH, 128]`` and ``k, v`` ``[B, Sk, KVH, 128]`` and fills pinned host tensors ``out, dq``
    (like q) and ``dk, dv`` (like k); it returns after enqueueing and making the caller's current
    stream wait for the last download, so ``torch.cuda.current_stream().synchronize()`` (or any
    later work on that stream) sees the results.

    ``head_groups`` chunks per batch element (it must divide KVH): more chunks shorten the
    pipeline's fill and drain, fewer keep each launch large enough to fill the GPU.
    """

    def __init__(self, device: torch.device, seqlen: int, heads_q: int, heads_k: int, slots: int = 3,
                 seqlen_k: int | None = None, head_groups: int = 2):
        if heads_k % head_groups != 0 or heads_q % heads_k != 0:
            raise ValueError(f"head_groups={head_groups} must divide heads_k={heads_k} (and heads_k heads_q)")
        self.device = device
        self.slots = slots
        self.groups = head_groups
        self.heads_q, self.heads_k = heads_q, heads_k
        self.seqlen_q = seqlen
        self.seqlen_k = seqlen if seqlen_k is None else seqlen_k
        self.s_in = torch.cuda.Stream(device)
        self.s_compute = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self.hq_c, self.hk_c = heads_q // head_groups, heads_k // head_groups
        shape_q = (1, self.seqlen_q, self.hq_c, 128)
        shape_k = (1, self.seqlen_k, self.hk_c, 128)

        def buf(shape):
            return torch.empty(shape, dtype=torch.bfloat16, device=device)
        self.dev_in = [{"q": buf(shape_q), "k": buf(shape_k), "v": buf(shape_k), "dout": buf(shape_q)}
                       for _ in range(slots)]
        self.dev_out = [{"out": buf(shape_q), "dq": buf(shape_q), "dk": buf(shape_k), "dv": buf(shape_k)}
                        for _ in range(slots)]
        self.ev_qkv = [torch.cuda.Event() for _ in range(slots)]        # q, k, v of the slot uploaded
        self.ev_dout = [torch.cuda.Event() for _ in range(slots)]       # dout uploaded
        self.ev_fwd = [torch.cuda.Event() for _ in range(slots)]        # out computed
        self.ev_bwd = [torch.cuda.Event() for _ in range(slots)]        # dq, dk, dv computed (inputs consumed)
        self.ev_downloaded = [torch.cuda.Event() for _ in range(slots)]
        self._lib = _cabi.load()

    def _copy(self, dev: torch.Tensor, host: torch.Tensor, b: int, g: int, kind: int,
              stream: torch.cuda.Stream) -> None:
        """One chunk of a [B, S, H, 128] host tensor: batch element b, heads [g * hc, (g + 1) * hc)."""
        seq, heads = host.size(1), host.size(2)
        hc = heads // self.groups
        row_bytes, pitch = hc * 256, heads * 256
        host_ptr = host.data_ptr() + (b * seq * heads + g * hc) * 256
        if kind == _H2D:
            rc = self._lib.b2a_copy_2d(dev.data_ptr(), row_bytes, host_ptr, pitch, row_bytes, seq, kind,
                                       ctypes.c_void_p(stream.cuda_stream))
        else:
            rc = self._lib.b2a_copy_2d(host_ptr, pitch, dev.data_ptr(), row_bytes, row_bytes, seq, kind,
                                       ctypes.c_void_p(stream.cuda_stream))
        _cabi.check(rc)

    def _check(self, host_in, host_out) -> int:
        batch = host_in["q"].size(0)
        want = {"q": (batch, self.seqlen_q, self.heads_q, 128), "dout": (batch, self.seqlen_q, self.heads_q, 128),
                "k": (batch, self.seqlen_k, self.heads_k, 128), "v": (batch, self.seqlen_k, self.heads_k, 128)}
        want.update(out=want["q"], dq=want["q"], dk=want["k"], dv=want["k"])
        for name in _IN + _OUT:
            t = host_in[name] if name in _IN else host_out[name]
            if t.device.type != "cpu" or not t.is_pinned() or t.dtype != torch.bfloat16 or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous pinned bf16 host tensor")
            if tuple(t.shape) != want[name]:
                raise ValueError(f"{name} must have shape {want[name]}, got {tuple(t.shape)}")
        return batch

    def run(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor], is_causal: bool) -> None:
        batch = self._check(host_in, host_out)
        caller = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(caller)
        for s in (self.s_in, self.s_compute, self.s_out):
            s.wait_event(start)

        with torch.cuda.device(self.device):
            for c in range(batch * self.groups):
                b, g = divmod(c, self.groups)
                slot = c % self.slots
                reuse = c >= self.slots
                i, o = self.dev_in[slot], self.dev_out[slot]
                if reuse:
                    self.s_in.wait_event(self.ev_bwd[slot])          # inputs of chunk c - slots consumed
                for name in ("q", "k", "v"):                         # the forward needs these three only
                    self._copy(i[name], host_in[name], b, g, _H2D, self.s_in)
                self.ev_qkv[slot].record(self.s_in)
                self._copy(i["dout"], host_in["dout"], b, g, _H2D, self.s_in)   # overlaps the forward
                self.ev_dout[slot].record(self.s_in)
                with torch.cuda.stream(self.s_compute):
                    self.s_compute.wait_event(self.ev_qkv[slot])
                    if reuse:
                        self.s_compute.wait_event(self.ev_downloaded[slot])   # outputs of chunk c - slots read
                    out, lse = _op.forward(i["q"], i["k"], i["v"], is_causal, return_lse=True)
                    o["out"].copy_(out)
                    self.ev_fwd[slot].record(self.s_compute)
                    self.s_compute.wait_event(self.ev_dout[slot])
                    _op.backward(i["dout"], i["q"], i["k"], i["v"], out, lse, is_causal,
                                 dq=o["dq"], dk=o["dk"], dv=o["dv"])
                    self.ev_bwd[slot].record(self.s_compute)
                self.s_out.wait_event(self.ev_fwd[slot])
                self._copy(o["out"], host_out["out"], b, g, _D2H, self.s_out)    # overlaps the backward
                self.s_out.wait_event(self.ev_bwd[slot])
                for name in ("dq", "dk", "dv"):
                    self._copy(o[name], host_out[name], b, g, _D2H, self.s_out)
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
    HostPipeline(device, q.size(1), q.size(2), k.size(2), seqlen_k=k.size(1),
                 head_groups=2 if k.size(2) % 2 == 0 else 1).run(host_in, host_out, is_causal)
