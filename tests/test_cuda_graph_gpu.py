"""The forward and backward launches can be captured into a CUDA graph and replayed: the
library allocates nothing, every launch and memset goes to the caller's stream, and the work
scheduler's counters are reset by captured memset nodes.  Replays must reproduce the eager
results (out, dk, dv bit for bit; dq too in deterministic mode)."""
from __future__ import annotations

import pytest
import torch

import min_fa3_op
from gpu_util import make_bshd

pytestmark = pytest.mark.gpu


def test_forward_backward_capture_and_replay():
    q, k, v, dout = make_bshd(55, 2, 1024, 8, 2)
    qc, kc, vc, dc = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    # Eager run first: also performs the one-time per-device kernel configuration.
    out_e, lse_e = min_fa3_op.forward(qc, kc, vc, True, return_lse=True)
    dq_e, dk_e, dv_e = min_fa3_op.backward(dc, qc, kc, vc, out_e, lse_e, True, deterministic=True)
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            out_g, lse_g = min_fa3_op.forward(qc, kc, vc, True, return_lse=True)
            dq_g, dk_g, dv_g = min_fa3_op.backward(dc, qc, kc, vc, out_g, lse_g, True, deterministic=True)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        for t in (out_g, dq_g, dk_g, dv_g):
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out_g, out_e) and torch.equal(lse_g, lse_e)
        assert torch.equal(dq_g, dq_e) and torch.equal(dk_g, dk_e) and torch.equal(dv_g, dv_e)

    # New inputs through the same graph: copy into the captured buffers and replay.
    q2, k2, v2, d2 = make_bshd(56, 2, 1024, 8, 2)
    qc.copy_(q2.cuda()); kc.copy_(k2.cuda()); vc.copy_(v2.cuda()); dc.copy_(d2.cuda())
    graph.replay()
    torch.cuda.synchronize()
    out_n, lse_n = min_fa3_op.forward(qc, kc, vc, True, return_lse=True)
    dq_n, dk_n, dv_n = min_fa3_op.backward(dc, qc, kc, vc, out_n, lse_n, True, deterministic=True)
    torch.cuda.synchronize()
    assert torch.equal(out_g, out_n) and torch.equal(dq_g, dq_n) and torch.equal(dk_g, dk_n) and torch.equal(dv_g, dv_n)
