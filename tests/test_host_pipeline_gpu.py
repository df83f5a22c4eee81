"""Host-buffer pipeline on the GPU: results must equal the plain device-tensor calls over the
whole batch (out, dk, dv bit-exact: same kernels on the same data in the same order; dq up to
the order-dependent fp32 accumulation), including when the pipeline object is reused."""
from __future__ import annotations

import pytest
import torch

import min_fa3_op
from gpu_util import make_bshd
from min_fa3_demo_b200.host_pipeline import HostPipeline

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("groups", [1, 2])
@pytest.mark.parametrize("causal", [True, False])
def test_pipeline_equals_direct_calls(causal, groups):
    b, s, qh, kvh = 5, 384, 8, 2
    q, k, v, dout = make_bshd(77, b, s, qh, kvh)
    host_in = {"q": q.pin_memory(), "k": k.pin_memory(), "v": v.pin_memory(), "dout": dout.pin_memory()}
    host_out = {"out": torch.empty_like(q).pin_memory(), "dq": torch.empty_like(q).pin_memory(),
                "dk": torch.empty_like(k).pin_memory(), "dv": torch.empty_like(v).pin_memory()}
    dev = torch.device("cuda", 0)
    pipe = HostPipeline(dev, s, qh, kvh, head_groups=groups)
    out, lse = min_fa3_op.forward(q.cuda(), k.cuda(), v.cuda(), causal, return_lse=True)
    dq, dk, dv = min_fa3_op.backward(dout.cuda(), q.cuda(), k.cuda(), v.cuda(), out, lse, causal)
    for _ in range(2):                      # second pass reuses slots, streams and events
        for t in host_out.values():
            t.zero_()
        pipe.run(host_in, host_out, causal)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(host_out["out"], out.cpu())
        assert torch.equal(host_out["dk"], dk.cpu())
        assert torch.equal(host_out["dv"], dv.cpu())
        diff = (host_out["dq"].float() - dq.cpu().float()).abs().max().item()
        assert diff <= 2.0 ** -6 * max(1.0, dq.float().abs().max().item())


def test_pipeline_rejects_pageable_memory():
    q, k, v, dout = make_bshd(78, 1, 128, 2, 2)
    pipe = HostPipeline(torch.device("cuda", 0), 128, 2, 2)
    host_in = {"q": q, "k": k, "v": v, "dout": dout}
    host_out = {n: torch.empty_like(t).pin_memory() for n, t in (("out", q), ("dq", q), ("dk", k), ("dv", v))}
    with pytest.raises(ValueError, match="pinned"):
        pipe.run(host_in, host_out, True)
