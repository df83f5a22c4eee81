"""Differentiable front end on the GPU: gradients through ``attention`` / ``attention_varlen``
equal the explicit forward + backward calls and meet the accuracy rule against the oracle."""
from __future__ import annotations

import pytest
import torch

import min_fa3_op
from gpu_util import assert_within, make_bshd, make_varlen
from min_fa3_demo_b200 import autograd as ag
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal", [True, False])
def test_bshd_autograd_matches_explicit_calls(causal):
    q, k, v, dout = make_bshd(31, 2, 640, 8, 2)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    out = ag.attention(qc, kc, vc, causal, deterministic=True)
    out.backward(dout.cuda())
    ref_out, lse = min_fa3_op.forward(q.cuda(), k.cuda(), v.cuda(), causal, return_lse=True)
    dq, dk, dv = min_fa3_op.backward(dout.cuda(), q.cuda(), k.cuda(), v.cuda(), ref_out, lse, causal, deterministic=True)
    assert torch.equal(out, ref_out)
    assert torch.equal(qc.grad, dq) and torch.equal(kc.grad, dk) and torch.equal(vc.grad, dv)
    rq, rk, rv = orc.bshd_backward(q, k, v, dout, causal)
    e = orc.bf16_attention_error(q, k, v, causal, dout)
    assert_within("dQ", qc.grad, rq, e["dq"])
    assert_within("dK", kc.grad, rk, e["dk"])
    assert_within("dV", vc.grad, rv, e["dv"])


def test_varlen_autograd_matches_explicit_calls():
    lengths = [300, 1, 1029, 128]
    q, k, v, dout, cu = make_varlen(32, lengths, 4, 2)
    cuc = cu.cuda()
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    out = ag.attention_varlen(qc, kc, vc, cuc, cuc, max(lengths), max(lengths), True, deterministic=True)
    out.backward(dout.cuda())
    ref_out, lse = min_fa3_op.forward_varlen(q.cuda(), k.cuda(), v.cuda(), cuc, cuc, max(lengths), max(lengths), True,
                                             cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, return_lse=True)
    dq, dk, dv = min_fa3_op.backward_varlen(dout.cuda(), q.cuda(), k.cuda(), v.cuda(), ref_out, lse, cuc, cuc,
                                            max(lengths), max(lengths), True, deterministic=True)
    assert torch.equal(out, ref_out)
    assert torch.equal(qc.grad, dq) and torch.equal(kc.grad, dk) and torch.equal(vc.grad, dv)


def test_operators_compose_with_other_autograd_nodes():
    # A projection before and a reduction after the attention: gradients flow through both.
    q, k, v, _ = make_bshd(33, 1, 256, 4, 4)
    w = torch.eye(128, device="cuda", dtype=torch.bfloat16).requires_grad_()
    qc = q.cuda()
    out = ag.attention(qc @ w, k.cuda(), v.cuda(), True)
    out.float().square().mean().backward()
    assert w.grad is not None and torch.isfinite(w.grad.float()).all() and w.grad.float().abs().sum() > 0
