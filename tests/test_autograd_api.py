"""Differentiable front end, CPU part: the torch.library operators exist, carry fake (meta)
implementations with the right shapes, and refuse CPU tensors (there is no CPU fallback)."""
from __future__ import annotations

import pytest
import torch

from min_fa3_demo_b200 import autograd as ag


def test_operators_are_registered_with_schemas():
    assert str(torch.ops.b200attn.fwd.default._schema).startswith("b200attn::fwd(Tensor q, Tensor k, Tensor v, bool is_causal)")
    assert "bool deterministic" in str(torch.ops.b200attn.bwd.default._schema)


def test_fake_implementations_give_shapes_and_dtypes():
    q = torch.empty(2, 384, 8, 128, dtype=torch.bfloat16, device="meta")
    k = torch.empty(2, 512, 2, 128, dtype=torch.bfloat16, device="meta")
    out, lse = torch.ops.b200attn.fwd(q, k, k, True)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    assert lse.shape == (2, 8, 384) and lse.dtype == torch.float32
    dq, dk, dv = torch.ops.b200attn.bwd(out, q, k, k, out, lse, True, False)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape


def test_cpu_tensors_are_rejected():
    q = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, requires_grad=True)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ag.attention(q, q, q, True)
    cu = torch.tensor([0, 128], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ag.attention_varlen(q[0], q[0], q[0], cu, cu, 128, 128, True)
