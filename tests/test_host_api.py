"""Host-side behaviour of the min_fa3_op mirror that needs no GPU: launch-grid override
resolution and argument validation order/messages (reference: bindings.cpp:32-62, 240-331;
include/min_fa3_launch_override.h:16-52; csrc/backward/min_fa3_bwd_bindings.cu:156-190)."""
from __future__ import annotations

import pytest
import torch

import min_fa3_op
from min_fa3_demo_b200 import min_fa3_op as op


def test_root_module_reexports_api():
    for name in ("forward", "forward_varlen", "backward", "backward_varlen"):
        assert getattr(min_fa3_op, name) is getattr(op, name)


def test_resolve_launch_grid_shape():
    assert op._debug_resolve_launch_grid_shape(132) == (132, 1, 1)
    assert op._debug_resolve_launch_grid_shape(132, manual_block_count=7) == (7, 1, 1)
    with pytest.raises(ValueError, match="only supports the current 1D persistent grid"):
        op._debug_resolve_launch_grid_shape(4, 2, 1, manual_block_count=7)
    with pytest.raises(ValueError, match="must be greater than 0"):
        op._debug_resolve_launch_grid_shape(4, manual_block_count=0)
    with pytest.raises(ValueError, match="32-bit grid.x"):
        op._debug_resolve_launch_grid_shape(4, manual_block_count=2**31)
    with pytest.raises(RuntimeError, match="auto_grid_x must be between 0"):
        op._debug_resolve_launch_grid_shape(-1)


def _bshd(b=1, s=8, h=2, d=128, dtype=torch.bfloat16):
    return torch.zeros(b, s, h, d, dtype=dtype)


def test_forward_rejects_bad_inputs_before_any_launch():
    q, k, v = _bshd(), _bshd(), _bshd()
    with pytest.raises(ValueError, match="manual_block_count must be greater than 0"):
        op.forward(q, k, v, True, manual_block_count=-3)
    with pytest.raises(RuntimeError, match="q must be a CUDA tensor"):
        op.forward(q, k, v, True)


def test_backward_rejects_bad_inputs_before_any_launch():
    q = _bshd()
    lse = torch.zeros(1, 2, 8)
    with pytest.raises(RuntimeError, match="q must be a CUDA tensor"):
        op.backward(q, q, q, q, q, lse, True)


@pytest.mark.parametrize("bad,msg", [
    (dict(dtype=torch.float16), "must have dtype torch.bfloat16"),
    (dict(d=64), "must have head_dim D=128"),
])
def test_check_helpers_messages(bad, msg):
    t = _bshd(**bad)
    # the device check comes first in the reference; emulate a CUDA tensor by checking the
    # remaining rules directly
    with pytest.raises(RuntimeError, match=msg):
        op._check(t.dtype == torch.bfloat16, "q must have dtype torch.bfloat16")
        op._check(t.size(3) == 128, "q must have head_dim D=128")


def test_varlen_host_checks():
    cu_dev_like = torch.tensor([0, 4, 8], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="must have dtype torch.int32"):
        op._check_cu_seqlens_host(torch.tensor([0, 4, 8]), cu_dev_like, "cu_seqlens_q_host")
    with pytest.raises(RuntimeError, match="same length as its CUDA cu_seqlens tensor"):
        op._check_cu_seqlens_host(torch.tensor([0, 8], dtype=torch.int32), cu_dev_like,
                                  "cu_seqlens_q_host")
    op._check_cu_seqlens_host(cu_dev_like.clone(), cu_dev_like, "cu_seqlens_q_host")
