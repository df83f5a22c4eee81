"""Context-parallel metadata validation runs on the host before any launch; the texts follow
the reference bindings (csrc/mega_ring_min_fa3_varlen_ring_bindings.cu:404-470), whose
negative test matches on them
(scripts/test_mega_ring/mega_ring_test_min_fa3_varlen_backward_validation_multi_rank.py:48-224)."""
from __future__ import annotations

import pytest
import torch

from min_fa3_demo_b200 import ring


def i32(*values):
    return torch.tensor(list(values), dtype=torch.int32)


def validate(cu, glens, sizes, starts, *, world=4, rank=0, causal=True, rows=4096, cap_rows=None, max_len=4096):
    q = torch.empty(int(cu[-1]), 2, 128, dtype=torch.bfloat16)
    arena = torch.empty(cap_rows if cap_rows is not None else world * rows, 2, 128, dtype=torch.bfloat16)
    return ring._validate_ring_metadata(q, arena, i32(*cu), i32(*cu), i32(*glens), i32(*sizes), i32(*starts),
                                        world, rank, causal, max_len, max_len)


def test_valid_metadata_returns_capacity():
    # rank 0 of 4: member of the 4-ring and the 2-ring at start 0, not of the single-rank doc on rank 3
    assert validate([0, 512, 1024, 1024], [2048, 1024, 256], [4, 2, 1], [0, 0, 3]) == 4096


@pytest.mark.parametrize("kwargs,msg", [
    (dict(cu=[0, 512], glens=[2048], sizes=[3], starts=[0]), "ring_sizes_host must contain only 1, 2, 4, or 8"),
    (dict(cu=[0, 256, 768], glens=[512, 2048], sizes=[2, 4], starts=[0, 0]),
     "batch must be ordered by non-increasing ring size"),
    (dict(cu=[0, 512], glens=[1024], sizes=[2], starts=[1]), "invalid aligned ring range"),
    (dict(cu=[0, 512], glens=[1024], sizes=[2], starts=[4]), "invalid aligned ring range"),
    (dict(cu=[0, 512], glens=[2050], sizes=[4], starts=[0]), "global length must be divisible by ring size"),
    (dict(cu=[0, 256], glens=[2048], sizes=[4], starts=[0]), "does not match hierarchical ring metadata"),
    (dict(cu=[0, 384], glens=[1536], sizes=[4], starts=[0]), "causal CP half length must be 128-aligned"),
    (dict(cu=[0, 100], glens=[100], sizes=[1], starts=[0]), "128-row aligned"),
    (dict(cu=[0, 512], glens=[0], sizes=[1], starts=[0]), "global_seqlens_host must be positive"),
    (dict(cu=[0, 512], glens=[512], sizes=[1], starts=[0], max_len=256), "must cover every local sequence"),
    (dict(cu=[0, 512], glens=[512], sizes=[1], starts=[0], cap_rows=4 * 256), "exceeds rank_kv_capacity"),
    (dict(cu=[0, 512], glens=[512], sizes=[1], starts=[0], cap_rows=4 * 200), "128-row aligned"),
    (dict(cu=[0, 512], glens=[512], sizes=[1], starts=[0], cap_rows=4 * 4096 + 1), "divisible by world_size"),
])
def test_invalid_metadata_is_rejected_before_any_launch(kwargs, msg):
    with pytest.raises(RuntimeError, match=msg):
        validate(**kwargs)


def test_non_member_rank_must_hold_no_tokens():
    # rank 3 is outside the ring [0, 2): its local length must be 0
    with pytest.raises(RuntimeError, match="does not match hierarchical ring metadata"):
        validate([0, 512], [1024], [2], [0], rank=3)
    assert validate([0, 0], [1024], [2], [0], rank=3) == 4096


def test_host_vectors_are_checked():
    q = torch.empty(512, 2, 128, dtype=torch.bfloat16)
    arena = torch.empty(4 * 1024, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="ring_sizes_host must have dtype torch.int32"):
        ring._validate_ring_metadata(q, arena, i32(0, 512), i32(0, 512), i32(512),
                                     torch.tensor([1]), i32(0), 4, 0, True, 512, 512)
    with pytest.raises(RuntimeError, match=r"ring_starts_host must have shape \[B\]"):
        ring._validate_ring_metadata(q, arena, i32(0, 512), i32(0, 512), i32(512), i32(1), i32(0, 0),
                                     4, 0, True, 512, 512)


# Planner output always passes the host-side validation of the Python entry points.
from hypothesis import given, settings, strategies as st  # noqa: E402

from min_fa3_demo_b200 import balancer as bal  # noqa: E402


@settings(max_examples=25, deadline=None)
@given(lengths=st.lists(st.integers(min_value=1, max_value=64).map(lambda n: n * 256), min_size=1, max_size=8),
       world=st.sampled_from([2, 4, 8]), causal=st.booleans())
def test_planner_output_passes_python_validation(lengths, world, causal):
    plan = bal.assign_hierarchical_rings(lengths, world, causal)
    cap = ((max(plan.rank_tokens) + 127) // 128) * 128
    for rank in range(world):
        lens, cu = bal.local_layout(plan, rank)
        q = torch.empty(cu[-1], 2, 128, dtype=torch.bfloat16)
        arena = torch.empty(world * cap, 2, 128, dtype=torch.bfloat16)
        got = ring._validate_ring_metadata(q, arena, i32(*cu), i32(*cu), i32(*plan.global_lengths),
                                           i32(*plan.ring_sizes), i32(*plan.ring_starts), world, rank, causal,
                                           max(max(lens), 1), max(max(lens), 1))
        assert got == cap
