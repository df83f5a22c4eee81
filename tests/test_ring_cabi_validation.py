"""The C ABI validates context-parallel metadata on the host before it touches the device, so
the native entry point can be exercised without a GPU: invalid placements must come back as
B2A_ERR_INVALID_ARGUMENT with a message, never as a launch.  (Pointers are dummies; a valid
placement proceeds to the device query, which fails cleanly on a machine without a GPU.)"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from min_fa3_demo_b200 import _cabi


def call(cu, glens, sizes, starts, *, world=4, rank=0, cap=4096, causal=1, comp=140, comm=8, heads=(8, 2),
         workspace_bytes=0):
    lib = _cabi.load()
    arrs = [np.asarray(a, dtype=np.int32) for a in (cu, glens, sizes, starts)]
    a = _cabi.RingFwdArgs()
    dummy = 0x1000
    a.q = a.out = a.lse = a.arena_k = a.arena_v = a.workspace = dummy
    for r in range(world):
        a.peer_k[r] = dummy
        a.peer_v[r] = dummy
    a.cu_seqlens_q_host, a.global_seqlens_host, a.ring_sizes_host, a.ring_starts_host = (x.ctypes.data for x in arrs)
    a.batch, a.world_size, a.rank, a.rank_kv_capacity = len(glens), world, rank, cap
    a.total_q = int(cu[-1])
    a.heads_q, a.heads_k, a.head_dim, a.is_causal = heads[0], heads[1], 128, causal
    a.num_comp_sm, a.num_comm_sm = comp, comm
    a.workspace_bytes = workspace_bytes     # 0: even a valid call stops at the workspace check, never launches
    rc = lib.b2a_ring_fwd(ctypes.byref(a), None)
    return rc, lib.b2a_last_error().decode()


@pytest.mark.parametrize("kwargs,fragment", [
    (dict(cu=[0, 512], glens=[2048], sizes=[3], starts=[0]), "ring size must be 1, 2, 4 or 8"),
    (dict(cu=[0, 256, 768], glens=[512, 2048], sizes=[2, 4], starts=[0, 0]), "non-increasing ring size"),
    (dict(cu=[0, 512], glens=[1024], sizes=[2], starts=[1]), "ring"),
    (dict(cu=[0, 512], glens=[2050], sizes=[4], starts=[0]), "multiple of ring size"),
    (dict(cu=[0, 384], glens=[1536], sizes=[4], starts=[0]), "halves must be multiples of 128"),
    (dict(cu=[0, 100], glens=[100], sizes=[1], starts=[0]), "multiple of 128"),
    (dict(cu=[0, 512], glens=[2048], sizes=[4], starts=[0], world=3), "world size must be 1, 2, 4 or 8"),
    (dict(cu=[0, 512], glens=[2048], sizes=[4], starts=[0], cap=100), "rank_kv_capacity"),
    (dict(cu=[0, 512], glens=[2048], sizes=[4], starts=[0], heads=(8, 3)), "heads_q % heads_k"),
    (dict(cu=[0, 512], glens=[2048], sizes=[4], starts=[0], comp=0), "num_comp_sm must be positive"),
])
def test_invalid_metadata_is_rejected_before_any_device_call(kwargs, fragment):
    rc, msg = call(**kwargs)
    assert rc == _cabi.B2A_ERR_INVALID_ARGUMENT, (rc, msg)
    assert fragment in msg, msg


def test_valid_metadata_passes_validation():
    # rank 0 of 4: member of the 4-ring and of the 2-ring at start 0, not of the document on rank 3
    rc, msg = call(cu=[0, 512, 1024, 1024], glens=[2048, 1024, 256], sizes=[4, 2, 1], starts=[0, 0, 3])
    # The metadata is accepted; the call then stops at the device query (no GPU) or at the
    # workspace-size check (GPU present) -- in both cases before anything is launched.
    assert rc in (_cabi.B2A_ERR_CUDA, _cabi.B2A_ERR_WORKSPACE_TOO_SMALL, _cabi.B2A_ERR_UNSUPPORTED_DEVICE), (rc, msg)


# --------------------------------------------------------------------------------------
# Planner <-> launcher contract: every plan the placement planner produces passes the native
# metadata validation on every rank (checked without a GPU: the call stops at the device query
# or at the workspace-size check, never at "invalid argument").
# --------------------------------------------------------------------------------------
from hypothesis import given, settings, strategies as st  # noqa: E402

from min_fa3_demo_b200 import balancer as bal  # noqa: E402


@settings(max_examples=25, deadline=None)
@given(lengths=st.lists(st.integers(min_value=1, max_value=64).map(lambda n: n * 256), min_size=1, max_size=8),
       world=st.sampled_from([2, 4, 8]), causal=st.booleans())
def test_planner_output_is_accepted_by_the_launcher(lengths, world, causal):
    plan = bal.assign_hierarchical_rings(lengths, world, causal)
    cap = max(plan.rank_tokens)
    cap = ((cap + 127) // 128) * 128
    for rank in range(world):
        _, cu = bal.local_layout(plan, rank)
        rc, msg = call(cu=cu, glens=plan.global_lengths, sizes=plan.ring_sizes, starts=plan.ring_starts,
                       world=world, rank=rank, cap=max(cap, 128), causal=int(causal))
        assert rc != _cabi.B2A_ERR_INVALID_ARGUMENT, (rank, msg)


# --------------------------------------------------------------------------------------
# Backward entry point: a sharded document needs copy CTAs for the second pull of the remote
# K/V -- unless the caller states that the forward's blocks are still in the arena.
# --------------------------------------------------------------------------------------
def call_bwd(*, comm, kv_resident):
    lib = _cabi.load()
    cu, glens, sizes, starts = (np.asarray(a, dtype=np.int32) for a in ([0, 512], [2048], [4], [0]))
    a = _cabi.RingBwdArgs()
    dummy = 0x1000
    a.dout = a.q = a.out = a.lse = a.dq = a.dk = a.dv = a.arena_k = a.arena_v = a.workspace = dummy
    for r in range(4):
        a.peer_k[r] = a.peer_v[r] = a.dk_accum_peer[r] = a.dv_accum_peer[r] = a.completion_peer[r] = dummy
    a.cu_seqlens_q_host, a.global_seqlens_host, a.ring_sizes_host, a.ring_starts_host = (
        x.ctypes.data for x in (cu, glens, sizes, starts))
    a.batch, a.world_size, a.rank, a.rank_kv_capacity = 1, 4, 0, 4096
    a.total_q = a.local_total_k = 512
    a.heads_q, a.heads_k, a.head_dim, a.is_causal = 8, 2, 128, 1
    a.num_comp_sm, a.num_comm_sm, a.kv_resident = 140, comm, kv_resident
    a.workspace_bytes = 0                  # a valid call stops at the workspace check at the latest
    rc = lib.b2a_ring_bwd(ctypes.byref(a), None)
    return rc, lib.b2a_last_error().decode()


def test_backward_without_copy_ctas_needs_resident_kv():
    rc, msg = call_bwd(comm=0, kv_resident=0)
    assert rc == _cabi.B2A_ERR_INVALID_ARGUMENT and "num_comm_sm must be positive" in msg, (rc, msg)
    for comm, resident in ((0, 1), (8, 0), (8, 1)):
        rc, msg = call_bwd(comm=comm, kv_resident=resident)
        assert rc in (_cabi.B2A_ERR_CUDA, _cabi.B2A_ERR_WORKSPACE_TOO_SMALL, _cabi.B2A_ERR_UNSUPPORTED_DEVICE), (rc, msg)
