"""Host-side argument validation of the context-parallel backward, walked through the negative
cases of the reference's own test
(scripts/test_mega_ring/mega_ring_test_min_fa3_varlen_backward_validation_multi_rank.py:48-224):
every case must raise ``RuntimeError`` whose text contains the substring the reference test
matches on, before anything is launched.  The table is restated here for an 8-rank world and
runs on the CPU: the dense tensors are CPU tensors (the validator's ``device_type`` argument
stands in for "cuda"), the parallel tensors are bare ``TKParallelTensor`` objects without peers.

One case differs from the reference table.  ``accumulator_capacity`` there passes accumulators
that are *larger* than needed and expects a rejection, i.e. it was written for an exact-size
rule; the reference binding checks ``numel >= KVH * padded_rank_capacity * 128``
(csrc/backward/min_fa3_bwd_bindings.cu:636-640), and its own benchmarks allocate more than the
minimum (ring_test/benchmark_topology_backward.py:459-497).  This implementation follows the
binding, so the case is exercised with accumulators one element too small.
"""
from __future__ import annotations

import pytest
import torch

from min_fa3_demo_b200 import ring
from min_fa3_demo_b200.parallel import TKParallelTensor

WORLD = 8
Q_HEADS, KV_HEADS, HEAD_DIM = 16, 8, 128
BASE_RANK_CAPACITY = 512


def int32(values):
    return torch.tensor(values, dtype=torch.int32)


def noncontiguous_int32(values):
    storage = torch.empty((2 * len(values),), dtype=torch.int32)
    view = storage[::2]
    view.copy_(int32(values))
    assert not view.is_contiguous()
    return view


def parallel(shape, dtype, rank):
    """A parallel tensor without peers: enough for the host-side checks, which never dereference
    ``raw_ptrs_``."""
    t = TKParallelTensor.__new__(TKParallelTensor)
    t.data_ = torch.zeros(shape, dtype=dtype)
    t.local_rank_, t.local_world_size_ = rank, WORLD
    t.raw_ptrs_ = [0] * WORLD
    t._imported = []
    return t


def make_cases(rank):
    valid_global, valid_rings, valid_starts = int32([2048]), int32([8]), int32([0])
    nonmember_lengths = [0] * WORLD
    nonmember_lengths[rank] = 128
    nonmember_lengths[(rank + 1) % WORLD] = 128
    base = dict(global_=valid_global, rings=valid_rings, starts=valid_starts)
    return [
        dict(name="host_cu_seqlens_dtype", expected="host cu_seqlens tensors must have dtype int32",
             q_lengths=[0], q_host_override=torch.tensor([0, 0], dtype=torch.int64), **base),
        dict(name="topology_metadata_device", expected="global_seqlens_host must be a CPU tensor",
             q_lengths=[0], global_=valid_global.to("meta"), rings=valid_rings, starts=valid_starts),
        dict(name="topology_metadata_dtype", expected="global_seqlens_host must have dtype int32",
             q_lengths=[0], global_=torch.tensor([2048], dtype=torch.int64), rings=valid_rings, starts=valid_starts),
        dict(name="topology_metadata_shape", expected="ring_starts_host must have shape [B]",
             q_lengths=[0], global_=valid_global, rings=valid_rings, starts=int32([0, 0])),
        dict(name="topology_metadata_contiguity", expected="ring_sizes_host must be contiguous",
             q_lengths=[0, 0], global_=int32([2048, 1024]), rings=noncontiguous_int32([8, 4]), starts=int32([0, 4])),
        dict(name="unordered_ring_sizes", expected="batch must be ordered by non-increasing ring size",
             q_lengths=[256 if rank < 2 else 0, 256 if rank < 4 else 0], global_=int32([512, 1024]),
             rings=int32([2, 4]), starts=int32([0, 0])),
        dict(name="unsupported_ring_size", expected="ring_sizes_host must contain only 1, 2, 4, or 8",
             q_lengths=[0], global_=int32([384]), rings=int32([3]), starts=int32([0])),
        dict(name="misaligned_ring_start", expected="invalid aligned ring range",
             q_lengths=[0], global_=int32([512]), rings=int32([2]), starts=int32([1])),
        dict(name="ring_range_crosses_world", expected="invalid aligned ring range",
             q_lengths=[0], global_=int32([512]), rings=int32([2]), starts=int32([WORLD])),
        dict(name="global_length_not_divisible", expected="global length must be divisible by ring size",
             q_lengths=[0], global_=int32([1025]), rings=int32([8]), starts=int32([0])),
        dict(name="nonmember_has_local_rows", expected="local q/k length does not match ring metadata",
             q_lengths=nonmember_lengths, global_=int32([128] * WORLD), rings=int32([1] * WORLD),
             starts=int32(list(range(WORLD)))),
        dict(name="member_length_mismatch", expected="local q/k length does not match ring metadata",
             q_lengths=[128], **base),
        dict(name="self_attention_length_mismatch", expected="self-attention q_len == k_len",
             q_lengths=[128], k_lengths=[256], **base),
        dict(name="local_length_alignment", expected="every local q/k length must be 128-row aligned",
             q_lengths=[130], global_=int32([1040]), rings=valid_rings, starts=valid_starts),
        dict(name="arena_capacity_insufficient", expected="local_total_k must fit in rank_kv_capacity",
             q_lengths=[256], arena="small", **base),
        dict(name="arena_capacity_unaligned", expected="rank_kv_capacity must be 128-row aligned",
             q_lengths=[128], global_=int32([1024]), rings=valid_rings, starts=valid_starts, arena="unaligned"),
        dict(name="causal_half_unaligned", expected="G2/G4/G8 local half length must be 128-row aligned",
             q_lengths=[128], global_=int32([1024]), rings=valid_rings, starts=valid_starts),
        dict(name="accumulator_dtype", expected="remote dK/dV accumulators must have dtype float32",
             q_lengths=[256], accum="dtype", **base),
        dict(name="accumulator_capacity", expected="remote dK/dV accumulators must each contain",
             q_lengths=[256], accum="short", **base),
        dict(name="completion_shape", expected="remote_dkv_completion must be a one-element int32 parallel tensor",
             q_lengths=[256], completion="shape", **base),
    ]


def cu(lengths):
    out = [0]
    for n in lengths:
        out.append(out[-1] + n)
    return int32(out)


def run_case(case, rank):
    arenas = {"base": BASE_RANK_CAPACITY, "small": 128, "unaligned": 129}
    cap = arenas[case.get("arena", "base")]
    remote_k = parallel([WORLD * cap, KV_HEADS, HEAD_DIM], torch.bfloat16, rank)
    remote_v = parallel([WORLD * cap, KV_HEADS, HEAD_DIM], torch.bfloat16, rank)
    guard = KV_HEADS * (BASE_RANK_CAPACITY + (WORLD + 1) * 128) * HEAD_DIM
    accum = case.get("accum", "guard")
    if accum == "dtype":
        acc = [parallel([1], torch.bfloat16, rank) for _ in range(2)]
    elif accum == "short":
        need = ring.dkv_accum_numel(KV_HEADS, 256, 1)
        acc = [parallel([need - 1], torch.float32, rank) for _ in range(2)]
    else:
        acc = [parallel([guard], torch.float32, rank) for _ in range(2)]
    completion = parallel([2 if case.get("completion") == "shape" else 1], torch.int32, rank)

    q_lengths = case["q_lengths"]
    k_lengths = case.get("k_lengths", q_lengths)
    cu_q_host, cu_k_host = cu(q_lengths), cu(k_lengths)
    total_q = int(cu_q_host[-1])
    q = torch.zeros((total_q, Q_HEADS, HEAD_DIM), dtype=torch.bfloat16)
    lse = torch.zeros((Q_HEADS, total_q), dtype=torch.float32)
    return ring._validate_backward_mega_ring(
        torch.zeros_like(q), q, remote_k.data_, remote_v.data_, torch.zeros_like(q), lse, cu_q_host.clone(),
        cu_k_host.clone(), 256, 256, case.get("q_host_override", cu_q_host), cu_k_host, remote_k, remote_v,
        acc[0], acc[1], completion, 1, 1, case["global_"], case["rings"], case["starts"], True, device_type="cpu")


CASE_NAMES = [c["name"] for c in make_cases(0)]


def test_table_has_the_twenty_reference_cases():
    assert len(CASE_NAMES) == 20 and len(set(CASE_NAMES)) == 20


@pytest.mark.parametrize("rank", [0, 3, 7])
@pytest.mark.parametrize("index", range(20), ids=CASE_NAMES)
def test_invalid_backward_arguments_raise_the_reference_text(index, rank):
    case = make_cases(rank)[index]
    with pytest.raises(RuntimeError) as info:
        run_case(case, rank)
    assert case["expected"] in str(info.value), f"{case['name']}: got {info.value!r}"


@pytest.mark.parametrize("rank", [0, 5])
def test_valid_arguments_pass_and_return_the_layout(rank):
    case = dict(q_lengths=[256], global_=int32([2048]), rings=int32([8]), starts=int32([0]))
    world, got_rank, cap, batch, local_total_k = run_case(case, rank)
    assert (world, got_rank, cap, batch, local_total_k) == (WORLD, rank, BASE_RANK_CAPACITY, 1, 256)


def test_accumulator_rule_is_the_reference_formula():
    # KVH * round128(logical_rank_capacity + B * 128) * 128 (min_fa3_bwd_bindings.cu:630-640)
    assert ring.dkv_accum_numel(8, 16384, 1) == 8 * (16384 + 128) * 128
    assert ring.dkv_accum_numel(2, 300, 3) == 2 * 768 * 128
