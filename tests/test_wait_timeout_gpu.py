"""A bounded device-side wait that runs out, on one GPU, without faulting or hanging anything.

Every spin wait of the kernels has a time limit; when it passes, the waiter records
(wait site, CTA) in the workspace's status word and returns, and the host reads it with
``b2a_check_status``.  The wait chosen here is the single-thread kernel that ends the
context-parallel backward: it waits until the rank's completion counter reaches the world
size.  The test presets the counter to -5 (the protocol wants 0), so the one signal of a
world-size-1 run leaves it at -4 and the wait must give up after its limit -- shortened to
50 ms through ``b2a_set_wait_timeout_ns``.  The kernel returns by itself, the context stays
usable, and the same call with a properly zeroed counter then succeeds.
"""
from __future__ import annotations

import time

import pytest
import torch

import min_fa3_op
from gpu_util import assert_within, make_varlen
from min_fa3_demo_b200 import _cabi
from min_fa3_demo_b200.ring import dkv_accum_numel
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def test_completion_wait_runs_out_and_reports_status():
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    lengths, qh, kvh = [256, 128], 4, 2
    q, k, v, dout, cu = make_varlen(5, lengths, qh, kvh)
    cap = 384
    arena_k = torch.zeros(cap, kvh, 128, dtype=torch.bfloat16, device=dev)
    arena_v = torch.zeros_like(arena_k)
    arena_k[:k.size(0)], arena_v[:v.size(0)] = k.to(dev), v.to(dev)
    rk = min_fa3_op.TKParallelTensor(arena_k, local_rank=0, local_world_size=1, multicast=False)
    rv = min_fa3_op.TKParallelTensor(arena_v, local_rank=0, local_world_size=1, multicast=False)
    numel = dkv_accum_numel(kvh, cap, len(lengths))
    acc_k = min_fa3_op.TKParallelTensor([numel], torch.float32, 0, 1, False)
    acc_v = min_fa3_op.TKParallelTensor([numel], torch.float32, 0, 1, False)
    done = min_fa3_op.TKParallelTensor([1], torch.int32, 0, 1, False)
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    meta = dict(global_seqlens_host=torch.tensor(lengths, dtype=torch.int32),
                ring_sizes_host=torch.ones(2, dtype=torch.int32), ring_starts_host=torch.zeros(2, dtype=torch.int32))
    qd, dd, cud = q.to(dev), dout.to(dev), cu.to(dev)
    out, lse = min_fa3_op.forward_varlen_mega_ring(
        qd, arena_k, arena_v, cud, cud, 256, 256, True, cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, remote_k=rk,
        remote_v=rv, num_comp_sm=sm, num_comm_sm=0, return_lse=True, **meta)

    def backward():
        return min_fa3_op.backward_varlen_mega_ring(
            dd, qd, arena_k, arena_v, out, lse, cud, cud, 256, 256, cu_seqlens_q_host=cu, cu_seqlens_k_host=cu,
            remote_k=rk, remote_v=rv, remote_dk_accum=acc_k, remote_dv_accum=acc_v, remote_dkv_completion=done,
            num_comp_sm=sm, num_comm_sm=0, **meta)

    with pytest.raises(RuntimeError, match="wait timeout must be between"):
        _cabi.check(lib.b2a_set_wait_timeout_ns(10))
    _cabi.check(lib.b2a_set_wait_timeout_ns(5_000_000))      # 5 ms; the completion wait gets 10x
    try:
        acc_k.data_.zero_(); acc_v.data_.zero_()
        done.data_.fill_(-5)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        backward()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        with pytest.raises(RuntimeError, match=r"bounded wait timed out \(wait site 26"):
            min_fa3_op.check_last_status("backward_varlen_mega_ring")
        assert 0.04 <= elapsed < 2.0, f"the wait should give up after about 50 ms, took {elapsed:.3f} s"
        assert done.data_.item() == -4          # the rank's own signal arrived; nothing else did
    finally:
        _cabi.check(lib.b2a_set_wait_timeout_ns(0))          # back to the default

    # The context is intact: the same call with the counter zeroed as the protocol demands succeeds.
    acc_k.data_.zero_(); acc_v.data_.zero_(); done.data_.zero_()
    torch.cuda.synchronize()
    dq, dk, dv = backward()
    torch.cuda.synchronize()
    min_fa3_op.check_last_status("backward_varlen_mega_ring")
    assert done.data_.item() == 1
    rq, rk_, rv_ = orc.varlen_backward(q, k, v, dout, cu.tolist(), cu.tolist(), True)
    e = {"dq": 0.0, "dk": 0.0, "dv": 0.0}
    for i in range(len(lengths)):
        s, t = int(cu[i]), int(cu[i + 1])
        errs = orc.bf16_attention_error(q[s:t][None], k[s:t][None], v[s:t][None], True, dout[s:t][None])
        for key in e:
            e[key] = max(e[key], errs[key])
    assert_within("dQ", dq, rq, e["dq"])
    assert_within("dK", dk, rk_, e["dk"])
    assert_within("dV", dv, rv_, e["dv"])
