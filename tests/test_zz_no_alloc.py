"""``b2a_fwd_noalloc``: the forward entry point for callers that cannot allocate device memory
(a plugin living inside a fixed memory pool, a real-time loop that must stay away from the
allocator).  Its scratch is an array built into the library, so the test calls it through the
C ABI with inputs and outputs only and compares with ``b2a_fwd`` given an ordinary workspace.
Two calls in a row check that the shared scratch is re-initialised correctly by each call.
This file sorts last so that a run stopping at the first failure has already run the rest.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from min_fa3_demo_b200 import _cabi

pytestmark = pytest.mark.gpu


def _args(q, k, v, out, lse, causal, cu=None, max_len=0):
    a = _cabi.FwdArgs()
    a.q, a.k, a.v, a.out, a.lse = (t.data_ptr() for t in (q, k, v, out, lse))
    if cu is None:
        b, s, qh = q.shape[0], q.shape[1], q.shape[2]
        a.batch, a.seqlen_q, a.seqlen_k = b, s, k.shape[1]
        a.total_q, a.total_k = b * s, b * k.shape[1]
        a.heads_q, a.heads_k = qh, k.shape[2]
    else:
        a.cu_seqlens_q = a.cu_seqlens_k = cu.data_ptr()
        a.batch, a.seqlen_q, a.seqlen_k = cu.numel() - 1, max_len, max_len
        a.total_q, a.total_k = q.shape[0], k.shape[0]
        a.heads_q, a.heads_k = q.shape[1], k.shape[1]
    a.head_dim = 128
    a.is_causal = int(causal)
    return a


def _run_with_workspace(lib, a):
    varlen = 1 if a.cu_seqlens_q else 0
    nbytes = lib.b2a_fwd_workspace_bytes(a.batch, a.total_q, varlen)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _cabi.check(lib.b2a_fwd(ctypes.byref(a), stream))
    torch.cuda.synchronize()


def _run_noalloc(lib, a):
    a.workspace, a.workspace_bytes = None, 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _cabi.check(lib.b2a_fwd_noalloc(ctypes.byref(a), stream))
    torch.cuda.synchronize()


def test_noalloc_forward_matches_regular_entry_point_twice_in_a_row():
    lib = _cabi.load()
    gen = torch.Generator().manual_seed(2024)

    # call 1: fixed-length BSHD, causal, GQA
    q = torch.randn(2, 512, 8, 128, generator=gen).to(torch.bfloat16).cuda()
    k = torch.randn(2, 512, 2, 128, generator=gen).to(torch.bfloat16).cuda()
    v = torch.randn(2, 512, 2, 128, generator=gen).to(torch.bfloat16).cuda()
    ref_out, ref_lse = torch.empty_like(q), torch.empty(2, 8, 512, device="cuda")
    _run_with_workspace(lib, _args(q, k, v, ref_out, ref_lse, True))
    out, lse = torch.full_like(q, 7.0), torch.full((2, 8, 512), 7.0, device="cuda")
    _run_noalloc(lib, _args(q, k, v, out, lse, True))
    # same kernel, same inputs: the tolerance of the other forward tests is 2x a bf16 error,
    # here the results are in fact identical
    assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)

    # call 2, right after: packed varlen with ragged documents (uses the work list in the
    # shared scratch, which still holds call 1's header)
    lengths = [300, 77, 512, 1, 129]
    cu = torch.tensor([0, 300, 377, 889, 890, 1019], dtype=torch.int32, device="cuda")
    qv = torch.randn(1019, 4, 128, generator=gen).to(torch.bfloat16).cuda()
    kv = torch.randn(1019, 2, 128, generator=gen).to(torch.bfloat16).cuda()
    vv = torch.randn(1019, 2, 128, generator=gen).to(torch.bfloat16).cuda()
    ref_out, ref_lse = torch.empty_like(qv), torch.empty(4, 1019, device="cuda")
    _run_with_workspace(lib, _args(qv, kv, vv, ref_out, ref_lse, True, cu, max(lengths)))
    for _ in range(2):
        out, lse = torch.full_like(qv, 7.0), torch.full((4, 1019), 7.0, device="cuda")
        _run_noalloc(lib, _args(qv, kv, vv, out, lse, True, cu, max(lengths)))
        assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)
        # the status word of the built-in scratch is read by passing no workspace
        assert lib.b2a_check_status(None, None) == _cabi.B2A_OK, _cabi.last_error()

    # and the result is right on its own account, not only equal to the other entry point
    from oracle import attention_oracle as orc
    cu_list = cu.cpu().tolist()
    want_out, want_lse = orc.varlen_forward(qv.cpu(), kv.cpu(), vv.cpu(), cu_list, cu_list, True)
    assert (out.float().cpu() - want_out).abs().max().item() <= 1.6e-2
    assert (lse.cpu() - want_lse).abs().max().item() <= 1e-3


def test_noalloc_rejects_problems_beyond_its_scratch():
    lib = _cabi.load()
    limit = lib.b2a_fwd_noalloc_scratch_limit()
    assert limit == 64 * 1024
    # a packed batch of 2.2M tokens needs a work list larger than the built-in scratch;
    # the check happens before any pointer is touched
    a = _cabi.FwdArgs()
    a.q = a.k = a.v = a.out = a.lse = 256
    a.cu_seqlens_q = a.cu_seqlens_k = 256
    a.batch, a.total_q, a.total_k = 16, 2_200_000, 2_200_000
    a.heads_q = a.heads_k = 1
    a.head_dim = 128
    rc = lib.b2a_fwd_noalloc(ctypes.byref(a), None)
    assert rc == _cabi.B2A_ERR_WORKSPACE_TOO_SMALL
    assert "built-in scratch" in _cabi.last_error()
