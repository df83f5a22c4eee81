"""Running (out, lse) merge of the forward epilogue on one GPU (``merge_running = 1``; reference:
include/min_fa3_epilogue.h:404-506, ring_test/ring_common.py:59-73).

* the kernel's merge against the golden vector recorded from the reference's own
  ``update_out_and_lse`` (tests/golden/merge_bf16.npz): the block result (O_b, L_b) is forced to
  the fixture's values by giving every query exactly one key;
* split-K: attention over all keys equals two merged calls over the two parts of the keys, and
  both equal the oracle;
* the ring-step decomposition of a causal sequence: second-half queries over the first-half keys
  (unmasked) merged with the second-half keys (causal).
"""
from __future__ import annotations

import math

import pytest
import torch

from conftest import from_bf16_bits, load_golden
from gpu_util import LSE_ATOL, bound, make_varlen
from min_fa3_demo_b200.min_fa3_op import _call_fwd, check_device_status
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def run_fwd(q, k, v, cu_q, cu_k, causal, out=None, lse=None, merge=False):
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    heads_q, heads_k = q.size(1), k.size(1)
    if out is None:
        out = torch.zeros_like(qd) if merge else torch.empty_like(qd)
        fill = float("-inf") if merge else 0.0
        lse = torch.full((heads_q, q.size(0)), fill, dtype=torch.float32, device=DEV)
    lens_q = (cu_q[1:] - cu_q[:-1]).tolist()
    lens_k = (cu_k[1:] - cu_k[:-1]).tolist()
    ws = _call_fwd(qd, kd, vd, out, lse, cu_q=cu_q.to(DEV), cu_k=cu_k.to(DEV), batch=cu_q.numel() - 1,
                   seqlen_q=max(lens_q), seqlen_k=max(lens_k), heads_q=heads_q, heads_k=heads_k,
                   is_causal=causal, merge_running=merge)
    torch.cuda.synchronize()
    check_device_status(ws)
    return out, lse


def split3(x: torch.Tensor):
    """x (fp32) as a sum of three bf16 numbers (24 mantissa bits in all)."""
    a = x.to(torch.bfloat16)
    b = (x - a.float()).to(torch.bfloat16)
    c = (x - a.float() - b.float()).to(torch.bfloat16)
    return a, b, c


def test_merge_epilogue_reproduces_the_reference_merge_fixture():
    g = load_golden("merge_bf16")
    out_a, out_b = from_bf16_bits(g["out_a"]), from_bf16_bits(g["out_b"])          # [16, 4, 128]
    lse_a, lse_b = torch.from_numpy(g["lse_a"]), torch.from_numpy(g["lse_b"])      # [4, 16]
    tokens, heads = out_a.size(0), out_a.size(1)
    # One key per query: O_b = v exactly, and LSE_b = q.k / sqrt(128) with k = (1, 1, 1, 0, ...) and the
    # first three components of q holding lse_b * sqrt(128) split into three bf16 terms.
    k = torch.zeros(tokens, heads, 128, dtype=torch.bfloat16)
    k[:, :, :3] = 1.0
    q = torch.zeros(tokens, heads, 128, dtype=torch.bfloat16)
    a, b, c = split3(lse_b.t().contiguous() * math.sqrt(128.0))
    q[:, :, 0], q[:, :, 1], q[:, :, 2] = a, b, c
    cu = torch.arange(tokens + 1, dtype=torch.int32)
    out, lse = run_fwd(q, k, out_b, cu, cu, False, out=out_a.to(DEV).clone(), lse=lse_a.to(DEV).clone(), merge=True)
    want_out, want_lse = torch.from_numpy(g["merged_out"]), torch.from_numpy(g["merged_lse"])
    torch.testing.assert_close(lse.cpu(), want_lse, rtol=0, atol=1e-4)
    # the kernel rounds the merged output to bf16
    torch.testing.assert_close(out.float().cpu(), want_out, rtol=2.0 ** -8, atol=1e-3)
    # and the oracle's merge is the same function
    o_or, l_or = orc.merge_out_lse(out_a.float(), lse_a, out_b.float(), lse_b)
    torch.testing.assert_close(o_or, want_out, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(l_or, want_lse, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("lengths", [[300, 128, 77], [1024, 513]])
def test_split_k_merge_equals_single_call_and_oracle(lengths):
    qh, kvh = 8, 2
    q, k, v, _dout, cu = make_varlen(11, lengths, qh, kvh)
    first = [(n + 1) // 2 for n in lengths]
    rest = [n - f for n, f in zip(lengths, first)]
    k1 = torch.cat([k[int(cu[i]): int(cu[i]) + first[i]] for i in range(len(lengths))])
    v1 = torch.cat([v[int(cu[i]): int(cu[i]) + first[i]] for i in range(len(lengths))])
    k2 = torch.cat([k[int(cu[i]) + first[i]: int(cu[i + 1])] for i in range(len(lengths))])
    v2 = torch.cat([v[int(cu[i]) + first[i]: int(cu[i + 1])] for i in range(len(lengths))])
    cu1 = torch.tensor([0, *torch.tensor(first).cumsum(0).tolist()], dtype=torch.int32)
    cu2 = torch.tensor([0, *torch.tensor(rest).cumsum(0).tolist()], dtype=torch.int32)

    whole, lse_whole = run_fwd(q, k, v, cu, cu, False)
    out, lse = run_fwd(q, k1, v1, cu, cu1, False, merge=True)              # merges into (0, -inf)
    part_out, part_lse = out.clone(), lse.clone()
    out, lse = run_fwd(q, k2, v2, cu, cu2, False, out=out, lse=lse, merge=True)

    ref_out, ref_lse = orc.varlen_forward(q, k, v, cu.tolist(), cu.tolist(), False)
    e = max(orc.bf16_attention_error(q[int(cu[i]):int(cu[i + 1])][None], k[int(cu[i]):int(cu[i + 1])][None],
                                     v[int(cu[i]):int(cu[i + 1])][None], False)["o"] for i in range(len(lengths)))
    for name, got_o, got_l in (("single call", whole, lse_whole), ("two merged calls", out, lse)):
        err = (got_o.float().cpu() - ref_out).abs().max().item()
        assert err <= bound(e), f"{name}: O error {err:.3e} exceeds {bound(e):.3e}"
        assert (got_l.cpu() - ref_lse).abs().max().item() <= LSE_ATOL, name
    # the first call alone is plain attention over the first part of the keys
    p_out, p_lse = orc.varlen_forward(q, k1, v1, cu.tolist(), cu1.tolist(), False)
    assert (part_out.float().cpu() - p_out).abs().max().item() <= bound(e)
    assert (part_lse.cpu() - p_lse).abs().max().item() <= LSE_ATOL
    # and the kernel's merge agrees with the oracle's merge of the two oracle parts
    o2, l2 = orc.varlen_forward(q, k2, v2, cu.tolist(), cu2.tolist(), False)
    m_out, m_lse = orc.merge_out_lse(p_out, p_lse, o2, l2)
    assert (out.float().cpu() - m_out).abs().max().item() <= bound(e)
    assert (lse.cpu() - m_lse).abs().max().item() <= LSE_ATOL


def test_causal_sequence_as_two_merged_ring_steps():
    qh, kvh, s = 8, 2, 1024
    q, k, v, _dout, cu = make_varlen(12, [s], qh, kvh)
    half = s // 2
    cu_h = torch.tensor([0, half], dtype=torch.int32)
    q2 = q[half:].contiguous()
    # step 0: own (diagonal) chunk with the causal mask; step 1: the earlier chunk, unmasked
    out, lse = run_fwd(q2, k[half:].contiguous(), v[half:].contiguous(), cu_h, cu_h, True, merge=True)
    out, lse = run_fwd(q2, k[:half].contiguous(), v[:half].contiguous(), cu_h, cu_h, False, out=out, lse=lse,
                       merge=True)
    ref_out, ref_lse = orc.varlen_forward(q, k, v, [0, s], [0, s], True)
    e = orc.bf16_attention_error(q[None], k[None], v[None], True)["o"]
    err = (out.float().cpu() - ref_out[half:]).abs().max().item()
    assert err <= bound(e), f"O error {err:.3e} exceeds {bound(e):.3e}"
    assert (lse.cpu() - ref_lse[:, half:]).abs().max().item() <= LSE_ATOL


@pytest.mark.parametrize("rows,blocks", [(333, 4), (1024, 3), (64, 8)])
def test_ring_step_copies_and_computes_in_one_launch(rows, blocks):
    """The ring step's copy CTAs (``prefetch_*`` fields of the forward arguments) ride in the
    attention launch: the prefetch buffers end up bit-exact copies of the source buffers -- whole
    32 KiB pieces plus a shorter tail -- and the attention result is the one of a launch without
    copy CTAs.  The source stands in for another rank's K/V (here: other buffers of the same GPU)."""
    qh, kvh = 4, 2
    q, k, v, _dout, cu = make_varlen(21, [rows], qh, kvh)
    gen = torch.Generator().manual_seed(22)
    src_k = torch.randn(rows, kvh, 128, generator=gen).to(torch.bfloat16).to(DEV)
    src_v = torch.randn(rows, kvh, 128, generator=gen).to(torch.bfloat16).to(DEV)
    dst_k = torch.full_like(src_k, -7.0)
    dst_v = torch.full_like(src_v, -7.0)
    qd, kd, vd, cud = q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV)

    def call(prefetch):
        out = torch.zeros_like(qd)
        lse = torch.full((qh, rows), float("-inf"), dtype=torch.float32, device=DEV)
        ws = _call_fwd(qd, kd, vd, out, lse, cu_q=cud, cu_k=cud, batch=1, seqlen_q=rows, seqlen_k=rows,
                       heads_q=qh, heads_k=kvh, is_causal=True, merge_running=True, grid_blocks=16,
                       prefetch=prefetch)
        torch.cuda.synchronize()
        check_device_status(ws)
        return out, lse

    plain_out, plain_lse = call(None)
    out, lse = call((src_k.data_ptr(), src_v.data_ptr(), dst_k, dst_v, blocks))
    assert torch.equal(dst_k, src_k) and torch.equal(dst_v, src_v)
    assert torch.equal(out, plain_out) and torch.equal(lse, plain_lse)
    ref_out, ref_lse = orc.varlen_forward(q, k, v, [0, rows], [0, rows], True)
    e = orc.bf16_attention_error(q[None], k[None], v[None], True)["o"]
    assert (out.float().cpu() - ref_out).abs().max().item() <= bound(e)
    assert (lse.cpu() - ref_lse).abs().max().item() <= LSE_ATOL
