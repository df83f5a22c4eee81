"""Backward parity on the GPU: dQ, dK, dV from the CUDA path (through min_fa3_op -> C ABI)
against the fp32 autograd oracle and the reference's golden fixtures.  Acceptance: each
gradient within 2x the max-abs error of a bf16 PyTorch attention against the oracle."""
from __future__ import annotations

import pytest
import torch

import min_fa3_op
from conftest import from_bf16_bits, load_golden
from gpu_util import assert_lse, assert_within, bound, make_bshd, make_varlen, varlen_bf16_errors
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def fwd_bwd_bshd(q, k, v, dout, causal, **kw):
    qc, kc, vc, dc = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    out, lse = min_fa3_op.forward(qc, kc, vc, causal, return_lse=True)
    grads = min_fa3_op.backward(dc, qc, kc, vc, out, lse, causal, **kw)
    torch.cuda.synchronize()
    return out, lse, grads


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,s,qh,kvh", [
    (1, 128, 32, 32),      # reference backward test default
    (1, 129, 4, 2),
    (2, 1024, 16, 4),      # benchmark configuration 1
    (1, 333, 2, 1),
    (2, 640, 8, 8),
    (1, 1, 2, 2),
])
def test_bshd_backward_vs_oracle(b, s, qh, kvh, causal):
    q, k, v, dout = make_bshd(4321 + s, b, s, qh, kvh)
    _, _, (dq, dk, dv) = fwd_bwd_bshd(q, k, v, dout, causal)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    rq, rk, rv = orc.bshd_backward(q, k, v, dout, causal)
    e = orc.bf16_attention_error(q, k, v, causal, dout)
    assert_within("dQ", dq, rq, e["dq"])
    assert_within("dK", dk, rk, e["dk"])
    assert_within("dV", dv, rv, e["dv"])


@pytest.mark.parametrize("sq,sk", [(256, 512), (300, 200)])
def test_bshd_backward_rectangular_causal(sq, sk):
    q, k, v, dout = make_bshd(5, 1, sq, 4, 2, sk=sk)
    _, _, (dq, dk, dv) = fwd_bwd_bshd(q, k, v, dout, True)
    rq, rk, rv = orc.bshd_backward(q, k, v, dout, True)
    e = orc.bf16_attention_error(q, k, v, True, dout)
    assert_within("dQ", dq, rq, e["dq"])
    assert_within("dK", dk, rk, e["dk"])
    assert_within("dV", dv, rv, e["dv"])


@pytest.mark.parametrize("tag,causal", [("full", False), ("causal", True)])
def test_bshd_backward_golden(tag, causal):
    g = load_golden(f"bshd_{tag}")
    q, k, v, dout = (from_bf16_bits(g[n]) for n in ("q", "k", "v", "dout"))
    _, _, grads = fwd_bwd_bshd(q, k, v, dout, causal)
    e = orc.bf16_attention_error(q, k, v, causal, dout)
    for ours, name in zip(grads, ("dq", "dk", "dv")):
        assert_within(name, ours, torch.from_numpy(g[name]), e[name])


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("lengths,qh,kvh", [
    ([128, 129], 4, 2),
    ([128, 111, 94, 128, 111, 94], 8, 2),       # S - 17*(i%3), the reference's uneven case
    ([1, 700, 255, 257, 1024, 3], 4, 4),
    ([37] * 40, 2, 2),
    ([200, 0, 77, 0], 4, 2),                             # empty documents inside and at the end
    ([0, 128], 2, 2),                                    # ... and in front
])
def test_varlen_backward_vs_oracle(lengths, qh, kvh, causal):
    q, k, v, dout, cu = make_varlen(7 + len(lengths), lengths, qh, kvh)
    qc, kc, vc, dc, cuc = q.cuda(), k.cuda(), v.cuda(), dout.cuda(), cu.cuda()
    out, lse = min_fa3_op.forward_varlen(qc, kc, vc, cuc, cuc, max(lengths), max(lengths), causal,
                                         cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, return_lse=True)
    dq, dk, dv = min_fa3_op.backward_varlen(dc, qc, kc, vc, out, lse, cuc, cuc, max(lengths),
                                            max(lengths), causal)
    torch.cuda.synchronize()
    rq, rk, rv = orc.varlen_backward(q, k, v, dout, cu.tolist(), cu.tolist(), causal)
    e = varlen_bf16_errors(q, k, v, dout, cu, causal)
    assert_within("dQ", dq, rq, e["dq"])
    assert_within("dK", dk, rk, e["dk"])
    assert_within("dV", dv, rv, e["dv"])


def test_varlen_document_without_keys():
    """A document with query rows but no keys: O = 0 and LSE = -inf for its rows (reference:
    include/min_fa3_epilogue.h:557-631), and they contribute nothing to any gradient."""
    gen = torch.Generator().manual_seed(23)
    cu_q = torch.tensor([0, 64, 194, 194 + 300], dtype=torch.int32)
    cu_k = torch.tensor([0, 0, 130, 130 + 300], dtype=torch.int32)
    q = torch.randn(494, 4, 128, generator=gen).to(torch.bfloat16)
    dout = torch.randn(494, 4, 128, generator=gen).to(torch.bfloat16)
    k = torch.randn(430, 2, 128, generator=gen).to(torch.bfloat16)
    v = torch.randn(430, 2, 128, generator=gen).to(torch.bfloat16)
    qc, kc, vc, dc = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    out, lse = min_fa3_op.forward_varlen(qc, kc, vc, cu_q.cuda(), cu_k.cuda(), 300, 300, False,
                                         cu_seqlens_q_host=cu_q, cu_seqlens_k_host=cu_k, return_lse=True)
    dq, dk, dv = min_fa3_op.backward_varlen(dc, qc, kc, vc, out, lse, cu_q.cuda(), cu_k.cuda(), 300, 300, False)
    torch.cuda.synchronize()
    assert bool((out[:64] == 0).all()) and bool(torch.isinf(lse[:, :64]).all()) and bool((lse[:, :64] < 0).all())
    assert bool((dq[:64] == 0).all())
    ref_out, ref_lse = orc.varlen_forward(q, k, v, cu_q.tolist(), cu_k.tolist(), False)
    rq, rk, rv = orc.varlen_backward(q, k, v, dout, cu_q.tolist(), cu_k.tolist(), False)
    errs = {"o": 0.0, "dq": 0.0, "dk": 0.0, "dv": 0.0}
    for (qs, qe), (ks, ke) in (((64, 194), (0, 130)), ((194, 494), (130, 430))):
        e = orc.bf16_attention_error(q[qs:qe][None], k[ks:ke][None], v[ks:ke][None], False, dout[qs:qe][None])
        errs = {key: max(errs[key], e[key]) for key in errs}
    assert_within("O", out, ref_out, errs["o"])
    assert_lse(lse, ref_lse)
    assert_within("dQ", dq, rq, errs["dq"])
    assert_within("dK", dk, rk, errs["dk"])
    assert_within("dV", dv, rv, errs["dv"])


@pytest.mark.parametrize("tag,causal", [("full", False), ("causal", True)])
def test_varlen_backward_golden(tag, causal):
    g = load_golden(f"varlen_{tag}")
    q, k, v, dout = (from_bf16_bits(g[n]) for n in ("q", "k", "v", "dout"))
    cu = torch.from_numpy(g["cu_seqlens"])
    lengths = (cu[1:] - cu[:-1]).tolist()
    qc, kc, vc, dc, cuc = q.cuda(), k.cuda(), v.cuda(), dout.cuda(), cu.cuda()
    out, lse = min_fa3_op.forward_varlen(qc, kc, vc, cuc, cuc, max(lengths), max(lengths), causal,
                                         cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, return_lse=True)
    grads = min_fa3_op.backward_varlen(dc, qc, kc, vc, out, lse, cuc, cuc, max(lengths),
                                       max(lengths), causal)
    e = varlen_bf16_errors(q, k, v, dout, cu, causal)
    for ours, name in zip(grads, ("dq", "dk", "dv")):
        assert_within(name, ours, torch.from_numpy(g[name]), e[name])


def test_backward_writes_into_caller_buffers():
    # reference: scripts/test_min_fa3/test_min_fa3_backward.py:60-75
    q, k, v, dout = make_bshd(8, 1, 256, 4, 2)
    qc, kc, vc, dc = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    out, lse = min_fa3_op.forward(qc, kc, vc, True, return_lse=True)
    expected = min_fa3_op.backward(dc, qc, kc, vc, out, lse, True)
    buffers = (torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc))
    got = min_fa3_op.backward(dc, qc, kc, vc, out, lse, True, dq=buffers[0], dk=buffers[1],
                              dv=buffers[2])
    assert all(r.data_ptr() == b.data_ptr() for r, b in zip(got, buffers))
    for a, b, name in zip(got, expected, ("dq", "dk", "dv")):
        # dK / dV are accumulated in a fixed order; dQ uses fp32 atomics (order may vary)
        if name == "dq":
            assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -6
        else:
            assert torch.equal(a, b), name


def test_backward_rejects_bad_lse_shape():
    # reference: scripts/test_min_fa3/test_min_fa3_backward.py:95-103
    q, k, v, dout = make_bshd(9, 1, 128, 4, 2)
    qc, kc, vc, dc = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    out, lse = min_fa3_op.forward(qc, kc, vc, True, return_lse=True)
    bad = torch.empty((1, 4, 129), device="cuda", dtype=torch.float32)
    with pytest.raises(RuntimeError, match=r"softmax_lse must have shape \[B, QH, Sq\]"):
        min_fa3_op.backward(dc, qc, kc, vc, out, bad, True)
    with pytest.raises(RuntimeError, match="dq must have shape"):
        min_fa3_op.backward(dc, qc, kc, vc, out, lse, True, dq=torch.empty_like(kc))


@pytest.mark.parametrize("causal", [False, True])
def test_full_size_backward_properties(causal):
    """Config 2 (B=4, S=8192, QH=32, KVH=8).  Size-independent identities of softmax attention:
    sum_k dV[k] = sum_q dO[q] per KV head (rows of P sum to one), and
    sum_i q_i . dq_i = sum_j k_j . dk_j per KV head (S depends on q and k only through q.k)."""
    torch.manual_seed(1)
    b, s, qh, kvh = 4, 8192, 32, 8
    q = torch.randn(b, s, qh, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(b, s, kvh, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(b, s, kvh, 128, device="cuda").to(torch.bfloat16)
    dout = torch.randn(b, s, qh, 128, device="cuda").to(torch.bfloat16)
    out, lse = min_fa3_op.forward(q, k, v, causal, return_lse=True)
    dq, dk, dv = min_fa3_op.backward(dout, q, k, v, out, lse, causal)
    for t in (dq, dk, dv):
        assert torch.isfinite(t.float()).all()

    g = qh // kvh
    dv_sum = dv.float().sum(dim=1)                                        # [B, KVH, D]
    do_sum = dout.float().view(b, s, kvh, g, 128).sum(dim=(1, 3))         # [B, KVH, D]
    scale = do_sum.abs().max().item()
    assert (dv_sum - do_sum).abs().max().item() <= 2e-2 * scale

    qdq = (q.float() * dq.float()).view(b, s, kvh, g, 128).sum(dim=(1, 3, 4))   # [B, KVH]
    kdk = (k.float() * dk.float()).sum(dim=(1, 3))                              # [B, KVH]
    denom = (q.float() * dq.float()).abs().view(b, s, kvh, g, 128).sum(dim=(1, 3, 4))
    assert ((qdq - kdk).abs() / denom).max().item() <= 2e-3

    # one KV head group of batch 0, first 1024 keys/queries of a causal problem, is itself a
    # complete attention problem: check it against the fp32 oracle
    if causal:
        n = 512
        qs, ks, vs, ds = (t[:1, :n].contiguous() for t in (q, k, v, dout))
        o2, l2 = min_fa3_op.forward(qs, ks, vs, True, return_lse=True)
        g2 = min_fa3_op.backward(ds, qs, ks, vs, o2, l2, True)
        # dQ of the prefix equals dQ of the full problem (rows < n only see keys < n)
        assert (g2[0].float() - dq[:1, :n].float()).abs().max().item() <= 3e-2
        rq, rk, rv = orc.bshd_backward(qs[:, :, :4].cpu(), ks[:, :, :1].cpu(), vs[:, :, :1].cpu(),
                                       ds[:, :, :4].cpu(), True)
        assert (g2[0][:, :, :4].float().cpu() - rq).abs().max().item() <= 3e-2


# --------------------------------------------------------------------------------------
# deterministic=True: dQ is accumulated in ascending key-block order, so repeated calls are
# bitwise identical (the reference checks four repeats:
# scripts/test_min_fa3_backward.py:77-93); the result must still meet the accuracy rule.
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("causal", [False, True])
def test_bshd_backward_deterministic_repeats_bitwise(causal):
    b, s, qh, kvh = 2, 2048, 8, 2
    q, k, v, dout = make_bshd(99, b, s, qh, kvh)
    qc, kc, vc, dc = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    out, lse = min_fa3_op.forward(qc, kc, vc, causal, return_lse=True)
    runs = [min_fa3_op.backward(dc, qc, kc, vc, out, lse, causal, deterministic=True) for _ in range(4)]
    torch.cuda.synchronize()
    for other in runs[1:]:
        for name, a, b_ in zip(("dq", "dk", "dv"), runs[0], other):
            assert torch.equal(a, b_), f"{name} differs between repeated deterministic calls"
    rq, rk, rv = orc.bshd_backward(q, k, v, dout, causal)
    e = orc.bf16_attention_error(q, k, v, causal, dout)
    assert_within("dQ", runs[0][0], rq, e["dq"])
    assert_within("dK", runs[0][1], rk, e["dk"])
    assert_within("dV", runs[0][2], rv, e["dv"])


def test_varlen_backward_deterministic_repeats_bitwise():
    lengths = [1500, 77, 640, 1, 2049, 333]
    q, k, v, dout, cu = make_varlen(17, lengths, 8, 2)
    qc, kc, vc, dc, cuc = q.cuda(), k.cuda(), v.cuda(), dout.cuda(), cu.cuda()
    out, lse = min_fa3_op.forward_varlen(qc, kc, vc, cuc, cuc, max(lengths), max(lengths), True,
                                         cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, return_lse=True)
    runs = [min_fa3_op.backward_varlen(dc, qc, kc, vc, out, lse, cuc, cuc, max(lengths), max(lengths), True,
                                       deterministic=True) for _ in range(4)]
    plain = min_fa3_op.backward_varlen(dc, qc, kc, vc, out, lse, cuc, cuc, max(lengths), max(lengths), True)
    torch.cuda.synchronize()
    for other in runs[1:]:
        for name, a, b_ in zip(("dq", "dk", "dv"), runs[0], other):
            assert torch.equal(a, b_), f"{name} differs between repeated deterministic calls"
    # Same arithmetic as the default path up to the order of the fp32 dQ additions.
    assert torch.equal(runs[0][1], plain[1]) and torch.equal(runs[0][2], plain[2])
    scale = max(1.0, plain[0].float().abs().max().item())
    assert (runs[0][0].float() - plain[0].float()).abs().max().item() <= 2.0 ** -6 * scale


# --------------------------------------------------------------------------------------
# Benchmark configuration 3 at full size: 65,536 packed tokens, 34 log-normal documents of
# 128 ... 7,731 tokens (not multiples of 128), QH=32, KVH=8.  O and LSE of sampled rows of
# every document (all heads) and dQ / dK / dV of one KV-head group on a subset of documents
# (longest, shortest and four in between) against the fp32 oracle under the acceptance rule.
# --------------------------------------------------------------------------------------
def test_config3_full_size_against_oracle():
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from bench import varlen_lengths

    lens = varlen_lengths()
    assert sum(lens) == 65536 and min(lens) >= 1
    qh, kvh, group = 32, 8, 4
    total = sum(lens)
    gen = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(total, qh, 128, device="cuda", generator=gen).to(torch.bfloat16)
    k = torch.randn(total, kvh, 128, device="cuda", generator=gen).to(torch.bfloat16)
    v = torch.randn(total, kvh, 128, device="cuda", generator=gen).to(torch.bfloat16)
    dout = torch.randn(total, qh, 128, device="cuda", generator=gen).to(torch.bfloat16)
    cu = torch.tensor([0, *torch.tensor(lens).cumsum(0).tolist()], dtype=torch.int32)
    cud = cu.cuda()
    mx = max(lens)
    out, lse = min_fa3_op.forward_varlen(q, k, v, cud, cud, mx, mx, True, cu_seqlens_q_host=cu,
                                         cu_seqlens_k_host=cu, return_lse=True)
    dq, dk, dv = min_fa3_op.backward_varlen(dout, q, k, v, out, lse, cud, cud, mx, mx, True)
    torch.cuda.synchronize()
    min_fa3_op.check_last_status()
    assert all(torch.isfinite(t.float()).all() for t in (out, lse, dq, dk, dv))

    # forward: up to 12 sampled rows per document, all heads
    for i, n in enumerate(lens):
        s0 = int(cu[i])
        rows = sorted({0, n - 1, n // 2, min(n - 1, 127), min(n - 1, 128), max(0, n - 129),
                       *[(7919 * (j + 1) * (i + 1)) % n for j in range(6)]})
        rows_t = torch.tensor(rows)
        qs = q[s0 + rows_t].cpu()
        ks, vs = k[s0:s0 + n].cpu(), v[s0:s0 + n].cpu()
        ref_o, ref_l = orc.attention_positions(qs, ks, vs, rows_t, torch.arange(n))
        # bf16 yardstick on the same rows: bf16 scores / probabilities / output
        sc = torch.einsum("qhd,khd->hqk", qs, ks.repeat_interleave(group, dim=1)).float() * (128 ** -0.5)
        sc = sc.masked_fill(torch.arange(n)[None, None, :] > rows_t[None, :, None], float("-inf"))
        pb = torch.softmax(sc, dim=-1).to(torch.bfloat16)
        ob = torch.einsum("hqk,khd->qhd", pb, vs.repeat_interleave(group, dim=1))
        e = (ob.float() - ref_o).abs().max().item()
        err = (out[s0 + rows_t].float().cpu() - ref_o).abs().max().item()
        assert err <= bound(e), f"doc {i} (len {n}): O error {err:.3e} exceeds {bound(e):.3e}"
        lerr = (lse[:, s0 + rows_t].cpu() - ref_l).abs().max().item()
        assert lerr <= 1e-3, f"doc {i} (len {n}): LSE error {lerr:.3e}"

    # backward: one KV-head group (query heads 28..31, KV head 7), whole documents
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    chosen = {order[-1], order[0], order[len(order) // 4], order[len(order) // 2], order[(3 * len(order)) // 4],
              order[-3]}
    for i in sorted(chosen):
        s0, n = int(cu[i]), lens[i]
        qs, ds = q[s0:s0 + n, 28:32].cpu()[None], dout[s0:s0 + n, 28:32].cpu()[None]
        ks, vs = k[s0:s0 + n, 7:8].cpu()[None], v[s0:s0 + n, 7:8].cpu()[None]
        rq, rk, rv = orc.bshd_backward(qs, ks, vs, ds, True)
        e = orc.bf16_attention_error(qs, ks, vs, True, ds)
        assert_within(f"dQ doc {i} (len {n})", dq[s0:s0 + n, 28:32][None], rq, e["dq"])
        # dK / dV of KV head 7 only receive contributions from query heads 28..31
        assert_within(f"dK doc {i} (len {n})", dk[s0:s0 + n, 7:8][None], rk, e["dk"])
        assert_within(f"dV doc {i} (len {n})", dv[s0:s0 + n, 7:8][None], rv, e["dv"])
