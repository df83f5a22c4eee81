"""The synthetic workloads of bench.py: shapes, length distributions and the algorithmic FLOP
counts the reported TFLOPS are based on (14 * QH * D * sum over documents of L(L+1)/2 for causal
attention, forward 4x and backward 10x of QH * D * visible pairs)."""
from __future__ import annotations

import importlib.util
from pathlib import Path

import pytest

from min_fa3_demo_b200 import balancer as bal

ROOT = Path(__file__).resolve().parents[1]
spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_headline_workload_flops():
    w = dict(bench.WORKLOAD)
    assert (w["batch"], w["seqlen"], w["heads_q"], w["heads_k"], w["head_dim"], w["causal"]) == (4, 8192, 32, 8, 128, True)
    fwd, bwd = bench.step_flops(w)
    assert fwd == pytest.approx(2.199e12, rel=1e-3)
    assert fwd + bwd == pytest.approx(7.697e12, rel=1e-3)
    w["causal"] = False
    fwd, bwd = bench.step_flops(w)
    assert fwd + bwd == pytest.approx(1.539e13, rel=1e-3)


def test_varlen_lengths_fill_exactly_and_respect_the_clip():
    lens = bench.varlen_lengths()
    assert sum(lens) == 65536 and min(lens) >= 1 and max(lens) <= 32768
    assert (len(lens), max(lens), min(lens)) == (34, 7731, 128)     # the seed-0 realisation
    assert lens == bench.varlen_lengths()                            # deterministic
    assert any(n % 128 for n in lens), "lengths are meant to be ragged"


def test_ring_varlen_documents_place_on_eight_ranks():
    lengths = bal.sample_mixture_lengths(0, target_tokens=131072)
    lengths[-1] -= sum(lengths) - 131072
    assert sum(lengths) == 131072 and all(n % 256 == 0 and n > 0 for n in lengths)
    plan = bal.assign_hierarchical_rings(lengths, 8, True)
    assert plan.feasible
    assert sum(plan.rank_tokens) == 131072
    for rank in range(8):
        lens, cu = bal.local_layout(plan, rank)
        assert cu[-1] == plan.rank_tokens[rank] and all(n % 128 == 0 for n in lens)


def test_recorded_dram_traffic_is_tied_to_the_kernel_sources(tmp_path, monkeypatch):
    """The DRAM traffic in the bench line comes from a committed ncu capture; it is only reported
    while the backward kernel's sources still hash to what the capture measured."""
    import json

    digest = bench.kernel_source_digest()
    assert len(digest) == 64
    record = json.loads((ROOT / "profiles" / "bwd_kernel_traffic.json").read_text())
    assert record["dram_bytes_per_launch"] == record["scale_to_bench_workload"] * (
        record["dram_bytes_read_captured"] + record["dram_bytes_write_captured"])
    got = bench.recorded_traffic()
    if record["kernel_source_sha256"] == digest:
        assert got["traffic"] == record["dram_bytes_per_launch"]
    else:
        assert got["traffic"] is None and "stale" in got["traffic_note"]
    # a changed source makes the record stale
    monkeypatch.setattr(bench, "kernel_source_digest", lambda: "0" * 64)
    stale = bench.recorded_traffic()
    assert stale["traffic"] is None and "stale" in stale["traffic_note"]


def test_both_arms_report_the_same_config_record():
    cfg = bench.workload_config(1)
    assert cfg["workload"] == bench.WORKLOAD["name"] and cfg["flops_per_step_per_gpu"] == sum(bench.step_flops())
    assert bench.workload_config(8)["parallelism"].startswith("8 independent")


def test_key_row_gradient_checker_equals_autograd():
    """The bench's dK / dV checker for sampled key rows (from every query row, given O and LSE)
    is the same function as fp32 autograd through dense causal attention."""
    import torch

    torch.manual_seed(0)
    tokens, qh, kvh = 96, 4, 2
    q, dout = (torch.randn(tokens, qh, 128).to(torch.bfloat16) for _ in range(2))
    k, v = (torch.randn(tokens, kvh, 128).to(torch.bfloat16) for _ in range(2))
    pos = torch.arange(tokens)
    out, lse, grads = bench._dense_rows(q, k, v, pos, pos, dout)
    rows = torch.tensor([0, 5, 95])
    dk, dv = bench._key_rows_grads(q, dout, out, lse.t().contiguous(), pos, k[rows], v[rows], pos[rows])
    torch.testing.assert_close(dk, grads[1][rows], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(dv, grads[2][rows], rtol=1e-4, atol=1e-4)


def test_ring_parity_checker_accepts_exact_results_and_rejects_a_wrong_document():
    """The full-size parity record of the ring workloads, run on the CPU for one rank: exact
    fp32 results of a three-document batch pass with ratios near zero; the same results with one
    document's output rows swapped for another's fail."""
    import torch

    torch.manual_seed(1)
    glens, sizes, starts = [256, 128, 384], [1, 1, 1], [0, 0, 0]
    qh, kvh, total = 4, 2, 768
    q, dout = (torch.randn(total, qh, 128).to(torch.bfloat16) for _ in range(2))
    k, v = (torch.randn(total, kvh, 128).to(torch.bfloat16) for _ in range(2))
    outs, lses, dqs, dks, dvs = [], [], [], [], []
    begin = 0
    for n in glens:
        pos = torch.arange(n)
        sl = slice(begin, begin + n)
        o, l, g = bench._dense_rows(q[sl], k[sl], v[sl], pos, pos, dout[sl])
        outs.append(o); lses.append(l); dqs.append(g[0]); dks.append(g[1]); dvs.append(g[2])
        begin += n
    out, lse = torch.cat(outs), torch.cat(lses, dim=1)
    grads = (torch.cat(dqs), torch.cat(dks), torch.cat(dvs))
    dev = torch.device("cpu")
    good = bench._ring_workload_parity(0, 1, dev, None, glens, sizes, starts, q, k, v, dout, out, lse, grads, total)
    assert good["pass"] and max(good["worst_err_over_bound"].values()) < 0.05
    wrong = out.clone()
    wrong[256:384] = out[0:128]
    bad = bench._ring_workload_parity(0, 1, dev, None, glens, sizes, starts, q, k, v, dout, wrong, lse, grads, total)
    assert not bad["pass"] and bad["worst_err_over_bound"]["o"] > 1.0
