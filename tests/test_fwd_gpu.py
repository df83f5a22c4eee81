"""Forward parity on the GPU: the CUDA path (through min_fa3_op -> C ABI) against the CPU
oracle and the reference's golden fixtures.  Acceptance: O within 2x the max-abs error of a
bf16 PyTorch attention against the fp32 oracle, LSE within 1e-3 absolute."""
from __future__ import annotations

import pytest
import torch

import min_fa3_op
from conftest import from_bf16_bits, load_golden
from gpu_util import (assert_lse, assert_within, bound, make_bshd, make_varlen, varlen_bf16_errors)
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def run_bshd(q, k, v, causal, **kw):
    out, lse = min_fa3_op.forward(q.cuda(), k.cuda(), v.cuda(), causal, return_lse=True, **kw)
    torch.cuda.synchronize()
    return out, lse


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,s,qh,kvh", [
    (1, 128, 32, 32),      # reference test default shape
    (1, 129, 4, 2),        # one row past a tile
    (2, 1024, 16, 4),      # benchmark configuration 1
    (1, 333, 2, 1),        # ragged, MQA
    (3, 640, 8, 8),
    (1, 1, 2, 2),          # single token
])
def test_bshd_forward_vs_oracle(b, s, qh, kvh, causal):
    q, k, v, _ = make_bshd(1234 + s, b, s, qh, kvh)
    out, lse = run_bshd(q, k, v, causal)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    assert lse.shape == (b, qh, s) and lse.dtype == torch.float32
    ref_out, ref_lse = orc.bshd_forward(q, k, v, causal)
    e = orc.bf16_attention_error(q, k, v, causal)["o"]
    assert_within("O", out, ref_out, e)
    assert_lse(lse, ref_lse)


@pytest.mark.parametrize("sq,sk", [(256, 512), (128, 1000), (300, 200), (512, 128)])
def test_bshd_forward_rectangular_causal(sq, sk):
    # bottom-right aligned mask; with sq > sk the first rows see no key: O = 0, LSE = -inf
    q, k, v, _ = make_bshd(77, 1, sq, 4, 2, sk=sk)
    out, lse = run_bshd(q, k, v, True)
    ref_out, ref_lse = orc.bshd_forward(q, k, v, True)
    e = orc.bf16_attention_error(q, k, v, True)["o"]
    assert_within("O", out, ref_out, max(e, 4e-3))
    assert_lse(lse, ref_lse)
    if sq > sk:
        assert torch.all(out[0, : sq - sk] == 0)


@pytest.mark.parametrize("tag,causal", [("full", False), ("causal", True)])
def test_bshd_forward_golden(tag, causal):
    g = load_golden(f"bshd_{tag}")
    q, k, v = (from_bf16_bits(g[n]) for n in ("q", "k", "v"))
    out, _ = run_bshd(q, k, v, causal)
    golden = from_bf16_bits(g["out_bf16"]).float()
    e = orc.bf16_attention_error(q, k, v, causal)["o"]
    # the golden output is itself rounded to bf16: allow that rounding on top of the rule
    assert (out.float().cpu() - golden).abs().max().item() <= bound(e) + 2.0 ** -8 * golden.abs().max().item()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("lengths,qh,kvh", [
    ([128, 129], 4, 2),                                  # reference varlen default
    ([128, 111, 94, 128, 111, 94], 8, 2),                # S - 17*(i%3), reference backward test
    ([1, 700, 255, 257, 1024, 3], 4, 4),
    ([2048], 2, 1),
    ([37] * 40, 2, 2),                                   # many short documents
    ([200, 0, 77, 0], 4, 2),                             # empty documents inside and at the end
    ([0, 128], 2, 2),                                    # ... and in front
])
def test_varlen_forward_vs_oracle(lengths, qh, kvh, causal):
    q, k, v, dout, cu = make_varlen(99 + len(lengths), lengths, qh, kvh)
    out, lse = min_fa3_op.forward_varlen(
        q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), max(lengths), max(lengths), causal,
        cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, return_lse=True)
    torch.cuda.synchronize()
    assert lse.shape == (qh, sum(lengths))
    ref_out, ref_lse = orc.varlen_forward(q, k, v, cu.tolist(), cu.tolist(), causal)
    e = varlen_bf16_errors(q, k, v, dout, cu, causal)["o"]
    assert_within("O", out, ref_out, e)
    assert_lse(lse, ref_lse)


@pytest.mark.parametrize("tag,causal", [("full", False), ("causal", True)])
def test_varlen_forward_golden(tag, causal):
    g = load_golden(f"varlen_{tag}")
    q, k, v = (from_bf16_bits(g[n]) for n in ("q", "k", "v"))
    cu = torch.from_numpy(g["cu_seqlens"])
    lengths = (cu[1:] - cu[:-1]).tolist()
    out = min_fa3_op.forward_varlen(
        q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), max(lengths), max(lengths), causal,
        cu_seqlens_q_host=cu, cu_seqlens_k_host=cu)
    golden = from_bf16_bits(g["out_bf16"]).float()
    assert (out.float().cpu() - golden).abs().max().item() <= 2e-2


def test_varlen_different_q_and_k_lengths():
    gen = torch.Generator().manual_seed(5)
    q_lens, k_lens = [100, 260, 7], [300, 260, 90]
    cu_q = torch.tensor([0, 100, 360, 367], dtype=torch.int32)
    cu_k = torch.tensor([0, 300, 560, 650], dtype=torch.int32)
    q = torch.randn(367, 4, 128, generator=gen).to(torch.bfloat16)
    k = torch.randn(650, 2, 128, generator=gen).to(torch.bfloat16)
    v = torch.randn(650, 2, 128, generator=gen).to(torch.bfloat16)
    for causal in (False, True):
        out, lse = min_fa3_op.forward_varlen(
            q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), max(q_lens), max(k_lens), causal,
            cu_seqlens_q_host=cu_q, cu_seqlens_k_host=cu_k, return_lse=True)
        ref_out, ref_lse = orc.varlen_forward(q, k, v, cu_q.tolist(), cu_k.tolist(), causal)
        assert_within("O", out, ref_out, 4e-3)
        assert_lse(lse, ref_lse)


@pytest.mark.parametrize("blocks", [1, 7, 500])
def test_manual_block_count_gives_same_result(blocks):
    q, k, v, _ = make_bshd(11, 2, 1024, 8, 2)
    base, base_lse = run_bshd(q, k, v, True)
    out, lse = run_bshd(q, k, v, True, manual_block_count=blocks)
    assert torch.equal(out, base) and torch.equal(lse, base_lse)


def test_forward_error_behaviour_on_gpu():
    q, k, v, _ = make_bshd(3, 1, 128, 6, 4)
    with pytest.raises(RuntimeError, match="qhead % kvhead == 0"):
        min_fa3_op.forward(q.cuda(), k.cuda(), v.cuda(), True)
    q, k, v, _ = make_bshd(3, 1, 128, 4, 4)
    with pytest.raises(RuntimeError, match="must be contiguous BSHD"):
        min_fa3_op.forward(q.cuda().transpose(1, 2), k.cuda(), v.cuda(), True)
    cu = torch.tensor([0, 100, 128], dtype=torch.int32)
    qv, kv, vv = q[0].cuda(), k[0].cuda(), v[0].cuda()
    bad = torch.tensor([0, 100, 127], dtype=torch.int32)
    with pytest.raises(RuntimeError, match=r"cu_seqlens_q_host\[-1\] must equal q.size\(0\)"):
        min_fa3_op.forward_varlen(qv, kv, vv, cu.cuda(), cu.cuda(), 100, 100, True,
                                  cu_seqlens_q_host=bad, cu_seqlens_k_host=cu)


# ---------------------------------------------------------------------------------------
# Full benchmark sizes: size-independent properties
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("causal", [False, True])
def test_full_size_rows_against_oracle_and_properties(causal):
    """Config 2 (B=4, S=8192, QH=32, KVH=8): sampled query rows against the CPU oracle, and
    the prefix property of causal attention."""
    torch.manual_seed(0)
    b, s, qh, kvh = 4, 8192, 32, 8
    q = torch.randn(b, s, qh, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(b, s, kvh, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(b, s, kvh, 128, device="cuda").to(torch.bfloat16)
    out, lse = min_fa3_op.forward(q, k, v, causal, return_lse=True)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()

    # sampled rows of (batch 3, query heads 28..31 -> kv head 7) against the fp32 oracle
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 4095, 4096, 8063, 8064, 8191])
    qs = q[3, rows][:, 28:32].cpu()
    ks, vs = k[3, :, 7:8].cpu(), v[3, :, 7:8].cpu()
    qpos = rows if causal else None
    kpos = torch.arange(s) if causal else None
    ref_out, ref_lse = orc.attention_positions(qs, ks, vs, qpos, kpos)
    assert (out[3, rows][:, 28:32].float().cpu() - ref_out).abs().max().item() <= 1.6e-2
    assert (lse[3, 28:32][:, rows].cpu() - ref_lse).abs().max().item() <= 1e-3

    if causal:
        # prefix property: the first n rows only depend on the first n keys
        n = 1536
        out_prefix = min_fa3_op.forward(q[:, :n].contiguous(), k[:, :n].contiguous(),
                                        v[:, :n].contiguous(), True)
        assert (out_prefix.float() - out[:, :n].float()).abs().max().item() <= 1.6e-2
    else:
        # permuting the keys (K and V together) does not change non-causal attention
        perm = torch.randperm(s, device="cuda")
        out_perm = min_fa3_op.forward(q, k[:, perm].contiguous(), v[:, perm].contiguous(), False)
        assert (out_perm.float() - out.float()).abs().max().item() <= 1.6e-2

    # rows of P sum to one: with V = 1 the output is exactly one
    ones = torch.ones_like(v)
    out_ones = min_fa3_op.forward(q, k, ones, causal)
    assert (out_ones.float() - 1.0).abs().max().item() <= 2.0 ** -7
