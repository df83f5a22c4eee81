"""CPU fp32 oracle for the attention path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This module restates, in plain fp32 PyTorch on the CPU, the reference functions that the
reference project's own tests use as ground truth for its attention operator.  Only
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
it, and only as the checker; the product (``min_fa3_demo_b200``) never does.

Parity pin: ``tests/golden/`` holds outputs of the reference's own Python reference
functions (imported from the reference checkout by ``tests/golden/make_golden.py``) on small
seeded inputs; ``tests/test_oracle_golden.py`` checks every function here against them.

Reference functions restated (paths relative to the reference project):
  * dense GQA attention through SDPA ........ scripts/test_min_fa3/test_min_fa3.py:26-37
  * per-document varlen loop ................ scripts/test_min_fa3/test_min_fa3_varlen.py:43-62
  * fp32 autograd backward .................. scripts/test_min_fa3/test_min_fa3_backward.py:16-36
  * varlen autograd backward ................ scripts/test_min_fa3/test_min_fa3_varlen_backward.py:25-52
  * explicit-position attention (out, lse) .. ring_test/utils.py:174-195
  * zigzag global positions ................. ring_test/ring_common.py:539-599
  * hierarchical sub-ring reference ......... ring_test/utils.py:198-273
  * running (out, lse) merge ................ ring_test/ring_common.py:59-73
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

HEAD_DIM = 128


# --------------------------------------------------------------------------------------
# core: attention with explicit positions, fp32, returns (out, lse)
# --------------------------------------------------------------------------------------
def attention_positions(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    query_positions: Optional[torch.Tensor],
    key_positions: Optional[torch.Tensor],
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of ``q [Tq,QH,D]`` over ``k,v [Tk,KVH,D]``; key j is visible to query i when
    ``key_positions[j] <= query_positions[i]`` (no mask when positions are None).

    Returns fp32 ``out [Tq,QH,D]`` and natural-log ``lse [QH,Tq]``; a row with no visible key
    gets ``out = 0`` and ``lse = -inf``.  Follows ring_test/utils.py:174-195 (which casts
    ``out`` to bf16; the cast is left to the caller here).
    """
    qf, kf, vf = q.float(), k.float(), v.float()
    repeat = q.size(1) // k.size(1)
    if repeat != 1:
        kf = kf.repeat_interleave(repeat, dim=1)
        vf = vf.repeat_interleave(repeat, dim=1)
    scores = torch.einsum("qhd,khd->hqk", qf, kf) * (q.size(-1) ** -0.5)
    if query_positions is not None:
        if key_positions is None:
            raise ValueError("causal oracle requires key positions")
        visible = key_positions.unsqueeze(0) <= query_positions.unsqueeze(1)
        scores = scores.masked_fill(~visible.unsqueeze(0), float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    probs = torch.softmax(scores, dim=-1)
    probs = torch.nan_to_num(probs, nan=0.0)
    out = torch.einsum("hqk,khd->qhd", probs, vf)
    return out, lse


def _causal_positions(sq: int, sk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Bottom-right aligned causal rule (hopper_compat/mask.h:88): key j visible to query i
    when j <= i + (sk - sq)."""
    return torch.arange(sq) + (sk - sq), torch.arange(sk)


# --------------------------------------------------------------------------------------
# BSHD / varlen forward
# --------------------------------------------------------------------------------------
def bshd_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q [B,S,QH,D]``, ``k,v [B,Sk,KVH,D]`` -> fp32 ``out [B,S,QH,D]``, ``lse [B,QH,S]``
    (scripts/test_min_fa3/test_min_fa3.py:26-37; LSE layout bindings.cpp:268)."""
    outs, lses = [], []
    for b in range(q.size(0)):
        qp, kp = _causal_positions(q.size(1), k.size(1)) if is_causal else (None, None)
        o, l = attention_positions(q[b], k[b], v[b], qp, kp)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def bshd_forward_sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool
                      ) -> torch.Tensor:
    """The reference test's literal formulation: fp32 ``F.scaled_dot_product_attention`` with
    ``enable_gqa`` (scripts/test_min_fa3/test_min_fa3.py:26-37).  Requires Sq == Sk when causal
    (SDPA's causal mask is top-left aligned)."""
    qb = q.permute(0, 2, 1, 3).float()
    kb = k.permute(0, 2, 1, 3).float()
    vb = v.permute(0, 2, 1, 3).float()
    out = F.scaled_dot_product_attention(qb, kb, vb, is_causal=is_causal,
                                         enable_gqa=qb.size(1) != kb.size(1))
    return out.permute(0, 2, 1, 3).contiguous()


def varlen_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: Sequence[int],
                   cu_seqlens_k: Sequence[int], is_causal: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packed ``q [Tq,QH,D]``, ``k,v [Tk,KVH,D]`` -> fp32 ``out [Tq,QH,D]``, ``lse [QH,Tq]``
    (scripts/test_min_fa3/test_min_fa3_varlen.py:43-62; LSE layout bindings.cpp:334)."""
    outs, lses = [], []
    for i in range(len(cu_seqlens_q) - 1):
        qs, qe = int(cu_seqlens_q[i]), int(cu_seqlens_q[i + 1])
        ks, ke = int(cu_seqlens_k[i]), int(cu_seqlens_k[i + 1])
        qp, kp = _causal_positions(qe - qs, ke - ks) if is_causal else (None, None)
        o, l = attention_positions(q[qs:qe], k[ks:ke], v[ks:ke], qp, kp)
        outs.append(o)
        lses.append(l)
    return torch.cat(outs, dim=0), torch.cat(lses, dim=1)


# --------------------------------------------------------------------------------------
# backward (fp32 autograd through the same math)
# --------------------------------------------------------------------------------------
def bshd_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dout: torch.Tensor,
                  is_causal: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp32 ``(dq, dk, dv)`` (scripts/test_min_fa3/test_min_fa3_backward.py:16-36)."""
    qr = q.detach().float().requires_grad_()
    kr = k.detach().float().requires_grad_()
    vr = v.detach().float().requires_grad_()
    out, _ = bshd_forward(qr, kr, vr, is_causal)
    return torch.autograd.grad(out, (qr, kr, vr), dout.float())


def varlen_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dout: torch.Tensor,
                    cu_seqlens_q: Sequence[int], cu_seqlens_k: Sequence[int], is_causal: bool
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp32 ``(dq, dk, dv)`` for packed inputs
    (scripts/test_min_fa3/test_min_fa3_varlen_backward.py:25-52)."""
    qr = q.detach().float().requires_grad_()
    kr = k.detach().float().requires_grad_()
    vr = v.detach().float().requires_grad_()
    out, _ = varlen_forward(qr, kr, vr, cu_seqlens_q, cu_seqlens_k, is_causal)
    return torch.autograd.grad(out, (qr, kr, vr), dout.float())


# --------------------------------------------------------------------------------------
# context-parallel helpers
# --------------------------------------------------------------------------------------
def zigzag_positions(ring_size: int, ring_rank: int, local_len: int) -> torch.Tensor:
    """Global positions of a rank's ``[front | back]`` zigzag shard: half-chunks ``r`` and
    ``2G-1-r`` of a sequence cut into ``2G`` halves (ring_test/ring_common.py:563-583)."""
    if local_len % 2 != 0:
        raise ValueError(f"zigzag layout needs an even local length, got {local_len}")
    half = local_len // 2
    ar = torch.arange(half, dtype=torch.int64)
    return torch.cat([ar + ring_rank * half, ar + (2 * ring_size - 1 - ring_rank) * half])


def zigzag_ring_forward(q: torch.Tensor, k_by_rank: torch.Tensor, v_by_rank: torch.Tensor,
                        rank: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Causal attention of one rank's zigzag shard ``q [L,QH,D]`` over every rank's K/V
    ``[W,L,KVH,D]`` (ring_test/ring_common.py:539-599, single document)."""
    world, local_len = k_by_rank.size(0), k_by_rank.size(1)
    key_pos = torch.cat([zigzag_positions(world, r, local_len) for r in range(world)])
    q_pos = zigzag_positions(world, rank, local_len)
    return attention_positions(q, k_by_rank.reshape(world * local_len, *k_by_rank.shape[2:]),
                               v_by_rank.reshape(world * local_len, *v_by_rank.shape[2:]),
                               q_pos, key_pos)


def hierarchical_forward(q: torch.Tensor, k_by_rank: List[torch.Tensor], v_by_rank: List[torch.Tensor],
                         rank_lengths: List[List[int]], global_lengths: Sequence[int],
                         ring_sizes: Sequence[int], ring_starts: Sequence[int], rank: int,
                         is_causal: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Hierarchical sub-ring reference (ring_test/utils.py:198-273).

    Document ``b`` of global length ``L_b`` lives on ranks ``[start_b, start_b + G_b)``, each
    holding ``L_b / G_b`` tokens in zigzag order (plain order when ``G_b == 1``).
    ``k_by_rank[r]`` is rank r's packed local K ``[sum_b len_r_b, KVH, D]`` and
    ``rank_lengths[r][b]`` its local length of document b.  Returns this rank's packed fp32
    ``out`` and ``lse [QH, local_total]``.
    """
    outs, lses = [], []
    q_off = 0
    for b, (glen, g, start) in enumerate(zip(global_lengths, ring_sizes, ring_starts)):
        mine = rank_lengths[rank][b]
        if mine == 0:
            continue
        local_len = glen // g
        q_b = q[q_off:q_off + mine]
        q_off += mine
        k_parts, v_parts, kpos = [], [], []
        for src in range(start, start + g):
            off = sum(rank_lengths[src][:b])
            k_parts.append(k_by_rank[src][off:off + local_len])
            v_parts.append(v_by_rank[src][off:off + local_len])
            if is_causal and g > 1:
                kpos.append(zigzag_positions(g, src - start, local_len))
        if is_causal and g > 1:
            qp, kp = zigzag_positions(g, rank - start, local_len), torch.cat(kpos)
        elif is_causal:
            qp, kp = torch.arange(local_len), torch.arange(local_len)
        else:
            qp, kp = None, None
        o, l = attention_positions(q_b, torch.cat(k_parts), torch.cat(v_parts), qp, kp)
        outs.append(o)
        lses.append(l)
    if not outs:
        return q.new_zeros(q.shape, dtype=torch.float32), torch.empty((q.size(1), 0))
    return torch.cat(outs), torch.cat(lses, dim=1)


def merge_out_lse(out: torch.Tensor, lse: torch.Tensor, block_out: torch.Tensor,
                  block_lse: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Running merge of two partial attentions (ring_test/ring_common.py:59-73):
    ``out [T,H,D]``, ``lse [H,T]`` merged with a block of the same layout.
    ``L = logaddexp(L_p, L_b)``, ``O = O_p - sigmoid(L_b - L_p) * (O_p - O_b)``; a pair of
    ``-inf`` rows stays ``(0, -inf)`` (min_fa3_epilogue.h:145-163)."""
    out = out.float()
    block_out = block_out.float()
    lp = lse.transpose(0, 1).unsqueeze(-1)
    lb = block_lse.transpose(0, 1).unsqueeze(-1)
    both_empty = torch.isinf(lp) & torch.isinf(lb) & (lp < 0) & (lb < 0)
    gate = torch.sigmoid(lb - lp)
    gate = torch.where(both_empty, torch.zeros_like(gate), gate)
    merged = out - gate * (out - block_out)
    merged = torch.where(both_empty.expand_as(merged), torch.zeros_like(merged), merged)
    new_lse = torch.logaddexp(lp, lb)
    return merged, new_lse.squeeze(-1).transpose(0, 1).contiguous()


# --------------------------------------------------------------------------------------
# acceptance rule
# --------------------------------------------------------------------------------------
def bf16_attention_error(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool,
                         dout: Optional[torch.Tensor] = None) -> dict:
    """Max-abs error of a bf16 PyTorch attention (SDPA on bf16 tensors, autograd for the
    gradients) against the fp32 oracle on the same BSHD inputs.  The acceptance bound for the
    CUDA path is 2x these numbers (O, dQ, dK, dV) and 1e-3 absolute on LSE."""
    out_ref, _ = bshd_forward(q, k, v, is_causal)
    qb = q.detach().permute(0, 2, 1, 3).to(torch.bfloat16).requires_grad_()
    kb = k.detach().permute(0, 2, 1, 3).to(torch.bfloat16).requires_grad_()
    vb = v.detach().permute(0, 2, 1, 3).to(torch.bfloat16).requires_grad_()
    if is_causal and q.size(1) != k.size(1):
        sq, sk = q.size(1), k.size(1)
        mask = torch.arange(sk)[None, :] <= (torch.arange(sq)[:, None] + (sk - sq))
        out_b = F.scaled_dot_product_attention(qb, kb, vb, attn_mask=mask,
                                               enable_gqa=qb.size(1) != kb.size(1))
    else:
        out_b = F.scaled_dot_product_attention(qb, kb, vb, is_causal=is_causal,
                                               enable_gqa=qb.size(1) != kb.size(1))
    res = {"o": (out_b.permute(0, 2, 1, 3).float() - out_ref).abs().max().item()}
    if dout is not None:
        dq_ref, dk_ref, dv_ref = bshd_backward(q, k, v, dout, is_causal)
        gq, gk, gv = torch.autograd.grad(out_b, (qb, kb, vb),
                                         dout.permute(0, 2, 1, 3).to(torch.bfloat16))
        res["dq"] = (gq.permute(0, 2, 1, 3).float() - dq_ref).abs().max().item()
        res["dk"] = (gk.permute(0, 2, 1, 3).float() - dk_ref).abs().max().item()
        res["dv"] = (gv.permute(0, 2, 1, 3).float() - dv_ref).abs().max().item()
    return res


def attention_flops(doc_lengths: Sequence[int], heads_q: int, is_causal: bool,
                    head_dim: int = HEAD_DIM) -> Tuple[float, float]:
    """Algorithmic (fwd, bwd) FLOPs: ``vis(L) = L(L+1)/2`` causal, ``L^2`` otherwise;
    fwd = 4*QH*D*sum(vis), bwd = 10*QH*D*sum(vis)
    (ring_test/benchmark_topology_forward.py:455-470)."""
    vis = sum(l * (l + 1) / 2 if is_causal else float(l) * l for l in doc_lengths)
    return 4.0 * heads_q * head_dim * vis, 10.0 * heads_q * head_dim * vis
