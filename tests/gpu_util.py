"""Helpers for the GPU parity tests: inputs, tolerances, per-document comparison."""
from __future__ import annotations

from typing import Sequence

import torch

from oracle import attention_oracle as orc

LSE_ATOL = 1e-3            # absolute LSE tolerance of the acceptance rule
ERR_FACTOR = 2.0           # outputs/gradients: <= 2x the error of a bf16 PyTorch attention
ERR_FLOOR = 2.0 ** -9      # never demand better than half a bf16 ulp at 1.0


def make_bshd(seed: int, b: int, sq: int, qh: int, kvh: int, sk: int | None = None):
    """Seeded N(0,1) bf16 q, k, v, dout on the CPU."""
    gen = torch.Generator().manual_seed(seed)
    sk = sk or sq
    q = torch.randn(b, sq, qh, 128, generator=gen).to(torch.bfloat16)
    k = torch.randn(b, sk, kvh, 128, generator=gen).to(torch.bfloat16)
    v = torch.randn(b, sk, kvh, 128, generator=gen).to(torch.bfloat16)
    dout = torch.randn(b, sq, qh, 128, generator=gen).to(torch.bfloat16)
    return q, k, v, dout


def make_varlen(seed: int, lengths: Sequence[int], qh: int, kvh: int):
    gen = torch.Generator().manual_seed(seed)
    total = sum(lengths)
    q = torch.randn(total, qh, 128, generator=gen).to(torch.bfloat16)
    k = torch.randn(total, kvh, 128, generator=gen).to(torch.bfloat16)
    v = torch.randn(total, kvh, 128, generator=gen).to(torch.bfloat16)
    dout = torch.randn(total, qh, 128, generator=gen).to(torch.bfloat16)
    cu = torch.tensor([0, *torch.tensor(list(lengths)).cumsum(0).tolist()], dtype=torch.int32)
    return q, k, v, dout, cu


def bound(e_bf16: float) -> float:
    return ERR_FACTOR * max(e_bf16, ERR_FLOOR)


def assert_within(name: str, ours: torch.Tensor, ref: torch.Tensor, e_bf16: float) -> None:
    err = (ours.float().cpu() - ref).abs().max().item()
    assert err <= bound(e_bf16), (
        f"{name}: max abs error {err:.3e} exceeds {ERR_FACTOR}x the bf16-PyTorch error "
        f"{e_bf16:.3e}")


def assert_lse(ours: torch.Tensor, ref: torch.Tensor) -> None:
    ours = ours.float().cpu()
    finite = torch.isfinite(ref)
    assert torch.equal(torch.isinf(ours) & (ours < 0), ~finite), "LSE -inf pattern differs"
    err = (ours[finite] - ref[finite]).abs().max().item() if finite.any() else 0.0
    assert err <= LSE_ATOL, f"LSE max abs error {err:.3e} exceeds {LSE_ATOL}"


def varlen_bf16_errors(q, k, v, dout, cu, causal) -> dict:
    """Worst per-document bf16-PyTorch error (the acceptance yardstick for packed inputs)."""
    worst = {"o": 0.0, "dq": 0.0, "dk": 0.0, "dv": 0.0}
    for i in range(cu.numel() - 1):
        s, e = int(cu[i]), int(cu[i + 1])
        if e == s:
            continue
        errs = orc.bf16_attention_error(q[s:e][None], k[s:e][None], v[s:e][None], causal,
                                        dout[s:e][None])
        for key in worst:
            worst[key] = max(worst[key], errs[key])
    return worst
