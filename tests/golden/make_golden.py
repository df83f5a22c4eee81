"""Generate the golden fixtures in this directory from the reference project's own Python
reference functions.

Usage: ``python tests/golden/make_golden.py --reference <path to the reference checkout>``

The reference's ground-truth functions are plain PyTorch and run on the CPU, but its test
modules import the compiled extension at the top; a stand-in ``min_fa3_op`` module is
registered first so that only the reference *functions* are used.  Inputs are small, seeded
and stored with the outputs, so the fixtures do not depend on RNG stability.  bf16 tensors
are stored as their int16 bit patterns.
"""

from __future__ import annotations

import argparse
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

OUT_DIR = Path(__file__).resolve().parent


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy()


def randn_bf16(gen: torch.Generator, *shape, scale: float = 1.0) -> torch.Tensor:
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", required=True, type=Path)
    args = parser.parse_args()
    ref = args.reference.resolve()

    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ref / "scripts" / "test_mega_ring"))
    sys.modules["min_fa3_op"] = types.ModuleType("min_fa3_op")
    t_fwd = _load(ref / "scripts/test_min_fa3/test_min_fa3.py", "ref_test_fwd")
    t_bwd = _load(ref / "scripts/test_min_fa3/test_min_fa3_backward.py", "ref_test_bwd")
    t_vfwd = _load(ref / "scripts/test_min_fa3/test_min_fa3_varlen.py", "ref_test_vfwd")
    t_vbwd = _load(ref / "scripts/test_min_fa3/test_min_fa3_varlen_backward.py", "ref_test_vbwd")
    ring_common = _load(ref / "ring_test/ring_common.py", "ref_ring_common")
    ring_utils = _load(ref / "ring_test/utils.py", "ref_ring_utils")
    mega = _load(ref / "scripts/test_mega_ring/mega_ring_test_min_fa3_varlen_ring_multi_rank.py",
                 "mega_ring_test_min_fa3_varlen_ring_multi_rank")

    torch.manual_seed(0)
    gen = torch.Generator().manual_seed(20260713)

    # 1) BSHD forward + backward, causal and non-causal, GQA 4/2.
    for causal in (False, True):
        q = randn_bf16(gen, 1, 72, 4, 128)
        k = randn_bf16(gen, 1, 72, 2, 128)
        v = randn_bf16(gen, 1, 72, 2, 128)
        dout = randn_bf16(gen, 1, 72, 4, 128)
        out = t_fwd.reference_flash(q, k, v, causal)                 # bf16
        dq, dk, dv = t_bwd.reference_backward(q, k, v, dout, causal)  # fp32
        np.savez_compressed(
            OUT_DIR / f"bshd_{'causal' if causal else 'full'}.npz",
            q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v), dout=bf16_bits(dout),
            out_bf16=bf16_bits(out), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())

    # 2) varlen forward + backward with ragged lengths (reference default style S - 17*(i%3)).
    lengths = t_vbwd.make_lengths(3, 40)
    cu = torch.tensor([0, *torch.tensor(lengths).cumsum(0).tolist()], dtype=torch.int32)
    total = int(cu[-1])
    for causal in (False, True):
        q = randn_bf16(gen, total, 4, 128)
        k = randn_bf16(gen, total, 2, 128)
        v = randn_bf16(gen, total, 2, 128)
        dout = randn_bf16(gen, total, 4, 128)
        out = t_vfwd.reference_varlen(q, k, v, cu, cu, causal)
        dq, dk, dv = t_vbwd.reference_backward(q, k, v, dout, cu, cu, causal)
        np.savez_compressed(
            OUT_DIR / f"varlen_{'causal' if causal else 'full'}.npz",
            cu_seqlens=cu.numpy(), q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
            dout=bf16_bits(dout), out_bf16=bf16_bits(out), dq=dq.numpy(), dk=dk.numpy(),
            dv=dv.numpy())

    # 3) explicit-position attention with (out, lse).
    q = randn_bf16(gen, 40, 4, 128)
    k = randn_bf16(gen, 56, 2, 128)
    v = randn_bf16(gen, 56, 2, 128)
    qpos = torch.randint(0, 56, (40,), generator=gen)
    kpos = torch.randperm(56, generator=gen)
    out, lse = ring_utils.attention_reference(q, k, v, qpos, kpos)
    out_nc, lse_nc = ring_utils.attention_reference(q, k, v, None, None)
    np.savez_compressed(OUT_DIR / "positions.npz", q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
                        qpos=qpos.numpy(), kpos=kpos.numpy(), out_bf16=bf16_bits(out),
                        lse=lse.numpy(), out_nc_bf16=bf16_bits(out_nc), lse_nc=lse_nc.numpy())

    # 4) zigzag ring reference: world 4, one document, local length 32 per rank.
    world, local_len = 4, 16
    k_by = randn_bf16(gen, world, local_len, 2, 128)
    v_by = randn_bf16(gen, world, local_len, 2, 128)
    q_by = randn_bf16(gen, world, local_len, 4, 128)
    outs = [ring_common.reference_zigzag_ring_varlen(q_by[r], k_by, v_by, 1, local_len, r)
            for r in range(world)]
    np.savez_compressed(OUT_DIR / "zigzag.npz", q=bf16_bits(q_by), k=bf16_bits(k_by),
                        v=bf16_bits(v_by), out_bf16=bf16_bits(torch.stack(outs)))

    # 5) mega-ring dense reference: rank-major K/V arena, 2 documents, world 2.
    world = 2
    lens = [16, 32]
    cu = torch.tensor([0, 16, 48], dtype=torch.int32)
    local_total = 48
    k_arena = randn_bf16(gen, world * local_total, 2, 128)
    v_arena = randn_bf16(gen, world * local_total, 2, 128)
    res = {}
    for rank in range(world):
        q = randn_bf16(gen, local_total, 4, 128)
        res[f"q{rank}"] = bf16_bits(q)
        for causal in (False, True):
            out = mega.reference_mega_ring_varlen(q, k_arena, v_arena, cu, cu, causal, rank, world)
            res[f"out{rank}_{'causal' if causal else 'full'}_bf16"] = bf16_bits(out)
    np.savez_compressed(OUT_DIR / "mega_ring.npz", cu_seqlens=cu.numpy(), k=bf16_bits(k_arena),
                        v=bf16_bits(v_arena), **res)

    # 6) hierarchical sub-rings: world 4; doc0 on all 4 ranks, doc1 on ranks 2-3, doc2 on rank 1.
    world = 4
    global_lengths, ring_sizes, ring_starts = [64, 32, 12], [4, 2, 1], [0, 2, 1]
    rank_lengths = []
    for r in range(world):
        row = []
        for glen, g, s in zip(global_lengths, ring_sizes, ring_starts):
            row.append(glen // g if s <= r < s + g else 0)
        rank_lengths.append(row)
    max_local = max(sum(row) for row in rank_lengths)
    gathered_k = torch.zeros(world, max_local, 2, 128, dtype=torch.bfloat16)
    gathered_v = torch.zeros(world, max_local, 2, 128, dtype=torch.bfloat16)
    qs = []
    for r in range(world):
        n = sum(rank_lengths[r])
        gathered_k[r, :n] = randn_bf16(gen, n, 2, 128)
        gathered_v[r, :n] = randn_bf16(gen, n, 2, 128)
        qs.append(randn_bf16(gen, n, 4, 128))
    res = {}
    for r in range(world):
        local_cu = torch.tensor([0, *torch.tensor(rank_lengths[r]).cumsum(0).tolist()])
        for causal in (False, True):
            out, lse = ring_utils.hierarchical_reference(
                qs[r], gathered_k, gathered_v, rank_lengths, local_cu, global_lengths, ring_sizes,
                ring_starts, r, causal)
            tag = "causal" if causal else "full"
            res[f"q{r}"] = bf16_bits(qs[r])
            res[f"out{r}_{tag}_bf16"] = bf16_bits(out)
            res[f"lse{r}_{tag}"] = lse.numpy()
    np.savez_compressed(OUT_DIR / "hierarchical.npz", k=bf16_bits(gathered_k), v=bf16_bits(gathered_v),
                        rank_lengths=np.array(rank_lengths), global_lengths=np.array(global_lengths),
                        ring_sizes=np.array(ring_sizes), ring_starts=np.array(ring_starts), **res)

    # 7) running (out, lse) merge.
    out_a = torch.randn(16, 4, 128, generator=gen)
    lse_a = torch.randn(4, 16, generator=gen)
    out_b = randn_bf16(gen, 16, 4, 128)
    lse_b = torch.randn(4, 16, generator=gen)
    run_out, run_lse = ring_common.update_out_and_lse(None, None, out_a, lse_a)
    run_out, run_lse = ring_common.update_out_and_lse(run_out, run_lse, out_b, lse_b)
    np.savez_compressed(OUT_DIR / "merge.npz", out_a=out_a.numpy(), lse_a=lse_a.numpy(),
                        out_b=bf16_bits(out_b), lse_b=lse_b.numpy(), merged_out=run_out.numpy(),
                        merged_lse=run_lse.squeeze(-1).transpose(0, 1).contiguous().numpy())

    # 8) the same merge with a running output that is exactly representable in bf16 (the CUDA
    # epilogue keeps the running output in bf16 between steps, min_fa3_epilogue.h:404-506), so a
    # kernel can be held to this fixture without an input-rounding allowance.
    gen8 = torch.Generator().manual_seed(88)
    out_a = randn_bf16(gen8, 16, 4, 128).float()
    lse_a = torch.randn(4, 16, generator=gen8)
    out_b = randn_bf16(gen8, 16, 4, 128)
    lse_b = torch.randn(4, 16, generator=gen8)
    run_out, run_lse = ring_common.update_out_and_lse(None, None, out_a, lse_a)
    run_out, run_lse = ring_common.update_out_and_lse(run_out, run_lse, out_b, lse_b)
    np.savez_compressed(OUT_DIR / "merge_bf16.npz", out_a=bf16_bits(out_a), lse_a=lse_a.numpy(),
                        out_b=bf16_bits(out_b), lse_b=lse_b.numpy(), merged_out=run_out.numpy(),
                        merged_lse=run_lse.squeeze(-1).transpose(0, 1).contiguous().numpy())

    for path in sorted(OUT_DIR.glob("*.npz")):
        print(f"{path.name}: {path.stat().st_size} bytes")


if __name__ == "__main__":
    main()
