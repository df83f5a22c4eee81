"""Host side of the context-parallel path with two real ranks (gloo, CPU): placement ->
per-rank layouts -> zigzag sharding -> K/V exchange -> attention of the local shard, checked
against attention over the unsharded documents.  The exchange stands in for the peer copies of
the CUDA path (same rank-major K/V layout, same metadata), the arithmetic is the CPU oracle."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from min_fa3_demo_b200 import balancer as bal
from min_fa3_demo_b200 import ring
from oracle import attention_oracle as orc

QH, KVH, D = 4, 2, 128
LENGTHS = [1024, 512, 256, 768]        # 1024 and 512 may be split over two ranks (multiples of 512)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _shard(full: torch.Tensor, g: int, r: int) -> torch.Tensor:
    """Rank r's zigzag shard of one document (plain copy for a ring of one)."""
    if g == 1:
        return full
    return full[orc.zigzag_positions(g, r, full.size(0) // g)]


def _worker(rank: int, world: int, port: int, causal: bool, results) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = bal.assign_hierarchical_rings(LENGTHS, world, causal)
        lens, cu = bal.local_layout(plan, rank)
        # Every rank derives the same plan; the metadata passes the launch-time validation.
        gathered = [None] * world
        dist.all_gather_object(gathered, (plan.global_lengths, plan.ring_sizes, plan.ring_starts))
        assert all(g == gathered[0] for g in gathered)
        cap = max(sum(bal.local_layout(plan, r)[0]) for r in range(world))
        cap = ((cap + 127) // 128) * 128
        q_meta = torch.empty(cu[-1], QH, D, dtype=torch.bfloat16)
        arena_meta = torch.empty(world * cap, KVH, D, dtype=torch.bfloat16)
        i32 = lambda v: torch.tensor(list(v), dtype=torch.int32)
        got_cap = ring._validate_ring_metadata(q_meta, arena_meta, i32(cu), i32(cu), i32(plan.global_lengths),
                                               i32(plan.ring_sizes), i32(plan.ring_starts), world, rank, causal,
                                               max(lens), max(lens))
        assert got_cap == cap

        # Documents are generated identically on every rank, then sharded.
        gen = torch.Generator().manual_seed(5)
        docs = []
        for length in plan.global_lengths:
            docs.append(tuple(torch.randn(length, h, D, generator=gen).to(torch.bfloat16).float()
                              for h in (QH, KVH, KVH)))
        local_q, local_k, local_v = [], [], []
        for (fq, fk, fv), g, s in zip(docs, plan.ring_sizes, plan.ring_starts):
            if s <= rank < s + g:
                local_q.append(_shard(fq, g, rank - s))
                local_k.append(_shard(fk, g, rank - s))
                local_v.append(_shard(fv, g, rank - s))
        q = torch.cat(local_q)
        k = torch.cat(local_k)
        v = torch.cat(local_v)
        assert q.size(0) == cu[-1]

        # K/V exchange into the rank-major arena layout [world * cap, KVH, D].
        pad = lambda t: torch.cat([t, t.new_zeros(cap - t.size(0), KVH, D)])
        k_all = [torch.empty(cap, KVH, D) for _ in range(world)]
        v_all = [torch.empty(cap, KVH, D) for _ in range(world)]
        dist.all_gather(k_all, pad(k))
        dist.all_gather(v_all, pad(v))
        rank_lengths = [bal.local_layout(plan, r)[0] for r in range(world)]
        k_by_rank = [k_all[r][:sum(rank_lengths[r])] for r in range(world)]
        v_by_rank = [v_all[r][:sum(rank_lengths[r])] for r in range(world)]
        out, lse = orc.hierarchical_forward(q, k_by_rank, v_by_rank, rank_lengths, plan.global_lengths,
                                            plan.ring_sizes, plan.ring_starts, rank, causal)

        # Reference: attention over each whole document, then this rank's rows of it.
        off = 0
        worst = 0.0
        for (fq, fk, fv), g, s in zip(docs, plan.ring_sizes, plan.ring_starts):
            if not (s <= rank < s + g):
                continue
            ref_out, ref_lse = orc.varlen_forward(fq, fk, fv, [0, fq.size(0)], [0, fk.size(0)], causal)
            rows = slice(None) if g == 1 else orc.zigzag_positions(g, rank - s, fq.size(0) // g)
            n = fq.size(0) // g
            worst = max(worst, (out[off:off + n] - ref_out[rows]).abs().max().item(),
                        (lse[:, off:off + n] - ref_lse[:, rows]).abs().max().item())
            off += n
        results[rank] = (worst, sum(lens))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal", [True, False])
def test_two_rank_placement_sharding_and_exchange(causal):
    world = 2
    port = _free_port()
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, causal, results), nprocs=world, join=True)
    assert set(results.keys()) == {0, 1}
    assert sum(tokens for _, tokens in results.values()) == sum(LENGTHS)
    for rank, (worst, _) in results.items():
        assert worst < 2e-5, f"rank {rank}: sharded attention differs from the unsharded one by {worst}"


# ---------------------------------------------------------------------------------------
# The benchmark's full-size parity record, on two real ranks: exact results of a mixed batch
# (one document on a ring of two, one on each rank alone) must pass, and a rank whose output
# rows of the shared document are in the wrong zigzag order must make the vote fail everywhere.
# ---------------------------------------------------------------------------------------
PARITY_DOCS = [(1024, 2, 0), (256, 1, 0), (384, 1, 1)]        # (global length, ring size, ring start)


def _parity_worker(rank: int, world: int, port: int, corrupt: bool, results) -> None:
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dev = torch.device("cpu")
        gen = torch.Generator().manual_seed(9)
        parts = {name: [] for name in ("q", "k", "v", "dout", "out", "lse", "dq", "dk", "dv")}
        for (glen, g, start) in PARITY_DOCS:
            qg, dg = (torch.randn(glen, QH, D, generator=gen).to(torch.bfloat16) for _ in range(2))
            kg, vg = (torch.randn(glen, KVH, D, generator=gen).to(torch.bfloat16) for _ in range(2))
            if not start <= rank < start + g:
                continue
            pos = torch.arange(glen)
            o, l, grads = bench._dense_rows(qg, kg, vg, pos, pos, dg)
            mine = bench._zigzag_positions(g, rank - start, glen // g, dev)
            if corrupt and rank == 1 and g == 2:
                half = mine.numel() // 2
                o = o.clone()
                o[mine] = o[torch.cat([mine[half:], mine[:half]])]     # halves of the shard swapped
            for name, t in (("q", qg), ("k", kg), ("v", vg), ("dout", dg), ("out", o), ("dq", grads[0]),
                            ("dk", grads[1]), ("dv", grads[2])):
                parts[name].append(t[mine])
            parts["lse"].append(l[:, mine])
        cat = {name: torch.cat(ts, dim=1 if name == "lse" else 0) for name, ts in parts.items()}
        cap = 1024
        rec = bench._ring_workload_parity(rank, world, dev, dist, [d[0] for d in PARITY_DOCS],
                                          [d[1] for d in PARITY_DOCS], [d[2] for d in PARITY_DOCS],
                                          cat["q"], cat["k"], cat["v"], cat["dout"], cat["out"], cat["lse"],
                                          (cat["dq"], cat["dk"], cat["dv"]), cap)
        results[rank] = (rec["pass"], rec["worst_err_over_bound"])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("corrupt", [False, True])
def test_bench_parity_record_on_two_ranks(corrupt):
    world = 2
    port = _free_port()
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_parity_worker, args=(world, port, corrupt, results), nprocs=world, join=True)
    assert set(results.keys()) == {0, 1}
    for rank, (ok, worst) in results.items():
        if corrupt:
            assert not ok and worst["o"] > 1.0, f"rank {rank} accepted a shard in the wrong order: {worst}"
        else:
            assert ok and max(worst.values()) < 0.05, f"rank {rank}: {worst}"
