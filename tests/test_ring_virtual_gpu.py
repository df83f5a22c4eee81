"""Context-parallel forward with several ranks emulated on ONE GPU, through the C ABI.

Every "virtual rank" owns a K/V arena on the same device; rank r's launch gets the other
arenas as its peer pointers.  The forward kernel never waits for another rank's launch (a rank
only reads the slices the owners wrote before the launch), so the W launches simply run one
after the other on one stream.  This executes, on a single-GPU machine, everything a real
multi-GPU forward executes except the NVLink hop: the copy CTAs (peer -> shared -> own arena),
the per-block ready flags and their bounded waits, the zigzag virtual block map, hierarchical
sub-rings (8 virtual ranks: rings of 8, 4, 2 and 1), and the one-chunk layout of unmasked rings
(shards of 384 rows).

The backward is not emulated this way: it ends with a wait for the other ranks' completion
signals, which would never come from launches queued behind it on the same GPU.
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from gpu_util import LSE_ATOL  # noqa: E402
from min_fa3_demo_b200 import _cabi  # noqa: E402
from mp_worker import SENTINEL, build_problem, doc_bounds, meta, oracle_forward, ring_docs_for  # noqa: E402

pytestmark = pytest.mark.gpu

QH, KVH, CAP = 8, 2, 2048


def launch_rank(lib, rank, world, q, out, lse, arenas_k, arenas_v, cu, docs, causal, ws, stats, comm=8):
    g, s, st = meta(docs)
    a = _cabi.RingFwdArgs()
    a.q, a.out, a.lse = q.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.arena_k, a.arena_v = arenas_k[rank].data_ptr(), arenas_v[rank].data_ptr()
    for r in range(world):
        a.peer_k[r] = arenas_k[r].data_ptr()
        a.peer_v[r] = arenas_v[r].data_ptr()
    a.cu_seqlens_q_host = cu.data_ptr()
    a.global_seqlens_host, a.ring_sizes_host, a.ring_starts_host = g.data_ptr(), s.data_ptr(), st.data_ptr()
    a.stats = stats.data_ptr()
    a.batch, a.world_size, a.rank, a.rank_kv_capacity = len(docs), world, rank, CAP
    a.total_q, a.heads_q, a.heads_k, a.head_dim = q.size(0), QH, KVH, 128
    a.is_causal = int(causal)
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    a.num_comp_sm, a.num_comm_sm = sm - comm, comm
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _cabi.check(lib.b2a_ring_fwd(ctypes.byref(a), stream))
    return (g, s, st)   # keep the host arrays alive until the caller synchronises


def expected_stats(docs, rank, causal):
    """(query-tile visits, K/V tile reads) the kernel must count for one rank: every 128-row query
    tile of every head once, and per tile the unmasked blocks of the chunks before its own plus the
    causal part of its own chunk."""
    visits = reads = 0
    for (glen, g, start) in docs:
        if not start <= rank < start + g:
            continue
        rr, llen = rank - start, glen // g
        halves = 2 if (causal and g > 1) else 1
        hb = (llen // halves) // 128
        for h in range(halves):
            if causal:
                chunks = 0 if g == 1 else (rr if h == 0 else 2 * g - 1 - rr)
            else:
                chunks = g
            for t in range(hb):
                visits += QH
                reads += QH * (chunks * hb + (t + 1 if causal else 0))
    return visits, reads


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_virtual_ranks_forward_matches_oracle(world, causal):
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    docs = ring_docs_for(world, causal)
    problems = [build_problem(world, r, docs, QH, KVH, causal, 4242 + causal) for r in range(world)]
    arenas_k = [torch.full((world * CAP, KVH, 128), SENTINEL, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    arenas_v = [torch.full((world * CAP, KVH, 128), SENTINEL, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    for r, (_q, k, v, _d, _cu, _o) in enumerate(problems):
        arenas_k[r][r * CAP: r * CAP + k.size(0)] = k.to(dev)
        arenas_v[r][r * CAP: r * CAP + v.size(0)] = v.to(dev)
    torch.cuda.synchronize()

    for rep in range(2):   # flags and tickets live in the workspace and must reset between launches
        keep, results = [], []
        for r, (q, k, _v, _d, cu, _o) in enumerate(problems):
            qd = q.to(dev)
            out = torch.full((q.size(0), QH, 128), SENTINEL, dtype=torch.bfloat16, device=dev)
            lse = torch.full((QH, q.size(0)), SENTINEL, dtype=torch.float32, device=dev)
            stats = torch.zeros(2, dtype=torch.int64, device=dev)
            nbytes = lib.b2a_ring_fwd_workspace_bytes(len(docs), world, CAP, q.size(0))
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            keep.append((qd, launch_rank(lib, r, world, qd, out, lse, arenas_k, arenas_v, cu, docs, causal, ws, stats)))
            results.append((out, lse, ws, stats))
        torch.cuda.synchronize()
        for r, (q, k, v, _d, cu, odocs) in enumerate(problems):
            out, lse, ws, stats = results[r]
            _cabi.check(lib.b2a_check_status(ctypes.c_void_p(ws.data_ptr()), None))
            ref_o, ref_l = oracle_forward(odocs, causal)
            tol = doc_bounds(odocs, causal)
            eo = (out.float().cpu() - ref_o).abs().max().item()
            el = (lse.cpu() - ref_l).abs().max().item()
            assert eo <= tol["o"], f"rank {r} rep {rep}: O error {eo:.3e} exceeds {tol['o']:.3e}"
            assert el <= LSE_ATOL, f"rank {r} rep {rep}: LSE error {el:.3e}"
            assert tuple(stats.tolist()) == expected_stats(docs, r, causal), "device-side work counters"
            # rows past the local slice were never addressed by any ring
            tail = arenas_k[r][r * CAP + k.size(0): (r + 1) * CAP]
            assert bool((tail.float() == SENTINEL).all().item())

    # Every remote block a rank fetched is a bit-exact copy of its owner's rows
    # (reference: scripts/test_mega_ring/mega_ring_test_min_fa3_varlen_hybrid_multi_rank.py:357-400).
    for r in range(world):
        for s in range(world):
            if s == r:
                continue
            mine = arenas_k[r][s * CAP:(s + 1) * CAP]
            theirs = arenas_k[s][s * CAP:(s + 1) * CAP]
            fetched = (mine.float() != SENTINEL).flatten(1).any(dim=1)
            assert torch.equal(mine[fetched], theirs[fetched])
            mine_v = arenas_v[r][s * CAP:(s + 1) * CAP]
            assert torch.equal(mine_v[fetched], arenas_v[s][s * CAP:(s + 1) * CAP][fetched])
        if world > 1 and causal is False:
            assert int(((arenas_k[r].float() != SENTINEL).flatten(1).any(dim=1)).sum()) > problems[r][1].size(0)
