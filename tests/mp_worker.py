"""Multi-rank worker for the context-parallel GPU tests.  Launched by tests/test_ring_gpu.py as
``python -m torch.distributed.run --nproc-per-node W tests/mp_worker.py <case>`` (one rank per GPU)
or run in-process with world size 1.  Every rank builds the same global problem from a seed,
keeps its zigzag shard, runs the CUDA path and checks it against the CPU oracle; failures are
voted across ranks so that every rank exits with the same status
(reference: scripts/test_min_fa3/test_min_fa3_varlen_ring_multi_rank.py:46-53)."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import min_fa3_op  # noqa: E402
from gpu_util import LSE_ATOL, bound  # noqa: E402
from min_fa3_demo_b200.ring import dkv_accum_numel  # noqa: E402
from oracle import attention_oracle as orc  # noqa: E402

SENTINEL = -123.0
BASE_SEED = 20260713


def setup():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return rank, world, torch.device("cuda", local_rank)


def barrier(world):
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()


def vote(ok: bool, world: int, what: str, rank: int) -> None:
    flag = torch.tensor([0 if ok else 1], device="cuda", dtype=torch.int32)
    if world > 1:
        dist.all_reduce(flag)
    if flag.item() != 0:
        raise SystemExit(f"[rank {rank}] {what}: FAILED on {flag.item()} rank(s)")
    if rank == 0:
        print(f"{what}: ok", flush=True)


def local_positions(g: int, r: int, local_len: int, causal: bool) -> torch.Tensor:
    """Global token positions of ring member r's shard (zigzag halves for causal rings)."""
    if g == 1:
        return torch.arange(local_len)
    if causal:
        return orc.zigzag_positions(g, r, local_len)
    return torch.arange(local_len) + r * local_len


def build_problem(world: int, rank: int, docs, qh: int, kvh: int, causal: bool, seed: int):
    """docs: list of (global_len, ring_size, ring_start), ring sizes non-increasing.
    Returns this rank's packed q, k, v, dout (bf16 CPU), cu_seqlens and, per member document,
    the global tensors for the oracle."""
    gen = torch.Generator().manual_seed(seed)
    q_parts, k_parts, v_parts, d_parts, lens, oracle_docs = [], [], [], [], [], []
    for (glen, g, start) in docs:
        qg = torch.randn(glen, qh, 128, generator=gen).to(torch.bfloat16)
        kg = torch.randn(glen, kvh, 128, generator=gen).to(torch.bfloat16)
        vg = (torch.randn(glen, kvh, 128, generator=gen) * 0.5).to(torch.bfloat16)
        dg = torch.randn(glen, qh, 128, generator=gen).to(torch.bfloat16)
        member = start <= rank < start + g
        if not member:
            lens.append(0)
            continue
        pos = local_positions(g, rank - start, glen // g, causal)
        q_parts.append(qg[pos]); k_parts.append(kg[pos]); v_parts.append(vg[pos]); d_parts.append(dg[pos])
        lens.append(glen // g)
        oracle_docs.append((qg, kg, vg, dg, pos))
    cu = torch.tensor([0, *torch.tensor(lens).cumsum(0).tolist()], dtype=torch.int32)

    def cat(parts, heads):
        return torch.cat(parts) if parts else torch.zeros(0, heads, 128, dtype=torch.bfloat16)
    return cat(q_parts, qh), cat(k_parts, kvh), cat(v_parts, kvh), cat(d_parts, qh), cu, oracle_docs


def oracle_forward(oracle_docs, causal):
    outs, lses = [], []
    for (qg, kg, vg, _dg, pos) in oracle_docs:
        kpos = torch.arange(kg.size(0)) if causal else None
        o, l = orc.attention_positions(qg[pos], kg, vg, pos if causal else None, kpos)
        outs.append(o); lses.append(l)
    return torch.cat(outs), torch.cat(lses, dim=1)


def doc_bounds(oracle_docs, causal) -> dict:
    """Acceptance bounds for this rank's outputs: 2x the max-abs error of a bf16 PyTorch attention
    against the fp32 oracle on the same global documents (worst document), as in the single-GPU
    tests; LSE is held to 1e-3 absolute by the callers."""
    worst = {"o": 0.0, "dq": 0.0, "dk": 0.0, "dv": 0.0}
    for (qg, kg, vg, dg, _pos) in oracle_docs:
        errs = orc.bf16_attention_error(qg[None], kg[None], vg[None], causal, dg[None])
        for key in worst:
            worst[key] = max(worst[key], errs[key])
    return {key: bound(val) for key, val in worst.items()}


def oracle_grads(oracle_docs, causal):
    """fp32 autograd over each global document, restricted to this rank's rows."""
    rq, rk, rv, ro = [], [], [], []
    for (qg, kg, vg, dg, pos) in oracle_docs:
        qf, kf, vf = (t.float().requires_grad_() for t in (qg, kg, vg))
        p_all = torch.arange(qg.size(0))
        o, _ = orc.attention_positions(qf, kf, vf, p_all if causal else None, p_all if causal else None)
        gq, gk, gv = torch.autograd.grad(o, (qf, kf, vf), dg.float())
        rq.append(gq[pos]); rk.append(gk[pos]); rv.append(gv[pos]); ro.append(o.detach()[pos])
    return torch.cat(rq), torch.cat(rk), torch.cat(rv), torch.cat(ro)


def make_accumulators(world, dev, kvh, cap, batch):
    numel = dkv_accum_numel(kvh, cap, batch)
    acc_k = min_fa3_op.TKParallelTensor([numel], torch.float32, dev.index, world, False)
    acc_v = min_fa3_op.TKParallelTensor([numel], torch.float32, dev.index, world, False)
    done = min_fa3_op.TKParallelTensor([1], torch.int32, dev.index, world, False)
    return acc_k, acc_v, done


def make_arena(world, rank, cap, local_k, local_v, dev):
    """Rank-major K/V arenas as parallel tensors; only the owner slice is written, the rest keeps
    a sentinel (reference: ...hybrid_multi_rank.py:159-189)."""
    kvh = local_k.size(1)
    ak = torch.full((world * cap, kvh, 128), SENTINEL, dtype=torch.bfloat16, device=dev)
    av = torch.full((world * cap, kvh, 128), SENTINEL, dtype=torch.bfloat16, device=dev)
    n = local_k.size(0)
    ak[rank * cap: rank * cap + n] = local_k.to(dev)
    av[rank * cap: rank * cap + n] = local_v.to(dev)
    rk = min_fa3_op.TKParallelTensor(ak, local_rank=dev.index, local_world_size=world, multicast=False)
    rv = min_fa3_op.TKParallelTensor(av, local_rank=dev.index, local_world_size=world, multicast=False)
    return rk, rv


def meta(docs):
    g = torch.tensor([d[0] for d in docs], dtype=torch.int32)
    s = torch.tensor([d[1] for d in docs], dtype=torch.int32)
    st = torch.tensor([d[2] for d in docs], dtype=torch.int32)
    return g, s, st


def ring_docs_for(world: int, causal: bool = True):
    """A hierarchical mix: all-rank documents, sub-rings, single-rank documents.  Without a causal
    mask a shard need not split into two 128-aligned halves: the mix then holds shards of 384 rows."""
    docs = [(world * 512, world, 0), (world * (256 if causal else 384), world, 0)]
    if world >= 4:
        half = world // 2
        docs += [(half * 512, half, 0), (half * 256, half, half)]
    if world >= 8:
        docs += [(2 * 256, 2, 2), (2 * 512, 2, world - 2)]
    if world >= 2:
        docs += [(512, 1, 0), (256, 1, world - 1), (128, 1, 1 % world)]
    else:
        docs += [(384, 1, 0)]
    return docs


def case_mega_ring_fwd(rank, world, dev):
    qh, kvh = 8, 2
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    for causal in (True, False):
        docs = ring_docs_for(world, causal)
        q, k, v, _d, cu, odocs = build_problem(world, rank, docs, qh, kvh, causal, BASE_SEED + causal)
        tol = doc_bounds(odocs, causal)
        cap = 2048
        rk, rv = make_arena(world, rank, cap, k, v, dev)
        barrier(world)
        g, s, st = meta(docs)
        lens = (cu[1:] - cu[:-1]).tolist()
        out = torch.full((q.size(0), qh, 128), SENTINEL, dtype=torch.bfloat16, device=dev)
        lse = torch.full((qh, q.size(0)), SENTINEL, dtype=torch.float32, device=dev)
        stats = torch.zeros(2, dtype=torch.int64, device=dev)
        ok = True
        for rep in range(3):   # repeated launches: flags and tickets must reset correctly
            min_fa3_op.forward_varlen_mega_ring(
                q.to(dev), rk.data_, rv.data_, cu.to(dev), cu.to(dev), max(max(lens), 1), max(max(lens), 1), causal,
                cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, remote_k=rk, remote_v=rv,
                num_comp_sm=sm - 8, num_comm_sm=8, global_seqlens_host=g, ring_sizes_host=s,
                ring_starts_host=st, out=out, lse=lse, return_lse=True, stats=stats)
            torch.cuda.synchronize()
            try:
                min_fa3_op.check_last_status("forward_varlen_mega_ring")
            except RuntimeError as exc:
                print(f"[rank {rank}] device status: {exc}", flush=True)
                ok = False
            if q.size(0) > 0:
                ref_o, ref_l = oracle_forward(odocs, causal)
                eo = (out.float().cpu() - ref_o).abs().max().item()
                el = (lse.cpu() - ref_l).abs().max().item()
                if not (eo <= tol["o"] and el <= LSE_ATOL):
                    print(f"[rank {rank}] causal={causal} rep={rep}: O err {eo:.3e} (bound {tol['o']:.3e}) "
                          f"LSE err {el:.3e}", flush=True)
                    ok = False
            barrier(world)
        # arena rows never addressed by any ring keep their sentinel
        tail = rk.data_[rank * cap + k.size(0): (rank + 1) * cap]
        ok = ok and bool((tail.float() == SENTINEL).all().item())
        ok = ok and stats[0].item() > 0 if q.size(0) > 0 else ok
        vote(ok, world, f"mega_ring_fwd causal={causal} world={world}", rank)
        barrier(world)


def case_remote_load(rank, world, dev):
    # bit-exact peer copy (reference: scripts/test_min_fa3/test_parallel_remote_load.py:77-90)
    torch.manual_seed(100 + rank)
    t = torch.randn(512, 1024, device=dev).to(torch.bfloat16)
    pt = min_fa3_op.create_parallel_tensor(t, local_rank=dev.index, local_world_size=world)
    vec = torch.randn(64, 4096, device=dev).to(torch.bfloat16)
    pv = min_fa3_op.create_parallel_tensor(vec, local_rank=dev.index, local_world_size=world)
    barrier(world)
    ok = True
    for src in range(world):
        got = min_fa3_op.parallel_remote_load(pt, src, num_blocks=16)
        gotv = min_fa3_op.parallel_remote_load_vec(pv, src, output=torch.empty_like(vec))
        expect, expectv = t.clone(), vec.clone()
        if world > 1:
            dist.broadcast(expect, src)
            dist.broadcast(expectv, src)
        torch.cuda.synchronize()
        ok = ok and torch.equal(got, expect) and torch.equal(gotv, expectv)
    try:
        min_fa3_op.parallel_remote_load(pv, 0)
        ok = False
    except RuntimeError as exc:
        ok = ok and "currently supports 2D" not in str(exc)
    vote(ok, world, f"parallel_remote_load world={world}", rank)
    barrier(world)


def case_ring_steps(rank, world, dev):
    """Plain (non-zigzag) ring built from forward_varlen_ring steps, as the reference's
    benchmark loop does (ring_test/homogeneous_all_cp_microbench/benchmark_ring_forward.py:446-482).
    Every step with a successor runs attention and the peer copy in one launch (num_comm_sm > 0)."""
    qh, kvh, local = 4, 2, 384
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    for causal in (False, True):
        gen = torch.Generator().manual_seed(7 + causal)
        qg = torch.randn(world * local, qh, 128, generator=gen).to(torch.bfloat16)
        kg = torch.randn(world * local, kvh, 128, generator=gen).to(torch.bfloat16)
        vg = torch.randn(world * local, kvh, 128, generator=gen).to(torch.bfloat16)
        sl = slice(rank * local, (rank + 1) * local)
        q, k, v = qg[sl].to(dev), kg[sl].to(dev), vg[sl].to(dev)
        rk = min_fa3_op.create_parallel_tensor(k, local_rank=dev.index, local_world_size=world)
        rv = min_fa3_op.create_parallel_tensor(v, local_rank=dev.index, local_world_size=world)
        cu = torch.tensor([0, 128, local], dtype=torch.int32)
        barrier(world)
        pk = [torch.empty_like(k), torch.empty_like(k)]
        pvv = [torch.empty_like(v), torch.empty_like(v)]
        cur_k, cur_v, out, lse = k, v, None, None
        ok = True
        for step in range(world):
            if causal and step > rank:
                break
            nxt = (rank - step - 1 + world) % world
            comm = 4 if step + 1 < world else 0
            out, lse = min_fa3_op.forward_varlen_ring(
                q, cur_k, cur_v, cu.to(dev), cu.to(dev), 256, 256, causal and step == 0,
                cu_seqlens_q_host=cu, cu_seqlens_k_host=cu, remote_k=rk, remote_v=rv, src_rank=nxt,
                num_comp_sm=sm - 4, num_comm_sm=comm, ring_step=step, prefetch_k=pk[step % 2],
                prefetch_v=pvv[step % 2], out=out, lse=lse, return_lse=True)
            if step + 1 < world:
                torch.cuda.synchronize()
                # the prefetched buffers are bit-exact copies of the source rank's K/V
                # (reference: scripts/test_min_fa3/test_min_fa3_varlen_ring_multi_rank.py:192-196)
                src = slice(nxt * local, (nxt + 1) * local)
                ok = ok and torch.equal(pk[step % 2].cpu(), kg[src]) and torch.equal(pvv[step % 2].cpu(), vg[src])
                cur_k, cur_v = pk[step % 2], pvv[step % 2]
        torch.cuda.synchronize()
        try:
            min_fa3_op.check_last_status("forward_varlen_ring")
        except RuntimeError as exc:
            print(f"[rank {rank}] device status: {exc}", flush=True)
            ok = False
        # two documents per rank: document j of every rank forms one global sequence in rank order
        outs, lses, e_bf16 = [], [], 0.0
        for (a, b) in ((0, 128), (128, local)):
            n = b - a
            kk = torch.cat([kg[r * local + a: r * local + b] for r in range(world)])
            vv = torch.cat([vg[r * local + a: r * local + b] for r in range(world)])
            qq = torch.cat([qg[r * local + a: r * local + b] for r in range(world)])
            qpos = torch.arange(n) + rank * n if causal else None
            kpos = torch.arange(world * n) if causal else None
            o, l = orc.attention_positions(qg[rank * local + a: rank * local + b], kk, vv, qpos, kpos)
            outs.append(o); lses.append(l)
            e_bf16 = max(e_bf16, orc.bf16_attention_error(qq[None], kk[None], vv[None], causal)["o"])
        eo = (out.float().cpu() - torch.cat(outs)).abs().max().item()
        el = (lse.cpu() - torch.cat(lses, dim=1)).abs().max().item()
        if not (eo <= bound(e_bf16) and el <= LSE_ATOL):
            print(f"[rank {rank}] ring steps causal={causal}: O err {eo:.3e} (bound {bound(e_bf16):.3e}) "
                  f"LSE err {el:.3e}", flush=True)
            ok = False
        vote(ok, world, f"forward_varlen_ring steps causal={causal} world={world}", rank)
        barrier(world)


def case_mega_ring_bwd(rank, world, dev):
    """dQ / dK / dV of the context-parallel backward against fp32 autograd over the global
    documents (dense reference as in ...backward_multi_rank.py:95-122, oracle-side).  The first
    repetition pulls the remote K/V again like the reference's backward, the second one works on
    what the forward left in the arena (``kv_resident``)."""
    qh, kvh = 8, 2
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    for causal in (True, False):
        docs = ring_docs_for(world, causal)
        q, k, v, dout, cu, odocs = build_problem(world, rank, docs, qh, kvh, causal, BASE_SEED + 11 + causal)
        tol = doc_bounds(odocs, causal)
        cap = 2048
        rk, rv = make_arena(world, rank, cap, k, v, dev)
        acc_k, acc_v, done = make_accumulators(world, dev, kvh, cap, len(docs))
        g, s, st = meta(docs)
        lens = (cu[1:] - cu[:-1]).tolist()
        mx = max(max(lens), 1)
        qd, dd, cud = q.to(dev), dout.to(dev), cu.to(dev)
        barrier(world)
        ok = True
        for rep in range(2):
            out, lse = min_fa3_op.forward_varlen_mega_ring(
                qd, rk.data_, rv.data_, cud, cud, mx, mx, causal, cu_seqlens_q_host=cu, cu_seqlens_k_host=cu,
                remote_k=rk, remote_v=rv, num_comp_sm=sm - 8, num_comm_sm=8, global_seqlens_host=g,
                ring_sizes_host=s, ring_starts_host=st, return_lse=True)
            acc_k.data_.zero_(); acc_v.data_.zero_(); done.data_.zero_()
            barrier(world)
            dq, dk, dv = min_fa3_op.backward_varlen_mega_ring(
                dd, qd, rk.data_, rv.data_, out, lse, cud, cud, mx, mx, cu_seqlens_q_host=cu,
                cu_seqlens_k_host=cu, remote_k=rk, remote_v=rv, remote_dk_accum=acc_k, remote_dv_accum=acc_v,
                remote_dkv_completion=done, num_comp_sm=sm - 8, num_comm_sm=8, global_seqlens_host=g,
                ring_sizes_host=s, ring_starts_host=st, is_causal=causal, kv_resident=(rep == 1))
            torch.cuda.synchronize()
            try:
                min_fa3_op.check_last_status("backward_varlen_mega_ring")
            except RuntimeError as exc:
                print(f"[rank {rank}] device status: {exc}", flush=True)
                ok = False
            ok = ok and done.data_.item() == world
            if odocs:
                rq, rkk, rvv, _ro = oracle_grads(odocs, causal)
                for name, got, ref in (("dq", dq, rq), ("dk", dk, rkk), ("dv", dv, rvv)):
                    err = (got.float().cpu() - ref).abs().max().item()
                    if not err <= tol[name]:
                        print(f"[rank {rank}] causal={causal} rep={rep} {name}: err {err:.3e} bound {tol[name]:.3e}",
                              flush=True)
                        ok = False
            barrier(world)
        vote(ok, world, f"mega_ring_bwd causal={causal} world={world}", rank)
        barrier(world)


def case_ring_autograd(rank, world, dev):
    """The differentiable context-parallel front end (RingAttention): gradients of this rank's
    shard against fp32 autograd over the global documents.  Two layers share one object and run
    forward, forward, backward, backward (the order of a training step): the second forward
    overwrites the K/V arena, and the first layer's backward must still see its own K/V."""
    from min_fa3_demo_b200.autograd import RingAttention
    qh, kvh = 8, 2
    causal = True
    docs = ring_docs_for(world, causal)
    problems = [build_problem(world, rank, docs, qh, kvh, causal, BASE_SEED + 21 + layer) for layer in range(2)]
    lens = (problems[0][4][1:] - problems[0][4][:-1]).tolist()
    ring = RingAttention(2048, kvh, is_causal=causal, device=dev)
    ok = True
    for rep in range(2):
        leaves, outs = [], []
        for (q, k, v, _dout, _cu, _odocs) in problems:
            qd, kd, vd = (t.to(dev).requires_grad_() for t in (q, k, v))
            leaves.append((qd, kd, vd))
            outs.append(ring(qd, kd, vd, lens, [d[0] for d in docs], [d[1] for d in docs], [d[2] for d in docs]))
        for layer in (1, 0):
            outs[layer].backward(problems[layer][3].to(dev))
        torch.cuda.synchronize()
        for layer, (q, k, v, dout, _cu, odocs) in enumerate(problems):
            if not odocs:
                continue
            tol = doc_bounds(odocs, causal)
            rq, rkk, rvv, ro = oracle_grads(odocs, causal)
            qd, kd, vd = leaves[layer]
            for name, key, got, ref in (("out", "o", outs[layer].detach(), ro), ("dq", "dq", qd.grad, rq),
                                        ("dk", "dk", kd.grad, rkk), ("dv", "dv", vd.grad, rvv)):
                err = (got.float().cpu() - ref).abs().max().item()
                if not err <= tol[key]:
                    print(f"[rank {rank}] ring_autograd rep={rep} layer={layer} {name}: err {err:.3e} "
                          f"bound {tol[key]:.3e}", flush=True)
                    ok = False
        barrier(world)
    vote(ok, world, f"ring_autograd world={world}", rank)
    barrier(world)


def case_empty_rank(rank, world, dev):
    """A rank that holds no token of any document still takes part in the forward and in the
    backward's completion protocol (reference: csrc/mega_ring_min_fa3_varlen_ring_bindings.cu:568-575)."""
    if world < 2:
        if rank == 0:
            print("empty_rank: needs at least 2 ranks, skipped", flush=True)
        return
    qh, kvh, causal = 4, 2, True
    members = 1 << ((world - 1).bit_length() - 1)                 # largest power of two below world
    docs = []
    if members > 1:
        docs.append((members * 512, members, 0))
    docs += [(384 if r % 2 == 0 else 256, 1, r) for r in range(world - 1)]   # the last rank gets nothing
    q, k, v, dout, cu, odocs = build_problem(world, rank, docs, qh, kvh, causal, BASE_SEED + 31)
    assert (rank == world - 1) == (q.size(0) == 0), "test layout: exactly the last rank is empty"
    cap = 2048
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    rk, rv = make_arena(world, rank, cap, k, v, dev)
    acc_k, acc_v, done = make_accumulators(world, dev, kvh, cap, len(docs))
    g, s_, st = meta(docs)
    lens = (cu[1:] - cu[:-1]).tolist()
    mx = max(max(lens), 1)
    qd, dd, cud = q.to(dev), dout.to(dev), cu.to(dev)
    barrier(world)
    out, lse = min_fa3_op.forward_varlen_mega_ring(
        qd, rk.data_, rv.data_, cud, cud, mx, mx, causal, cu_seqlens_q_host=cu, cu_seqlens_k_host=cu,
        remote_k=rk, remote_v=rv, num_comp_sm=sm - 8, num_comm_sm=8, global_seqlens_host=g,
        ring_sizes_host=s_, ring_starts_host=st, return_lse=True)
    acc_k.data_.zero_(); acc_v.data_.zero_(); done.data_.zero_()
    barrier(world)
    dq, dk, dv = min_fa3_op.backward_varlen_mega_ring(
        dd, qd, rk.data_, rv.data_, out, lse, cud, cud, mx, mx, cu_seqlens_q_host=cu, cu_seqlens_k_host=cu,
        remote_k=rk, remote_v=rv, remote_dk_accum=acc_k, remote_dv_accum=acc_v, remote_dkv_completion=done,
        num_comp_sm=sm - 8, num_comm_sm=8, global_seqlens_host=g, ring_sizes_host=s_, ring_starts_host=st,
        is_causal=causal)
    torch.cuda.synchronize()
    ok = done.data_.item() == world and tuple(out.shape) == tuple(q.shape) and tuple(dk.shape) == tuple(k.shape)
    try:
        min_fa3_op.check_last_status("backward_varlen_mega_ring")
    except RuntimeError as exc:
        print(f"[rank {rank}] device status: {exc}", flush=True)
        ok = False
    if odocs:
        tol = doc_bounds(odocs, causal)
        rq, rkk, rvv, ro = oracle_grads(odocs, causal)
        for name, key, got, ref in (("out", "o", out, ro), ("dq", "dq", dq, rq), ("dk", "dk", dk, rkk),
                                    ("dv", "dv", dv, rvv)):
            err = (got.float().cpu() - ref).abs().max().item()
            if not err <= tol[key]:
                print(f"[rank {rank}] empty_rank {name}: err {err:.3e} bound {tol[key]:.3e}", flush=True)
                ok = False
    barrier(world)
    vote(ok, world, f"empty_rank world={world}", rank)
    barrier(world)


CASES = {"empty_rank": case_empty_rank, "ring_autograd": case_ring_autograd, "mega_ring_bwd": case_mega_ring_bwd, "mega_ring_fwd": case_mega_ring_fwd, "remote_load": case_remote_load, "ring_steps": case_ring_steps}


def main(argv):
    rank, world, dev = setup()
    names = argv[1:] or list(CASES)
    for name in names:
        CASES[name](rank, world, dev)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv)
