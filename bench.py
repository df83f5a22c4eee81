"""Benchmark of the attention hot path: forward + backward on synthetic inputs.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU attention

One step is one forward + backward pass over the workload.  At every N the workload is
benchmark configuration 2 per GPU (BSHD, causal, B=4, S=8192, QH=32, KVH=8, d=128, bf16 N(0,1)
from a fixed seed): each rank owns an independent batch, there is no data-path collective,
scaling is weak.  Printed numbers use the causal-discounted algorithmic FLOPs
``14 * QH * D * sum_docs L(L+1)/2`` per step (forward 4x, backward 10x).

The JSON line carries: ``value`` (whole-job TFLOPS with inputs resident in HBM, CUDA events,
max over ranks), ``e2e`` (same metric from pinned host buffers to pinned host buffers through
``min_fa3_demo_b200.host_pipeline``: upload, ``min_fa3_op`` calls and download of successive
batch elements overlapped, all inside the timed region), ``roofline`` (dominant kernel = the
backward main kernel, timed live with CUDA events around each launch), ``cpu_baseline``
(fp32 PyTorch SDPA forward + autograd backward on the host cores, a bounded sample) and
``clocks`` sampled with nvidia-smi during the timed region.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = dict(name="bshd_causal_B4_S8192_QH32_KVH8_D128", batch=4, seqlen=8192, heads_q=32,
                heads_k=8, head_dim=128, causal=True)
METRIC = "fwd+bwd attention TFLOPS (causal FLOPs), whole job; per-GPU value and % of bf16 peak alongside"
UNIT = "TFLOPS"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0


def step_flops(w=WORKLOAD):
    s = w["seqlen"]
    vis = s * (s + 1) / 2 if w["causal"] else float(s) * s
    unit = w["heads_q"] * w["head_dim"] * vis * w["batch"]
    return 4.0 * unit, 10.0 * unit


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["bf16_tflops"]), float(data.get("bf16_tflops_sustained", 0.0)), "measured"
    return FALLBACK_BF16_TFLOPS, 1400.0, "fallback"


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons in the background."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.samples = []
        self.proc = None
        self.thread = None
        self.window = [None, None]   # sample-count marks bracketing the timed region

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def mark_begin(self):
        self.window[0] = len(self.samples)

    def mark_end(self):
        self.window[1] = len(self.samples)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        lo = self.window[0] or 0
        hi = self.window[1] if self.window[1] is not None else len(self.samples)
        # keep one sample either side so that short timed regions still see a reading
        chosen = self.samples[max(lo - 1, 0):hi + 1]
        for parts in chosen:
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------
# CPU baseline / reference arm
# --------------------------------------------------------------------------------------
def cpu_attention_sample(seconds_budget: float, seed: int = 0):
    """Times the reference's CPU-capable attention (fp32 SDPA + autograd backward,
    scripts/test_min_fa3/test_min_fa3_backward.py:16-36) on KV-head groups of the workload:
    one group = one batch element, one KV head and its QH/KVH query heads at full S.
    Returns (TFLOPS, groups timed, seconds)."""
    import torch.nn.functional as F

    w = WORKLOAD
    torch.set_num_threads(os.cpu_count() or 1)
    g = w["heads_q"] // w["heads_k"]
    gen = torch.Generator().manual_seed(seed)
    s = w["seqlen"]
    fwd, bwd = step_flops()
    group_flops = (fwd + bwd) / (w["batch"] * w["heads_k"])
    done, t0 = 0, time.perf_counter()
    while True:
        q = torch.randn(1, g, s, 128, generator=gen).to(torch.bfloat16).float().requires_grad_()
        k = torch.randn(1, 1, s, 128, generator=gen).to(torch.bfloat16).float().requires_grad_()
        v = torch.randn(1, 1, s, 128, generator=gen).to(torch.bfloat16).float().requires_grad_()
        dout = torch.randn(1, g, s, 128, generator=gen).to(torch.bfloat16).float()
        if done == 0:
            t0 = time.perf_counter()   # exclude the first input generation
        out = F.scaled_dot_product_attention(q, k, v, is_causal=w["causal"], enable_gqa=g != 1)
        torch.autograd.grad(out, (q, k, v), dout)
        done += 1
        elapsed = time.perf_counter() - t0
        if elapsed >= seconds_budget or done >= w["batch"] * w["heads_k"]:
            break
    return done * group_flops / elapsed / 1e12, done, elapsed


def cpu_baseline_record(seconds_budget: float) -> dict:
    tflops, groups, secs = cpu_attention_sample(seconds_budget)
    w = WORKLOAD
    return {"value": tflops, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{groups} of {w['batch'] * w['heads_k']} (batch, KV-head) groups of the workload "
                      f"(each {w['heads_q'] // w['heads_k']} query heads x 1 KV head, S={w['seqlen']}, causal), "
                      f"fp32 torch SDPA forward + autograd backward, {secs:.1f} s"}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(min(args.warmup, 1)):
        cpu_attention_sample(2.0)
    values, t0 = [], time.perf_counter()
    per_step_budget = max(2.0, min(10.0, 90.0 / max(args.steps, 1)))
    samples = []
    for _ in range(args.steps):
        tflops, groups, secs = cpu_attention_sample(per_step_budget)
        values.append(tflops)
        samples.append((groups, secs))
    value = statistics.mean(values)
    fwd, bwd = step_flops()
    w = WORKLOAD
    sample = (f"each step: {samples[0][0]} of {w['batch'] * w['heads_k']} (batch, KV-head) groups, fp32 torch SDPA "
              f"forward + autograd backward on CPU, ~{per_step_budget:.0f} s; value = mean over steps")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": (fwd + bwd) / (value * 1e12) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "note": "ms_per_step extrapolates the sampled rate to the full workload"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# CUDA arm
# --------------------------------------------------------------------------------------
def run_cuda_arm(args) -> None:
    import torch.distributed as dist

    import min_fa3_op
    from min_fa3_demo_b200 import _cabi

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.load()   # raises if the CUDA library is missing

    w = WORKLOAD
    b, s, qh, kvh = w["batch"], w["seqlen"], w["heads_q"], w["heads_k"]
    causal = w["causal"]
    gen = torch.Generator(device="cpu").manual_seed(1000 * 0 + rank)
    host = {}
    for name, heads in (("q", qh), ("k", kvh), ("v", kvh), ("dout", qh)):
        t = torch.empty(b, s, heads, 128, dtype=torch.bfloat16).pin_memory()
        t.copy_(torch.randn(b, s, heads, 128, generator=gen).to(torch.bfloat16))
        host[name] = t
    q, k, v, dout = (host[n].to(dev, non_blocking=True) for n in ("q", "k", "v", "dout"))
    torch.cuda.synchronize()

    def step_resident():
        out, lse = min_fa3_op.forward(q, k, v, causal, return_lse=True)
        return out, min_fa3_op.backward(dout, q, k, v, out, lse, causal)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    fwd_flops, bwd_flops = step_flops()
    flops = fwd_flops + bwd_flops

    # ---- device-resident timing -------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_resident()
    barrier()
    lib.b2a_profile_enable(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark_begin()
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    barrier()
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = e0.elapsed_time(e1)
    buf = (ctypes.c_float * 256)()
    n_bwd = lib.b2a_profile_read(1, buf, 256)
    bwd_ms = [buf[i] for i in range(n_bwd)]
    n_fwd = lib.b2a_profile_read(0, buf, 256)
    fwd_ms = [buf[i] for i in range(n_fwd)]
    lib.b2a_profile_enable(0)
    t = torch.tensor([ms_total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps

    # ---- end to end through the public API with host buffers ---------------------------
    from min_fa3_demo_b200.host_pipeline import HostPipeline
    host_out = {"out": torch.empty_like(host["q"]).pin_memory(), "dq": torch.empty_like(host["q"]).pin_memory(),
                "dk": torch.empty_like(host["k"]).pin_memory(), "dv": torch.empty_like(host["v"]).pin_memory()}
    pipeline = HostPipeline(dev, s, qh, kvh, head_groups=args.e2e_head_groups)

    def step_e2e():
        # Host q, k, v, dout in; host out, dq, dk, dv back: upload, kernels and download of
        # successive batch elements overlap on three streams.
        pipeline.run(host, host_out, causal)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms = None
    if not args.skip_e2e:
        for _ in range(2):
            step_e2e()
        barrier()
        e0.record()
        for _ in range(e2e_steps):
            step_e2e()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item() / e2e_steps
    h2d = sum(host[n].numel() * 2 for n in ("q", "k", "v", "dout"))
    d2h = sum(t.numel() * 2 for t in host_out.values())

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    burst, sustained, peak_kind = measured_peaks()
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    bwd_avg_ms = statistics.mean(bwd_ms) if bwd_ms else None
    achieved = bwd_flops / (bwd_avg_ms * 1e-3) / 1e12 if bwd_avg_ms else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "batch_per_gpu": b, "seq_len": s, "heads_q": qh,
                   "heads_k": kvh, "head_dim": 128, "causal": causal,
                   "parallelism": f"{world} independent replica(s), no data-path collective",
                   "l2": "inputs larger than L2 (1.7 GB of tensors per step vs 126 MB L2)",
                   "flops_per_step_per_gpu": flops},
        "tflops_per_gpu": value / world,
        "pct_of_bf16_peak": {f"{peak_kind}_burst": 100.0 * value / world / burst,
                             f"{peak_kind}_sustained": 100.0 * value / world / sustained if sustained else None,
                             "nominal_dense_2250": 100.0 * value / world / NOMINAL_BF16_TFLOPS},
        "kernel_ms": {"fwd_kernel": statistics.mean(fwd_ms) if fwd_ms else None,
                      "bwd_kernel": bwd_avg_ms,
                      "fwd_tflops": fwd_flops / (statistics.mean(fwd_ms) * 1e-3) / 1e12 if fwd_ms else None},
        "roofline": {"bound": "tensor", "kernel": "bwd_kernel", "achieved": achieved, "peak": sustained or burst,
                     "peak_kind": f"{peak_kind} sustained cuBLAS bf16 (kernel timed inside a long step)",
                     "unit": "TFLOP/s", "frac": achieved / (sustained or burst) if achieved else None,
                     "frac_of_burst": achieved / burst if achieved else None,
                     "traffic": None},
        "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12 if e2e_ms else None, "unit": UNIT,
                "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "min_fa3_demo_b200.host_pipeline.HostPipeline.run (pinned host tensors in and out; "
                       "(batch element, KV-head group) chunks pipelined over upload / compute / download streams)"},
        "gpu_launches": 4 * args.steps,
        "gpu_launches_note": "per step: fwd_kernel, bwd_preprocess_kernel, bwd_kernel, bwd_postprocess_kernel",
        "clocks": clocks,
    }
    if world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_record(args.cpu_seconds)
    traffic_file = ROOT / "profiles" / "bwd_kernel_traffic.json"
    if traffic_file.exists():
        line["roofline"]["traffic"] = json.loads(traffic_file.read_text()).get("dram_bytes_per_launch")
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# Ring context-parallel workload (benchmark configuration 4)
# --------------------------------------------------------------------------------------
def run_ring_workload(args) -> None:
    """One 131,072-token causal sequence (QH=32, KVH=8, d=128), zigzag-sharded over the N ranks;
    K/V of the other ranks is pulled over NVLink inside the attention launch.  Strong scaling:
    the problem is fixed, so whole-job TFLOPS = total FLOPs / max-over-ranks time.  Forward and
    backward are timed separately and summed; the backward time excludes the forward and the
    accumulator zeroing + barrier that must precede every backward call (the reference's protocol,
    ring_test/homogeneous_all_cp_microbench/benchmark_ring_backward.py:413-446)."""
    import torch.distributed as dist

    import min_fa3_op

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from min_fa3_demo_b200 import balancer as bal

    varlen = args.workload == "ring_varlen"
    if varlen:
        # Config 5: mixture-distributed documents, load-balanced placement on sub-rings.
        qh, kvh = 64, 8
        lengths = bal.sample_mixture_lengths(0, target_tokens=args.ring_tokens)
        lengths[-1] -= sum(lengths) - args.ring_tokens      # last document truncated to fill
        if world > 1:
            plan = bal.assign_hierarchical_rings(lengths, world, True)
            glens, sizes, starts = plan.global_lengths, plan.ring_sizes, plan.ring_starts
            lens, cu_list = bal.local_layout(plan, rank)
            cap = max(sum(bal.local_layout(plan, r)[0]) for r in range(world))
            balance = {"compute_deviation": plan.compute_deviation, "token_deviation": plan.token_deviation,
                       "feasible": plan.feasible, "ring_sizes": sorted(set(sizes), reverse=True)}
        else:
            glens, sizes, starts = list(lengths), [1] * len(lengths), [0] * len(lengths)
            lens = list(lengths)
            cu_list = [0]
            for n in lens:
                cu_list.append(cu_list[-1] + n)
            cap, balance = cu_list[-1], None
    else:
        # Config 4: one sequence over all ranks.
        qh, kvh = 32, 8
        glens, sizes, starts = [args.ring_tokens], [world], [0]
        lens = [args.ring_tokens // world]
        cu_list = [0, lens[0]]
        cap, balance = lens[0], None
    total = sum(glens)
    cap = ((cap + 127) // 128) * 128
    local = cu_list[-1]
    max_len = max(lens)
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    q = torch.randn(local, qh, 128, device=dev, generator=gen).to(torch.bfloat16)
    k = torch.randn(local, kvh, 128, device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(local, kvh, 128, device=dev, generator=gen).to(torch.bfloat16)
    dout = torch.randn(local, qh, 128, device=dev, generator=gen).to(torch.bfloat16)
    cu = torch.tensor(cu_list, dtype=torch.int32)
    cud = cu.to(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    if world == 1:
        def fwd():
            return min_fa3_op.forward_varlen(q, k, v, cud, cud, max_len, max_len, True, cu_seqlens_q_host=cu,
                                             cu_seqlens_k_host=cu, return_lse=True)

        def bwd(out, lse):
            return min_fa3_op.backward_varlen(dout, q, k, v, out, lse, cud, cud, max_len, max_len, True)

        def reset():
            pass
    else:
        arena_k = torch.zeros(world * cap, kvh, 128, dtype=torch.bfloat16, device=dev)
        arena_v = torch.zeros_like(arena_k)
        arena_k[rank * cap:rank * cap + local] = k
        arena_v[rank * cap:rank * cap + local] = v
        rk = min_fa3_op.TKParallelTensor(arena_k, local_rank=local_rank, local_world_size=world, multicast=False)
        rv = min_fa3_op.TKParallelTensor(arena_v, local_rank=local_rank, local_world_size=world, multicast=False)
        acc_k = min_fa3_op.TKParallelTensor([kvh * cap * 128], torch.float32, local_rank, world, False)
        acc_v = min_fa3_op.TKParallelTensor([kvh * cap * 128], torch.float32, local_rank, world, False)
        done = min_fa3_op.TKParallelTensor([1], torch.int32, local_rank, world, False)
        meta = dict(global_seqlens_host=torch.tensor(glens, dtype=torch.int32),
                    ring_sizes_host=torch.tensor(sizes, dtype=torch.int32),
                    ring_starts_host=torch.tensor(starts, dtype=torch.int32))
        comm = args.ring_comm_sm

        def fwd():
            return min_fa3_op.forward_varlen_mega_ring(
                q, rk.data_, rv.data_, cud, cud, max_len, max_len, True, cu_seqlens_q_host=cu,
                cu_seqlens_k_host=cu, remote_k=rk, remote_v=rv, num_comp_sm=sm - comm, num_comm_sm=comm,
                return_lse=True, **meta)

        def bwd(out, lse):
            return min_fa3_op.backward_varlen_mega_ring(
                dout, q, rk.data_, rv.data_, out, lse, cud, cud, max_len, max_len, cu_seqlens_q_host=cu,
                cu_seqlens_k_host=cu, remote_k=rk, remote_v=rv, remote_dk_accum=acc_k, remote_dv_accum=acc_v,
                remote_dkv_completion=done, num_comp_sm=sm - comm, num_comm_sm=comm, **meta)

        def reset():
            acc_k.data_.zero_()
            acc_v.data_.zero_()
            done.data_.zero_()
            barrier()

    if args.ring_impl == "allgather" and world > 1:
        if varlen:
            raise SystemExit("--ring-impl allgather is implemented for the single-sequence ring workload")
        # Comparison baseline built from library collectives: every rank gathers all K/V (NCCL
        # all_gather), restores global token order, and runs plain varlen attention for its two
        # zigzag halves as two documents whose keys are the global prefix each half may see
        # (causal, bottom-right aligned); backward scatters dK/dV of the two prefixes back to
        # global order and reduce_scatters them to their owners.
        half = local // 2
        chunks = 2 * world
        kv_shape = (world, local, kvh, 128)
        # chunk c of the global sequence lives on rank (c if c < world else chunks-1-c), front or back half
        order = torch.empty(chunks, dtype=torch.long)
        for c in range(chunks):
            r_own = c if c < world else chunks - 1 - c
            order[c] = r_own * 2 + (0 if c < world else 1)
        order_dev = order.to(dev)
        inv_dev = torch.argsort(order_dev)
        n_front, n_back = (rank + 1) * half, (chunks - rank) * half
        cu_q2 = torch.tensor([0, half, 2 * half], dtype=torch.int32)
        cu_k2 = torch.tensor([0, n_front, n_front + n_back], dtype=torch.int32)
        cu_q2d, cu_k2d = cu_q2.to(dev), cu_k2.to(dev)
        gk = torch.empty(kv_shape, dtype=torch.bfloat16, device=dev)
        gv = torch.empty(kv_shape, dtype=torch.bfloat16, device=dev)
        state = {}

        def global_order(t):      # [world, local, ...] in rank order -> [chunks * half, ...] in token order
            return t.view(chunks, half, kvh, 128).index_select(0, order_dev).reshape(chunks * half, kvh, 128)

        def fwd():
            dist.all_gather_into_tensor(gk, k)
            dist.all_gather_into_tensor(gv, v)
            kg, vg = global_order(gk), global_order(gv)
            k2 = torch.cat([kg[:n_front], kg[:n_back]])
            v2 = torch.cat([vg[:n_front], vg[:n_back]])
            state["k2"], state["v2"] = k2, v2
            return min_fa3_op.forward_varlen(q, k2, v2, cu_q2d, cu_k2d, half, n_back, True, cu_seqlens_q_host=cu_q2,
                                             cu_seqlens_k_host=cu_k2, return_lse=True)

        def bwd(out, lse):
            dq, dk2, dv2 = min_fa3_op.backward_varlen(dout, q, state["k2"], state["v2"], out, lse, cu_q2d, cu_k2d,
                                                      half, n_back, True)
            outs = []
            for d2 in (dk2, dv2):
                g = torch.zeros(chunks * half, kvh, 128, dtype=torch.float32, device=dev)
                g[:n_front] += d2[:n_front].float()
                g[:n_back] += d2[n_front:].float()
                # back to rank order [world, local, ...] and reduce_scatter to the owners
                g = g.view(chunks, half, kvh, 128).index_select(0, inv_dev).reshape(world, local, kvh, 128)
                mine = torch.empty(local, kvh, 128, dtype=torch.float32, device=dev)
                dist.reduce_scatter_tensor(mine, g)
                outs.append(mine.to(torch.bfloat16))
            return dq, outs[0], outs[1]

        def reset():
            pass

    barrier()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    fwd_ms, bwd_ms = [], []
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for it in range(max(args.warmup, 3) + args.steps):
        if it == max(args.warmup, 3):
            sampler.mark_begin()
        barrier()
        e[0].record()
        out, lse = fwd()
        e[1].record()
        reset()
        e[2].record()
        bwd(out, lse)
        e[3].record()
        torch.cuda.synchronize()
        t = torch.tensor([e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3])], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)   # per-iteration max over ranks
        if it >= max(args.warmup, 3):
            fwd_ms.append(t[0].item())
            bwd_ms.append(t[1].item())
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        vis = sum(n * (n + 1) / 2 for n in glens)
        f_flops, b_flops = 4.0 * qh * 128 * vis, 10.0 * qh * 128 * vis
        fm, bm = statistics.mean(fwd_ms), statistics.mean(bwd_ms)
        burst, sustained, peak_kind = measured_peaks()
        value = (f_flops + b_flops) / ((fm + bm) * 1e-3) / 1e12
        # K/V bytes rank 0 pulls per forward: for every document whose ring it is in, the shards of
        # the other ring members (rank 0 holds the first and the last chunk of a zigzag ring, so it
        # sees all of them).
        ingress = sum((g - 1) * (n // g) for n, g, st in zip(glens, sizes, starts) if st == 0 and g > 1)
        ingress *= kvh * 128 * 2 * 2
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": fm + bm, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": (f"ring_varlen_cp_causal_T{total}_docs{len(glens)}_QH{qh}_KVH{kvh}_D128" if varlen
                                    else f"ring_cp_causal_S{total}_QH{qh}_KVH{kvh}_D128"),
                       "tokens_rank0": local, "documents": len(glens), "placement": balance,
                       "parallelism": (f"cp{world} hierarchical zigzag sub-rings (load-balanced placement), "
                                       "K/V pulled over NVLink in-kernel" if varlen else
                                       f"cp{world} zigzag ring, K/V pulled over NVLink in-kernel")
                       if world > 1 else "single GPU (efficiency baseline)",
                       "copy_ctas": args.ring_comm_sm if world > 1 and args.ring_impl == "fused" else 0,
                       "exchange": ("in-kernel peer loads (fused)" if args.ring_impl == "fused" else
                                    "NCCL all_gather of K/V + reduce_scatter of dK/dV (comparison baseline)"),
                       "l2": "inputs larger than L2"},
            "tflops_per_gpu": value / world, "fwd_ms": fm, "bwd_ms": bm,
            "fwd_tflops_per_gpu": f_flops / (fm * 1e-3) / 1e12 / world,
            "bwd_tflops_per_gpu": b_flops / (bm * 1e-3) / 1e12 / world,
            "pct_of_bf16_peak": {f"{peak_kind}_burst": 100.0 * value / world / burst,
                                 f"{peak_kind}_sustained": 100.0 * value / world / sustained if sustained else None,
                                 "nominal_dense_2250": 100.0 * value / world / NOMINAL_BF16_TFLOPS},
            "nvlink": {"kv_ingress_bytes_rank0_fwd": ingress,
                       "achieved_gbs_over_fwd_kernel": ingress / (fm * 1e-3) / 1e9 if world > 1 else 0.0},
            "gpu_launches": 4 * args.steps, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# Packed varlen workload (benchmark configuration 3)
# --------------------------------------------------------------------------------------
def varlen_lengths(total: int = 65536, seed: int = 0):
    """Document lengths of config 3: log-normal (median 1,500, sigma 1.2) clipped to
    [128, 32768], drawn until ``total`` tokens are reached, the last one truncated to fill."""
    import math

    import numpy as np
    rng = np.random.default_rng(seed)
    out, acc = [], 0
    while acc < total:
        n = int(min(max(round(rng.lognormal(math.log(1500.0), 1.2)), 128), 32768))
        n = min(n, total - acc)
        out.append(n)
        acc += n
    return out


def run_varlen_workload(args) -> None:
    """65,536 packed tokens of causal attention on one GPU (QH=32, KVH=8, d=128), forward +
    backward through ``forward_varlen`` / ``backward_varlen``; inputs resident in HBM."""
    import min_fa3_op
    from min_fa3_demo_b200 import _cabi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    _cabi.load()
    qh, kvh = 32, 8
    lens = varlen_lengths()
    total = sum(lens)
    cu_list = [0]
    for n in lens:
        cu_list.append(cu_list[-1] + n)
    cu = torch.tensor(cu_list, dtype=torch.int32)
    cud = cu.to(dev)
    gen = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn(total, qh, 128, device=dev, generator=gen).to(torch.bfloat16)
    k = torch.randn(total, kvh, 128, device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(total, kvh, 128, device=dev, generator=gen).to(torch.bfloat16)
    dout = torch.randn(total, qh, 128, device=dev, generator=gen).to(torch.bfloat16)
    max_len = max(lens)

    def step():
        out, lse = min_fa3_op.forward_varlen(q, k, v, cud, cud, max_len, max_len, True, cu_seqlens_q_host=cu,
                                             cu_seqlens_k_host=cu, return_lse=True)
        return min_fa3_op.backward_varlen(dout, q, k, v, out, lse, cud, cud, max_len, max_len, True)

    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark_begin()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    sampler.mark_end()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    vis = sum(n * (n + 1) / 2 for n in lens)
    flops = 14.0 * qh * 128 * vis
    burst, sustained, peak_kind = measured_peaks()
    value = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"varlen_causal_T{total}_docs{len(lens)}_QH{qh}_KVH{kvh}_D128",
                   "longest_document": max_len, "shortest_document": min(lens),
                   "l2": "inputs larger than L2", "flops_per_step_per_gpu": flops},
        "tflops_per_gpu": value,
        "pct_of_bf16_peak": {f"{peak_kind}_burst": 100.0 * value / burst,
                             f"{peak_kind}_sustained": 100.0 * value / sustained if sustained else None,
                             "nominal_dense_2250": 100.0 * value / NOMINAL_BF16_TFLOPS},
        "gpu_launches": 6 * args.steps,
        "gpu_launches_note": "per step: 2 x varlen_plan_kernel, fwd_kernel, bwd_preprocess_kernel, bwd_kernel, "
                             "bwd_postprocess_kernel",
        "clocks": clocks}), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=30)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("cuda", "reference"), default="cuda")
    parser.add_argument("--cpu-seconds", type=float, default=15.0,
                        help="time budget of the CPU baseline sample (N=1 only)")
    parser.add_argument("--batch", type=int, default=None,
                        help="override the per-GPU batch (smaller cases for profiler captures)")
    parser.add_argument("--workload", choices=("bshd", "varlen", "ring", "ring_varlen"), default="bshd",
                        help="bshd: config 2 replicas (default); varlen: config 3 (65,536 packed tokens, 1 GPU); "
                             "ring: config 4, one long causal sequence over N ranks; ring_varlen: config 5, "
                             "131,072 packed tokens placed on hierarchical sub-rings over N ranks")
    parser.add_argument("--non-causal", action="store_true", help="bshd workload without the causal mask")
    parser.add_argument("--ring-tokens", type=int, default=131072)
    parser.add_argument("--ring-comm-sm", type=int, default=8)
    parser.add_argument("--ring-impl", choices=("fused", "allgather"), default="fused",
                        help="ring workload: fused = K/V pulled inside the attention launch (the product); "
                             "allgather = comparison baseline, NCCL all_gather of K/V + plain varlen attention + "
                             "NCCL reduce_scatter of dK/dV")
    parser.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg")
    parser.add_argument("--e2e-head-groups", type=int, default=2,
                        help="chunks per batch element in the host-buffer pipeline (must divide the KV heads)")
    parser.add_argument("--skip-cpu-baseline", action="store_true", help="skip the CPU baseline leg")
    args = parser.parse_args()
    if args.non_causal:
        WORKLOAD["causal"] = False
        WORKLOAD["name"] = WORKLOAD["name"].replace("bshd_causal", "bshd_noncausal")
    if args.batch is not None:
        WORKLOAD["batch"] = args.batch
        WORKLOAD["name"] = WORKLOAD["name"].replace("_B4_", f"_B{args.batch}_")
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload in ("ring", "ring_varlen"):
        run_ring_workload(args)
    elif args.workload == "varlen":
        run_varlen_workload(args)
    else:
        run_cuda_arm(args)


if __name__ == "__main__":
    main()
