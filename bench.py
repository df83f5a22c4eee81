"""Benchmark of the attention hot path: forward + backward on synthetic inputs.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU attention

One step is one forward + backward pass over the workload.  At every N the headline workload
is benchmark configuration 2 per GPU (BSHD, causal, B=4, S=8192, QH=32, KVH=8, d=128, bf16
N(0,1) from a fixed seed): each rank owns an independent batch, there is no data-path
collective, scaling is weak.  For N >= 2 the same run then executes the path that shards --
context parallel, benchmark configuration 4: one 131,072-token causal sequence zigzag-sharded
over the N ranks with the K/V exchange inside the attention kernels -- times it with the
reference's protocol, times the same problem on rank 0 alone (T(1)), checks every rank's
results against fp32 PyTorch, and reports all of it as ``config.ring_cp`` (and as a JSON line
of its own before the headline line).  Printed numbers use the causal-discounted algorithmic
FLOPs ``14 * QH * D * sum_docs L(L+1)/2`` per step (forward 4x, backward 10x).

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


def workload_config(world: int) -> dict:
    """The ``config`` record of the headline workload; the same dict in both arms."""
    w = WORKLOAD
    fwd, bwd = step_flops()
    return {"workload": w["name"], "batch_per_gpu": w["batch"], "seq_len": w["seqlen"], "heads_q": w["heads_q"],
            "heads_k": w["heads_k"], "head_dim": 128, "causal": w["causal"],
            "parallelism": f"{world} independent replica(s), no data-path collective",
            "l2": "inputs larger than L2 (1.7 GB of tensors per step vs 126 MB L2)",
            "flops_per_step_per_gpu": fwd + bwd}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["bf16_tflops"]), float(data.get("bf16_tflops_sustained", 0.0)), "measured"
    return FALLBACK_BF16_TFLOPS, 1400.0, "fallback"


def kernel_source_digest() -> str:
    """SHA-256 over the backward kernel's sources: ties a recorded ncu capture to the code it measured."""
    import hashlib
    h = hashlib.sha256()
    for name in ("b2a_bwd.cuh", "b2a_bwd.cu", "b2a_ptx.cuh"):
        h.update((ROOT / "min_fa3_demo_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()


def recorded_traffic() -> dict:
    """DRAM bytes per launch of the dominant kernel from the committed ncu capture
    (profiles/bwd_kernel_traffic.json: read + write bytes of one launch at a smaller batch, scaled by
    the batch ratio).  A number taken under a profiler cannot be produced inside this run, so it is a
    record; it is reported only while the kernel sources still hash to what the capture measured,
    otherwise ``traffic`` is null and the note says the record is stale."""
    path = ROOT / "profiles" / "bwd_kernel_traffic.json"
    if not path.exists():
        return {"traffic": None, "traffic_note": "no ncu capture recorded"}
    rec = json.loads(path.read_text())
    if rec.get("kernel_source_sha256") != kernel_source_digest():
        return {"traffic": None, "traffic_note": "recorded ncu capture is stale: the kernel sources changed since "
                                                 f"{rec.get('captured_case')} was captured"}
    return {"traffic": rec.get("dram_bytes_per_launch"),
            "traffic_note": f"ncu capture of {rec.get('captured_case')} scaled x{rec.get('scale_to_bench_workload')} "
                            "(traffic is proportional to the batch), kernel sources unchanged since"}


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
        "config": workload_config(args.gpus),
        "sampled": "each step times a bounded sample of the workload's (batch, KV-head) groups on the host cores; "
                   "ms_per_step extrapolates the sampled rate to the full workload",
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
        return out, min_fa3_op.backward(dout, q, k, v, out, lse, causal, deterministic=w.get("deterministic", False))

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

    # ---- context parallel on the same N ranks (N >= 2) -------------------------------------------
    ring_cp = None
    if world > 1 and not args.skip_ring:
        del q, k, v, dout, pipeline
        torch.cuda.empty_cache()
        ring_cp = ring_cp_leg(args, rank, local_rank, world, dev, dist)

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
        "config": workload_config(world),
        "tflops_per_gpu": value / world,
        "pct_of_bf16_peak": {f"{peak_kind}_burst": 100.0 * value / world / burst,
                             f"{peak_kind}_sustained": 100.0 * value / world / sustained if sustained else None,
                             "nominal_dense_2250": 100.0 * value / world / NOMINAL_BF16_TFLOPS},
        "kernel_ms": {"fwd_kernel": statistics.mean(fwd_ms) if fwd_ms else None,
                      "bwd_kernel": bwd_avg_ms,
                      "fwd_tflops": fwd_flops / (statistics.mean(fwd_ms) * 1e-3) / 1e12 if fwd_ms else None},
        "roofline": {"bound": "tensor", "kernel": "bwd_kernel", "achieved": achieved, "peak": burst,
                     "peak_kind": f"{peak_kind} burst cuBLAS bf16 (the timed region is a fraction of a second, "
                                  "well short of the seconds-long loop behind the sustained figure)",
                     "unit": "TFLOP/s", "frac": achieved / burst if achieved else None,
                     "frac_of_sustained": achieved / sustained if achieved and sustained else None,
                     "traffic": None},  # filled from the recorded ncu capture below
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
    line["roofline"].update(recorded_traffic())
    if ring_cp is not None:
        # The path that shards: reported beside the replica headline (whose `value` stays the
        # configuration-2 number at every N) and as a line of its own.
        line["config"]["ring_cp"] = ring_cp
        print(json.dumps({"record": "ring_cp", **ring_cp}), flush=True)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# Context-parallel leg of the default multi-GPU run (benchmark configuration 4)
# --------------------------------------------------------------------------------------
def _zigzag_positions(world: int, rank: int, local: int, device) -> torch.Tensor:
    """Global positions of a rank's [front | back] shard: chunks r and 2W-1-r of 2W equal chunks."""
    half = local // 2
    ar = torch.arange(half, device=device)
    if world == 1:
        return torch.arange(local, device=device)
    return torch.cat([ar + rank * half, ar + (2 * world - 1 - rank) * half])


def _dense_rows(qs, k, v, qpos, kpos, dout=None, low_precision=False):
    """Checker, plain PyTorch on the GPU: causal attention of a few query rows ``qs [R, QH, 128]``
    over keys ``k, v [T, KVH, 128]`` with explicit positions (key j visible to row i when
    ``kpos[j] <= qpos[i]``).  fp32 throughout, or -- ``low_precision`` -- with bf16 scores,
    probabilities and products, the yardstick of the acceptance rule.  Returns ``out [R, QH, 128]``,
    ``lse [QH, R]`` and, with ``dout``, the gradients with respect to qs, k and v."""
    dt = torch.bfloat16 if low_precision else torch.float32
    group = qs.size(1) // k.size(1)
    leaves = [t.detach().to(dt).requires_grad_(dout is not None) for t in (qs, k, v)]
    q_, k_, v_ = leaves
    rows, kvh, t = qs.size(0), k.size(1), k.size(0)
    qg = q_.view(rows, kvh, group, 128)
    scores = torch.einsum("rhgd,thd->hgrt", qg, k_).float() * (128 ** -0.5)
    scores = scores.masked_fill((kpos[None, :] > qpos[:, None])[None, None], float("-inf"))
    lse = torch.logsumexp(scores, dim=-1).reshape(kvh * group, rows)
    probs = torch.softmax(scores, dim=-1).to(dt)
    out = torch.einsum("hgrt,thd->rhgd", probs, v_).reshape(rows, kvh * group, 128)
    grads = None
    if dout is not None:
        grads = torch.autograd.grad(out, leaves, dout.to(dt))
    return out.detach().float(), lse.detach(), grads


def _bound(e_low_precision: float) -> float:
    # acceptance rule: 2x the error of a bf16 PyTorch attention, never tighter than half a bf16 ulp at 1
    return 2.0 * max(e_low_precision, 2.0 ** -9)


def _key_rows_grads(qf, dof, of, lsef, qpos, kj, vj, kpos_j, low_precision=False):
    """Checker, plain PyTorch on the GPU: dK and dV of a few key rows ``kj, vj [R, KVH, 128]`` of one
    causal document from ALL its query rows ``qf, dof, of [T, QH, 128]`` with their log-sum-exp
    ``lsef [T, QH]`` (the O and LSE rows are the run's own, themselves checked on sampled rows):
    dV_j = sum_i P_ij dO_i and dK_j = scale * sum_i P_ij (dO_i . v_j - D_i) q_i with
    P_ij = exp(scale * q_i . k_j - LSE_i) and D_i = dO_i . O_i.  ``low_precision`` computes scores,
    probabilities, dS and the results in bf16, the yardstick of the acceptance rule."""
    t, qh = qf.size(0), qf.size(1)
    kvh = kj.size(1)
    group = qh // kvh
    scale = 128 ** -0.5
    dt = torch.bfloat16 if low_precision else torch.float32      # bf16: products and results rounded too
    qg = qf.to(dt).view(t, kvh, group, 128)
    dog = dof.to(dt).view(t, kvh, group, 128)
    dsum = (dof.float() * of.float()).sum(-1).view(t, kvh, group)
    lse = lsef.view(t, kvh, group)
    s_ = torch.einsum("thgd,rhd->thgr", qg, kj.to(dt)).float() * scale
    p_ = torch.exp(s_ - lse[..., None])
    p_ = p_.masked_fill((kpos_j[None, :] > qpos[:, None])[:, None, None, :], 0.0)
    dp = torch.einsum("thgd,rhd->thgr", dog, vj.to(dt)).float()
    ds = p_ * (dp - dsum[..., None])
    dv = torch.einsum("thgr,thgd->rhd", p_.to(dt), dog).float()
    dk = torch.einsum("thgr,thgd->rhd", ds.to(dt), qg).float() * scale
    return dk, dv


def _ring_workload_parity(rank, world, dev, dist, glens, sizes, starts, q, k, v, dout, out, lse, grads, cap):
    """Sampled-row check of a context-parallel run at its full size: for up to three of this
    rank's documents (largest, smallest, median), all heads, O / LSE / dQ of a few local query
    rows against plain fp32 PyTorch over the document's K/V, and dK / dV of a few local key rows
    from all query rows of the document -- the document's tensors are gathered from its ring
    members (checker plumbing: all_gathers of the local tensors).  Bound: 2x the error of the same
    computation with bf16 scores / probabilities, LSE 1e-3.  The verdict is voted over all ranks."""
    dq, dk, dv = grads

    def layout(r):
        lens = [n // g if st <= r < st + g else 0 for n, g, st in zip(glens, sizes, starts)]
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        return lens, cu

    def gathered(t):
        """[world, cap, ...] copy of every rank's local rows (zero padded)."""
        pad = torch.zeros((cap,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
        pad[:t.size(0)] = t
        if world == 1:
            return pad[None]
        full = torch.empty((world * cap,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
        dist.all_gather_into_tensor(full, pad)          # rank-major concatenation along the rows
        return full.view((world,) + tuple(pad.shape))
    gk, gv, gq, gdo, go = (gathered(t) for t in (k, v, q, dout, out))
    gl = gathered(lse.t().contiguous())                    # [world, cap, QH]
    lens, cu = layout(rank)
    mine = sorted((d for d in range(len(glens)) if lens[d] > 0), key=lambda d: glens[d])
    picks_d = sorted({mine[0], mine[len(mine) // 2], mine[-1]}) if mine else []
    worst = {"o": 0.0, "lse": 0.0, "dq": 0.0, "dk": 0.0, "dv": 0.0}
    checked = 0
    for d in picks_d:
        g, st, n = sizes[d], starts[d], lens[d]
        offs = [layout(m)[1][d] for m in range(st, st + g)]

        def doc(t):
            return torch.cat([t[m, off:off + n] for m, off in zip(range(st, st + g), offs)])
        kf, vf = doc(gk), doc(gv)
        pos = torch.cat([_zigzag_positions(g, m - st, n, dev) for m in range(st, st + g)])
        mypos = _zigzag_positions(g, rank - st, n, dev)
        rows = torch.tensor(sorted({0, n // 2 - 1, n // 2, n - 1, (104729 * (rank + 3)) % n, (7919 * (d + 5)) % n}),
                            device=dev)
        sel = rows + cu[d]
        ref_o, ref_l, ref_g = _dense_rows(q[sel], kf, vf, mypos[rows], pos, dout[sel])
        low_o, _low_l, low_g = _dense_rows(q[sel], kf, vf, mypos[rows], pos, dout[sel], low_precision=True)
        b_o = _bound((low_o - ref_o).abs().max().item())
        b_q = _bound((low_g[0].float() - ref_g[0]).abs().max().item())
        worst["o"] = max(worst["o"], (out[sel].float() - ref_o).abs().max().item() / b_o)
        worst["lse"] = max(worst["lse"], (lse[:, sel] - ref_l).abs().max().item() / 1e-3)
        worst["dq"] = max(worst["dq"], (dq[sel].float() - ref_g[0]).abs().max().item() / b_q)
        # dK / dV of a few local key rows from every query row of the document
        krows = torch.tensor(sorted({0, n // 2, n - 1, (15485863 * (rank + 1)) % n}), device=dev)
        ksel = krows + cu[d]
        operands = (doc(gq), doc(gdo), doc(go), doc(gl), pos, k[ksel], v[ksel], mypos[krows])
        ref_dk, ref_dv = _key_rows_grads(*operands)
        low_dk, low_dv = _key_rows_grads(*operands, low_precision=True)
        worst["dk"] = max(worst["dk"], (dk[ksel].float() - ref_dk).abs().max().item()
                          / _bound((low_dk - ref_dk).abs().max().item()))
        worst["dv"] = max(worst["dv"], (dv[ksel].float() - ref_dv).abs().max().item()
                          / _bound((low_dv - ref_dv).abs().max().item()))
        checked += rows.numel() + krows.numel()
    ok = all(x <= 1.0 for x in worst.values())
    keys = ("o", "lse", "dq", "dk", "dv")
    t = torch.tensor([1.0 if ok else 0.0, -float(checked)] + [-worst[key] for key in keys], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return {"pass": bool(t[0].item() == 1.0),
            "rule": "up to three documents per rank, all heads: O / LSE / dQ of sampled local query rows against "
                    "fp32 PyTorch over the document's K/V, dK / dV of sampled local key rows from all query rows "
                    "of the document; bound 2x the error of the same computation with bf16 scores / "
                    "probabilities, LSE 1e-3; worst ratio over all ranks",
            "worst_err_over_bound": {key: -t[2 + i].item() for i, key in enumerate(keys)},
            "rows_checked_max_rank": int(-t[1].item())}


def ring_cp_leg(args, rank: int, local_rank: int, world: int, dev, dist) -> dict:
    """Context parallel on all N ranks of the run: one 131,072-token causal sequence (QH 32, KVH 8,
    d 128), zigzag-sharded, K/V pulled over NVLink inside the attention launches, dK/dV added into
    the owner's accumulators.  Timing follows the reference's protocol
    (ring_test/benchmark_topology_forward.py:382-411, .../benchmark_ring_backward.py:413-446):
    CUDA events around forward and backward separately, per-iteration maximum over ranks, mean of
    the maxima; the accumulator zeroing + barrier before each backward is outside the timed part.
    In the same run rank 0 alone times the same 131,072-token problem on one GPU (T(1)), and every
    rank checks its results against a plain fp32 PyTorch computation on the GPU: O / LSE / dQ of
    sampled local rows of the full-size problem (all heads), and every output of a 2,048-token
    zigzag problem (all heads)."""
    import min_fa3_op
    from min_fa3_demo_b200 import _cabi
    from min_fa3_demo_b200.ring import dkv_accum_numel

    torch.backends.cuda.matmul.allow_tf32 = False
    lib = _cabi.load()
    qh, kvh, tokens = 32, 8, args.ring_tokens
    local = tokens // world
    cap = local
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    comm = args.ring_comm_sm
    warm = 3
    steps = max(3, min(args.steps, 10))

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()

    arena_k = torch.zeros(world * cap, kvh, 128, dtype=torch.bfloat16, device=dev)
    arena_v = torch.zeros_like(arena_k)
    rk = min_fa3_op.TKParallelTensor(arena_k, local_rank=local_rank, local_world_size=world, multicast=False)
    rv = min_fa3_op.TKParallelTensor(arena_v, local_rank=local_rank, local_world_size=world, multicast=False)
    accum = dkv_accum_numel(kvh, cap, 1)
    acc_k = min_fa3_op.TKParallelTensor([accum], torch.float32, local_rank, world, False)
    acc_v = min_fa3_op.TKParallelTensor([accum], torch.float32, local_rank, world, False)
    done = min_fa3_op.TKParallelTensor([1], torch.int32, local_rank, world, False)

    def run_ring(q, k, v, dout, glen, kv_resident=False):
        """One forward + backward of a single zigzag-sharded document of ``glen`` global tokens."""
        n = q.size(0)
        cu = torch.tensor([0, n], dtype=torch.int32)
        cud = cu.to(dev)
        meta = dict(global_seqlens_host=torch.tensor([glen], dtype=torch.int32),
                    ring_sizes_host=torch.tensor([world], dtype=torch.int32),
                    ring_starts_host=torch.tensor([0], dtype=torch.int32))
        arena_k[rank * cap:rank * cap + n] = k
        arena_v[rank * cap:rank * cap + n] = v
        barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        out, lse = min_fa3_op.forward_varlen_mega_ring(
            q, rk.data_, rv.data_, cud, cud, n, n, True, cu_seqlens_q_host=cu, cu_seqlens_k_host=cu,
            remote_k=rk, remote_v=rv, num_comp_sm=sm - comm, num_comm_sm=comm, return_lse=True, **meta)
        ev[1].record()
        acc_k.data_.zero_()
        acc_v.data_.zero_()
        done.data_.zero_()
        barrier()
        ev[2].record()
        dq, dk, dv = min_fa3_op.backward_varlen_mega_ring(
            dout, q, rk.data_, rv.data_, out, lse, cud, cud, n, n, cu_seqlens_q_host=cu, cu_seqlens_k_host=cu,
            remote_k=rk, remote_v=rv, remote_dk_accum=acc_k, remote_dv_accum=acc_v, remote_dkv_completion=done,
            num_comp_sm=sm - comm, num_comm_sm=comm, kv_resident=kv_resident, **meta)
        ev[3].record()
        torch.cuda.synchronize()
        times = torch.tensor([ev[0].elapsed_time(ev[1]), ev[2].elapsed_time(ev[3])], device=dev)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        return (out, lse, dq, dk, dv), times

    # ---- timed runs at full size --------------------------------------------------------
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    q = torch.randn(local, qh, 128, device=dev, generator=gen).to(torch.bfloat16)
    k = torch.randn(local, kvh, 128, device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(local, kvh, 128, device=dev, generator=gen).to(torch.bfloat16)
    dout = torch.randn(local, qh, 128, device=dev, generator=gen).to(torch.bfloat16)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    fwd_ms, bwd_ms, results = [], [], None
    for it in range(warm + steps):
        if it == warm:
            sampler.mark_begin()
        results, t = run_ring(q, k, v, dout, tokens)
        if it >= warm:
            fwd_ms.append(t[0].item())
            bwd_ms.append(t[1].item())
    sampler.mark_end()
    clocks_ring = sampler.stop() if rank == 0 else None
    # The same backward on the K/V blocks the forward left in the arena (no second pull); the
    # headline bwd_ms above is the self-contained call, as the reference times it.
    bwd_resident_ms = []
    for it in range(4):
        _res, t = run_ring(q, k, v, dout, tokens, kv_resident=True)
        if it >= 1:
            bwd_resident_ms.append(t[1].item())
    status_ok = True
    try:
        min_fa3_op.check_last_status()
    except RuntimeError as exc:
        status_ok = False
        print(f"[rank {rank}] ring leg device status: {exc}", file=sys.stderr, flush=True)

    # ---- parity, full size: sampled local rows against fp32 PyTorch over the gathered K/V -----
    out, lse, dq, dk, dv = results
    gk = torch.empty(world, local, kvh, 128, dtype=torch.bfloat16, device=dev)
    gv = torch.empty_like(gk)
    dist.all_gather_into_tensor(gk, k)      # checker plumbing, not the product's data path
    dist.all_gather_into_tensor(gv, v)
    kpos = torch.cat([_zigzag_positions(world, r, local, dev) for r in range(world)])
    qpos_all = _zigzag_positions(world, rank, local, dev)
    half = local // 2
    picks = sorted({0, 1, 127, 128, half - 1, half, half + 1, local - 129, local - 128, local - 1,
                    *[(104729 * (j + 1) * (rank + 3)) % local for j in range(22)]})
    rows = torch.tensor(picks, device=dev)
    kf, vf = gk.view(-1, kvh, 128), gv.view(-1, kvh, 128)
    ref_o, ref_l, ref_g = _dense_rows(q[rows], kf, vf, qpos_all[rows], kpos, dout[rows])
    low_o, _low_l, low_g = _dense_rows(q[rows], kf, vf, qpos_all[rows], kpos, dout[rows], low_precision=True)
    full = {
        "rows_per_rank": len(picks),
        "o_err": (out[rows].float() - ref_o).abs().max().item(),
        "o_bound": _bound((low_o - ref_o).abs().max().item()),
        "lse_err": (lse[:, rows] - ref_l).abs().max().item(), "lse_bound": 1e-3,
        "dq_err": (dq[rows].float() - ref_g[0]).abs().max().item(),
        "dq_bound": _bound((low_g[0].float() - ref_g[0]).abs().max().item()),
    }
    del gk, gv, kf, vf, ref_o, ref_l, ref_g, low_o, low_g

    # ---- parity, 2,048-token zigzag problem: every output, all heads ----------------------------
    small_tokens = max(2048, 256 * world)
    s_local = small_tokens // world
    gen_s = torch.Generator(device=dev).manual_seed(77)           # same global problem on every rank
    qg = torch.randn(small_tokens, qh, 128, device=dev, generator=gen_s).to(torch.bfloat16)
    kg = torch.randn(small_tokens, kvh, 128, device=dev, generator=gen_s).to(torch.bfloat16)
    vg = torch.randn(small_tokens, kvh, 128, device=dev, generator=gen_s).to(torch.bfloat16)
    dg = torch.randn(small_tokens, qh, 128, device=dev, generator=gen_s).to(torch.bfloat16)
    mine = _zigzag_positions(world, rank, s_local, dev)
    (so, sl, sdq, sdk, sdv), _ = run_ring(qg[mine].contiguous(), kg[mine].contiguous(), vg[mine].contiguous(),
                                          dg[mine].contiguous(), small_tokens)
    pos = torch.arange(small_tokens, device=dev)
    ref_o, ref_l, ref_g = _dense_rows(qg, kg, vg, pos, pos, dg)
    low_o, _l, low_g = _dense_rows(qg, kg, vg, pos, pos, dg, low_precision=True)
    small = {"tokens": small_tokens,
             "o_err": (so.float() - ref_o[mine]).abs().max().item(),
             "o_bound": _bound((low_o - ref_o).abs().max().item()),
             "lse_err": (sl - ref_l[:, mine]).abs().max().item(), "lse_bound": 1e-3}
    for name, got, idx in (("dq", sdq, 0), ("dk", sdk, 1), ("dv", sdv, 2)):
        small[f"{name}_err"] = (got.float() - ref_g[idx][mine]).abs().max().item()
        small[f"{name}_bound"] = _bound((low_g[idx].float() - ref_g[idx]).abs().max().item())
    try:
        min_fa3_op.check_last_status()
    except RuntimeError as exc:
        status_ok = False
        print(f"[rank {rank}] ring parity device status: {exc}", file=sys.stderr, flush=True)

    def passes(rec):
        return all(rec[key] <= rec[key.replace("_err", "_bound")] for key in rec if key.endswith("_err"))
    ok_local = status_ok and passes(full) and passes(small)
    flag = torch.tensor([0 if ok_local else 1], device=dev, dtype=torch.int32)
    dist.all_reduce(flag)
    # worst error / bound ratio over ranks, per quantity
    keys = [("full", key) for key in full if key.endswith("_err")] + [("small", key) for key in small if key.endswith("_err")]
    ratios = torch.tensor([(full if w == "full" else small)[key] / (full if w == "full" else small)[key.replace("_err", "_bound")]
                           for w, key in keys], device=dev)
    dist.all_reduce(ratios, op=dist.ReduceOp.MAX)

    # ---- peer copy probe: every rank pulls its neighbour's K slice with the library's copy kernel --
    probe_bytes = local * kvh * 128 * 2
    landing = torch.empty(local, kvh, 128, dtype=torch.bfloat16, device=dev)
    src = rk.raw_ptrs_[(rank + 1) % world] + ((rank + 1) % world) * cap * kvh * 256
    probe = {}
    for blocks in (8, 32, 128):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        reps = 4
        lib.b2a_peer_copy(ctypes.c_void_p(landing.data_ptr()), ctypes.c_void_p(src), probe_bytes, blocks, None, stream)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            lib.b2a_peer_copy(ctypes.c_void_p(landing.data_ptr()), ctypes.c_void_p(src), probe_bytes, blocks, None, stream)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        probe[f"{blocks}_ctas_gbs"] = probe_bytes / (t.item() * 1e-3) / 1e9
    del landing

    # ---- T(1): the same problem on rank 0 alone ------------------------------------------------------
    barrier()
    t1 = torch.zeros(3, device=dev)
    clocks_t1 = None
    if rank == 0:
        del q, k, v, dout, results, out, lse, dq, dk, dv
        torch.cuda.empty_cache()
        gen1 = torch.Generator(device=dev).manual_seed(4242)
        q1 = torch.randn(tokens, qh, 128, device=dev, generator=gen1).to(torch.bfloat16)
        k1 = torch.randn(tokens, kvh, 128, device=dev, generator=gen1).to(torch.bfloat16)
        v1 = torch.randn(tokens, kvh, 128, device=dev, generator=gen1).to(torch.bfloat16)
        d1 = torch.randn(tokens, qh, 128, device=dev, generator=gen1).to(torch.bfloat16)
        cu1 = torch.tensor([0, tokens], dtype=torch.int32)
        cu1d = cu1.to(dev)
        sampler1 = ClockSampler(local_rank)
        sampler1.start()
        f_ms, b_ms = [], []
        for it in range(1 + 2):
            if it == 1:
                sampler1.mark_begin()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            o1, l1 = min_fa3_op.forward_varlen(q1, k1, v1, cu1d, cu1d, tokens, tokens, True, cu_seqlens_q_host=cu1,
                                               cu_seqlens_k_host=cu1, return_lse=True)
            ev[1].record()
            min_fa3_op.backward_varlen(d1, q1, k1, v1, o1, l1, cu1d, cu1d, tokens, tokens, True)
            ev[2].record()
            torch.cuda.synchronize()
            if it >= 1:
                f_ms.append(ev[0].elapsed_time(ev[1]))
                b_ms.append(ev[1].elapsed_time(ev[2]))
        sampler1.mark_end()
        clocks_t1 = sampler1.stop()
        t1 = torch.tensor([statistics.mean(f_ms), statistics.mean(b_ms), 1.0], device=dev)
        del q1, k1, v1, d1, o1, l1
        torch.cuda.empty_cache()
    barrier()

    fm, bm = statistics.mean(fwd_ms), statistics.mean(bwd_ms)
    vis = tokens * (tokens + 1) / 2
    f_flops, b_flops = 4.0 * qh * 128 * vis, 10.0 * qh * 128 * vis
    ingress = (world - 1) * local * kvh * 128 * 2 * 2         # rank 0 sees every other shard: K and V
    burst, sustained, peak_kind = measured_peaks()
    rec = {
        "workload": f"ring_cp_causal_S{tokens}_QH{qh}_KVH{kvh}_D128", "n_gpus": world, "gpus_active": world,
        "parallelism": f"cp{world} zigzag ring, K/V pulled over NVLink in-kernel, dK/dV added into the owner's "
                       "accumulators over NVLink",
        "steps": steps, "warmup": warm,
        "timing": "CUDA events, forward and backward separately, per-iteration max over ranks, mean; the "
                  "accumulator zeroing + barrier before each backward is not timed (reference protocol)",
        "fwd_ms": fm, "bwd_ms": bm, "ms_per_step": fm + bm,
        "bwd_kv_resident_ms": statistics.mean(bwd_resident_ms),
        "tflops_per_gpu": (f_flops + b_flops) / ((fm + bm) * 1e-3) / 1e12 / world,
        "fwd_tflops_per_gpu": f_flops / (fm * 1e-3) / 1e12 / world,
        "bwd_tflops_per_gpu": b_flops / (bm * 1e-3) / 1e12 / world,
        "pct_of_bf16_peak_burst": 100.0 * (f_flops + b_flops) / ((fm + bm) * 1e-3) / 1e12 / world / burst,
        "copy_ctas": comm,
        "kv_ingress_bytes_rank0_fwd": ingress, "kv_ingress_gbs": ingress / (fm * 1e-3) / 1e9,
        "peer_copy_probe": {"bytes": probe_bytes, "what": "b2a_peer_copy of the neighbour rank's K slice, all "
                            "ranks at once, max over ranks", **probe},
        "parity": {"pass": flag.item() == 0, "device_status_ok": status_ok,
                   "rule": "max-abs error <= 2x the error of the same computation with bf16 scores/probabilities "
                           "(both against fp32 PyTorch on the GPU); LSE <= 1e-3",
                   "worst_err_over_bound": {f"{w}.{key[:-4]}": ratios[i].item() for i, (w, key) in enumerate(keys)},
                   "rank0_full_size_sampled_rows": full, "rank0_small_problem": small},
    }
    if rank == 0:
        t1f, t1b = t1[0].item(), t1[1].item()
        mhz_n = (clocks_ring or {}).get("sm_mhz")
        mhz_1 = (clocks_t1 or {}).get("sm_mhz")
        rec.update({
            "t1_fwd_ms": t1f, "t1_bwd_ms": t1b, "t1_ms": t1f + t1b,
            "t1_what": "same 131,072-token causal problem through forward_varlen / backward_varlen on rank 0 "
                       "alone, measured in this run (1 warm-up + 2 timed steps)",
            "sm_mhz": {"ring": mhz_n, "t1": mhz_1}, "clocks_ring": clocks_ring, "clocks_t1": clocks_t1,
            "efficiency": (t1f + t1b) / (world * (fm + bm)),
            "efficiency_fwd": t1f / (world * fm), "efficiency_bwd": t1b / (world * bm),
            "efficiency_clock_normalised": ((t1f + t1b) * mhz_1) / (world * (fm + bm) * mhz_n)
            if mhz_1 and mhz_n else None,
        })
    return rec


# --------------------------------------------------------------------------------------
# Ring context-parallel workload (benchmark configuration 4)
# --------------------------------------------------------------------------------------
def run_ring_workload(args, doc_lengths=None, emit=True):
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
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    from min_fa3_demo_b200 import balancer as bal

    varlen = args.workload in ("ring_varlen", "ring_dataset")
    if varlen:
        # Config 5: mixture-distributed documents, load-balanced placement on sub-rings
        # (or the document lengths of one dataset-shaped batch, given by the caller).
        qh, kvh = 64, 8
        if doc_lengths is not None:
            lengths = list(doc_lengths)
        else:
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
        from min_fa3_demo_b200.ring import dkv_accum_numel
        accum = dkv_accum_numel(kvh, cap, len(glens))
        acc_k = min_fa3_op.TKParallelTensor([accum], torch.float32, local_rank, world, False)
        acc_v = min_fa3_op.TKParallelTensor([accum], torch.float32, local_rank, world, False)
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

    if args.ring_impl == "nccl_ring" and world > 1:
        if varlen:
            raise SystemExit("--ring-impl nccl_ring is implemented for the single-sequence ring workload")
        # Second comparison baseline: the classic ring schedule with a library transport.  K/V
        # shards travel rank to rank with NCCL send/recv (posted before the step's attention so
        # that they overlap it); each step runs the plain attention kernels on the visiting shard
        # and merges into the running (out, lse) through the kernel's merge epilogue.  Per step the
        # two zigzag halves of q are two documents: against the own shard [front | front+back]
        # with the causal mask, against an earlier rank's shard its front half for both, against
        # a later rank's shard nothing for the front half and the whole shard for the back half.
        # Backward: dQ partials are summed in fp32; the fp32 dK/dV of a shard travel with it and
        # take one more hop home at the end.
        from min_fa3_demo_b200.min_fa3_op import _call_fwd
        half = local // 2
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        cu_q2 = torch.tensor([0, half, local], dtype=torch.int32).to(dev)
        cu_k_own = torch.tensor([0, half, half + local], dtype=torch.int32).to(dev)
        cu_k_early = torch.tensor([0, half, local], dtype=torch.int32).to(dev)
        cu_k_late = torch.tensor([0, 0, local], dtype=torch.int32).to(dev)
        recv_kv = [(torch.empty_like(k), torch.empty_like(v)) for _ in range(2)]
        recv_g = [(torch.empty(local, kvh, 128, dtype=torch.float32, device=dev),
                   torch.empty(local, kvh, 128, dtype=torch.float32, device=dev)) for _ in range(2)]

        def step_operands(src, kb, vb):
            if src == rank:
                return torch.cat([kb[:half], kb]), torch.cat([vb[:half], vb]), cu_k_own, True, local
            if src < rank:
                return (torch.cat([kb[:half], kb[:half]]), torch.cat([vb[:half], vb[:half]]), cu_k_early, False,
                        half)
            return kb, vb, cu_k_late, False, local

        def exchange(send, recv):
            ops = [dist.P2POp(dist.isend, t, nxt) for t in send] + [dist.P2POp(dist.irecv, t, prv) for t in recv]
            return dist.batch_isend_irecv(ops)

        def fwd():
            out = torch.zeros_like(q)
            lse = torch.full((qh, local), float("-inf"), dtype=torch.float32, device=dev)
            kb, vb = k, v
            for s in range(world):
                works = exchange((kb, vb), recv_kv[s & 1]) if s < world - 1 else []
                k2, v2, cu_k2, causal, max_k = step_operands((rank - s) % world, kb, vb)
                _call_fwd(q, k2, v2, out, lse, cu_q=cu_q2, cu_k=cu_k2, batch=2, seqlen_q=half, seqlen_k=max_k,
                          heads_q=qh, heads_k=kvh, is_causal=causal, merge_running=True)
                for w in works:
                    w.wait()
                if s < world - 1:
                    kb, vb = recv_kv[s & 1]
            return out, lse

        def bwd(out, lse):
            dq_acc = torch.zeros(local, qh, 128, dtype=torch.float32, device=dev)
            gk = torch.zeros(local, kvh, 128, dtype=torch.float32, device=dev)   # dK / dV of the visiting shard
            gv = torch.zeros_like(gk)
            kb, vb = k, v
            g_works = []
            for s in range(world):
                src = (rank - s) % world
                kv_works = exchange((kb, vb), recv_kv[s & 1]) if s < world - 1 else []
                k2, v2, cu_k2, causal, max_k = step_operands(src, kb, vb)
                dq_p, dk2, dv2 = min_fa3_op.backward_varlen(dout, q, k2, v2, out, lse, cu_q2, cu_k2, half, max_k,
                                                            causal)
                dq_acc += dq_p
                for w in g_works:          # the visiting shard's gradients so far have arrived
                    w.wait()
                if s > 0:
                    gk, gv = recv_g[(s - 1) & 1]
                for acc, part in ((gk, dk2), (gv, dv2)):
                    if src == rank:
                        acc[:half] += part[:half]
                        acc += part[half:]
                    elif src < rank:
                        acc[:half] += part[:half]
                        acc[:half] += part[half:]
                    else:
                        acc += part
                g_works = exchange((gk, gv), recv_g[s & 1])      # on to the next holder (last hop: home)
                for w in kv_works:
                    w.wait()
                if s < world - 1:
                    kb, vb = recv_kv[s & 1]
            for w in g_works:
                w.wait()
            dk_mine, dv_mine = recv_g[(world - 1) & 1]
            return dq_acc.to(torch.bfloat16), dk_mine.to(torch.bfloat16), dv_mine.to(torch.bfloat16)

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
        grads = bwd(out, lse)
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
    torch.backends.cuda.matmul.allow_tf32 = False
    parity = _ring_workload_parity(rank, world, dev, dist, glens, sizes, starts, q, k, v, dout, out, lse,
                                   grads, cap)
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
                       "exchange": {"fused": "in-kernel peer loads (fused)",
                                    "allgather": "NCCL all_gather of K/V + reduce_scatter of dK/dV (comparison "
                                                 "baseline)",
                                    "nccl_ring": "NCCL send/recv ring of K/V and fp32 dK/dV shards, one attention "
                                                 "call per ring step (comparison baseline)"}[args.ring_impl],
                       "l2": "inputs larger than L2"},
            "tflops_per_gpu": value / world, "fwd_ms": fm, "bwd_ms": bm,
            "fwd_tflops_per_gpu": f_flops / (fm * 1e-3) / 1e12 / world,
            "bwd_tflops_per_gpu": b_flops / (bm * 1e-3) / 1e12 / world,
            "pct_of_bf16_peak": {f"{peak_kind}_burst": 100.0 * value / world / burst,
                                 f"{peak_kind}_sustained": 100.0 * value / world / sustained if sustained else None,
                                 "nominal_dense_2250": 100.0 * value / world / NOMINAL_BF16_TFLOPS},
            "nvlink": {"kv_ingress_bytes_rank0_fwd": ingress,
                       "achieved_gbs_over_fwd_kernel": ingress / (fm * 1e-3) / 1e9 if world > 1 else 0.0},
            "gpu_launches": 4 * args.steps, "clocks": clocks, "parity": parity,
        }
        if emit:
            print(json.dumps(line), flush=True)
        else:
            line["flops"] = f_flops + b_flops
            return line
    if world > 1 and emit:
        dist.destroy_process_group()
    return None


def run_ring_virtual(args) -> None:
    """Forward of the ring workload with the ranks emulated on ONE GPU: every virtual rank owns a
    K/V arena on the same device and gets the others' as its peer pointers; the W launches run one
    after the other (the forward never waits for another rank's launch).  Everything a real
    multi-GPU forward executes runs except the NVLink hop, so the per-rank times separate what the
    work lists and the copy CTAs cost from what the link costs.  T(1) is the same sequence through
    ``forward_varlen`` on the same GPU."""
    import min_fa3_op
    from min_fa3_demo_b200 import _cabi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _cabi.load()
    world, tokens, comm = args.virtual_ranks, args.ring_tokens, args.ring_comm_sm
    qh, kvh = 32, 8
    local = tokens // world
    cap = local
    gen = torch.Generator(device=dev).manual_seed(1)

    def rand(rows, heads):
        return torch.randn(rows, heads, 128, device=dev, generator=gen).to(torch.bfloat16)
    arenas_k = [rand(world * cap, kvh) for _ in range(world)]
    arenas_v = [rand(world * cap, kvh) for _ in range(world)]
    q = rand(local, qh)
    out = torch.empty_like(q)
    lse = torch.empty(qh, local, device=dev)
    cu = torch.tensor([0, local], dtype=torch.int32)
    meta = [torch.tensor([x], dtype=torch.int32) for x in (tokens, world, 0)]
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    nbytes = lib.b2a_ring_fwd_workspace_bytes(1, world, cap, local)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    warm, steps = max(args.warmup, 3), args.steps
    sampler = ClockSampler(0)
    sampler.start()
    sampler.mark_begin()
    per_rank = {}
    for r in range(world):
        a = _cabi.RingFwdArgs()
        a.q, a.out, a.lse = q.data_ptr(), out.data_ptr(), lse.data_ptr()
        a.arena_k, a.arena_v = arenas_k[r].data_ptr(), arenas_v[r].data_ptr()
        for x in range(world):
            a.peer_k[x], a.peer_v[x] = arenas_k[x].data_ptr(), arenas_v[x].data_ptr()
        a.cu_seqlens_q_host = cu.data_ptr()
        a.global_seqlens_host, a.ring_sizes_host, a.ring_starts_host = (m.data_ptr() for m in meta)
        a.batch, a.world_size, a.rank, a.rank_kv_capacity = 1, world, r, cap
        a.total_q, a.heads_q, a.heads_k, a.head_dim, a.is_causal = local, qh, kvh, 128, 1
        a.num_comp_sm, a.num_comm_sm = sm - comm, comm
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
        times = []
        for it in range(warm + steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _cabi.check(lib.b2a_ring_fwd(ctypes.byref(a), stream))
            e1.record()
            torch.cuda.synchronize()
            if it >= warm:
                times.append(e0.elapsed_time(e1))
        _cabi.check(lib.b2a_check_status(ctypes.c_void_p(ws.data_ptr()), None))
        per_rank[r] = statistics.mean(times)
    del arenas_k, arenas_v
    torch.cuda.empty_cache()
    q1, k1, v1 = rand(tokens, qh), rand(tokens, kvh), rand(tokens, kvh)
    cu1 = torch.tensor([0, tokens], dtype=torch.int32)
    cu1d = cu1.to(dev)
    times = []
    for it in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        min_fa3_op.forward_varlen(q1, k1, v1, cu1d, cu1d, tokens, tokens, True, cu_seqlens_q_host=cu1,
                                  cu_seqlens_k_host=cu1)
        e1.record()
        torch.cuda.synchronize()
        if it >= 1:
            times.append(e0.elapsed_time(e1))
    sampler.mark_end()
    clocks = sampler.stop()
    t1 = statistics.mean(times)
    slowest = max(per_rank.values())
    flops = 4.0 * qh * 128 * tokens * (tokens + 1) / 2
    print(json.dumps({
        "metric": "forward attention TFLOPS (causal FLOPs) of the slowest virtual rank x ranks", "unit": "TFLOPS",
        "value": flops / (slowest * 1e-3) / 1e12 / world, "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": slowest, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"ring_virtual_fwd_causal_S{tokens}_QH{qh}_KVH{kvh}_D128", "virtual_ranks": world,
                   "copy_ctas": comm, "l2": "inputs larger than L2"},
        "fwd_ms_per_rank": per_rank, "t1_fwd_ms": t1, "t1_over_ranks_ms": t1 / world,
        "efficiency_fwd_slowest_rank": t1 / world / slowest,
        "gpu_launches": world * (warm + steps) + 3, "clocks": clocks}), flush=True)


def run_ring_dataset(args) -> None:
    """Dataset-shaped context-parallel runs (the reference's benchmark_dataset protocol,
    benchmark_logs/*/benchmark_dataset.log: packed batches of ~131,072 tokens whose document
    lengths follow a dataset's length histogram, placed by the load balancer on hierarchical
    sub-rings; reported as TFLOPS/GPU weighted over the cases, i.e. total FLOPs / total time).
    The histogram comes from a file in the reference's format (``--length-buckets``, e.g. the
    reference checkout's dataset/sequence_length_buckets.json, with ``--dataset`` naming the entry)
    or, without one, from the synthetic log-normal / Pareto mixture stand-in."""
    import torch.distributed as dist

    from min_fa3_demo_b200 import balancer as bal

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.length_buckets:
        tables = bal.load_length_buckets(args.length_buckets)
        if args.dataset not in tables:
            raise SystemExit(f"--dataset {args.dataset!r} is not in {args.length_buckets} (has: {sorted(tables)})")
        counts, source = tables[args.dataset], f"{args.dataset} ({args.length_buckets})"
    else:
        counts, source = bal.synthetic_length_buckets(), "synthetic log-normal/Pareto mixture histogram"
    cases = bal.generate_dataset_length_cases(counts, args.ring_tokens, args.dataset_seed, args.cases)
    records = []
    for lengths in cases:
        rec = run_ring_workload(args, doc_lengths=lengths, emit=False)
        if rank == 0:
            records.append(rec)
    if rank == 0:
        flops = sum(r["flops"] for r in records)
        seconds = sum(r["ms_per_step"] for r in records) * 1e-3
        fwd_s = sum(r["fwd_ms"] for r in records) * 1e-3
        burst, sustained, peak_kind = measured_peaks()
        value = flops / seconds / 1e12
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": seconds * 1e3 / len(records), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"ring_dataset_T{args.ring_tokens}_QH64_KVH8_D128", "length_histogram": source,
                       "cases": len(records), "seed": args.dataset_seed,
                       "documents_per_case": [r["config"]["documents"] for r in records],
                       "weighting": "total FLOPs / total time over the cases (forward + backward)"},
            "tflops_per_gpu": value / world,
            "fwd_tflops_per_gpu": sum(r["flops"] for r in records) * (4.0 / 14.0) / fwd_s / 1e12 / world,
            "pct_of_bf16_peak": {f"{peak_kind}_burst": 100.0 * value / world / burst},
            "per_case_tflops_per_gpu": [r["tflops_per_gpu"] for r in records],
            "per_case_placement": [r["config"]["placement"] for r in records],
            "parity": {"pass": all(r["parity"]["pass"] for r in records), "rule": records[0]["parity"]["rule"],
                       "worst_err_over_bound": {key: max(r["parity"]["worst_err_over_bound"][key] for r in records)
                                                for key in ("o", "lse", "dq", "dk", "dv")}},
            "gpu_launches": 4 * args.steps * len(records), "clocks": records[-1]["clocks"]}), flush=True)
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
    lib = _cabi.load()
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
    lib.b2a_profile_enable(1)
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
    buf = (ctypes.c_float * 256)()
    kernel_ms = {}
    for name, slot in (("fwd_kernel", 0), ("bwd_kernel", 1)):
        n = lib.b2a_profile_read(slot, buf, 256)
        kernel_ms[name] = statistics.mean(buf[i] for i in range(n)) if n else None
    lib.b2a_profile_enable(0)
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
        "kernel_ms": kernel_ms,
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
    parser.add_argument("--workload", choices=("bshd", "varlen", "ring", "ring_varlen", "ring_dataset", "ring_virtual"),
                        default="bshd",
                        help="bshd: config 2 replicas (default); varlen: config 3 (65,536 packed tokens, 1 GPU); "
                             "ring: config 4, one long causal sequence over N ranks; ring_varlen: config 5, "
                             "131,072 packed tokens placed on hierarchical sub-rings over N ranks; ring_dataset: "
                             "several such batches whose document lengths follow a dataset length histogram; "
                             "ring_virtual: the ring forward with --virtual-ranks ranks emulated on one GPU")
    parser.add_argument("--virtual-ranks", type=int, default=4, choices=(2, 4, 8),
                        help="ring_virtual: number of emulated ranks")
    parser.add_argument("--length-buckets", default=None,
                        help="ring_dataset: length-histogram file in the reference's format "
                             "(dataset/sequence_length_buckets.json of the reference checkout)")
    parser.add_argument("--dataset", default="arxiv", help="ring_dataset: entry of the histogram file")
    parser.add_argument("--cases", type=int, default=4, help="ring_dataset: packed batches to run")
    parser.add_argument("--dataset-seed", type=int, default=0)
    parser.add_argument("--non-causal", action="store_true", help="bshd workload without the causal mask")
    parser.add_argument("--deterministic", action="store_true",
                        help="bshd workload with the backward's fixed dQ accumulation order (bit-identical repeats)")
    parser.add_argument("--ring-tokens", type=int, default=131072)
    parser.add_argument("--ring-comm-sm", type=int, default=8)
    parser.add_argument("--ring-impl", choices=("fused", "allgather", "nccl_ring"), default="fused",
                        help="ring workload: fused = K/V pulled inside the attention launch (the product); "
                             "allgather = comparison baseline, NCCL all_gather of K/V + plain varlen attention + "
                             "NCCL reduce_scatter of dK/dV; nccl_ring = second baseline, K/V (and dK/dV) shards passed "
                             "rank to rank with NCCL send/recv, one plain attention call per ring step")
    parser.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg")
    parser.add_argument("--skip-ring", action="store_true",
                        help="N >= 2: skip the context-parallel leg (131,072-token ring) of the default run")
    parser.add_argument("--e2e-head-groups", type=int, default=2,
                        help="chunks per batch element in the host-buffer pipeline (must divide the KV heads)")
    parser.add_argument("--skip-cpu-baseline", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--print-kernel-digest", action="store_true",
                        help="print the hash of the backward kernel sources (recorded beside an ncu traffic capture) and exit")
    args = parser.parse_args()
    if args.print_kernel_digest:
        print(kernel_source_digest())
        return
    if args.non_causal:
        WORKLOAD["causal"] = False
        WORKLOAD["name"] = WORKLOAD["name"].replace("bshd_causal", "bshd_noncausal")
    if args.deterministic:
        WORKLOAD["deterministic"] = True
        WORKLOAD["name"] += "_deterministic_dq"
    if args.batch is not None:
        WORKLOAD["batch"] = args.batch
        WORKLOAD["name"] = WORKLOAD["name"].replace("_B4_", f"_B{args.batch}_")
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "ring_dataset":
        run_ring_dataset(args)
    elif args.workload == "ring_virtual":
        run_ring_virtual(args)
    elif args.workload in ("ring", "ring_varlen"):
        run_ring_workload(args)
    elif args.workload == "varlen":
        run_varlen_workload(args)
    else:
        run_cuda_arm(args)


if __name__ == "__main__":
    main()
