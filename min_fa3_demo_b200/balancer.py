"""Document -> (ring size, ring start) placement for hierarchical context parallelism.

Same contract as the reference planner ``balancer.assign_hierarchical_rings``
(``balancer/load_balancer.py:902-1085``): every document gets a ring of 1/2/4/8 consecutive
ranks starting at a multiple of the ring size ("buddy" rings); a causal document may only use
ring size G > 1 when ``length % (256 * G) == 0`` (``load_balancer.py:121-131``: both zigzag
halves of every member stay 128-row aligned), a non-causal one when ``length % (128 * G) == 0``; the result lists the documents sorted by
``(-ring_size, ring_start, original index)`` (``load_balancer.py:1053-1060``), which is the
order the context-parallel kernels require (ring sizes non-increasing).  Each ring member
holds ``length / G`` tokens and, thanks to the zigzag split, ``compute / G`` of the work.

The search itself is this repository's own and much simpler than the reference's Pareto beam
search: longest-processing-time greedy over all legal (size, start) candidates with a
lexicographic (compute peak, token peak, communication) objective, followed by single-document
re-placement moves, then moves of two documents at once, until no move improves the objective.  It is a host-side planner off the
timed path; placements are legal and deterministic, and balance quality is tested against
recorded results of the reference planner on the same inputs.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

RING_SIZES = (1, 2, 4, 8)
MAX_SEQUENCE_TOKENS = 128 * 1024
# Ring-aware rounding of sampled lengths (balancer/sampler.py:18-24, 111-123).
_ALIGNMENT_TIERS = ((2 * 1024, 256), (4 * 1024, 512), (8 * 1024, 1024), (16 * 1024, 2048))
_LARGE_ALIGNMENT = 2048


@dataclass(frozen=True)
class HybridWorkload:
    """Placement plus balance metrics (field names follow balancer/load_balancer.py:32-67)."""

    global_lengths: List[int]
    ring_sizes: List[int]
    ring_starts: List[int]
    original_indices: List[int]
    rank_compute: List[float]
    rank_tokens: List[int]
    rank_communication: List[float]
    average_compute: float
    peak_compute: float
    average_tokens: float
    peak_tokens: int
    compute_balance_tolerance: float
    token_balance_tolerance: float
    feasible: bool
    repair_moves: int

    @property
    def compute_deviation(self) -> float:
        return _max_relative_deviation(self.rank_compute, self.average_compute)

    @property
    def token_deviation(self) -> float:
        return _max_relative_deviation(self.rank_tokens, self.average_tokens)

    @property
    def communication_amplification(self) -> float:
        return sum(self.rank_communication) / sum(self.global_lengths)


def _max_relative_deviation(values: Sequence[float], average: float) -> float:
    if average <= 0:
        return 0.0
    return max(abs(v - average) for v in values) / average


def attention_compute(length: int, is_causal: bool) -> int:
    """Score-matrix entries of one document (balancer/load_balancer.py:109-112)."""
    return length * (length + 1) // 2 if is_causal else length * length


def ring_communication_per_rank(length: int, ring_size: int) -> float:
    """K/V tokens each member pulls from the others (balancer/load_balancer.py:115-118)."""
    return 0.0 if ring_size == 1 else (ring_size - 1) * length / ring_size


def eligible_ring_sizes(length: int, world_size: int, is_causal: bool) -> List[int]:
    out = []
    for g in RING_SIZES:
        if g > world_size:
            continue
        if is_causal:
            if g == 1 or length % (256 * g) == 0:
                out.append(g)
        elif g == 1 or length % (128 * g) == 0:
            # The reference accepts any length divisible by the ring size here
            # (balancer/load_balancer.py:121-131), but its launch contract wants every member's
            # shard to be a multiple of 128 rows; asking for that already in the planner keeps every
            # plan launchable.
            out.append(g)
    return out


def align_sequence_length(length: int) -> int:
    """Round a sampled length up to its tier's alignment (balancer/sampler.py:111-123)."""
    alignment = _LARGE_ALIGNMENT
    for upper, a in _ALIGNMENT_TIERS:
        if length < upper:
            alignment = a
            break
    return min(MAX_SEQUENCE_TOKENS, ((length + alignment - 1) // alignment) * alignment)


def _objective(compute: np.ndarray, tokens: np.ndarray, comm: float, avg_c: float, avg_t: float,
               ctol: float, ttol: float, final: bool) -> Tuple[float, float, float, float]:
    """Lexicographic objective: compute-balance violation, token-balance violation (both zero
    inside the tolerances), then communication volume, then the compute spread (the larger of
    peak - average and average - minimum for complete placements, the peak before).  While documents
    are still being placed only overload counts; for complete placements underload counts too."""
    c_over = max(0.0, float(compute.max()) - (1.0 + ctol) * avg_c)
    t_over = max(0.0, float(tokens.max()) - (1.0 + ttol) * avg_t)
    if final:
        c_over = max(c_over, (1.0 - ctol) * avg_c - float(compute.min()))
        t_over = max(t_over, (1.0 - ttol) * avg_t - float(tokens.min()))
    spread = max(float(compute.max()) - avg_c, avg_c - float(compute.min())) if final else float(compute.max())
    return (c_over / max(avg_c, 1.0), t_over / max(avg_t, 1.0), comm, spread)


def assign_hierarchical_rings(lengths: Sequence[int], world_size: int, is_causal: bool,
                              compute_balance_tolerance: float = 0.05,
                              token_balance_tolerance: float = 0.10,
                              max_repair_iterations: int = 32) -> HybridWorkload:
    if world_size not in (2, 4, 8):
        raise ValueError(f"world_size must be 2, 4, or 8, got {world_size}")
    if not lengths or any(type(length) is not int or length <= 0 for length in lengths):
        raise ValueError("lengths must contain positive integers")
    for name, value in (("compute_balance_tolerance", compute_balance_tolerance),
                        ("token_balance_tolerance", token_balance_tolerance)):
        if not math.isfinite(value) or value < 0:
            raise ValueError(f"{name} must be finite and non-negative, got {value}")
    if type(max_repair_iterations) is not int or max_repair_iterations < 0:
        raise ValueError(f"max_repair_iterations must be a non-negative integer, got {max_repair_iterations}")

    n = len(lengths)
    work = [attention_compute(length, is_causal) for length in lengths]
    candidates: List[List[Tuple[int, int]]] = []
    for length in lengths:
        cands = [(g, s) for g in eligible_ring_sizes(length, world_size, is_causal)
                 for s in range(0, world_size, g)]
        candidates.append(cands)

    avg_c = float(sum(work)) / world_size
    avg_t = sum(lengths) / world_size
    ctol, ttol = compute_balance_tolerance, token_balance_tolerance
    order = sorted(range(n), key=lambda i: (-work[i], i))

    def solve(balance_first: bool):
        compute = np.zeros(world_size)
        tokens = np.zeros(world_size)
        comm = [0.0]
        placement: List[Tuple[int, int]] = [(1, 0)] * n

        def apply(i: int, cand: Tuple[int, int], sign: float) -> None:
            g, s = cand
            compute[s:s + g] += sign * work[i] / g
            tokens[s:s + g] += sign * lengths[i] / g
            comm[0] += sign * g * ring_communication_per_rank(lengths[i], g)

        def greedy_key():
            if balance_first:
                return (float(compute.max()), float(tokens.max()), comm[0])
            return _objective(compute, tokens, comm[0], avg_c, avg_t, ctol, ttol, False)

        for i in order:
            best, best_obj = None, None
            for cand in candidates[i]:
                apply(i, cand, +1.0)
                obj = greedy_key()
                apply(i, cand, -1.0)
                if best_obj is None or obj < best_obj:
                    best, best_obj = cand, obj
            placement[i] = best
            apply(i, best, +1.0)

        moves_box = [0]

        def pair_moves() -> bool:
            cur = _objective(compute, tokens, comm[0], avg_c, avg_t, ctol, ttol, True)
            movable = [i for i in order if len(candidates[i]) > 1]
            for a_pos, i in enumerate(movable):
                for k in movable[a_pos + 1:]:
                    ci, ck = placement[i], placement[k]
                    apply(i, ci, -1.0)
                    apply(k, ck, -1.0)
                    best, best_obj = None, cur
                    for cand_i in candidates[i]:
                        apply(i, cand_i, +1.0)
                        for cand_k in candidates[k]:
                            if cand_i == ci and cand_k == ck:
                                continue
                            apply(k, cand_k, +1.0)
                            obj = _objective(compute, tokens, comm[0], avg_c, avg_t, ctol, ttol, True)
                            apply(k, cand_k, -1.0)
                            if obj < best_obj:
                                best, best_obj = (cand_i, cand_k), obj
                        apply(i, cand_i, -1.0)
                    if best is not None:
                        placement[i], placement[k] = best
                        apply(i, best[0], +1.0)
                        apply(k, best[1], +1.0)
                        moves_box[0] += 2
                        return True          # back to the (cheaper) single-move pass
                    apply(i, ci, +1.0)
                    apply(k, ck, +1.0)
            return False

        # Local repair: move one document at a time while the objective improves (violations,
        # then communication, then -- at equal communication -- the compute spread).
        moves = 0
        for _ in range(max_repair_iterations):
            improved = False
            for i in order:
                current = placement[i]
                cur_obj = _objective(compute, tokens, comm[0], avg_c, avg_t, ctol, ttol, True)
                apply(i, current, -1.0)
                best, best_obj = current, cur_obj
                for cand in candidates[i]:
                    apply(i, cand, +1.0)
                    obj = _objective(compute, tokens, comm[0], avg_c, avg_t, ctol, ttol, True)
                    apply(i, cand, -1.0)
                    if obj < best_obj:
                        best, best_obj = cand, obj
                apply(i, best, +1.0)
                if best != current:
                    placement[i] = best
                    moves += 1
                    improved = True
            if not improved:
                # Single moves are exhausted: try moving two documents at once (typically two
                # equally long documents leaving a wide ring for two narrower ones side by side,
                # which a single move cannot do without breaking the balance).
                improved = pair_moves()
                if not improved:
                    break
        final = _objective(compute, tokens, comm[0], avg_c, avg_t, ctol, ttol, True)
        return final, placement, compute, tokens, moves_box[0] + moves

    # Two starting points: communication-first inside the tolerances, and balance-first (which
    # the repair pass then thins out); keep whichever ends with the better objective.
    final, placement, compute, tokens, moves = min((solve(False), solve(True)), key=lambda r: r[0])

    rows = sorted(range(n), key=lambda i: (-placement[i][0], placement[i][1], i))
    rank_comm = [0.0] * world_size
    for i in range(n):
        g, s = placement[i]
        for r in range(s, s + g):
            rank_comm[r] += ring_communication_per_rank(lengths[i], g)
    rank_tokens = [int(round(t)) for t in tokens]
    feasible = (_max_relative_deviation(list(compute), avg_c) <= compute_balance_tolerance + 1e-12 and
                _max_relative_deviation(rank_tokens, avg_t) <= token_balance_tolerance + 1e-12)
    return HybridWorkload(
        global_lengths=[lengths[i] for i in rows],
        ring_sizes=[placement[i][0] for i in rows],
        ring_starts=[placement[i][1] for i in rows],
        original_indices=rows,
        rank_compute=[float(c) for c in compute],
        rank_tokens=rank_tokens,
        rank_communication=rank_comm,
        average_compute=avg_c,
        peak_compute=float(compute.max()),
        average_tokens=avg_t,
        peak_tokens=max(rank_tokens),
        compute_balance_tolerance=compute_balance_tolerance,
        token_balance_tolerance=token_balance_tolerance,
        feasible=feasible,
        repair_moves=moves,
    )


def sample_mixture_lengths(seed: int, target_tokens: int = 131072, max_len: int = MAX_SEQUENCE_TOKENS
                           ) -> List[int]:
    """Synthetic document lengths of the varlen ring benchmark configuration: with probability
    0.7 log-normal (median 2000, sigma 1.0), else Pareto (alpha 1.1, minimum 8192), capped at
    ``max_len``, rounded up by :func:`align_sequence_length`, accumulated until the total reaches
    ``target_tokens``.  Stands in for the reference's dataset-shaped samplers
    (balancer/sampler.py:126-174), which need length histograms of corpora not available here."""
    rng = np.random.default_rng(seed)
    lengths: List[int] = []
    total = 0
    while total < target_tokens:
        if rng.random() < 0.7:
            raw = rng.lognormal(mean=math.log(2000.0), sigma=1.0)
        else:
            raw = 8192.0 * (1.0 + rng.pareto(1.1))
        length = align_sequence_length(int(min(max(round(raw), 1), max_len)))
        lengths.append(length)
        total += length
    return lengths


# --------------------------------------------------------------------------------------
# Dataset-shaped length sampling (reference: balancer/sampler.py:28-174)
# --------------------------------------------------------------------------------------
LENGTH_BUCKET_SIZE = 256


def load_length_buckets(path) -> dict:
    """Reads a length-histogram file in the reference's format (``dataset/sequence_length_buckets.json``:
    ``bucket_size`` 256, ``max_sequence_tokens`` 131072, ``interval`` "(lower, upper]",
    ``overflow_policy`` "clamp_to_last_bucket", and per dataset ``sample_count`` plus 512
    ``bucket_counts``) and returns ``{dataset: tuple(counts)}``.  The checks and their messages follow
    balancer/sampler.py:28-91.  The file itself belongs to the reference checkout and is not shipped here."""
    import json
    from pathlib import Path

    path = Path(path)
    try:
        payload = json.loads(path.read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as exc:
        raise RuntimeError(f"failed to load dataset bucket statistics from {path}") from exc
    if not isinstance(payload, dict):
        raise RuntimeError(f"bucket statistics in {path} must be a JSON object")
    if payload.get("bucket_size") != LENGTH_BUCKET_SIZE:
        raise RuntimeError(f"bucket_size in {path} must be {LENGTH_BUCKET_SIZE}, got {payload.get('bucket_size')!r}")
    if payload.get("max_sequence_tokens") != MAX_SEQUENCE_TOKENS:
        raise RuntimeError(f"max_sequence_tokens in {path} must be {MAX_SEQUENCE_TOKENS}, "
                           f"got {payload.get('max_sequence_tokens')!r}")
    if payload.get("interval") != "(lower, upper]":
        raise RuntimeError(f"interval in {path} must be '(lower, upper]'")
    if payload.get("overflow_policy") != "clamp_to_last_bucket":
        raise RuntimeError(f"overflow_policy in {path} must be 'clamp_to_last_bucket'")
    datasets = payload.get("datasets")
    if not isinstance(datasets, dict) or not datasets:
        raise RuntimeError(f"datasets in {path} must be a non-empty JSON object")
    expected = MAX_SEQUENCE_TOKENS // LENGTH_BUCKET_SIZE
    result = {}
    for name, stats in datasets.items():
        counts = stats.get("bucket_counts") if isinstance(stats, dict) else None
        if not isinstance(counts, list) or len(counts) != expected:
            raise RuntimeError(f"bucket_counts for {name!r} in {path} must contain {expected} entries")
        if any(type(c) is not int or c < 0 for c in counts):
            raise RuntimeError(f"bucket_counts for {name!r} in {path} must be non-negative integers")
        if sum(counts) != stats.get("sample_count"):
            raise RuntimeError(f"bucket_counts for {name!r} in {path} sum to {sum(counts)}, "
                               f"expected sample_count={stats.get('sample_count')!r}")
        result[name] = tuple(counts)
    return result


def synthetic_length_buckets(seed: int = 0, samples: int = 200000) -> Tuple[int, ...]:
    """A stand-in histogram for machines without the reference's dataset statistics: bucket counts of
    the 70/30 log-normal / Pareto mixture of benchmark configuration 5 (the same distribution
    ``sample_mixture_lengths`` draws from), in the file format's 512 buckets of 256 tokens."""
    rng = np.random.default_rng(seed)
    heavy = rng.random(samples) >= 0.7
    lengths = np.where(heavy, 8192.0 * (1.0 + rng.pareto(1.1, samples)),
                       rng.lognormal(math.log(2000.0), 1.0, samples))
    lengths = np.clip(np.rint(lengths), 1, MAX_SEQUENCE_TOKENS).astype(np.int64)
    buckets = np.minimum((lengths + LENGTH_BUCKET_SIZE - 1) // LENGTH_BUCKET_SIZE,
                         MAX_SEQUENCE_TOKENS // LENGTH_BUCKET_SIZE) - 1
    return tuple(int(c) for c in np.bincount(buckets, minlength=MAX_SEQUENCE_TOKENS // LENGTH_BUCKET_SIZE))


def generate_dataset_length_cases(bucket_counts: Sequence[int], target_tokens: int, seed: int, num_cases: int
                                  ) -> List[List[int]]:
    """``num_cases`` packed batches drawn from one ``random.Random(seed)`` stream, exactly as the
    reference sampler does (balancer/sampler.py:126-174): a bucket is drawn with probability
    proportional to its count, its upper bound is the sampled length, the last document of a batch is
    cut to the remaining budget, and every length is rounded up by the ring-aware tiers
    (``align_sequence_length``).  With the reference's histogram and the same seed the batches equal
    the reference's."""
    import random

    if num_cases <= 0:
        raise ValueError(f"num_cases must be positive, got {num_cases}")
    if target_tokens <= 0:
        raise ValueError(f"target_tokens must be positive, got {target_tokens}")
    counts = list(bucket_counts)
    total = sum(counts)
    if total <= 0:
        raise RuntimeError("bucket counts must contain at least one sample")
    rng = random.Random(seed)
    cases = []
    for _ in range(num_cases):
        lengths, remaining = [], target_tokens
        while remaining > 0:
            draw, cumulative, idx = rng.randrange(total), 0, 0
            for idx, count in enumerate(counts):
                cumulative += count
                if draw < cumulative:
                    break
            sampled = (idx + 1) * LENGTH_BUCKET_SIZE
            length = align_sequence_length(min(sampled, remaining, MAX_SEQUENCE_TOKENS))
            lengths.append(length)
            remaining = max(remaining - length, 0)
        cases.append(lengths)
    return cases


def local_layout(workload: HybridWorkload, rank: int) -> Tuple[List[int], List[int]]:
    """This rank's local document lengths (0 for rings it is not part of) and their cumulative
    offsets, in the placement's document order — the ``cu_seqlens`` a rank passes to the
    context-parallel entry points."""
    lens = []
    for length, g, s in zip(workload.global_lengths, workload.ring_sizes, workload.ring_starts):
        lens.append(length // g if s <= rank < s + g else 0)
    cu = [0]
    for length in lens:
        cu.append(cu[-1] + length)
    return lens, cu
