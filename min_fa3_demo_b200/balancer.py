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
    inside the tolerances), then communication volume, then the compute peak.  While documents
    are still being placed only overload counts; for complete placements underload counts too."""
    c_over = max(0.0, float(compute.max()) - (1.0 + ctol) * avg_c)
    t_over = max(0.0, float(tokens.max()) - (1.0 + ttol) * avg_t)
    if final:
        c_over = max(c_over, (1.0 - ctol) * avg_c - float(compute.min()))
        t_over = max(t_over, (1.0 - ttol) * avg_t - float(tokens.min()))
    return (c_over / max(avg_c, 1.0), t_over / max(avg_t, 1.0), comm, float(compute.max()))


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
                            if obj[:3] < best_obj[:3]:
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

        # Local repair: move one document at a time while (violations, communication) improve.
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
                    if obj[:3] < best_obj[:3]:
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
