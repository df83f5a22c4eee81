"""Placement planner: legality, ordering, determinism and balance quality against recorded
results of the reference planner (tests/golden/balancer_reference.json, written by
tests/golden/make_balancer_golden.py)."""
from __future__ import annotations

import json
from pathlib import Path

import pytest

from min_fa3_demo_b200 import balancer as bal

CASES = json.loads((Path(__file__).resolve().parent / "golden" / "balancer_reference.json").read_text())


def test_eligible_ring_sizes_follow_the_reference_rule():
    # causal: G > 1 needs length % (256 * G) == 0 (balancer/load_balancer.py:121-131)
    assert bal.eligible_ring_sizes(2048, 8, True) == [1, 2, 4, 8]
    assert bal.eligible_ring_sizes(1024, 8, True) == [1, 2, 4]
    assert bal.eligible_ring_sizes(768, 8, True) == [1]
    assert bal.eligible_ring_sizes(768, 4, False) == [1, 2]          # shards must stay multiples of 128 rows
    assert bal.eligible_ring_sizes(1024, 4, False) == [1, 2, 4]
    assert bal.eligible_ring_sizes(4096, 2, True) == [1, 2]


def test_alignment_tiers():
    assert bal.align_sequence_length(1) == 256
    assert bal.align_sequence_length(2047) == 2048
    assert bal.align_sequence_length(2049) == 2560
    assert bal.align_sequence_length(5000) == 5120
    assert bal.align_sequence_length(9000) == 10240
    assert bal.align_sequence_length(20000) == 20480
    assert bal.align_sequence_length(10**7) == bal.MAX_SEQUENCE_TOKENS


def test_argument_validation():
    with pytest.raises(ValueError, match="world_size must be 2, 4, or 8"):
        bal.assign_hierarchical_rings([1024], 3, True)
    with pytest.raises(ValueError, match="positive integers"):
        bal.assign_hierarchical_rings([1024, 0], 4, True)
    with pytest.raises(ValueError, match="compute_balance_tolerance"):
        bal.assign_hierarchical_rings([1024], 4, True, compute_balance_tolerance=-1.0)


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"w{c['world_size']}-s{c['seed']}-{'c' if c['is_causal'] else 'n'}")
def test_placement_is_legal_ordered_deterministic_and_balanced(case):
    lengths, world, causal = case["lengths"], case["world_size"], case["is_causal"]
    plan = bal.assign_hierarchical_rings(lengths, world, causal)
    again = bal.assign_hierarchical_rings(lengths, world, causal)
    assert (plan.global_lengths, plan.ring_sizes, plan.ring_starts) == \
        (again.global_lengths, again.ring_sizes, again.ring_starts)
    # every document placed exactly once
    assert sorted(plan.original_indices) == list(range(len(lengths)))
    assert [lengths[i] for i in plan.original_indices] == plan.global_lengths
    # legal buddy rings, sorted by (-ring size, ring start, original index)
    keys = []
    for length, g, s, idx in zip(plan.global_lengths, plan.ring_sizes, plan.ring_starts, plan.original_indices):
        assert g in bal.eligible_ring_sizes(length, world, causal)
        assert s % g == 0 and 0 <= s and s + g <= world
        keys.append((-g, s, idx))
    assert keys == sorted(keys)
    # per-rank accounting is consistent
    assert sum(plan.rank_tokens) == sum(lengths)
    assert sum(plan.rank_compute) == pytest.approx(sum(bal.attention_compute(l, causal) for l in lengths))
    # quality: feasible whenever the reference planner is, with at most 1.3x its communication volume
    if case["ref_feasible"]:
        assert plan.feasible
        assert plan.compute_deviation <= plan.compute_balance_tolerance + 1e-9
        assert plan.token_deviation <= plan.token_balance_tolerance + 1e-9
    assert sum(plan.rank_communication) <= 1.3 * case["ref_communication"] + 1.0


def test_mixture_sampler_and_local_layout():
    lengths = bal.sample_mixture_lengths(0)
    assert lengths == bal.sample_mixture_lengths(0)
    assert sum(lengths) >= 131072 and all(l % 256 == 0 and l <= bal.MAX_SEQUENCE_TOKENS for l in lengths)
    plan = bal.assign_hierarchical_rings(lengths, 8, True)
    total = 0
    for rank in range(8):
        lens, cu = bal.local_layout(plan, rank)
        assert cu[-1] == sum(lens) == plan.rank_tokens[rank]
        assert all(l % 128 == 0 for l in lens)
        total += cu[-1]
    assert total == sum(lengths)


# --------------------------------------------------------------------------------------
# Property test: whatever the lengths, a plan is legal (the launch-time metadata rules of the
# context-parallel entry points) and accounts for every token and every unit of work.
# --------------------------------------------------------------------------------------
from hypothesis import given, settings, strategies as st  # noqa: E402


@settings(max_examples=40, deadline=None)
@given(lengths=st.lists(st.integers(min_value=1, max_value=96).map(lambda n: n * 256), min_size=1, max_size=10),
       world=st.sampled_from([2, 4, 8]), causal=st.booleans())
def test_random_inputs_give_legal_plans(lengths, world, causal):
    plan = bal.assign_hierarchical_rings(lengths, world, causal)
    assert sorted(plan.global_lengths) == sorted(lengths)
    assert sorted(plan.original_indices) == list(range(len(lengths)))
    keys = [(-g, s, i) for g, s, i in zip(plan.ring_sizes, plan.ring_starts, plan.original_indices)]
    assert keys == sorted(keys)                                   # non-increasing ring size, then start
    for length, g, s in zip(plan.global_lengths, plan.ring_sizes, plan.ring_starts):
        assert g in bal.eligible_ring_sizes(length, world, causal)
        assert s % g == 0 and 0 <= s and s + g <= world
        assert (length // g) % 128 == 0 and (not causal or g == 1 or (length // g // 2) % 128 == 0)
    assert sum(plan.rank_tokens) == sum(lengths)
    assert sum(plan.rank_compute) == pytest.approx(sum(bal.attention_compute(n, causal) for n in lengths))
    for rank in range(world):
        lens, cu = bal.local_layout(plan, rank)
        assert cu[-1] == plan.rank_tokens[rank]


# --------------------------------------------------------------------------------------
# Dataset-shaped sampling (reference: balancer/sampler.py:28-174)
# --------------------------------------------------------------------------------------
def test_dataset_sampler_matches_recorded_reference_sampler():
    """Same histogram + same seed -> the batches of the reference's ``generate_dataset_length_cases``
    (recorded by tests/golden/make_balancer_golden.py on a synthetic histogram)."""
    import json
    from pathlib import Path

    golden = json.loads((Path(__file__).resolve().parent / "golden" / "sampler_reference.json").read_text())
    counts = bal.synthetic_length_buckets(seed=golden["histogram_seed"], samples=golden["histogram_samples"])
    assert len(counts) == 512 and sum(counts) == golden["histogram_samples"]
    for run in golden["runs"]:
        got = bal.generate_dataset_length_cases(counts, run["target_tokens"], run["seed"], len(run["cases"]))
        assert got == run["cases"]
        for lengths in got:
            assert sum(lengths) >= run["target_tokens"]
            assert all(n % 256 == 0 and 0 < n <= bal.MAX_SEQUENCE_TOKENS for n in lengths)


def test_length_bucket_file_format_is_the_reference_format(tmp_path):
    import json

    counts = [0] * 512
    counts[3], counts[40], counts[511] = 5, 2, 1
    good = {"bucket_size": 256, "max_sequence_tokens": 131072, "interval": "(lower, upper]",
            "overflow_policy": "clamp_to_last_bucket", "tokenizer": "none",
            "datasets": {"toy": {"sample_count": 8, "bucket_counts": counts}}}
    path = tmp_path / "buckets.json"
    path.write_text(json.dumps(good))
    loaded = bal.load_length_buckets(path)
    assert loaded == {"toy": tuple(counts)}
    cases = bal.generate_dataset_length_cases(loaded["toy"], 32768, 0, 2)
    assert len(cases) == 2 and all(sum(c) >= 32768 for c in cases)
    for key, value, fragment in (("bucket_size", 128, "bucket_size"), ("interval", "[lower, upper)", "interval"),
                                 ("overflow_policy", "drop", "overflow_policy")):
        bad = dict(good)
        bad[key] = value
        path.write_text(json.dumps(bad))
        with pytest.raises(RuntimeError, match=fragment):
            bal.load_length_buckets(path)
    bad = json.loads(json.dumps(good))
    bad["datasets"]["toy"]["sample_count"] = 9
    path.write_text(json.dumps(bad))
    with pytest.raises(RuntimeError, match="sum to 8"):
        bal.load_length_buckets(path)
    with pytest.raises(RuntimeError, match="failed to load"):
        bal.load_length_buckets(tmp_path / "missing.json")
