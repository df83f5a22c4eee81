"""Record results of the reference planner (``balancer.assign_hierarchical_rings``) on seeded
synthetic length sets, for the placement-quality tests.

Usage: ``python tests/golden/make_balancer_golden.py --reference <path to the reference checkout>``
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", required=True, type=Path)
    args = parser.parse_args()
    sys.path.insert(0, str(args.reference.resolve()))
    import balancer as ref_balancer  # the reference package

    from min_fa3_demo_b200.balancer import sample_mixture_lengths

    cases = []
    for world in (2, 4, 8):
        for seed in range(4):
            for causal in (True, False):
                lengths = sample_mixture_lengths(seed, 131072)
                ref = ref_balancer.assign_hierarchical_rings(lengths, world, is_causal=causal)
                cases.append({
                    "world_size": world, "seed": seed, "is_causal": causal, "lengths": lengths,
                    "ref_global_lengths": ref.global_lengths, "ref_ring_sizes": ref.ring_sizes,
                    "ref_ring_starts": ref.ring_starts, "ref_peak_compute": ref.peak_compute,
                    "ref_compute_deviation": ref.compute_deviation,
                    "ref_token_deviation": ref.token_deviation, "ref_feasible": ref.feasible,
                    "ref_communication": sum(ref.rank_communication),
                })
    out = Path(__file__).resolve().parent / "balancer_reference.json"
    out.write_text(json.dumps(cases))
    print(f"{out.name}: {out.stat().st_size} bytes, {len(cases)} cases")

    # The reference's dataset-shaped sampler (balancer/sampler.py:126-174) run on a SYNTHETIC
    # histogram (the mixture stand-in of this repository, not the reference's dataset statistics):
    # its per-dataset count table is swapped for the synthetic one for the duration of the call.
    from balancer import sampler as ref_sampler

    from min_fa3_demo_b200.balancer import synthetic_length_buckets
    counts = synthetic_length_buckets(seed=5, samples=50000)
    ref_sampler._DATASET_BUCKET_COUNTS["synthetic"] = counts
    sampled = []
    for target, seed, num in ((131072, 0, 3), (131072, 7, 2), (65536, 1, 2), (16384, 3, 2)):
        sampled.append({"target_tokens": target, "seed": seed,
                        "cases": ref_sampler.generate_dataset_length_cases("synthetic", target, seed, num)})
    out = Path(__file__).resolve().parent / "sampler_reference.json"
    out.write_text(json.dumps({"histogram_seed": 5, "histogram_samples": 50000, "runs": sampled}))
    print(f"{out.name}: {out.stat().st_size} bytes")


if __name__ == "__main__":
    main()
