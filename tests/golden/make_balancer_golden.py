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


if __name__ == "__main__":
    main()
