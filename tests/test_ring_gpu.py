"""Context-parallel GPU tests.  The checks live in tests/mp_worker.py (one process per GPU);
this file launches it: world size 1 on any GPU machine, and world size 2/4/8 through
torch.distributed.run when that many GPUs are visible."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = Path(__file__).resolve().parent / "mp_worker.py"


def run_worker(world: int, cases: list[str]) -> None:
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    if world == 1:
        for key in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE"):
            env.pop(key, None)
        cmd = [sys.executable, str(WORKER), *cases]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", "29517", str(WORKER), *cases]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(res.stdout[-4000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.parametrize("case", ["mega_ring_fwd", "remote_load", "ring_steps", "mega_ring_bwd", "ring_autograd"])
def test_single_rank(case):
    run_worker(1, [case])


def _multi_world() -> int:
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for w in (8, 4, 2):
        if n >= w:
            return w
    return 0


@pytest.mark.skipif(_multi_world() == 0, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("case", ["remote_load", "ring_steps", "mega_ring_fwd", "mega_ring_bwd", "ring_autograd", "empty_rank"])
def test_multi_rank(case):
    run_worker(_multi_world(), [case])
