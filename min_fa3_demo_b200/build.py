"""In-tree build of ``libb200attn.so`` (the C-ABI attention library) with nvcc for sm_100a.

Usage: ``python -m min_fa3_demo_b200.build [--force] [--verbose]``.

The library is compiled from ``csrc/*.cu`` straight into the package directory so that a
source checkout plus this one command is everything a GPU machine needs.  nvcc
cross-compiles without a GPU.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libb200attn.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def extra_flags() -> list[str]:
    """Additional nvcc flags from the environment (e.g. -DB2A_PHASES for phase timing probes)."""
    return os.environ.get("B2A_EXTRA_NVCC_FLAGS", "").split()


def find_nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    if candidate.exists():
        return str(candidate)
    found = shutil.which("nvcc")
    if found is None:
        raise RuntimeError("nvcc not found (set CUDA_HOME)")
    return found


def source_files() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC_DIR.glob("*.cu")) + list(CSRC_DIR.glob("*.cuh"))
                       + [PKG_DIR.parent / "include" / "b200attn.h"]):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS + extra_flags()).encode())
    return h.hexdigest()


def is_up_to_date() -> bool:
    stamp = BUILD_DIR / "stamp"
    return LIB_PATH.exists() and stamp.exists() and stamp.read_text() == _digest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if sources changed; returns its path."""
    if not force and is_up_to_date():
        return LIB_PATH
    nvcc = find_nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags(), *extra, "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}")
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, source_files()))

    link = [nvcc, "-shared", "-o", str(LIB_PATH), *[str(o) for o in objects]]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    (BUILD_DIR / "stamp").write_text(_digest())
    return LIB_PATH


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()
