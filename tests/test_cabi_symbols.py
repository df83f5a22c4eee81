"""The C-ABI library must load and export every function that include/b200attn.h declares
(no compute calls here: there is no GPU on the CPU test machine)."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from min_fa3_demo_b200 import _cabi, build

HEADER = Path(__file__).resolve().parents[1] / "include" / "b200attn.h"


def declared_functions() -> list[str]:
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2a_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _cabi.load()


def test_header_declares_functions():
    names = declared_functions()
    assert "b2a_fwd" in names and "b2a_bwd" in names and "b2a_last_error" in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"libb200attn.so does not export {name}"


def test_ctypes_table_covers_header():
    assert sorted(_cabi.SIGNATURES) == declared_functions()


def test_abi_version_and_error_text(lib):
    assert lib.b2a_abi_version() >= 1
    assert isinstance(_cabi.last_error(), str)


def test_struct_sizes_match_c_layout(tmp_path):
    # The header is plain C: compile it with the C compiler and compare every struct's size and
    # the offset of its last field with the ctypes mirror.
    import shutil
    import subprocess
    gcc = shutil.which("gcc") or shutil.which("cc")
    if gcc is None:
        pytest.skip("no C compiler")
    structs = {"b2a_fwd_args": (_cabi.FwdArgs, "prefetch_blocks"), "b2a_bwd_args": (_cabi.BwdArgs, "workspace_bytes"),
               "b2a_ring_fwd_args": (_cabi.RingFwdArgs, "workspace_bytes"),
               "b2a_ring_bwd_args": (_cabi.RingBwdArgs, "workspace_bytes")}
    lines = "".join(f'printf("{name} %zu %zu\\n", sizeof({name}), offsetof({name}, {last}));\n'
                    for name, (_, last) in structs.items())
    src = tmp_path / "sizes.c"
    src.write_text(f'#include <stdio.h>\n#include <stddef.h>\n#include "{HEADER}"\nint main(void) {{\n{lines}return 0;\n}}\n')
    exe = tmp_path / "sizes"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    for line in filter(None, out):
        name, size, off = line.split()
        mirror, last = structs[name]
        assert ctypes.sizeof(mirror) == int(size), name
        assert getattr(mirror, last).offset == int(off), name


def test_argument_validation_without_gpu(lib):
    # NULL args and bad sizes are rejected before any CUDA call.
    assert lib.b2a_fwd(None, None) == _cabi.B2A_ERR_INVALID_ARGUMENT
    assert "args must not be NULL" in _cabi.last_error()
    a = _cabi.FwdArgs()
    a.q = a.k = a.v = a.out = a.lse = 256
    a.head_dim = 64
    assert lib.b2a_fwd(ctypes.byref(a), None) == _cabi.B2A_ERR_INVALID_ARGUMENT
    assert "head_dim must be 128" in _cabi.last_error()
    a.head_dim, a.batch, a.heads_q, a.heads_k = 128, 1, 6, 4
    assert lib.b2a_fwd(ctypes.byref(a), None) == _cabi.B2A_ERR_INVALID_ARGUMENT
    assert "heads_q % heads_k" in _cabi.last_error()
    b = _cabi.BwdArgs()
    assert lib.b2a_bwd(ctypes.byref(b), None) == _cabi.B2A_ERR_INVALID_ARGUMENT


def test_workspace_sizes(lib):
    assert lib.b2a_fwd_workspace_bytes(4, 4 * 8192, 0) >= 16
    varlen = lib.b2a_fwd_workspace_bytes(34, 65536, 1)
    assert varlen >= 16 + (65536 // 256 + 34) * 8
    # backward: fp32 dQ accumulator dominates (heads_q * padded rows * 128 floats)
    bwd = lib.b2a_bwd_workspace_bytes(4, 4 * 8192, 4 * 8192, 32, 8, 0)
    assert bwd >= 32 * 4 * 8192 * 128 * 4
