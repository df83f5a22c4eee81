"""ctypes binding of ``libb200attn.so`` (declared in ``include/b200attn.h``).

The library is the product; there is no fallback.  ``load()`` raises if the shared object
is missing or does not export the expected symbols, so a machine without the CUDA build
fails loudly instead of silently computing somewhere else.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200attn.so"

B2A_OK = 0
B2A_ERR_INVALID_ARGUMENT = -1
B2A_ERR_CUDA = -2
B2A_ERR_WORKSPACE_TOO_SMALL = -3
B2A_ERR_UNSUPPORTED_DEVICE = -4
B2A_ERR_DEVICE_STATUS = -5


class FwdArgs(Structure):
    """Mirror of ``b2a_fwd_args``."""

    _fields_ = [
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("cu_seqlens_q", c_void_p),
        ("cu_seqlens_k", c_void_p),
        ("batch", c_int32),
        ("seqlen_q", c_int32),
        ("seqlen_k", c_int32),
        ("total_q", c_int32),
        ("total_k", c_int32),
        ("heads_q", c_int32),
        ("heads_k", c_int32),
        ("head_dim", c_int32),
        ("is_causal", c_int32),
        ("merge_running", c_int32),
        ("grid_blocks", c_int32),
        ("softmax_scale", c_float),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("prefetch_src_k", c_void_p),
        ("prefetch_src_v", c_void_p),
        ("prefetch_dst_k", c_void_p),
        ("prefetch_dst_v", c_void_p),
        ("prefetch_bytes", c_size_t),
        ("prefetch_blocks", c_int32),
    ]


class BwdArgs(Structure):
    """Mirror of ``b2a_bwd_args``."""

    _fields_ = [
        ("dout", c_void_p),
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("dq", c_void_p),
        ("dk", c_void_p),
        ("dv", c_void_p),
        ("cu_seqlens_q", c_void_p),
        ("cu_seqlens_k", c_void_p),
        ("batch", c_int32),
        ("seqlen_q", c_int32),
        ("seqlen_k", c_int32),
        ("total_q", c_int32),
        ("total_k", c_int32),
        ("heads_q", c_int32),
        ("heads_k", c_int32),
        ("head_dim", c_int32),
        ("is_causal", c_int32),
        ("deterministic", c_int32),
        ("grid_blocks", c_int32),
        ("softmax_scale", c_float),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


class RingFwdArgs(Structure):
    """Mirror of ``b2a_ring_fwd_args``."""

    _fields_ = [
        ("q", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("arena_k", c_void_p),
        ("arena_v", c_void_p),
        ("peer_k", c_void_p * 8),
        ("peer_v", c_void_p * 8),
        ("cu_seqlens_q_host", c_void_p),
        ("global_seqlens_host", c_void_p),
        ("ring_sizes_host", c_void_p),
        ("ring_starts_host", c_void_p),
        ("stats", c_void_p),
        ("batch", c_int32),
        ("world_size", c_int32),
        ("rank", c_int32),
        ("rank_kv_capacity", c_int32),
        ("total_q", c_int32),
        ("heads_q", c_int32),
        ("heads_k", c_int32),
        ("head_dim", c_int32),
        ("is_causal", c_int32),
        ("num_comp_sm", c_int32),
        ("num_comm_sm", c_int32),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


class RingBwdArgs(Structure):
    """Mirror of ``b2a_ring_bwd_args``."""

    _fields_ = [
        ("dout", c_void_p),
        ("q", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("dq", c_void_p),
        ("dk", c_void_p),
        ("dv", c_void_p),
        ("arena_k", c_void_p),
        ("arena_v", c_void_p),
        ("peer_k", c_void_p * 8),
        ("peer_v", c_void_p * 8),
        ("dk_accum_peer", c_void_p * 8),
        ("dv_accum_peer", c_void_p * 8),
        ("completion_peer", c_void_p * 8),
        ("cu_seqlens_q_host", c_void_p),
        ("global_seqlens_host", c_void_p),
        ("ring_sizes_host", c_void_p),
        ("ring_starts_host", c_void_p),
        ("batch", c_int32),
        ("world_size", c_int32),
        ("rank", c_int32),
        ("rank_kv_capacity", c_int32),
        ("total_q", c_int32),
        ("local_total_k", c_int32),
        ("heads_q", c_int32),
        ("heads_k", c_int32),
        ("head_dim", c_int32),
        ("is_causal", c_int32),
        ("num_comp_sm", c_int32),
        ("num_comm_sm", c_int32),
        ("kv_resident", c_int32),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


# symbol -> (restype, argtypes); must list every function include/b200attn.h declares.
SIGNATURES = {
    "b2a_abi_version": (c_int32, []),
    "b2a_last_error": (c_char_p, []),
    "b2a_fwd_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "b2a_fwd": (c_int32, [POINTER(FwdArgs), c_void_p]),
    "b2a_fwd_noalloc": (c_int32, [POINTER(FwdArgs), c_void_p]),
    "b2a_fwd_noalloc_scratch_limit": (c_size_t, []),
    "b2a_bwd_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32, c_int32, c_int32]),
    "b2a_bwd": (c_int32, [POINTER(BwdArgs), c_void_p]),
    "b2a_ipc_export": (c_int32, [c_void_p, c_void_p, POINTER(ctypes.c_uint64)]),
    "b2a_ipc_import": (c_int32, [c_void_p, ctypes.c_uint64, POINTER(c_void_p)]),
    "b2a_ipc_close": (c_int32, [c_void_p, ctypes.c_uint64]),
    "b2a_peer_copy": (c_int32, [c_void_p, c_void_p, c_size_t, c_int32, c_void_p, c_void_p]),
    "b2a_copy_2d": (c_int32, [c_void_p, c_size_t, c_void_p, c_size_t, c_size_t, c_size_t, c_int32, c_void_p]),
    "b2a_ring_fwd_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32]),
    "b2a_ring_fwd": (c_int32, [POINTER(RingFwdArgs), c_void_p]),
    "b2a_ring_bwd_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "b2a_ring_bwd": (c_int32, [POINTER(RingBwdArgs), c_void_p]),
    "b2a_check_status": (c_int32, [c_void_p, c_void_p]),
    "b2a_set_wait_timeout_ns": (c_int32, [ctypes.c_uint64]),
    "b2a_profile_enable": (c_int32, [c_int32]),
    "b2a_profile_read": (c_int32, [c_int32, POINTER(c_float), c_int32]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m min_fa3_demo_b200.build` "
            "(there is no non-CUDA fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise RuntimeError(f"{LIB_PATH} does not export {name}")
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().b2a_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Turn a non-zero return code into the Python exception the reference would raise."""
    if rc == B2A_OK:
        return
    msg = last_error()
    if rc == B2A_ERR_INVALID_ARGUMENT:
        raise RuntimeError(msg)
    raise RuntimeError(f"b200attn error {rc}: {msg}")
