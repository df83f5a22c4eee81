"""Host-side mirror of the reference's ``min_fa3_op`` Python API on top of ``libb200attn.so``.

Same function names, argument meaning, output shapes and error behaviour as the reference
(``min_fa3_op.py`` and the pybind layer ``bindings.cpp`` /
``csrc/backward/min_fa3_bwd_bindings.cu``), so a caller switches by changing the import.
PyTorch is used only for device memory and streams; every computation is a call through
the C ABI declared in ``include/b200attn.h``.  Without the CUDA library the import of the
entry points still works (for CPU-side argument checks) but every compute call raises.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional, Tuple, Union

import torch

from . import _cabi

__all__ = [
    "TKParallelTensor",
    "forward",
    "forward_varlen",
    "forward_varlen_ring",
    "forward_varlen_mega_ring",
    "backward",
    "backward_varlen",
    "backward_varlen_mega_ring",
    "create_parallel_tensor",
    "parallel_remote_load",
    "parallel_remote_load_vec",
    "_debug_resolve_launch_grid_shape",
    "check_last_status",
]

_INT32_MAX = 2**31 - 1
_UINT32_MAX = 2**32 - 1


def _check(cond: bool, msg: str) -> None:
    """TORCH_CHECK equivalent: the reference raises RuntimeError from its bindings."""
    if not cond:
        raise RuntimeError(msg)


# --------------------------------------------------------------------------------------
# launch-grid override (reference: include/min_fa3_launch_override.h:16-52)
# --------------------------------------------------------------------------------------
def _validate_manual_block_count(value, arg_name: str = "manual_block_count") -> Optional[int]:
    if value is None:
        return None
    value = int(value)
    if value <= 0:
        raise ValueError(
            f"{arg_name} must be greater than 0. The value is a thread-block count (grid.x), "
            "not a thread count."
        )
    if value > _INT32_MAX:
        raise ValueError(
            f"{arg_name} must fit in a positive 32-bit grid.x thread-block count. Got {value}."
        )
    return value


def _debug_resolve_launch_grid_shape(auto_grid_x, auto_grid_y=1, auto_grid_z=1, *,
                                     manual_block_count=None):
    """CPU-side helper for testing launch-grid override resolution (bindings.cpp:365-378)."""
    manual = _validate_manual_block_count(manual_block_count)
    dims = []
    for value, name in ((auto_grid_x, "auto_grid_x"), (auto_grid_y, "auto_grid_y"),
                        (auto_grid_z, "auto_grid_z")):
        value = int(value)
        _check(0 <= value <= _UINT32_MAX,
               f"{name} must be between 0 and {_UINT32_MAX}. Got {value}")
        dims.append(value)
    if manual is None:
        return tuple(dims)
    if dims[1] != 1 or dims[2] != 1:
        raise ValueError(
            "manual_block_count override only supports the current 1D persistent grid. "
            f"Automatic grid shape was ({dims[0]}, {dims[1]}, {dims[2]})."
        )
    return (manual, dims[1], dims[2])


# --------------------------------------------------------------------------------------
# argument checks (messages follow bindings.cpp:32-62 and min_fa3_bwd_bindings.cu:42-82)
# --------------------------------------------------------------------------------------
def _check_bshd(t: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.bfloat16, f"{name} must have dtype torch.bfloat16")
    _check(t.dim() == 4, f"{name} must have shape [B, S, H, D]")
    _check(t.size(3) == 128, f"{name} must have head_dim D=128")
    _check(t.is_contiguous(), f"{name} must be contiguous BSHD")


def _check_varlen_qkv(t: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.bfloat16, f"{name} must have dtype torch.bfloat16")
    _check(t.dim() == 3, f"{name} must have shape [total_tokens, H, D]")
    _check(t.size(2) == 128, f"{name} must have head_dim D=128")
    _check(t.is_contiguous(), f"{name} must be contiguous [total_tokens, H, D]")


def _check_cu_seqlens(t: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.int32, f"{name} must have dtype torch.int32")
    _check(t.dim() == 1, f"{name} must be 1D")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    _check(t.numel() >= 2, f"{name} must have shape [B + 1] with B >= 1")


def _check_cu_seqlens_host(t: torch.Tensor, device_t: torch.Tensor, name: str) -> None:
    _check(not t.is_cuda, f"{name} must be a CPU tensor")
    _check(t.dtype == torch.int32, f"{name} must have dtype torch.int32")
    _check(t.dim() == 1, f"{name} must be 1D")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    _check(t.numel() == device_t.numel(),
           f"{name} must have the same length as its CUDA cu_seqlens tensor")


def _check_bf16_cuda(t: torch.Tensor, name: str, dim: int) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.bfloat16, f"{name} must have dtype torch.bfloat16")
    _check(t.dim() == dim, f"{name} must have {dim} dimensions")
    _check(t.size(-1) == 128, f"{name} must have head_dim D=128")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _check_same_device(ref: torch.Tensor, t: torch.Tensor, name: str) -> None:
    _check(t.device == ref.device, f"{name} must be on the same CUDA device as q")


def _check_lse(lse: torch.Tensor, q: torch.Tensor) -> None:
    _check(lse.is_cuda, "softmax_lse must be a CUDA tensor")
    _check(lse.dtype == torch.float32, "softmax_lse must have dtype torch.float32")
    _check(lse.is_contiguous(), "softmax_lse must be contiguous")
    _check_same_device(q, lse, "softmax_lse")


def _check_bwd_cu_seqlens(t: torch.Tensor, q: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.int32, f"{name} must have dtype torch.int32")
    _check(t.dim() == 1 and t.numel() >= 2, f"{name} must have shape [B + 1]")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    _check_same_device(q, t, name)


def _grad_output(provided: Optional[torch.Tensor], like: torch.Tensor, name: str) -> torch.Tensor:
    if provided is None:
        return torch.empty_like(like)
    _check_bf16_cuda(provided, name, like.dim())
    _check_same_device(like, provided, name)
    _check(provided.shape == like.shape, f"{name} must have shape {list(like.shape)}")
    return provided


def _check_device_capability(device: torch.device, what: str) -> None:
    major, minor = torch.cuda.get_device_capability(device)
    _check(major == 10,
           f"{what} only supports Blackwell SM100. Current device capability is {major}.{minor}")


# --------------------------------------------------------------------------------------
# C-ABI plumbing
# --------------------------------------------------------------------------------------
def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    # Stream-ordered caching allocator: freed after enqueue is safe, like the reference's
    # per-call scratch tensors.
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _call_fwd(q, k, v, out, lse, *, cu_q, cu_k, batch, seqlen_q, seqlen_k, heads_q, heads_k,
              is_causal, merge_running=False, grid_blocks=0, prefetch=None):
    """``prefetch``: optional ``(src_k_ptr, src_v_ptr, dst_k, dst_v, blocks)`` -- that many extra
    CTAs of the launch copy ``dst_k.numel() * 2`` bytes from each source address first."""
    lib = _cabi.load()
    total_q = q.numel() // (heads_q * 128)
    total_k = k.numel() // (heads_k * 128)
    nbytes = lib.b2a_fwd_workspace_bytes(batch, total_q, 0 if cu_q is None else 1)
    ws = _workspace(nbytes, q.device)
    args = _cabi.FwdArgs()
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    args.out, args.lse = out.data_ptr(), lse.data_ptr()
    args.cu_seqlens_q, args.cu_seqlens_k = _ptr(cu_q), _ptr(cu_k)
    args.batch, args.seqlen_q, args.seqlen_k = batch, seqlen_q, seqlen_k
    args.total_q, args.total_k = total_q, total_k
    args.heads_q, args.heads_k, args.head_dim = heads_q, heads_k, 128
    args.is_causal = int(bool(is_causal))
    args.merge_running = int(bool(merge_running))
    args.grid_blocks = int(grid_blocks or 0)
    args.softmax_scale = 0.0
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    if prefetch is not None:
        src_k, src_v, dst_k, dst_v, blocks = prefetch
        args.prefetch_src_k, args.prefetch_src_v = src_k, src_v
        args.prefetch_dst_k, args.prefetch_dst_v = dst_k.data_ptr(), dst_v.data_ptr()
        args.prefetch_bytes = dst_k.numel() * dst_k.element_size()
        args.prefetch_blocks = int(blocks)
    with torch.cuda.device(q.device):
        _cabi.check(lib.b2a_fwd(ctypes.byref(args), _stream_ptr(q.device)))
    return ws


def _call_bwd(dout, q, k, v, out, lse, dq, dk, dv, *, cu_q, cu_k, batch, seqlen_q, seqlen_k,
              heads_q, heads_k, is_causal, deterministic):
    lib = _cabi.load()
    total_q = q.numel() // (heads_q * 128)
    total_k = k.numel() // (heads_k * 128)
    nbytes = lib.b2a_bwd_workspace_bytes(batch, total_q, total_k, heads_q, heads_k,
                                         0 if cu_q is None else 1)
    ws = _workspace(nbytes, q.device)
    args = _cabi.BwdArgs()
    args.dout, args.q, args.k, args.v = dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    args.out, args.lse = out.data_ptr(), lse.data_ptr()
    args.dq, args.dk, args.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    args.cu_seqlens_q, args.cu_seqlens_k = _ptr(cu_q), _ptr(cu_k)
    args.batch, args.seqlen_q, args.seqlen_k = batch, seqlen_q, seqlen_k
    args.total_q, args.total_k = total_q, total_k
    args.heads_q, args.heads_k, args.head_dim = heads_q, heads_k, 128
    args.is_causal = int(bool(is_causal))
    args.deterministic = int(bool(deterministic))
    args.grid_blocks = 0
    args.softmax_scale = 0.0
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    with torch.cuda.device(q.device):
        _cabi.check(lib.b2a_bwd(ctypes.byref(args), _stream_ptr(q.device)))
    return ws


def check_device_status(workspace: torch.Tensor) -> None:
    """Synchronise and raise if a kernel that used ``workspace`` reported a device-side error."""
    lib = _cabi.load()
    _cabi.check(lib.b2a_check_status(ctypes.c_void_p(workspace.data_ptr()),
                                     _stream_ptr(workspace.device)))


# Scratch of the most recent call of each entry point on this thread.  Keeping the tensor alive
# keeps the 16-byte header with the device status word readable after the call has returned.
_LAST = threading.local()


def _remember_workspace(entry_point: str, workspace: torch.Tensor) -> None:
    table = getattr(_LAST, "workspaces", None)
    if table is None:
        table = _LAST.workspaces = {}
    table[entry_point] = workspace


def check_last_status(entry_point: Optional[str] = None) -> None:
    """Synchronise and raise ``RuntimeError`` if the most recent call of ``entry_point`` (e.g.
    ``"forward"``, ``"backward_varlen_mega_ring"``; default: every entry point) made on this
    thread left a device-side error: a bounded wait that ran out, or a failed device check.
    The kernels never trap or hang on such an error; they record it and return, and this is how
    the host learns of it (the reference's device waits are unbounded and report nothing,
    include/mega_ring_semaphore.cuh:69-80)."""
    table = getattr(_LAST, "workspaces", None) or {}
    names = [entry_point] if entry_point is not None else list(table)
    for name in names:
        ws = table.get(name)
        if ws is not None:
            check_device_status(ws)


# --------------------------------------------------------------------------------------
# public API
# --------------------------------------------------------------------------------------
def forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool, *,
            manual_block_count: Optional[int] = None, return_lse: bool = False
            ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """BSHD attention forward (reference: ``forward``, bindings.cpp:240-278).

    q ``[B, S, QH, 128]``, k/v ``[B, Sk, KVH, 128]`` bf16 contiguous; returns ``out`` like q and,
    with ``return_lse``, the fp32 natural-log LSE ``[B, QH, S]``.
    """
    manual = _validate_manual_block_count(manual_block_count)
    _check_bshd(q, "q")
    _check_bshd(k, "k")
    _check_bshd(v, "v")
    _check(q.device == k.device and q.device == v.device, "q, k, v must be on the same CUDA device")
    _check(q.size(0) == k.size(0) and q.size(0) == v.size(0),
           "q, k, v must have the same batch size B")
    _check(k.size(1) == v.size(1), "k and v must have the same sequence length Sk")
    _check(k.size(2) == v.size(2), "k and v must have the same KV head count")
    _check(q.size(2) % k.size(2) == 0,
           "This demo requires qhead % kvhead == 0 for GQA/MQA. "
           f"Got qhead={q.size(2)}, kvhead={k.size(2)}")
    _check(v.size(3) == 128, "v must have head_dim D=128")
    _check_device_capability(q.device, "min_fa3_demo_b200")

    out = torch.empty_like(q)
    lse = torch.empty((q.size(0), q.size(2), q.size(1)), dtype=torch.float32, device=q.device)
    ws = _call_fwd(q, k, v, out, lse, cu_q=None, cu_k=None, batch=q.size(0), seqlen_q=q.size(1),
                   seqlen_k=k.size(1), heads_q=q.size(2), heads_k=k.size(2), is_causal=is_causal,
                   grid_blocks=manual or 0)
    _remember_workspace("forward", ws)
    if return_lse:
        return out, lse
    return out


def forward_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                   cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
                   max_seqlen_q: int, max_seqlen_k: int, is_causal: bool, *,
                   cu_seqlens_q_host: torch.Tensor, cu_seqlens_k_host: torch.Tensor,
                   manual_block_count: Optional[int] = None, return_lse: bool = False
                   ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Packed varlen attention forward (reference: ``forward_varlen``, bindings.cpp:280-363).

    q ``[total_q, QH, 128]``, k/v ``[total_k, KVH, 128]``; LSE layout ``[QH, total_q]``.
    """
    manual = _validate_manual_block_count(manual_block_count)
    max_seqlen_q, max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    _check_varlen_qkv(q, "q")
    _check_varlen_qkv(k, "k")
    _check_varlen_qkv(v, "v")
    _check_cu_seqlens(cu_seqlens_q, "cu_seqlens_q")
    _check_cu_seqlens(cu_seqlens_k, "cu_seqlens_k")
    _check_cu_seqlens_host(cu_seqlens_q_host, cu_seqlens_q, "cu_seqlens_q_host")
    _check_cu_seqlens_host(cu_seqlens_k_host, cu_seqlens_k, "cu_seqlens_k_host")
    _check(q.device == k.device and q.device == v.device, "q, k, v must be on the same CUDA device")
    _check(q.device == cu_seqlens_q.device and q.device == cu_seqlens_k.device,
           "q, k, v, cu_seqlens_q, and cu_seqlens_k must be on the same CUDA device")
    _check(k.size(1) == v.size(1), "k and v must have the same KV head count")
    _check(q.size(1) % k.size(1) == 0,
           "This demo requires qhead % kvhead == 0 for GQA/MQA. "
           f"Got qhead={q.size(1)}, kvhead={k.size(1)}")
    _check(v.size(2) == 128, "v must have head_dim D=128")
    _check(cu_seqlens_q.size(0) == cu_seqlens_k.size(0),
           "cu_seqlens_q and cu_seqlens_k must have the same length")
    _check(max_seqlen_q > 0 and max_seqlen_k > 0, "max_seqlen_q and max_seqlen_k must be positive")
    _check(max_seqlen_q <= _INT32_MAX and max_seqlen_k <= _INT32_MAX, "max seqlens must fit in int32")
    _check_device_capability(q.device, "min_fa3_demo_b200")

    batch = cu_seqlens_q_host.size(0) - 1
    _check(batch >= 1, "varlen demo requires batch size B >= 1")
    _check(int(cu_seqlens_q_host[0]) == 0, "cu_seqlens_q_host must start with 0")
    _check(int(cu_seqlens_k_host[0]) == 0, "cu_seqlens_k_host must start with 0")
    _check(int(cu_seqlens_q_host[batch]) == q.size(0),
           f"cu_seqlens_q_host[-1] must equal q.size(0). Got {int(cu_seqlens_q_host[batch])} "
           f"vs {q.size(0)}")
    _check(int(cu_seqlens_k_host[batch]) == k.size(0),
           f"cu_seqlens_k_host[-1] must equal k.size(0). Got {int(cu_seqlens_k_host[batch])} "
           f"vs {k.size(0)}")

    out = torch.empty_like(q)
    lse = torch.empty((q.size(1), q.size(0)), dtype=torch.float32, device=q.device)
    ws = _call_fwd(q, k, v, out, lse, cu_q=cu_seqlens_q, cu_k=cu_seqlens_k, batch=batch,
                   seqlen_q=max_seqlen_q, seqlen_k=max_seqlen_k, heads_q=q.size(1), heads_k=k.size(1),
                   is_causal=is_causal, grid_blocks=manual or 0)
    _remember_workspace("forward_varlen", ws)
    if return_lse:
        return out, lse
    return out


def backward(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
             out: torch.Tensor, softmax_lse: torch.Tensor, is_causal: bool, *,
             deterministic: bool = False, dq: Optional[torch.Tensor] = None,
             dk: Optional[torch.Tensor] = None, dv: Optional[torch.Tensor] = None
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """BSHD attention backward (reference: ``backward``, min_fa3_bwd_bindings.cu:156-253).

    Returns ``(dq, dk, dv)``; caller-provided buffers are written in place and returned.
    """
    _check_bf16_cuda(q, "q", 4)
    _check_bf16_cuda(k, "k", 4)
    _check_bf16_cuda(v, "v", 4)
    _check_bf16_cuda(out, "out", 4)
    _check_bf16_cuda(dout, "dout", 4)
    _check_lse(softmax_lse, q)
    _check_same_device(q, k, "k")
    _check_same_device(q, v, "v")
    _check_same_device(q, out, "out")
    _check_same_device(q, dout, "dout")
    _check(q.size(0) > 0 and q.size(1) > 0 and k.size(1) > 0, "B, Sq, and Sk must be positive")
    _check(q.size(0) == k.size(0) and q.size(0) == v.size(0), "q, k, v must have the same B")
    _check(k.size(1) == v.size(1), "k and v must have the same Sk")
    _check(k.size(2) == v.size(2), "k and v must have the same KV head count")
    _check(q.size(2) % k.size(2) == 0, "qhead must be divisible by kvhead")
    _check(out.shape == q.shape, "out must have the same shape as q")
    _check(dout.shape == q.shape, "dout must have the same shape as q")
    _check(tuple(softmax_lse.shape) == (q.size(0), q.size(2), q.size(1)),
           "softmax_lse must have shape [B, QH, Sq]")
    _check_device_capability(q.device, "min_fa3_demo_b200 backward")
    dq = _grad_output(dq, q, "dq")
    dk = _grad_output(dk, k, "dk")
    dv = _grad_output(dv, v, "dv")
    ws = _call_bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_q=None, cu_k=None, batch=q.size(0),
                   seqlen_q=q.size(1), seqlen_k=k.size(1), heads_q=q.size(2), heads_k=k.size(2),
                   is_causal=is_causal, deterministic=deterministic)
    _remember_workspace("backward", ws)
    return dq, dk, dv


def backward_varlen(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    out: torch.Tensor, softmax_lse: torch.Tensor, cu_seqlens_q: torch.Tensor,
                    cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int,
                    is_causal: bool, *, deterministic: bool = False,
                    dq: Optional[torch.Tensor] = None, dk: Optional[torch.Tensor] = None,
                    dv: Optional[torch.Tensor] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Packed varlen backward (reference: ``backward_varlen``, min_fa3_bwd_bindings.cu:255-357)."""
    max_seqlen_q, max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    _check_bf16_cuda(q, "q", 3)
    _check_bf16_cuda(k, "k", 3)
    _check_bf16_cuda(v, "v", 3)
    _check_bf16_cuda(out, "out", 3)
    _check_bf16_cuda(dout, "dout", 3)
    _check_lse(softmax_lse, q)
    _check_bwd_cu_seqlens(cu_seqlens_q, q, "cu_seqlens_q")
    _check_bwd_cu_seqlens(cu_seqlens_k, q, "cu_seqlens_k")
    _check_same_device(q, k, "k")
    _check_same_device(q, v, "v")
    _check_same_device(q, out, "out")
    _check_same_device(q, dout, "dout")
    _check(q.size(0) > 0 and k.size(0) > 0, "total_q and total_k must be positive")
    _check(k.size(0) == v.size(0), "k and v must have the same total_k")
    _check(k.size(1) == v.size(1), "k and v must have the same KV head count")
    _check(q.size(1) % k.size(1) == 0, "qhead must be divisible by kvhead")
    _check(out.shape == q.shape, "out must have the same shape as q")
    _check(dout.shape == q.shape, "dout must have the same shape as q")
    _check(cu_seqlens_q.numel() == cu_seqlens_k.numel(),
           "cu_seqlens_q and cu_seqlens_k must have the same B")
    _check(max_seqlen_q > 0 and max_seqlen_k > 0, "max seqlens must be positive")
    _check(max_seqlen_q <= _INT32_MAX and max_seqlen_k <= _INT32_MAX, "max seqlens must fit int32")
    _check(tuple(softmax_lse.shape) == (q.size(1), q.size(0)),
           "softmax_lse must have shape [QH, total_q]")
    _check_device_capability(q.device, "min_fa3_demo_b200 backward")
    dq = _grad_output(dq, q, "dq")
    dk = _grad_output(dk, k, "dk")
    dv = _grad_output(dv, v, "dv")
    ws = _call_bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_q=cu_seqlens_q, cu_k=cu_seqlens_k,
                   batch=cu_seqlens_q.numel() - 1, seqlen_q=max_seqlen_q, seqlen_k=max_seqlen_k,
                   heads_q=q.size(1), heads_k=k.size(1), is_causal=is_causal,
                   deterministic=deterministic)
    _remember_workspace("backward_varlen", ws)
    return dq, dk, dv


# Context-parallel entry points and peer-memory helpers live in their own modules; they are
# re-exported here so that this module carries the whole reference API surface.
from .parallel import (TKParallelTensor, _resolve_parallel_context, create_parallel_tensor,  # noqa: E402,F401
                       parallel_remote_load, parallel_remote_load_vec)

_RING_EXPORTS = ("backward_varlen_mega_ring", "forward_varlen_mega_ring", "forward_varlen_ring")


def __getattr__(name: str):
    # The ring module imports helpers from this one, so its entry points are resolved on first
    # use (either module may be imported first).
    if name in _RING_EXPORTS:
        from . import ring
        return getattr(ring, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
