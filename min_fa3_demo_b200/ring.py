"""Context-parallel entry points of the ``min_fa3_op`` API (single node, NVLink).

``forward_varlen_ring``       one ring step: attention over the current K/V merged into the
                              running (out, lse) while the next rank's K/V is prefetched
                              (reference: csrc/min_fa3_varlen_ring_bindings.cu:231-400).
``forward_varlen_mega_ring``  the whole zigzag / hierarchical CP forward in one launch
                              (reference: csrc/mega_ring_min_fa3_varlen_ring_bindings.cu:304-600).

Validation follows the reference bindings, including the texts its negative tests match on.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple, Union

import torch

from . import _cabi
from .min_fa3_op import (_INT32_MAX, _call_fwd, _check, _check_cu_seqlens, _check_cu_seqlens_host,
                         _check_device_capability, _check_varlen_qkv, _stream_ptr, _workspace)
from .parallel import TKParallelTensor

__all__ = ["forward_varlen_ring", "forward_varlen_mega_ring", "backward_varlen_mega_ring"]


def _check_parallel_base(t: TKParallelTensor, name: str) -> None:
    _check(isinstance(t, TKParallelTensor), f"{name} must be a TKParallelTensor")
    _check(t.data_.is_cuda, f"{name} must be CUDA-backed")
    _check(t.data_.dtype == torch.bfloat16, f"{name} must have dtype torch.bfloat16")
    _check(t.data_.dim() == 3 and t.data_.size(2) == 128, f"{name} must have shape [total_tokens, H, 128]")
    _check(t.data_.is_contiguous(), f"{name} must be contiguous")


def _check_out(t: torch.Tensor, q: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.bfloat16, f"{name} must have dtype torch.bfloat16")
    _check(t.shape == q.shape, f"{name} must have the same shape as q")
    _check(t.device == q.device, f"{name} must be on the same CUDA device as q")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _check_lse(t: torch.Tensor, q: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.float32, f"{name} must have dtype torch.float32")
    _check(t.dim() == 2, f"{name} must have shape [qhead, total_q]")
    _check(t.size(0) == q.size(1) and t.size(1) == q.size(0), f"{name} must have shape [qhead, total_q]")
    _check(t.device == q.device, f"{name} must be on the same CUDA device as q")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _check_host_vec(t: torch.Tensor, batch: int, name: str) -> None:
    _check(isinstance(t, torch.Tensor) and not t.is_cuda, f"{name} must be a CPU tensor")
    _check(t.dtype == torch.int32, f"{name} must have dtype torch.int32")
    _check(t.dim() == 1 and t.is_contiguous(), f"{name} must be a contiguous 1D tensor")
    _check(t.numel() == batch, f"{name} must have shape [B]. Got {t.numel()} vs B={batch}")


def _common_checks(q, k, v, cu_q, cu_k, cu_q_host, cu_k_host, max_q, max_k, num_comp_sm, num_comm_sm):
    _check_varlen_qkv(q, "q")
    _check_varlen_qkv(k, "k")
    _check_varlen_qkv(v, "v")
    _check_cu_seqlens(cu_q, "cu_seqlens_q")
    _check_cu_seqlens(cu_k, "cu_seqlens_k")
    _check_cu_seqlens_host(cu_q_host, cu_q, "cu_seqlens_q_host")
    _check_cu_seqlens_host(cu_k_host, cu_k, "cu_seqlens_k_host")
    _check(q.device == k.device and q.device == v.device, "q, k, v must be on the same CUDA device")
    _check(q.device == cu_q.device and q.device == cu_k.device,
           "q, k, v, cu_seqlens_q, and cu_seqlens_k must be on the same CUDA device")
    _check(k.size(1) == v.size(1), "k and v must have the same KV head count")
    _check(q.size(1) % k.size(1) == 0,
           f"This demo requires qhead % kvhead == 0 for GQA/MQA. Got qhead={q.size(1)}, kvhead={k.size(1)}")
    _check(v.size(2) == 128, "v must have head_dim D=128")
    _check(cu_q.size(0) == cu_k.size(0), "cu_seqlens_q and cu_seqlens_k must have the same length")
    _check(max_q > 0 and max_k > 0, "max_seqlen_q and max_seqlen_k must be positive")
    _check(max_q <= _INT32_MAX and max_k <= _INT32_MAX, "max seqlens must fit in int32")
    _check(num_comp_sm > 0, f"num_comp_sm must be positive. Got {num_comp_sm}")
    _check(num_comm_sm >= 0, f"num_comm_sm must be non-negative. Got {num_comm_sm}")


# --------------------------------------------------------------------------------------
# one ring step
# --------------------------------------------------------------------------------------
def forward_varlen_ring(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, is_causal, *,
                        cu_seqlens_q_host, cu_seqlens_k_host, remote_k: TKParallelTensor,
                        remote_v: TKParallelTensor, src_rank: int, num_comp_sm: int, num_comm_sm: int,
                        ring_step: int, prefetch_k, prefetch_v, out: Optional[torch.Tensor] = None,
                        lse: Optional[torch.Tensor] = None, return_lse: bool = False
                        ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Attention of ``q`` over the current ``k, v`` merged in place into the running
    ``out`` / ``lse`` (defaults: zeros / -inf), while ``num_comm_sm`` copy CTAs prefetch
    ``src_rank``'s K/V from the parallel tensors into ``prefetch_k`` / ``prefetch_v``.
    The copy runs on a side stream next to the attention kernel (limited to ``num_comp_sm``
    CTAs) and is joined before the call returns control of the stream."""
    max_seqlen_q, max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    num_comp_sm, num_comm_sm, src_rank, ring_step = (int(num_comp_sm), int(num_comm_sm), int(src_rank),
                                                    int(ring_step))
    prefetch_k = prefetch_k.data_ if isinstance(prefetch_k, TKParallelTensor) else prefetch_k
    prefetch_v = prefetch_v.data_ if isinstance(prefetch_v, TKParallelTensor) else prefetch_v
    _check_parallel_base(remote_k, "remote_k")
    _check_parallel_base(remote_v, "remote_v")
    _common_checks(q, k, v, cu_seqlens_q, cu_seqlens_k, cu_seqlens_q_host, cu_seqlens_k_host,
                   max_seqlen_q, max_seqlen_k, num_comp_sm, num_comm_sm)
    _check(remote_k.data_.device == q.device, "remote_k must be created on the same local CUDA device as q")
    _check(remote_v.data_.device == q.device, "remote_v must be created on the same local CUDA device as q")
    _check(remote_k.data_.shape == k.shape, "remote_k must have the same shape as local k")
    _check(remote_v.data_.shape == v.shape, "remote_v must have the same shape as local v")
    _check(remote_k.data_.data_ptr() != remote_v.data_.data_ptr(),
           "remote_k and remote_v must be separate TKParallelTensor allocations")
    _check(remote_k.local_rank_ == q.device.index, "remote_k local_rank must match q.device.index")
    _check(remote_v.local_rank_ == q.device.index, "remote_v local_rank must match q.device.index")
    _check(remote_k.local_world_size_ == remote_v.local_world_size_,
           "remote_k and remote_v must have the same local_world_size")
    _check(0 <= src_rank < remote_k.local_world_size_,
           f"src_rank must be in [0, local_world_size). Got src_rank={src_rank}, "
           f"local_world_size={remote_k.local_world_size_}")
    _check(ring_step >= 0, f"ring_step must be non-negative. Got {ring_step}")
    _check((prefetch_k is None) == (prefetch_v is None),
           "prefetch_k and prefetch_v must either both be provided or both be omitted")
    for buf, like, name in ((prefetch_k, k, "prefetch_k"), (prefetch_v, v, "prefetch_v")):
        if buf is not None:
            _check(buf.is_cuda and buf.dtype == torch.bfloat16 and buf.is_contiguous(),
                   f"{name} must be a contiguous CUDA bf16 tensor")
            _check(buf.shape == like.shape and buf.device == like.device,
                   f"{name} must have the same shape and device as local k/v")
    _check_device_capability(q.device, "min_fa3_demo_b200")
    batch = cu_seqlens_q_host.size(0) - 1
    _check(batch >= 1, "varlen demo requires batch size B >= 1")
    _check(int(cu_seqlens_q_host[0]) == 0, "cu_seqlens_q_host must start with 0")
    _check(int(cu_seqlens_k_host[0]) == 0, "cu_seqlens_k_host must start with 0")
    _check(int(cu_seqlens_q_host[batch]) == q.size(0),
           f"cu_seqlens_q_host[-1] must equal q.size(0). Got {int(cu_seqlens_q_host[batch])} vs {q.size(0)}")
    _check(int(cu_seqlens_k_host[batch]) == k.size(0),
           f"cu_seqlens_k_host[-1] must equal k.size(0). Got {int(cu_seqlens_k_host[batch])} vs {k.size(0)}")

    if out is None:
        out = torch.zeros_like(q)
    else:
        _check_out(out, q, "out")
    if lse is None:
        lse = torch.full((q.size(1), q.size(0)), float("-inf"), dtype=torch.float32, device=q.device)
    else:
        _check_lse(lse, q, "lse")

    main = torch.cuda.current_stream(q.device)
    side = None
    if num_comm_sm > 0:
        if prefetch_k is None:
            prefetch_k, prefetch_v = torch.empty_like(k), torch.empty_like(v)
        lib = _cabi.load()
        side = torch.cuda.Stream(device=q.device)
        side.wait_stream(main)
        nbytes = k.numel() * 2
        with torch.cuda.device(q.device), torch.cuda.stream(side):
            sp = ctypes.c_void_p(side.cuda_stream)
            _cabi.check(lib.b2a_peer_copy(ctypes.c_void_p(prefetch_k.data_ptr()),
                                          ctypes.c_void_p(remote_k.raw_ptrs_[src_rank]), nbytes,
                                          max(1, num_comm_sm // 2 or 1), None, sp))
            _cabi.check(lib.b2a_peer_copy(ctypes.c_void_p(prefetch_v.data_ptr()),
                                          ctypes.c_void_p(remote_v.raw_ptrs_[src_rank]), nbytes,
                                          max(1, num_comm_sm - num_comm_sm // 2), None, sp))
        prefetch_k.record_stream(side)
        prefetch_v.record_stream(side)
    _call_fwd(q, k, v, out, lse, cu_q=cu_seqlens_q, cu_k=cu_seqlens_k, batch=batch,
              seqlen_q=max_seqlen_q, seqlen_k=max_seqlen_k, heads_q=q.size(1), heads_k=k.size(1),
              is_causal=is_causal, merge_running=True, grid_blocks=num_comp_sm)
    if side is not None:
        main.wait_stream(side)
    if return_lse:
        return out, lse
    return out


# --------------------------------------------------------------------------------------
# hierarchical ring metadata (shared by forward and backward)
# --------------------------------------------------------------------------------------
def _validate_ring_metadata(q, k_arena, cu_q_host, cu_k_host, global_seqlens_host, ring_sizes_host,
                            ring_starts_host, world_size: int, rank: int, is_causal: bool,
                            max_seqlen_q: int, max_seqlen_k: int) -> int:
    """Checks of csrc/mega_ring_min_fa3_varlen_ring_bindings.cu:404-470; returns rank_kv_capacity."""
    batch = cu_q_host.size(0) - 1
    _check(batch >= 1, "varlen demo requires batch size B >= 1")
    _check(int(cu_q_host[0]) == 0, "cu_seqlens_q_host must start with 0")
    _check(int(cu_k_host[0]) == 0, "cu_seqlens_k_host must start with 0")
    _check(int(cu_q_host[batch]) == q.size(0),
           f"cu_seqlens_q_host[-1] must equal q.size(0). Got {int(cu_q_host[batch])} vs {q.size(0)}")
    local_total_k = int(cu_k_host[batch])
    _check(local_total_k >= 0, "cu_seqlens_k_host[-1] must be non-negative")
    _check(k_arena.size(0) % world_size == 0, "k and v arena rows must match and be divisible by world_size")
    cap = k_arena.size(0) // world_size
    _check(0 < cap <= _INT32_MAX, f"rank_kv_capacity must be positive and fit in int32. Got {cap}")
    _check(cap % 128 == 0, f"mega ring requires rank_kv_capacity to be 128-row aligned. Got {cap}")
    _check(local_total_k <= cap, f"local_total_k exceeds rank_kv_capacity. Got {local_total_k} vs {cap}")
    _check_host_vec(global_seqlens_host, batch, "global_seqlens_host")
    _check_host_vec(ring_sizes_host, batch, "ring_sizes_host")
    _check_host_vec(ring_starts_host, batch, "ring_starts_host")
    cq, ck = cu_q_host.tolist(), cu_k_host.tolist()
    glens, sizes, starts = global_seqlens_host.tolist(), ring_sizes_host.tolist(), ring_starts_host.tolist()
    prev = None
    for b in range(batch):
        q_len, k_len = cq[b + 1] - cq[b], ck[b + 1] - ck[b]
        _check(q_len >= 0 and k_len >= 0, f"cu_seqlens must be nondecreasing at batch={b}")
        _check(q_len % 128 == 0 and k_len % 128 == 0,
               f"mega ring requires every local q/k length to be 128-row aligned at batch={b}. "
               f"q_len={q_len}, k_len={k_len}")
        _check(glens[b] > 0, f"global_seqlens_host must be positive at batch={b}")
        _check(sizes[b] in (1, 2, 4, 8), f"ring_sizes_host must contain only 1, 2, 4, or 8. batch={b}, value={sizes[b]}")
        _check(prev is None or sizes[b] <= prev, f"batch must be ordered by non-increasing ring size. batch={b}")
        prev = sizes[b]
        _check(starts[b] >= 0 and starts[b] % sizes[b] == 0 and starts[b] + sizes[b] <= world_size,
               f"invalid aligned ring range at batch={b}: start={starts[b]}, size={sizes[b]}")
        _check(glens[b] % sizes[b] == 0, f"global length must be divisible by ring size at batch={b}")
        member = starts[b] <= rank < starts[b] + sizes[b]
        expected = glens[b] // sizes[b] if member else 0
        _check(q_len == expected and k_len == expected,
               f"local q/k length does not match hierarchical ring metadata at batch={b}. "
               f"expected={expected}, q_len={q_len}, k_len={k_len}")
        if is_causal and sizes[b] > 1 and member:
            _check(expected % 2 == 0, f"causal CP local length must be even at batch={b}")
            _check((expected // 2) % 128 == 0,
                   f"causal CP half length must be 128-aligned at batch={b}. half_len={expected // 2}")
        _check(q_len <= max_seqlen_q and k_len <= max_seqlen_k,
               "max_seqlen_q/max_seqlen_k must cover every local sequence")
    return cap


def _ring_arena_checks(q, k, v, remote_k, remote_v, what: str, allowed_worlds) -> Tuple[int, int]:
    _check(remote_k.data_.device == q.device, "remote_k must be created on the same local CUDA device as q")
    _check(remote_v.data_.device == q.device, "remote_v must be created on the same local CUDA device as q")
    _check(remote_k.data_.shape == k.shape, "remote_k must have the same shape as local k")
    _check(remote_v.data_.shape == v.shape, "remote_v must have the same shape as local v")
    _check(k.data_ptr() == remote_k.data_.data_ptr(),
           "k must be remote_k.data_ so compute and IPC use the same arena")
    _check(v.data_ptr() == remote_v.data_.data_ptr(),
           "v must be remote_v.data_ so compute and IPC use the same arena")
    _check(remote_k.data_.data_ptr() != remote_v.data_.data_ptr(),
           "remote_k and remote_v must be separate TKParallelTensor allocations")
    _check(remote_k.local_rank_ == q.device.index, "remote_k local_rank must match q.device.index")
    _check(remote_v.local_rank_ == q.device.index, "remote_v local_rank must match q.device.index")
    _check(remote_k.local_world_size_ == remote_v.local_world_size_,
           "remote_k and remote_v must have the same local_world_size")
    _check(remote_k.local_rank_ == remote_v.local_rank_, "remote_k and remote_v must have the same local_rank")
    world = remote_k.local_world_size_
    _check(world in allowed_worlds,
           f"{what} requires world_size in {{{', '.join(str(w) for w in allowed_worlds)}}}. Got {world}")
    return world, remote_k.local_rank_


def forward_varlen_mega_ring(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, is_causal, *,
                             cu_seqlens_q_host, cu_seqlens_k_host, remote_k: TKParallelTensor,
                             remote_v: TKParallelTensor, num_comp_sm: int, num_comm_sm: int,
                             global_seqlens_host, ring_sizes_host, ring_starts_host,
                             out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                             return_lse: bool = False, stats: Optional[torch.Tensor] = None
                             ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Whole context-parallel forward in one launch.  ``k`` / ``v`` are the rank-major arenas
    ``[world * rank_kv_capacity, KVH, 128]`` and must be ``remote_k.data_`` / ``remote_v.data_``;
    every rank writes its own slice ``[rank * cap, rank * cap + local_total_k)`` and all ranks
    synchronise before the call.  Documents are described by CPU int32 ``[B]`` tensors
    ``global_seqlens_host`` / ``ring_sizes_host`` / ``ring_starts_host`` (ring sizes 1/2/4/8,
    non-increasing, aligned starts); causal rings use the zigzag ``[front | back]`` layout.
    ``out`` / ``lse`` are fully overwritten (world size 1 is also accepted here)."""
    max_seqlen_q, max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    num_comp_sm, num_comm_sm = int(num_comp_sm), int(num_comm_sm)
    _check_parallel_base(remote_k, "remote_k")
    _check_parallel_base(remote_v, "remote_v")
    _common_checks(q, k, v, cu_seqlens_q, cu_seqlens_k, cu_seqlens_q_host, cu_seqlens_k_host,
                   max_seqlen_q, max_seqlen_k, num_comp_sm, num_comm_sm)
    world, rank = _ring_arena_checks(q, k, v, remote_k, remote_v, "hierarchical mega ring forward",
                                     (1, 2, 4, 8))
    _check_device_capability(q.device, "min_fa3_demo_b200")
    sm_count = torch.cuda.get_device_properties(q.device).multi_processor_count
    _check(num_comp_sm + num_comm_sm <= sm_count,
           f"num_comp_sm + num_comm_sm must not exceed the device SM count ({sm_count}). "
           f"Got {num_comp_sm + num_comm_sm}")
    cap = _validate_ring_metadata(q, k, cu_seqlens_q_host, cu_seqlens_k_host, global_seqlens_host,
                                  ring_sizes_host, ring_starts_host, world, rank, bool(is_causal),
                                  max_seqlen_q, max_seqlen_k)
    if out is None:
        out = torch.empty_like(q)
    else:
        _check_out(out, q, "out")
    if lse is None:
        lse = torch.empty((q.size(1), q.size(0)), dtype=torch.float32, device=q.device)
    else:
        _check_lse(lse, q, "lse")
    if stats is not None:
        _check(stats.is_cuda and stats.dtype == torch.int64 and stats.numel() == 2 and stats.is_contiguous(),
               "stats must be a contiguous CUDA int64 tensor with 2 elements")
    if q.size(0) == 0:
        return (out, lse) if return_lse else out

    lib = _cabi.load()
    batch = cu_seqlens_q_host.size(0) - 1
    nbytes = lib.b2a_ring_fwd_workspace_bytes(batch, world, cap, q.size(0))
    ws = _workspace(nbytes, q.device)
    a = _cabi.RingFwdArgs()
    a.q, a.out, a.lse = q.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.arena_k, a.arena_v = k.data_ptr(), v.data_ptr()
    for r in range(world):
        a.peer_k[r] = remote_k.raw_ptrs_[r]
        a.peer_v[r] = remote_v.raw_ptrs_[r]
    a.cu_seqlens_q_host = cu_seqlens_q_host.data_ptr()
    a.global_seqlens_host = global_seqlens_host.data_ptr()
    a.ring_sizes_host = ring_sizes_host.data_ptr()
    a.ring_starts_host = ring_starts_host.data_ptr()
    a.stats = stats.data_ptr() if stats is not None else None
    a.batch, a.world_size, a.rank, a.rank_kv_capacity = batch, world, rank, cap
    a.total_q, a.heads_q, a.heads_k, a.head_dim = q.size(0), q.size(1), k.size(1), 128
    a.is_causal = int(bool(is_causal))
    a.num_comp_sm, a.num_comm_sm = num_comp_sm, num_comm_sm
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    with torch.cuda.device(q.device):
        _cabi.check(lib.b2a_ring_fwd(ctypes.byref(a), _stream_ptr(q.device)))
    forward_varlen_mega_ring.last_workspace = ws
    if return_lse:
        return out, lse
    return out


# --------------------------------------------------------------------------------------
# context-parallel backward
# --------------------------------------------------------------------------------------
def _check_parallel_identity(t: TKParallelTensor, q: torch.Tensor, world: int, rank: int, name: str) -> None:
    # reference: csrc/backward/min_fa3_bwd_bindings.cu:359-373
    _check(isinstance(t, TKParallelTensor), f"{name} must be a TKParallelTensor")
    _check(t.data_.is_cuda, f"{name} must be CUDA-backed")
    _check(t.data_.device == q.device, f"{name} local view must be on q.device")
    _check(t.local_world_size_ == world, f"{name} world size mismatch")
    _check(t.local_rank_ == rank, f"{name} local rank mismatch")
    _check(len(t.raw_ptrs_) == world, f"{name} must expose one pointer per rank")


def backward_varlen_mega_ring(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                              max_seqlen_k, *, cu_seqlens_q_host, cu_seqlens_k_host,
                              remote_k: TKParallelTensor, remote_v: TKParallelTensor,
                              remote_dk_accum: TKParallelTensor, remote_dv_accum: TKParallelTensor,
                              remote_dkv_completion: TKParallelTensor, num_comp_sm: int, num_comm_sm: int,
                              global_seqlens_host, ring_sizes_host, ring_starts_host, is_causal: bool = True
                              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Context-parallel backward of ``forward_varlen_mega_ring`` (reference:
    ``backward_varlen_mega_ring``, csrc/backward/min_fa3_bwd_bindings.cu:375-722; causal like the
    reference by default, the non-causal ring is accepted too).

    ``k`` / ``v`` are the K/V arenas (``remote_k.data_`` / ``remote_v.data_``).  The fp32
    accumulators ``remote_dk_accum`` / ``remote_dv_accum`` (>= ``KVH * rank_kv_capacity * 128``
    floats) and the int32 ``remote_dkv_completion`` counter must be zeroed, and all ranks
    synchronised, before every call.  Returns ``dq [total_q, QH, 128]`` and compact
    ``dk, dv [local_total_k, KVH, 128]``."""
    from .min_fa3_op import _check_bf16_cuda, _check_same_device
    max_seqlen_q, max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    num_comp_sm, num_comm_sm = int(num_comp_sm), int(num_comm_sm)
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (out, "out"), (dout, "dout")):
        _check_bf16_cuda(t, name, 3)
    _check(softmax_lse.is_cuda and softmax_lse.dtype == torch.float32 and softmax_lse.is_contiguous(),
           "softmax_lse must be a contiguous CUDA float32 tensor")
    _check(tuple(softmax_lse.shape) == (q.size(1), q.size(0)), "softmax_lse must have shape [QH, total_q]")
    for t, name in ((k, "k"), (v, "v"), (out, "out"), (dout, "dout"), (softmax_lse, "softmax_lse")):
        _check_same_device(q, t, name)
    _check(out.shape == q.shape, "out must have the same shape as q")
    _check(dout.shape == q.shape, "dout must have the same shape as q")
    _check(k.size(1) == v.size(1), "k and v must have the same KV head count")
    _check(q.size(1) % k.size(1) == 0, "qhead must be divisible by kvhead")
    _check_cu_seqlens(cu_seqlens_q, "cu_seqlens_q")
    _check_cu_seqlens(cu_seqlens_k, "cu_seqlens_k")
    _check_cu_seqlens_host(cu_seqlens_q_host, cu_seqlens_q, "cu_seqlens_q_host")
    _check_cu_seqlens_host(cu_seqlens_k_host, cu_seqlens_k, "cu_seqlens_k_host")
    _check(num_comp_sm > 0, f"num_comp_sm must be positive. Got {num_comp_sm}")
    _check(num_comm_sm >= 0, f"num_comm_sm must be non-negative. Got {num_comm_sm}")
    _check_parallel_base(remote_k, "remote_k")
    _check_parallel_base(remote_v, "remote_v")
    world, rank = _ring_arena_checks(q, k, v, remote_k, remote_v, "mega ring backward", (1, 2, 4, 8))
    for t, name in ((remote_dk_accum, "remote_dk_accum"), (remote_dv_accum, "remote_dv_accum"),
                    (remote_dkv_completion, "remote_dkv_completion")):
        _check_parallel_identity(t, q, world, rank, name)
    _check(remote_dk_accum.data_.dtype == torch.float32 and remote_dv_accum.data_.dtype == torch.float32,
           "remote_dk_accum and remote_dv_accum must have dtype torch.float32")
    _check(remote_dkv_completion.data_.dtype == torch.int32 and remote_dkv_completion.data_.numel() >= 1,
           "remote_dkv_completion must be an int32 tensor with at least one element")
    _check_device_capability(q.device, "min_fa3_demo_b200 backward")
    sm_count = torch.cuda.get_device_properties(q.device).multi_processor_count
    _check(num_comp_sm + num_comm_sm <= sm_count,
           f"num_comp_sm + num_comm_sm must not exceed the device SM count ({sm_count}). "
           f"Got {num_comp_sm + num_comm_sm}")
    cap = _validate_ring_metadata(q, k, cu_seqlens_q_host, cu_seqlens_k_host, global_seqlens_host,
                                  ring_sizes_host, ring_starts_host, world, rank, bool(is_causal),
                                  max_seqlen_q, max_seqlen_k)
    need = k.size(1) * cap * 128
    _check(remote_dk_accum.data_.numel() >= need and remote_dv_accum.data_.numel() >= need,
           f"remote_dk_accum / remote_dv_accum need at least KVH * rank_kv_capacity * 128 = {need} floats")
    batch = cu_seqlens_q_host.size(0) - 1
    local_total_k = int(cu_seqlens_k_host[batch])

    dq = torch.empty_like(q)
    dk = torch.empty((local_total_k, k.size(1), 128), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty_like(dk)
    lib = _cabi.load()
    nbytes = lib.b2a_ring_bwd_workspace_bytes(batch, world, cap, q.size(0), q.size(1))
    ws = _workspace(nbytes, q.device)
    a = _cabi.RingBwdArgs()
    a.dout, a.q, a.out, a.lse = dout.data_ptr(), q.data_ptr(), out.data_ptr(), softmax_lse.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.arena_k, a.arena_v = k.data_ptr(), v.data_ptr()
    for r in range(world):
        a.peer_k[r] = remote_k.raw_ptrs_[r]
        a.peer_v[r] = remote_v.raw_ptrs_[r]
        a.dk_accum_peer[r] = remote_dk_accum.raw_ptrs_[r]
        a.dv_accum_peer[r] = remote_dv_accum.raw_ptrs_[r]
        a.completion_peer[r] = remote_dkv_completion.raw_ptrs_[r]
    a.cu_seqlens_q_host = cu_seqlens_q_host.data_ptr()
    a.global_seqlens_host = global_seqlens_host.data_ptr()
    a.ring_sizes_host = ring_sizes_host.data_ptr()
    a.ring_starts_host = ring_starts_host.data_ptr()
    a.batch, a.world_size, a.rank, a.rank_kv_capacity = batch, world, rank, cap
    a.total_q, a.local_total_k = q.size(0), local_total_k
    a.heads_q, a.heads_k, a.head_dim = q.size(1), k.size(1), 128
    a.is_causal = int(bool(is_causal))
    a.num_comp_sm, a.num_comm_sm = num_comp_sm, num_comm_sm
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    with torch.cuda.device(q.device):
        _cabi.check(lib.b2a_ring_bwd(ctypes.byref(a), _stream_ptr(q.device)))
    backward_varlen_mega_ring.last_workspace = ws
    return dq, dk, dv
