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
                         _check_device_capability, _check_varlen_qkv, _remember_workspace, _stream_ptr,
                         _workspace)
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
    ``src_rank``'s K/V from the parallel tensors into ``prefetch_k`` / ``prefetch_v`` -- all in
    one launch on the current stream (``num_comp_sm`` attention CTAs followed by ``num_comm_sm``
    copy CTAs, which join the attention work once their share of the copy is done).  With
    ``num_comm_sm == 0`` nothing is copied (csrc/min_fa3_varlen_ring_bindings.cu:343-348)."""
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

    # One launch, as in the reference (include/min_fa3_varlen_ring_launch.h:217): CTAs
    # [0, num_comp_sm) run attention, CTAs [num_comp_sm, num_comp_sm + num_comm_sm) first pull
    # src_rank's K/V through the peer mapping into the prefetch buffers.
    prefetch = None
    if num_comm_sm > 0 and k.numel() > 0:
        if prefetch_k is None:
            prefetch_k, prefetch_v = torch.empty_like(k), torch.empty_like(v)
        prefetch = (remote_k.raw_ptrs_[src_rank], remote_v.raw_ptrs_[src_rank], prefetch_k, prefetch_v,
                    num_comm_sm)
    ws = _call_fwd(q, k, v, out, lse, cu_q=cu_seqlens_q, cu_k=cu_seqlens_k, batch=batch,
                   seqlen_q=max_seqlen_q, seqlen_k=max_seqlen_k, heads_q=q.size(1), heads_k=k.size(1),
                   is_causal=is_causal, merge_running=True, grid_blocks=num_comp_sm, prefetch=prefetch)
    _remember_workspace("forward_varlen_ring", ws)
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
    _remember_workspace("forward_varlen_mega_ring", ws)
    if return_lse:
        return out, lse
    return out


# --------------------------------------------------------------------------------------
# context-parallel backward
# --------------------------------------------------------------------------------------
def dkv_accum_numel(heads_k: int, logical_rank_capacity: int, batch: int) -> int:
    """Floats each of ``remote_dk_accum`` / ``remote_dv_accum`` must hold: the reference's rule
    ``KVH * round128(logical_rank_capacity + B * 128) * 128``
    (csrc/backward/min_fa3_bwd_bindings.cu:630-640), where ``logical_rank_capacity`` is the largest
    number of key rows any rank holds and ``B`` the number of documents."""
    padded = ((int(logical_rank_capacity) + int(batch) * 128 + 127) // 128) * 128
    return int(heads_k) * padded * 128


def _check_parallel_identity(t, q: torch.Tensor, world: int, rank: int, name: str, device_type: str) -> None:
    # reference: csrc/backward/min_fa3_bwd_bindings.cu:359-373
    _check(isinstance(t, TKParallelTensor), f"{name} must be a TKParallelTensor")
    _check(t.data_.device.type == device_type, f"{name} must be CUDA-backed")
    _check(t.data_.device == q.device, f"{name} local view must be on q.device")
    _check(t.local_world_size_ == world, f"{name} world size mismatch")
    _check(t.local_rank_ == rank, f"{name} local rank mismatch")
    _check(len(t.raw_ptrs_) == world, f"{name} must expose one pointer per rank")


def _check_bwd_dense(t: torch.Tensor, name: str, device_type: str) -> None:
    # check_bf16_cuda, csrc/backward/min_fa3_bwd_bindings.cu:40-46
    _check(t.device.type == device_type, f"{name} must be a CUDA tensor")
    _check(t.dtype == torch.bfloat16, f"{name} must have dtype torch.bfloat16")
    _check(t.dim() == 3, f"{name} must have 3 dimensions")
    _check(t.size(-1) == 128, f"{name} must have head_dim D=128")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _validate_backward_mega_ring(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                 max_seqlen_k, cu_seqlens_q_host, cu_seqlens_k_host, remote_k, remote_v,
                                 remote_dk_accum, remote_dv_accum, remote_dkv_completion, num_comp_sm,
                                 num_comm_sm, global_seqlens_host, ring_sizes_host, ring_starts_host,
                                 is_causal: bool, device_type: str = "cuda") -> Tuple[int, int, int, int, int]:
    """Every host-side check of the context-parallel backward, in the order and with the texts of
    the reference binding (csrc/backward/min_fa3_bwd_bindings.cu:398-545, 622-640) and of the
    substrings its negative test matches on
    (scripts/test_mega_ring/mega_ring_test_min_fa3_varlen_backward_validation_multi_rank.py:48-224).
    Nothing is launched or allocated here.  Returns ``(world, rank, rank_kv_capacity, batch,
    local_total_k)``.  ``device_type`` exists for the CPU-only tests of this function."""
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (out, "out"), (dout, "dout")):
        _check_bwd_dense(t, name, device_type)
    _check(softmax_lse.device.type == device_type, "softmax_lse must be a CUDA tensor")
    _check(softmax_lse.dtype == torch.float32, "softmax_lse must have dtype torch.float32")
    _check(softmax_lse.is_contiguous(), "softmax_lse must be contiguous")
    _check(softmax_lse.device == q.device, "softmax_lse must be on the same CUDA device as q")
    for t, name in ((cu_seqlens_q, "cu_seqlens_q"), (cu_seqlens_k, "cu_seqlens_k")):
        _check(t.device.type == device_type, f"{name} must be a CUDA tensor")
        _check(t.dtype == torch.int32, f"{name} must have dtype torch.int32")
        _check(t.dim() == 1 and t.numel() >= 2, f"{name} must have shape [B + 1]")
        _check(t.is_contiguous(), f"{name} must be contiguous")
        _check(t.device == q.device, f"{name} must be on the same CUDA device as q")
    hosts = (cu_seqlens_q_host, cu_seqlens_k_host)
    _check(all(isinstance(t, torch.Tensor) and t.device.type == "cpu" for t in hosts),
           "host cu_seqlens tensors must be on CPU")
    _check(all(t.dtype == torch.int32 for t in hosts), "host cu_seqlens tensors must have dtype int32")
    _check(all(t.is_contiguous() for t in hosts), "host cu_seqlens tensors must be contiguous")
    _check(cu_seqlens_q_host.numel() == cu_seqlens_q.numel() and cu_seqlens_k_host.numel() == cu_seqlens_k.numel(),
           "host and device cu_seqlens lengths must match")
    _check(cu_seqlens_q.numel() == cu_seqlens_k.numel(), "cu_seqlens_q and cu_seqlens_k must have the same B")
    batch = cu_seqlens_q_host.numel() - 1
    for t, name in ((global_seqlens_host, "global_seqlens_host"), (ring_sizes_host, "ring_sizes_host"),
                    (ring_starts_host, "ring_starts_host")):
        _check(isinstance(t, torch.Tensor) and t.device.type == "cpu", f"{name} must be a CPU tensor")
        _check(t.dtype == torch.int32, f"{name} must have dtype int32")
        _check(t.dim() == 1 and t.numel() == batch, f"{name} must have shape [B]")
        _check(t.is_contiguous(), f"{name} must be contiguous")
    _check(all(t.device == q.device for t in (k, v, out, dout)), "all dense tensors must be on the same CUDA device")
    _check(out.shape == q.shape and dout.shape == q.shape, "out and dout must have the same shape as q")
    _check(q.size(1) > 0 and k.size(1) > 0, "qhead and kvhead must be positive")
    _check(q.size(1) % k.size(1) == 0, "qhead must be divisible by kvhead")
    _check(k.size(1) == v.size(1) and k.size(2) == v.size(2), "k/v shapes must match")
    _check(tuple(softmax_lse.shape) == (q.size(1), q.size(0)), "softmax_lse must have shape [QH, total_q]")
    # The reference wants both counts positive; a single-rank world has nothing to copy, so
    # num_comm_sm = 0 is accepted there.
    _check(num_comp_sm > 0 and num_comm_sm >= 0,
           "mega-ring backward requires positive compute and communication SM counts")
    if q.is_cuda:
        _check_device_capability(q.device, "min_fa3_demo_b200 backward")
        sm_count = torch.cuda.get_device_properties(q.device).multi_processor_count
        _check(num_comp_sm + num_comm_sm <= sm_count,
               f"num_comp_sm + num_comm_sm must not exceed the device SM count ({sm_count})")
    _check(isinstance(remote_k, TKParallelTensor), "remote_k must be a TKParallelTensor")
    world, rank = remote_k.local_world_size_, remote_k.local_rank_
    _check(world in (1, 2, 4, 8), "world_size must be one of 1, 2, 4, or 8")
    for t, name in ((remote_k, "remote_k"), (remote_v, "remote_v"), (remote_dk_accum, "remote_dk_accum"),
                    (remote_dv_accum, "remote_dv_accum"), (remote_dkv_completion, "remote_dkv_completion")):
        _check_parallel_identity(t, q, world, rank, name, device_type)
    _check(remote_k.data_.dtype == torch.bfloat16 and remote_v.data_.dtype == torch.bfloat16 and
           remote_k.data_.shape == k.shape and remote_v.data_.shape == v.shape,
           "remote_k/remote_v must match the concatenated bf16 k/v storage")
    _check(remote_k.data_.data_ptr() == k.data_ptr() and remote_v.data_.data_ptr() == v.data_ptr(),
           "k/v must be the local remote_k/remote_v IPC arena views")
    _check(remote_dk_accum.data_.dtype == torch.float32 and remote_dv_accum.data_.dtype == torch.float32,
           "remote dK/dV accumulators must have dtype float32")
    _check(remote_dkv_completion.data_.dtype == torch.int32 and remote_dkv_completion.data_.numel() == 1,
           "remote_dkv_completion must be a one-element int32 parallel tensor")

    cq, ck = cu_seqlens_q_host.tolist(), cu_seqlens_k_host.tolist()
    glens, sizes, starts = global_seqlens_host.tolist(), ring_sizes_host.tolist(), ring_starts_host.tolist()
    _check(cq[0] == 0 and ck[0] == 0, "cu_seqlens must start at zero")
    local_total_k = ck[batch]
    _check(k.size(0) == v.size(0) and k.size(0) % world == 0,
           "k/v arena rows must match and be divisible by world_size")
    cap = k.size(0) // world
    _check(0 < cap <= _INT32_MAX, "rank_kv_capacity must be positive and fit in int32")
    _check(cap % 128 == 0, f"rank_kv_capacity must be 128-row aligned. Got {cap}")
    _check(0 <= local_total_k <= cap,
           f"local_total_k must fit in rank_kv_capacity. Got {local_total_k} vs {cap}")
    _check(cq[batch] == q.size(0), "cu_seqlens_q_host[-1] must equal q.size(0)")
    prev, max_q, max_k = 8, 0, 0
    rank_rows = [0] * world
    for b in range(batch):
        q_len, k_len = cq[b + 1] - cq[b], ck[b + 1] - ck[b]
        _check(q_len >= 0 and k_len >= 0, f"cu_seqlens must be nondecreasing at batch={b}")
        _check(q_len == k_len, f"causal hybrid backward requires self-attention q_len == k_len at batch={b}")
        _check(q_len % 128 == 0, f"every local q/k length must be 128-row aligned at batch={b}")
        _check(glens[b] > 0, f"global_seqlens_host must be positive at batch={b}")
        _check(sizes[b] in (1, 2, 4, 8), f"ring_sizes_host must contain only 1, 2, 4, or 8 at batch={b}")
        _check(sizes[b] <= prev, f"batch must be ordered by non-increasing ring size at batch={b}")
        prev = sizes[b]
        _check(starts[b] >= 0 and starts[b] % sizes[b] == 0 and starts[b] + sizes[b] <= world,
               f"invalid aligned ring range at batch={b}: start={starts[b]}, size={sizes[b]}, world_size={world}")
        _check(glens[b] % sizes[b] == 0, f"global length must be divisible by ring size at batch={b}")
        member_rows = glens[b] // sizes[b]
        for owner in range(starts[b], starts[b] + sizes[b]):
            rank_rows[owner] += member_rows
            _check(rank_rows[owner] <= _INT32_MAX, "logical rank K/V capacity must fit in int32")
        member = starts[b] <= rank < starts[b] + sizes[b]
        expected = member_rows if member else 0
        _check(q_len == expected,
               f"local q/k length does not match ring metadata at batch={b}. expected={expected}, actual={q_len}")
        if is_causal and sizes[b] > 1 and member:
            _check(q_len % 2 == 0 and (q_len // 2) % 128 == 0,
                   f"G2/G4/G8 local half length must be 128-row aligned at batch={b}")
        max_q, max_k = max(max_q, q_len), max(max_k, k_len)
    _check(0 < max_seqlen_q <= _INT32_MAX and 0 < max_seqlen_k <= _INT32_MAX,
           "max seqlens must be positive int32 values")
    _check(max_q <= max_seqlen_q and max_k <= max_seqlen_k,
           "max_seqlen_q/max_seqlen_k must cover every local sequence")
    logical_cap = max(rank_rows)
    _check(0 < logical_cap <= cap,
           f"logical rank K/V capacity must be positive and fit in the reusable arena. Got {logical_cap} "
           f"vs arena capacity {cap}")
    need = dkv_accum_numel(k.size(1), logical_cap, batch)
    _check(remote_dk_accum.data_.numel() >= need and remote_dv_accum.data_.numel() >= need,
           "remote dK/dV accumulators must each contain (have capacity for) at least "
           f"KVH * padded_rank_capacity * 128 = {need} float elements")
    return world, rank, cap, batch, local_total_k


def backward_varlen_mega_ring(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                              max_seqlen_k, *, cu_seqlens_q_host, cu_seqlens_k_host,
                              remote_k: TKParallelTensor, remote_v: TKParallelTensor,
                              remote_dk_accum: TKParallelTensor, remote_dv_accum: TKParallelTensor,
                              remote_dkv_completion: TKParallelTensor, num_comp_sm: int, num_comm_sm: int,
                              global_seqlens_host, ring_sizes_host, ring_starts_host, is_causal: bool = True,
                              kv_resident: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Context-parallel backward of ``forward_varlen_mega_ring`` (reference:
    ``backward_varlen_mega_ring``, csrc/backward/min_fa3_bwd_bindings.cu:375-722; causal like the
    reference by default, the non-causal ring is accepted too).

    ``k`` / ``v`` are the K/V arenas (``remote_k.data_`` / ``remote_v.data_``).  The fp32
    accumulators ``remote_dk_accum`` / ``remote_dv_accum`` (at least ``dkv_accum_numel(KVH,
    logical_rank_capacity, B)`` floats, the reference's sizing rule) and the one-element int32
    ``remote_dkv_completion`` counter must be zeroed, and all ranks synchronised, before every
    call.  Returns ``dq [total_q, QH, 128]`` and compact ``dk, dv [local_total_k, KVH, 128]``.

    ``kv_resident`` (not in the reference, whose backward always pulls the remote K/V again):
    pass True when this rank's arena still holds what ``forward_varlen_mega_ring`` left there on
    the same metadata and K/V -- nothing crosses NVLink for K/V then and every CTA computes from
    the start.  With the default the call is self-contained like the reference's."""
    max_seqlen_q, max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    num_comp_sm, num_comm_sm = int(num_comp_sm), int(num_comm_sm)
    world, rank, cap, batch, local_total_k = _validate_backward_mega_ring(
        dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
        cu_seqlens_q_host, cu_seqlens_k_host, remote_k, remote_v, remote_dk_accum, remote_dv_accum,
        remote_dkv_completion, num_comp_sm, num_comm_sm, global_seqlens_host, ring_sizes_host,
        ring_starts_host, bool(is_causal))

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
    a.kv_resident = int(bool(kv_resident))
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    with torch.cuda.device(q.device):
        _cabi.check(lib.b2a_ring_bwd(ctypes.byref(a), _stream_ptr(q.device)))
    _remember_workspace("backward_varlen_mega_ring", ws)
    return dq, dk, dv
