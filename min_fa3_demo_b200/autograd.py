"""Differentiable front end: ``torch.library`` operators plus autograd formulas over the
``min_fa3_op`` kernels, and a context-parallel attention object that owns the peer-visible
buffers.

The reference exposes forward and backward as separate calls and leaves their pairing to the
caller (``min_fa3_op.py:25-52, 278-306``); its context-parallel backward additionally requires
the caller to zero three peer-visible buffers and synchronise all ranks before every call
(``csrc/backward/min_fa3_bwd_bindings.cu:375-722``, README "remote workspace reset").  This
module does the pairing once:

``attention(q, k, v, is_causal)``                 BSHD, differentiable
``attention_varlen(q, k, v, cu_seqlens, ...)``    packed varlen, differentiable
``RingAttention``                                  context parallel over a process group: owns the
                                                   K/V arenas, the fp32 dK/dV accumulators and the
                                                   completion counter, copies local K/V into the
                                                   arena, and performs the zero + barrier protocol

The dense operators are registered with ``torch.library.custom_op`` (namespace ``b200attn``)
with fake (meta) implementations, so they trace under ``torch.compile`` / fake tensors; there
is no CPU implementation — calling them with CPU tensors raises.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import min_fa3_op as _op


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the attention operators have no CPU implementation")


# ------------------------------------------------------------------------------------------
# torch.library operators (BSHD)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("b200attn::fwd", mutates_args=())
def _fwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    _require_cuda(q, "q")
    out, lse = _op.forward(q, k, v, is_causal, return_lse=True)
    return out, lse


@_fwd_op.register_fake
def _(q, k, v, is_causal):
    return torch.empty_like(q), q.new_empty((q.size(0), q.size(2), q.size(1)), dtype=torch.float32)


@torch.library.custom_op("b200attn::bwd", mutates_args=())
def _bwd_op(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
            lse: torch.Tensor, is_causal: bool, deterministic: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    _require_cuda(q, "q")
    dq, dk, dv = _op.backward(dout.contiguous(), q, k, v, out, lse, is_causal, deterministic=deterministic)
    return dq, dk, dv


@_bwd_op.register_fake
def _(dout, q, k, v, out, lse, is_causal, deterministic):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, is_causal: bool, deterministic: bool):
        out, lse = torch.ops.b200attn.fwd(q, k, v, is_causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.is_causal, ctx.deterministic = is_causal, deterministic
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = torch.ops.b200attn.bwd(dout, q, k, v, out, lse, ctx.is_causal, ctx.deterministic)
        return dq, dk, dv, None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = True, *,
              deterministic: bool = False) -> torch.Tensor:
    """Differentiable BSHD attention: q ``[B, S, QH, 128]``, k/v ``[B, Sk, KVH, 128]`` bf16."""
    return _Attention.apply(q, k, v, bool(is_causal), bool(deterministic))


# ------------------------------------------------------------------------------------------
# Packed varlen
# ------------------------------------------------------------------------------------------
class _AttentionVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, cu_q_host, cu_k_host, max_q: int, max_k: int, is_causal: bool,
                deterministic: bool):
        _require_cuda(q, "q")
        out, lse = _op.forward_varlen(q, k, v, cu_q, cu_k, max_q, max_k, is_causal,
                                      cu_seqlens_q_host=cu_q_host, cu_seqlens_k_host=cu_k_host, return_lse=True)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.args = (max_q, max_k, is_causal, deterministic)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, is_causal, deterministic = ctx.args
        dq, dk, dv = _op.backward_varlen(dout.contiguous(), q, k, v, out, lse, cu_q, cu_k, max_q, max_k, is_causal,
                                         deterministic=deterministic)
        return (dq, dk, dv) + (None,) * 8


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                     cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, is_causal: bool = True, *,
                     cu_seqlens_q_host: Optional[torch.Tensor] = None,
                     cu_seqlens_k_host: Optional[torch.Tensor] = None, deterministic: bool = False) -> torch.Tensor:
    """Differentiable packed attention: q ``[T, QH, 128]``, k/v ``[Tk, KVH, 128]``; the CPU copies of
    ``cu_seqlens`` are made here when the caller does not pass them (one device->host read)."""
    if cu_seqlens_q_host is None:
        cu_seqlens_q_host = cu_seqlens_q.cpu()
    if cu_seqlens_k_host is None:
        cu_seqlens_k_host = cu_seqlens_k.cpu()
    return _AttentionVarlen.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, cu_seqlens_q_host, cu_seqlens_k_host,
                                  int(max_seqlen_q), int(max_seqlen_k), bool(is_causal), bool(deterministic))


# ------------------------------------------------------------------------------------------
# Context parallel
# ------------------------------------------------------------------------------------------
class _RingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ring: "RingAttention", cu, cu_host, max_len: int, meta):
        generation = ring._load_kv(k, v)
        out, lse = _op.forward_varlen_mega_ring(
            q, ring.arena_k.data_, ring.arena_v.data_, cu, cu, max_len, max_len, ring.is_causal,
            cu_seqlens_q_host=cu_host, cu_seqlens_k_host=cu_host, remote_k=ring.arena_k, remote_v=ring.arena_v,
            num_comp_sm=ring.num_comp_sm, num_comm_sm=ring.num_comm_sm, return_lse=True, **meta)
        ctx.save_for_backward(q, k, v, out, lse, cu)
        ctx.ring, ctx.cu_host, ctx.max_len, ctx.meta = ring, cu_host, max_len, meta
        ctx.kv_rows, ctx.generation = k.size(0), generation
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        ring: RingAttention = ctx.ring
        resident = ring._generation == ctx.generation   # the forward's remote blocks are still in the arena
        if not resident:
            # Another forward has used the arena since this call's forward (several layers or
            # micro-batches share the object, or activation checkpointing re-ran a forward): put
            # this call's K/V back.  Every rank sees the same sequence of calls, so all of them
            # take this branch together (it contains barriers).
            ctx.generation = ring._load_kv(k, v)
        ring._reset_backward_buffers()
        dq, dk, dv = _op.backward_varlen_mega_ring(
            dout.contiguous(), q, ring.arena_k.data_, ring.arena_v.data_, out, lse, cu, cu, ctx.max_len, ctx.max_len,
            cu_seqlens_q_host=ctx.cu_host, cu_seqlens_k_host=ctx.cu_host, remote_k=ring.arena_k,
            remote_v=ring.arena_v, remote_dk_accum=ring.acc_k, remote_dv_accum=ring.acc_v,
            remote_dkv_completion=ring.done, num_comp_sm=ring.num_comp_sm, num_comm_sm=ring.num_comm_sm,
            is_causal=ring.is_causal, kv_resident=resident, **ctx.meta)
        return dq, dk[:ctx.kv_rows], dv[:ctx.kv_rows], None, None, None, None, None


class RingAttention:
    """Context-parallel attention over all ranks of one NVLink node (one process per GPU,
    ``torch.distributed`` initialised with NCCL before construction).

    The object owns everything the mega-ring entry points want from the caller: the rank-major
    K/V arenas (``rank_kv_capacity`` rows per rank), the fp32 dK/dV accumulators and the completion
    counter, all peer-visible.  ``__call__`` takes this rank's packed shard ``q, k, v``
    ``[T_local, H, 128]`` in the placement's document order (zigzag ``[front | back]`` halves for
    causal rings) with the placement metadata, and is differentiable.  Calls must be made by all
    ranks together, in the same order (they contain barriers).  One object may serve many layers
    or micro-batches: the arena holds the K/V of the latest forward, and a backward whose K/V has
    been overwritten since copies its saved K/V back first (one extra local copy and two
    barriers); with one object per layer that never happens.  ``max_documents`` bounds the
    number of documents per call (it sizes the fp32 dK/dV accumulators).
    """

    def __init__(self, rank_kv_capacity: int, heads_k: int, *, is_causal: bool = True, num_comm_sm: int = 8,
                 device: Optional[torch.device] = None, group=None, max_documents: int = 64):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.cap = ((int(rank_kv_capacity) + 127) // 128) * 128
        self.heads_k = heads_k
        self.is_causal = bool(is_causal)
        sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.num_comm_sm = num_comm_sm if self.world > 1 else 0
        self.num_comp_sm = sm - self.num_comm_sm
        local_rank = self.device.index

        def parallel(shape, dtype):
            t = torch.zeros(shape, dtype=dtype, device=self.device)
            return _op.TKParallelTensor(t, local_rank=local_rank, local_world_size=self.world, multicast=False)
        self.arena_k = parallel((self.world * self.cap, heads_k, 128), torch.bfloat16)
        self.arena_v = parallel((self.world * self.cap, heads_k, 128), torch.bfloat16)
        from .ring import dkv_accum_numel
        self.max_documents = int(max_documents)
        accum = dkv_accum_numel(heads_k, self.cap, self.max_documents)
        self.acc_k = parallel((accum,), torch.float32)
        self.acc_v = parallel((accum,), torch.float32)
        self.done = parallel((1,), torch.int32)
        self._generation = 0        # counts arena loads; identical on every rank

    def _barrier(self) -> None:
        torch.cuda.current_stream(self.device).synchronize()
        if self.world > 1:
            self.dist.barrier(self.group)

    def _load_kv(self, k: torch.Tensor, v: torch.Tensor) -> int:
        """Copies this rank's K/V into its arena slice (between two barriers) and returns the
        arena generation that now holds them."""
        if k.size(0) > self.cap:
            raise RuntimeError(f"local K/V has {k.size(0)} rows, the arena holds {self.cap} per rank")
        self._barrier()                       # nobody still reads the arena of a previous call
        lo = self.rank * self.cap
        self.arena_k.data_[lo:lo + k.size(0)].copy_(k.detach())
        self.arena_v.data_[lo:lo + v.size(0)].copy_(v.detach())
        self._barrier()                       # every rank's slice is in place
        self._generation += 1
        return self._generation

    def _reset_backward_buffers(self) -> None:
        self.acc_k.data_.zero_()
        self.acc_v.data_.zero_()
        self.done.data_.zero_()
        self._barrier()

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, local_lengths: Sequence[int],
                 global_lengths: Sequence[int], ring_sizes: Sequence[int], ring_starts: Sequence[int]) -> torch.Tensor:
        if len(local_lengths) > self.max_documents:
            raise RuntimeError(f"{len(local_lengths)} documents in one call, but the accumulators were sized "
                               f"for max_documents={self.max_documents}")
        cu_list: List[int] = [0]
        for n in local_lengths:
            cu_list.append(cu_list[-1] + int(n))
        cu_host = torch.tensor(cu_list, dtype=torch.int32)
        cu = cu_host.to(self.device)
        meta = dict(global_seqlens_host=torch.tensor(list(global_lengths), dtype=torch.int32),
                    ring_sizes_host=torch.tensor(list(ring_sizes), dtype=torch.int32),
                    ring_starts_host=torch.tensor(list(ring_starts), dtype=torch.int32))
        max_len = max(max(int(n) for n in local_lengths), 1)
        return _RingFn.apply(q, k, v, self, cu, cu_host, max_len, meta)
