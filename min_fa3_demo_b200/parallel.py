"""Peer-visible tensors and peer -> local copies (single node, NVLink).

Mirror of the reference's ``TKParallelTensor`` container, ``create_parallel_tensor`` and
``parallel_remote_load[_vec]`` (``min_fa3_op.py:145-275``, ``csrc/parallel/remote_load.cu``).
A parallel tensor is a local CUDA tensor of identical shape on every local rank plus the table
of device pointers under which each rank's copy is reachable from this process
(``raw_ptrs_``).  Pointers are exchanged once as CUDA-IPC handles through
``torch.distributed`` (the reference uses a ThunderKittens socket broker); construction is
therefore collective over the local ranks.  ``multicast`` must be False, as at every call
site of the reference.
"""

from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from . import _cabi

MAX_WORLD_SIZE = 8

# CUDA-IPC allocations already mapped into this process: handle bytes -> [base pointer, users].
# An allocation is opened once however many tensors live inside it.
_OPENED: dict = {}


def _env_int(name: str) -> Optional[int]:
    value = os.environ.get(name)
    return None if value is None else int(value)


def _resolve_parallel_context(local_rank: Optional[int], local_world_size: Optional[int]
                              ) -> Tuple[int, int]:
    """Fills in a missing local rank / local world size the way the reference does
    (min_fa3_op.py:145-178): an explicit argument wins, then ``LOCAL_RANK`` / ``LOCAL_WORLD_SIZE``
    from the launcher's environment, then the current CUDA device for the rank and the size of
    the initialised process group for the world.  A process group that spans more ranks than
    the local world size means several nodes, which peer mappings cannot cross: rejected with
    the reference's message."""
    group_size = dist.get_world_size() if dist.is_available() and dist.is_initialized() else None
    rank = local_rank if local_rank is not None else _env_int("LOCAL_RANK")
    if rank is None:
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is required for parallel_remote_load")
        rank = torch.cuda.current_device()
    world = local_world_size if local_world_size is not None else _env_int("LOCAL_WORLD_SIZE")
    if world is None:
        world = group_size
    if world is None:
        raise RuntimeError("local_world_size is required when LOCAL_WORLD_SIZE is not set "
                           "and torch.distributed is not initialized")
    if group_size is not None and group_size != world:
        raise RuntimeError("ThunderKittens parallel IPC path is single-node only: "
                           f"world_size={group_size}, local_world_size={world}")
    return int(rank), int(world)


class TKParallelTensor:
    """Local tensor ``data_`` plus ``raw_ptrs_[r]``: the address of rank r's copy as seen from
    this process.  Constructors (both collective over the local ranks):

    ``TKParallelTensor(tensor, *, local_rank, local_world_size, multicast=False)``
    ``TKParallelTensor(shape, dtype, local_rank, local_world_size, multicast)``
    """

    def __init__(self, tensor_or_shape: Union[torch.Tensor, Sequence[int]], dtype=None,
                 local_rank: Optional[int] = None, local_world_size: Optional[int] = None,
                 multicast: bool = False):
        if multicast:
            raise NotImplementedError("multicast parallel tensors are not supported (the attention "
                                      "path only uses multicast=False)")
        if local_rank is None or local_world_size is None:
            raise TypeError("local_rank and local_world_size are required")
        self.local_rank_ = int(local_rank)
        self.local_world_size_ = int(local_world_size)
        if not 1 <= self.local_world_size_ <= MAX_WORLD_SIZE:
            raise RuntimeError(f"local_world_size must be in [1, {MAX_WORLD_SIZE}], got "
                               f"{self.local_world_size_}")
        if isinstance(tensor_or_shape, torch.Tensor):
            tensor = tensor_or_shape
            if not tensor.is_cuda:
                raise ValueError("tensor must be a CUDA tensor")
            if not tensor.is_contiguous():
                raise ValueError("tensor must be contiguous")
            self.data_ = tensor
        else:
            if dtype is None:
                raise TypeError("dtype is required when constructing from a shape")
            self.data_ = torch.zeros(tuple(int(s) for s in tensor_or_shape), dtype=dtype,
                                     device=torch.device("cuda", self.local_rank_))
        self._imported: list = []
        self.raw_ptrs_ = self._exchange()

    # ---------------------------------------------------------------------------------
    def _exchange(self) -> List[int]:
        world = self.local_world_size_
        if world == 1:
            return [self.data_.data_ptr()]
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("torch.distributed must be initialised to build a parallel tensor "
                               "over more than one rank")
        if dist.get_world_size() != world:
            raise RuntimeError(f"process group has {dist.get_world_size()} ranks, expected {world}")
        lib = _cabi.load()
        rank = dist.get_rank()
        handle = (ctypes.c_ubyte * 64)()
        offset = ctypes.c_uint64(0)
        with torch.cuda.device(self.data_.device):
            _cabi.check(lib.b2a_ipc_export(ctypes.c_void_p(self.data_.data_ptr()), handle,
                                           ctypes.byref(offset)))
        mine = (bytes(handle), int(offset.value), tuple(self.data_.shape), str(self.data_.dtype))
        gathered: List = [None] * world
        dist.all_gather_object(gathered, mine)
        ptrs: List[int] = []
        for r, (h, off, shape, dt) in enumerate(gathered):
            if shape != mine[2] or dt != mine[3]:
                raise RuntimeError(f"parallel tensor shape/dtype mismatch between rank {rank} "
                                   f"{mine[2:]} and rank {r} {(shape, dt)}")
            if r == rank:
                ptrs.append(self.data_.data_ptr())
                continue
            key = (self.data_.device.index, h)
            entry = _OPENED.get(key)
            if entry is None:
                out = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                with torch.cuda.device(self.data_.device):
                    _cabi.check(lib.b2a_ipc_import(buf, ctypes.c_uint64(0), ctypes.byref(out)))
                entry = [int(out.value), 0]
                _OPENED[key] = entry
            entry[1] += 1
            ptrs.append(entry[0] + off)
            self._imported.append(key)
        return ptrs

    def close(self) -> None:
        """Unmap the peers' buffers (collective use must have finished)."""
        if not self._imported:
            return
        lib = _cabi.load()
        with torch.cuda.device(self.data_.device):
            for key in self._imported:
                entry = _OPENED.get(key)
                if entry is None:
                    continue
                entry[1] -= 1
                if entry[1] == 0:
                    lib.b2a_ipc_close(ctypes.c_void_p(entry[0]), ctypes.c_uint64(0))
                    del _OPENED[key]
        self._imported = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def create_parallel_tensor(tensor: torch.Tensor, *, local_rank: Optional[int] = None,
                           local_world_size: Optional[int] = None) -> TKParallelTensor:
    """Wrap a contiguous local CUDA tensor (reference: min_fa3_op.py:186-206)."""
    local_rank, local_world_size = _resolve_parallel_context(local_rank, local_world_size)
    if not tensor.is_cuda:
        raise ValueError("tensor must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise ValueError("tensor must be contiguous")
    if tensor.device.index != local_rank:
        raise ValueError(
            f"tensor device index ({tensor.device.index}) must match local_rank ({local_rank})"
        )
    return TKParallelTensor(tensor, local_rank=local_rank, local_world_size=local_world_size,
                            multicast=False)


# --------------------------------------------------------------------------------------
# peer -> local copy
# --------------------------------------------------------------------------------------
_TILE_SIDE = 128
_VEC_COLS = 4096


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_base_inputs(inp: TKParallelTensor, src_rank: int, num_blocks: int, op: str) -> None:
    # reference: csrc/parallel/remote_load.cu:280-295
    t = inp.data_
    _check(t.is_cuda, "input must be a CUDA tensor")
    _check(t.is_contiguous(), "input must be contiguous")
    _check(t.numel() > 0, "input must be non-empty")
    _check(t.dim() == 2, f"{op} currently supports 2D tensors only")
    _check(t.dtype == torch.bfloat16, f"{op} currently supports torch.bfloat16 only")
    _check(1 <= inp.local_world_size_ <= MAX_WORLD_SIZE,
           f"{op} currently supports local_world_size in [1, {MAX_WORLD_SIZE}]. "
           f"Got {inp.local_world_size_}")
    _check(0 <= src_rank < inp.local_world_size_,
           f"src_rank must be in [0, local_world_size). Got src_rank={src_rank}, "
           f"local_world_size={inp.local_world_size_}")
    _check(t.numel() <= 2**31 - 1, f"{op} only supports tensors with numel <= INT_MAX. Got {t.numel()}")
    _check(num_blocks > 0, f"{op} requires num_blocks > 0. Got {num_blocks}")
    _check(num_blocks <= 2**31 - 1, f"{op} requires num_blocks <= INT_MAX. Got {num_blocks}")


def _check_output(output: torch.Tensor, inp: TKParallelTensor) -> None:
    _check(output.device == inp.data_.device, "output must be on the same device as the local input shard")
    _check(output.shape == inp.data_.shape, "output must have the same shape as input")
    _check(output.dtype == inp.data_.dtype, "output must have the same dtype as input")


def _remote_load(inp: TKParallelTensor, src_rank: int, output: Optional[torch.Tensor],
                 num_blocks: int) -> torch.Tensor:
    if output is None:
        output = torch.empty_like(inp.data_)
    _check(output.is_contiguous(), "output must be contiguous")
    lib = _cabi.load()
    nbytes = inp.data_.numel() * inp.data_.element_size()
    with torch.cuda.device(inp.data_.device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(inp.data_.device).cuda_stream)
        _cabi.check(lib.b2a_peer_copy(ctypes.c_void_p(output.data_ptr()),
                                      ctypes.c_void_p(inp.raw_ptrs_[src_rank]), nbytes,
                                      int(num_blocks), None, stream))
    return output


def _as_parallel(input_tensor, local_rank, local_world_size) -> TKParallelTensor:
    if isinstance(input_tensor, TKParallelTensor):
        return input_tensor
    return create_parallel_tensor(input_tensor, local_rank=local_rank,
                                  local_world_size=local_world_size)


def parallel_remote_load(input_tensor: Union[torch.Tensor, TKParallelTensor], src_rank: int,
                         output: Optional[torch.Tensor] = None, num_blocks: Optional[int] = None,
                         local_rank: Optional[int] = None, local_world_size: Optional[int] = None
                         ) -> torch.Tensor:
    """Copy ``src_rank``'s copy of a 2-D bf16 parallel tensor (rows, cols multiples of 128) into
    a local tensor (reference: min_fa3_op.py:217-241, remote_load.cu:313-340)."""
    inp = _as_parallel(input_tensor, local_rank, local_world_size)
    if num_blocks is None:
        num_blocks = torch.cuda.get_device_properties(inp.local_rank_).multi_processor_count
    _check_base_inputs(inp, int(src_rank), int(num_blocks), "parallel_remote_load")
    _check(inp.data_.size(0) % _TILE_SIDE == 0,
           f"parallel_remote_load requires rows to be a multiple of {_TILE_SIDE}. Got rows={inp.data_.size(0)}")
    _check(inp.data_.size(1) % _TILE_SIDE == 0,
           f"parallel_remote_load requires cols to be a multiple of {_TILE_SIDE}. Got cols={inp.data_.size(1)}")
    if output is not None:
        _check_output(output, inp)
    return _remote_load(inp, int(src_rank), output, int(num_blocks))


def parallel_remote_load_vec(input_tensor: Union[torch.Tensor, TKParallelTensor], src_rank: int,
                             output: Optional[torch.Tensor] = None, num_blocks: Optional[int] = None,
                             local_rank: Optional[int] = None, local_world_size: Optional[int] = None
                             ) -> torch.Tensor:
    """Row-vector variant: cols must be 4096 (reference: min_fa3_op.py:251-275)."""
    inp = _as_parallel(input_tensor, local_rank, local_world_size)
    if num_blocks is None:
        num_blocks = torch.cuda.get_device_properties(inp.local_rank_).multi_processor_count
    _check_base_inputs(inp, int(src_rank), int(num_blocks), "parallel_remote_load_vec")
    _check(inp.data_.size(1) == _VEC_COLS,
           f"parallel_remote_load_vec currently supports cols={_VEC_COLS} only. Got cols={inp.data_.size(1)}")
    if output is not None:
        _check_output(output, inp)
    return _remote_load(inp, int(src_rank), output, int(num_blocks))
