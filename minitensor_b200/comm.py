"""Gradient exchange for data-parallel training: the ``mtb200_comm_*`` entry points (NCCL all-reduce behind
the C ABI) as a small Python object.

One process drives one GPU.  The 128-byte NCCL id is created on rank 0 and handed to the other ranks through
whatever channel the launcher offers; :meth:`Communicator.from_process_group` uses an initialised
``torch.distributed`` group for that hand-over only - the collectives themselves go through the library.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check

ID_BYTES = 128


class Communicator:
    def __init__(self, world_size: int, rank: int, device: int, unique_id: bytes):
        if len(unique_id) != ID_BYTES:
            raise ValueError(f"the NCCL id is {ID_BYTES} bytes, got {len(unique_id)}")
        self.lib = _lib.load()
        self.world_size, self.rank, self.device = int(world_size), int(rank), int(device)
        h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, ID_BYTES)
        check(self.lib.mtb200_comm_init_rank(self.world_size, self.rank, buf, self.device, C.byref(h)))
        self._h = h
        self._stream = None

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(ID_BYTES)
        check(_lib.load().mtb200_comm_unique_id(buf))
        return buf.raw

    @classmethod
    def from_process_group(cls, device: int) -> "Communicator":
        """Rank, world size and the id hand-over come from the default ``torch.distributed`` group."""
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised: nothing to exchange the NCCL id over")
        rank, world = dist.get_rank(), dist.get_world_size()
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(world, rank, device, box[0])

    def all_reduce_sum(self, t: torch.Tensor, stream: torch.cuda.Stream, scale: float = 1.0) -> None:
        """In place ``t = scale * sum over ranks of t`` (contiguous f32, on this communicator's device), enqueued
        on ``stream``."""
        if t.dtype != torch.float32 or not t.is_contiguous() or not t.is_cuda or t.device.index != self.device:
            raise ValueError("all_reduce_sum takes a contiguous float32 tensor on the communicator's device")
        if self._stream != stream.cuda_stream:
            check(self.lib.mtb200_comm_set_stream(self._h, self.rank, C.c_void_p(stream.cuda_stream)))
            self._stream = stream.cuda_stream
        check(self.lib.mtb200_allreduce_sum_f32(self._h, self.rank, C.c_void_p(t.data_ptr()), t.numel(), float(scale)))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.lib.mtb200_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
