"""Variable-size all-to-all of rows between the ranks of a group -- the one exchange step every route form uses.

Two transports behind one call:

* GPU ranks on the default NCCL group: the library's own communicator (``sgl_route_exchange``: grouped
  ``ncclSend`` / ``ncclRecv`` enqueued on the CURRENT stream by one foreign call; nothing to wait for on the host, the
  result is ordered by the stream).  Rows of any dtype travel as 32-bit words.
* anything else (CPU ranks on gloo, sub-groups): ``torch.distributed.all_to_all_single``.

The reference keeps a private ``ncclComm_t`` next to torch.distributed in the same way
(starrygl/utils/context.py:109-122, csrc/include/starrygl/commContext.cu.hpp:85-174).
"""
import ctypes as C
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _C


class NativeComm:
    """The library's NCCL communicator over all ranks of the default process group.  The unique id travels through the
    process group that already exists."""
    _instance: Optional["NativeComm"] = None

    def __init__(self, handle=None, rank=None, world=None):
        L = _C.lib()
        if handle is not None:                       # adopt a communicator somebody else created (DistContext)
            self.handle, self.rank, self.world, self._owned = handle, rank, world, False
            return
        rank, world = dist.get_rank(), dist.get_world_size()
        buf = C.create_string_buffer(128)
        if rank == 0:
            _C.check(L.sgl_comm_unique_id(buf, 128))
        box = [buf.raw]
        dist.broadcast_object_list(box, src=0)
        self.handle = C.c_void_p()
        _C.check(L.sgl_comm_init(C.byref(self.handle), rank, world, box[0]))
        self.rank, self.world, self._owned = rank, world, True

    @classmethod
    def get(cls) -> "NativeComm":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    @classmethod
    def adopt(cls, handle, rank: int, world: int):
        """Use an existing communicator (one made through ``DistContext``) for the routes of this process."""
        if cls._instance is None:
            cls._instance = cls(handle, rank, world)
        return cls._instance

    @classmethod
    def shutdown(cls):
        if cls._instance is not None:
            if cls._instance._owned:
                _C.lib().sgl_comm_destroy(cls._instance.handle)
            cls._instance = None


def use_native(t: torch.Tensor, group) -> bool:
    return (t.is_cuda and dist.is_initialized() and group in (None, dist.GroupMember.WORLD)
            and dist.get_backend() == "nccl")


class _Done:
    """Handle of an exchange that is ordered by the stream it was enqueued on: nothing to wait for."""

    def wait(self):
        return True


def _row_words(t: torch.Tensor) -> int:
    per_row = t.element_size()
    for d in t.shape[1:]:
        per_row *= int(d)
    if per_row % 4:
        raise _C.SglError(f"rows of {per_row} bytes cannot travel as 32-bit words (pad the row to a multiple of 4 bytes)")
    return per_row // 4


def exchange_rows(send: torch.Tensor, send_sizes: Sequence[int], recv: torch.Tensor, recv_sizes: Sequence[int], group=None):
    """Segment p of ``send`` (``send_sizes[p]`` rows) goes to rank p; segment q of ``recv`` arrives from rank q.
    Returns a handle whose ``wait()`` completes the exchange (a no-op for the stream-ordered native transport).
    ``send`` and ``recv`` must be contiguous and of equal row shape and dtype."""
    if not (send.is_contiguous() and recv.is_contiguous()):
        raise _C.SglError("exchange_rows needs contiguous buffers")
    if use_native(send, group):
        comm = NativeComm.get()
        if len(send_sizes) != comm.world or len(recv_sizes) != comm.world:
            raise ValueError(f"split sizes must have one entry per rank ({comm.world})")
        words = _row_words(send if send.dim() > 1 else send.view(-1, 1))
        h_send = (C.c_int64 * comm.world)(*[int(v) for v in send_sizes])
        h_recv = (C.c_int64 * comm.world)(*[int(v) for v in recv_sizes])
        _C.check(_C.lib().sgl_route_exchange(comm.handle, send.data_ptr() if send.numel() else None, h_send,
                                             recv.data_ptr() if recv.numel() else None, h_recv, words, _C.stream_ptr()))
        return _Done()
    world = dist.get_world_size(group)
    if len(send_sizes) != world or len(recv_sizes) != world:
        raise ValueError(f"split sizes must have one entry per rank ({world})")
    return dist.all_to_all_single(recv, send, [int(v) for v in recv_sizes], [int(v) for v in send_sizes], group=group,
                                  async_op=True)


def exchange_counts(send_counts: torch.Tensor, group=None) -> List[int]:
    """Every rank tells every other how many rows it will send; returns the counts this rank will receive (host list:
    they size the receive buffer, so this is the one place a route's set-up synchronises)."""
    send_counts = send_counts.to(torch.int64).contiguous()
    recv = torch.empty_like(send_counts)
    ones = [1] * send_counts.numel()
    exchange_rows(send_counts.view(-1, 1), ones, recv.view(-1, 1), ones, group).wait()
    return [int(v) for v in recv.tolist()]
