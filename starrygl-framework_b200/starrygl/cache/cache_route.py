"""Owner -> replica push of node rows between graph partitions (the "cache route").

Mirrors starrygl/cache/cache_route.py (``CommPlan`` :121-166, ``CacheUpdateFuture`` :172-198,
``CacheRoute.update_with_plan`` :211-277, ``CacheRouteManager`` :426-432) with a different wire format:
the reference sends three collectives per call (counts, write slots, rows) around two host synchronisations
and separate gather / scatter passes.  Here one kernel packs ``[row | ts | write slot]`` straight into the
send buffer (grouped by destination rank because the plan's ``send_indices`` are), ONE variable-size
all-to-all moves it over NCCL, and one kernel on the receiver scatters rows and timestamps to their slots.
The receive counts are exchanged once per plan and cached on it (``CommPlan.recv_sizes``), so a plan that is
reused -- or that was saved with its receive counts -- costs no host synchronisation at all.
"""
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _C, ops
from ..route.exchange import NativeComm, exchange_counts, exchange_rows, use_native

__all__ = ['CommPlan', 'CacheUpdateFuture', 'CacheRoute', 'CacheRouteManager', 'compute_layer_route']


@dataclass
class CommPlan:
    """What this rank sends during one slot: for every row the destination rank (sorted), the local row to
    read and the slot to write on the receiver."""
    send_ranks: torch.Tensor           # [S] destination rank of every row, ascending
    send_sizes: torch.Tensor           # [P] rows per destination rank
    send_indices: torch.Tensor         # [S] local row to read
    send_remote_indices: torch.Tensor  # [S] slot to write on the receiver
    recv_sizes: Optional[List[int]] = field(default=None, compare=False)   # [P] rows arriving per source rank
    _send_list: Optional[List[int]] = field(default=None, compare=False, repr=False)

    def __repr__(self):
        if self.is_empty():
            return "CommPlan(Empty)"
        return f"CommPlan(send={self.send_indices.numel()} items -> {int(torch.count_nonzero(self.send_sizes))} parts)"

    def is_empty(self) -> bool:
        return self.send_indices.numel() == 0

    def send_list(self) -> List[int]:
        if self._send_list is None:
            self._send_list = [int(v) for v in self.send_sizes.tolist()]
        return self._send_list

    def to(self, device: torch.device, non_blocking: bool = False):
        self.send_list()   # keep the host copy of the split sizes before the tensor leaves the host
        self.send_ranks = self.send_ranks.to(device, non_blocking=non_blocking)
        self.send_sizes = self.send_sizes.to(device, non_blocking=non_blocking)
        self.send_indices = self.send_indices.to(device, non_blocking=non_blocking)
        self.send_remote_indices = self.send_remote_indices.to(device, non_blocking=non_blocking)
        return self

    def pin_memory(self):
        self.send_ranks = self.send_ranks.pin_memory()
        self.send_sizes = self.send_sizes.pin_memory()
        self.send_indices = self.send_indices.pin_memory()
        self.send_remote_indices = self.send_remote_indices.pin_memory()
        return self

    @classmethod
    def empty(cls, num_parts: int):
        """A plan that sends nothing.  ``num_parts`` (the number of ranks) is required: the plan still takes part in
        the exchange, and a ``send_sizes`` of another length than its peers' would never match their collective."""
        if int(num_parts) < 1:
            raise ValueError("CommPlan.empty needs the number of ranks (num_parts >= 1)")
        return cls(send_ranks=torch.empty(0, dtype=torch.long), send_sizes=torch.zeros(int(num_parts), dtype=torch.long),
                   send_indices=torch.empty(0, dtype=torch.long), send_remote_indices=torch.empty(0, dtype=torch.long))


def compute_layer_route(layer_ids: Tensor, node_parts: Tensor, pid: int, replica_table, num_parts: int,
                        max_replicas_per_node: int = 0) -> Optional["CommPlan"]:
    """Build the plan of one layer on the GPU (reference: ``_compute_layer_route``, prepare_sample.py:266-310): the rows of
    nodes owned by partition ``pid`` -- for every node the row with its latest timestamp -- go to every other rank that
    holds a replica.  ``layer_ids`` is the layer's node-id list in (id, ts) order (what the batch builder returns);
    ``replica_table`` a ``CSRReplicaTable`` on the same GPU.  Returns ``None`` when nothing has to be sent (as the
    reference does); the receive sizes are not known yet and are exchanged on first use of the plan."""
    if not layer_ids.is_cuda:
        raise RuntimeError("compute_layer_route runs on the GPU")
    if max_replicas_per_node <= 0:
        max_replicas_per_node = max(num_parts - 1, 1)
    cap = layer_ids.numel() * max_replicas_per_node
    st = ops.StatusWord(layer_ids.device)
    ranks, rows, locs, sizes, total = ops.plan_route(layer_ids, node_parts.to(layer_ids.device), pid, replica_table.indptr,
                                                     replica_table.indices, replica_table.locs, num_parts, cap, status=st)
    n = int(total.item())
    st.check("compute_layer_route")
    if n == 0:
        return None
    return CommPlan(send_ranks=ranks[:n], send_sizes=sizes, send_indices=rows[:n], send_remote_indices=locs[:n])


class CacheUpdateFuture:
    """Handle of one push; ``wait()`` completes the collective and applies the remote writes."""

    def __init__(self, works, recv_ids: Optional[Tensor], recv_feats: Tensor, write_callback: Callable, mode: str,
                 width: int = 0):
        self.works = works
        self.recv_ids = recv_ids
        self.recv_feats = recv_feats
        self.write_callback = write_callback
        self.mode = mode
        self._width = width
        self._done = False

    def wait(self):
        if self._done:
            return
        self._done = True
        for work in self.works:
            if work is not None:
                work.wait()
        if self.recv_feats.shape[0] == 0:
            return
        if self.recv_ids is None:
            # wire rows are [payload(width) | slot as two 32-bit words]
            w = self._width
            state = getattr(self.write_callback, "fused_state", None)
            if state is not None:   # one kernel: slot decode + row scatter + timestamp scatter
                state.write_wire(self.recv_feats, w)
                return
            self.recv_ids = ops.wire_slots(self.recv_feats, w)
            self.recv_feats = self.recv_feats[:, :w]
        self.write_callback(self.recv_ids, self.recv_feats, self.mode)


class _NativeBinding:
    """Everything of one (plan, feature width) pair that does not change from call to call: device copies of the
    index arrays, host split arrays, send / receive buffers and the pre-converted argument list."""

    def __init__(self, plan: "CommPlan", recv_list, feats: Tensor, has_ts: bool, comm: NativeComm):
        import ctypes as C
        dev = feats.device
        self.send_idx = plan.send_indices.to(dev, torch.int64).contiguous()
        self.remote = plan.send_remote_indices.to(dev, torch.int64).contiguous()
        P = comm.world
        self.h_send = (C.c_int64 * P)(*plan.send_list())
        self.h_recv = (C.c_int64 * P)(*recv_list)
        self.dim = feats.shape[1]
        self.width = self.dim + (1 if has_ts else 0)
        self.n_send, self.n_recv = sum(plan.send_list()), sum(recv_list)
        pitch = ops.wire_pitch(self.width, False)
        self.send_buf = torch.empty(max(self.n_send, 1), pitch, dtype=torch.float32, device=dev)
        self.recv_buf = torch.empty(max(self.n_recv, 1), pitch, dtype=torch.float32, device=dev)
        self.status = ops.StatusWord(dev)


class CacheRoute:
    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def _use_native(self, t: Tensor) -> bool:
        return use_native(t, self.group)

    def _update_native(self, feats, plan, write_callback, local_ts):
        """GPU ranks on the default NCCL group: pack, grouped send/recv and (inside ``wait``) unpack are issued by the
        library on the current stream -- one foreign call to send, one to apply, no torch collective, no host sync."""
        comm = NativeComm.get()
        recv_list = self._exchange_counts(plan, feats.device)
        key = (feats.shape[1], local_ts is not None, feats.device)
        cache = plan.__dict__.setdefault("_native", {})
        b = cache.get(key)
        if b is None:
            b = cache[key] = _NativeBinding(plan, recv_list, feats, local_ts is not None, comm)
        L = _C.lib()
        ts = None if local_ts is None else local_ts.to(torch.float32).contiguous()
        rc = L.sgl_cache_route_step(comm.handle, feats.data_ptr(), feats.shape[0], b.dim, _C.ptr(ts), b.send_idx.data_ptr(),
                                    b.remote.data_ptr(), b.h_send, b.h_recv, b.send_buf.data_ptr(), b.recv_buf.data_ptr(),
                                    None, 0, None, 0, b.status.ptr(), _C.stream_ptr())
        _C.check(rc)
        fut = CacheUpdateFuture([], None, b.recv_buf[:b.n_recv], write_callback, 'cold', b.width)
        fut._keep = (feats, ts)     # inputs of kernels that may still be queued
        return [fut]

    def _exchange_counts(self, plan: CommPlan, device) -> List[int]:
        if plan.recv_sizes is None:
            # checked on the host BEFORE the collective: ranks whose split arrays differ in length would wait for each
            # other forever inside it
            if plan.send_sizes.numel() != self.world_size:
                raise ValueError(f"CommPlan.send_sizes has {plan.send_sizes.numel()} entries, the group has "
                                 f"{self.world_size} ranks (an empty plan must be built with CommPlan.empty(world_size))")
            if int(plan.send_sizes.sum()) != plan.send_indices.numel():
                raise ValueError("CommPlan.send_sizes does not add up to the number of send_indices")
            plan.recv_sizes = exchange_counts(plan.send_sizes.to(device), self.group)
        return plan.recv_sizes

    @torch.no_grad()
    def update_with_plan(self, local_features: Tensor, plan: CommPlan, write_callback: Callable,
                         slice_size: int = 0, local_ts: Optional[Tensor] = None) -> List[CacheUpdateFuture]:
        """Push ``local_features[plan.send_indices]`` (optionally with ``local_ts`` appended as last column) to the
        ranks of the plan.  ``write_callback(slots, rows, mode)`` runs on the receiver inside ``wait()``.
        ``slice_size`` is accepted for compatibility; the single packed message makes column slicing unnecessary.
        Every rank of the group must call this (an empty plan still takes part in the exchange)."""
        device = local_features.device
        feats = local_features.contiguous()
        if self._use_native(feats) and feats.dtype == torch.float32:
            return self._update_native(feats, plan, write_callback, local_ts)
        width = feats.shape[1] + (1 if local_ts is not None else 0)
        recv_list = self._exchange_counts(plan, device)
        send_list = plan.send_list()
        send_idx = plan.send_indices.to(device)
        remote = plan.send_remote_indices.to(device)
        packed = ops.route_pack(feats, local_ts, send_idx, remote_idx=remote)          # [S, wire pitch]
        recv = torch.empty(sum(recv_list), ops.wire_pitch(width, False), dtype=torch.float32, device=device)
        work = exchange_rows(packed, send_list, recv, recv_list, self.group)
        fut = CacheUpdateFuture([work], None, recv, write_callback, 'cold', width)
        fut._keep = packed
        return [fut]


class CacheRouteManager:
    _instance = None

    @classmethod
    def get_instance(cls, group: Optional[dist.ProcessGroup] = None) -> CacheRoute:
        if cls._instance is None:
            cls._instance = CacheRoute(group)
        return cls._instance

    @classmethod
    def reset(cls):
        cls._instance = None
