"""Per-partition node state (node memory / historical embeddings): ``[loc_nums, dim]`` float32 rows plus one
float32 timestamp per row.

Mirrors starrygl/cache/NodeState.py (``DistNodeState`` :8-82, ``HistoryLayerUpdater`` :229-282).  Reads and
writes are single fused kernels: the global->local slot lookup, the row copy and the timestamp copy happen in
one pass (the reference issues three indexing operations).  The state lives in GPU memory, or in pinned host
memory that the kernels address directly (the reference's "UVA" mode).
"""
from typing import List, Optional, Tuple, Union

import torch
from torch import Tensor

from .. import ops
from ..utils.partition_book import DistRouteIndex, PartitionState
from .cache_route import CacheRouteManager, CommPlan


def _compute_device():
    if not torch.cuda.is_available():
        raise RuntimeError("DistNodeState needs a CUDA device: its reads and writes are CUDA kernels")
    return torch.device("cuda", torch.cuda.current_device())


class DistNodeState:
    def __init__(self, state: PartitionState, dim: int, device: Union[str, torch.device] = 'cpu', pinned: bool = True):
        self.state = state
        self.node_mapper = state.node_mapper
        self.loc_nums = self.node_mapper.loc_nums
        self.dim = dim
        self.device = torch.device(device)
        self._alloc()
        self.status = None

    def _alloc(self):
        if self.device.type == 'cpu':
            # host-resident state: pinned, and aliased as device tensors the kernels read over the bus
            self._host = (torch.zeros(self.loc_nums, self.dim, dtype=torch.float32).pin_memory(),
                          torch.zeros(self.loc_nums, dtype=torch.float32).pin_memory())
            self.compute_device = _compute_device()
            self.data = self._host[0]
            self.ts = self._host[1]
            self._d_data, self._d_ts = self.data, self.ts   # pinned: the kernels address them in place
        else:
            self.compute_device = self.device
            self.data = torch.zeros(self.loc_nums, self.dim, dtype=torch.float32, device=self.device)
            self.ts = torch.zeros(self.loc_nums, dtype=torch.float32, device=self.device)
            self._d_data, self._d_ts = self.data, self.ts

    def _status(self):
        if self.status is None:
            self.status = ops.StatusWord(self.compute_device)
        return self.status

    def _ids_and_map(self, key):
        m = self.node_mapper
        raw = m.raw_ids(key, self.compute_device)
        if m.mode == 'offset':
            raw = raw - m.offset
        return raw.contiguous(), (m.g2l_map(self.compute_device) if m.mode == 'map' else None)

    def __getitem__(self, key: Union[Tensor, DistRouteIndex]) -> Tuple[Tensor, Tensor]:
        """(rows, timestamps) of the given global ids, on the GPU."""
        ids, g2l = self._ids_and_map(key)
        return ops.gather_rows(self._d_data, ids, map=g2l, ts_table=self._d_ts, status=self._status())

    def update(self, gids: Tensor, values: Tensor, ts: Optional[Tensor] = None):
        """Write rows (and timestamps) of the ids that are stored here; ids without a local slot are skipped."""
        ids, g2l = self._ids_and_map(gids)
        if ids.numel() == 0:
            return
        values = values.to(self.compute_device, torch.float32).contiguous()
        if ts is not None:
            ts = ts.to(self.compute_device, torch.float32).reshape(-1).contiguous()
        ops.scatter_rows(self._d_data, ids, values, map=g2l, ts_table=self._d_ts if ts is not None else None, ts=ts,
                         status=self._status())

    def write_packed(self, local_rows: Tensor, packed: Tensor):
        """rows ``packed[:, :-1]`` -> data[local_rows], ``packed[:, -1]`` -> ts[local_rows] in one kernel."""
        if local_rows.numel():
            ops.scatter_rows(self._d_data, local_rows.to(self.compute_device), packed.contiguous(), ts_table=self._d_ts,
                             split_last_col=True, status=self._status())

    def write_wire(self, wire: Tensor, width: int):
        """Apply received route rows ``[row | ts | slot]`` (the receive side of the cache route) in one kernel."""
        ops.route_unpack(wire, width, self._d_data, self._d_ts if width == self.dim + 1 else None, status=self._status())

    def to(self, device: Union[str, torch.device]):
        new_device = torch.device(device)
        if new_device != self.device:
            old_data, old_ts = self.data, self.ts
            self.device = new_device
            self._alloc()
            self.data.copy_(old_data)
            self.ts.copy_(old_ts)
        return self

    def reset(self):
        self.data.fill_(0)
        self.ts.fill_(0)

    def prefetch(self, gids: Tensor, stream: Optional[torch.cuda.Stream] = None):
        if stream is None:
            return self[gids]
        with torch.cuda.stream(stream):
            return self[gids]


class HistoryLayerUpdater:
    """Per-layer history stores plus the owner -> replica broadcast of freshly computed rows."""

    def __init__(self, node_states: List[DistNodeState]):
        self.node_states = node_states
        self.task = None

    def update(self, layer_idx: int, nids: torch.Tensor, feats: torch.Tensor, ts: torch.Tensor):
        if layer_idx < len(self.node_states):
            self.node_states[layer_idx].update(nids, feats, ts)

    def __call__(self, layer_idx, nids, feats, ts):
        self.update(layer_idx, nids, feats, ts)

    def update_embedding_and_broadcast(self, layer_idx: int, updated_emb: torch.Tensor, updated_ts: torch.Tensor,
                                       plan: CommPlan, indices: torch.Tensor) -> list:
        """1. write the rows locally; 2. send them (embedding || ts) to every rank holding a replica.  The remote
        writes are applied when the returned futures are waited on (at the latest by the next call)."""
        assert layer_idx < len(self.node_states), "Layer index out of range"
        if self.task is not None:
            for t in self.task:
                t.wait()
            self.task = None
        if plan is None or plan.is_empty():
            return []
        target_state = self.node_states[layer_idx]
        target_state.update(indices, updated_emb, updated_ts)

        def remote_write_callback(recv_indices, recv_data, mode):
            target_state.write_packed(recv_indices, recv_data)
        remote_write_callback.fused_state = target_state   # lets the future apply the wire rows in one kernel

        manager = CacheRouteManager.get_instance()
        futures = manager.update_with_plan(local_features=updated_emb, plan=plan, write_callback=remote_write_callback,
                                           local_ts=updated_ts.reshape(-1))
        self.task = futures
        return futures
