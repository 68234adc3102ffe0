"""Id bookkeeping of a partition: packed (partition, local) ids and global->local slot maps.

Mirrors starrygl/utils/partition_book.py of the reference (``DistRouteIndex`` :7-52, ``IDMapper`` :56-176,
``PartitionState`` :179-276).  On CUDA tensors the packing/unpacking runs in the library's kernels; the
global->local lookup itself is fused into the gather / scatter kernels (see ``starrygl.cache.NodeState``), the
``to_local`` method here exists for callers that want the slot tensor itself.
"""
from typing import Optional, Union

import torch
from torch import Tensor

from .. import ops


class DistRouteIndex:
    """64-bit id: bits 0-47 local index, bits 48-61 partition, bit 62 shared flag."""
    PART_SHIFT = 48
    SHARED_BIT = 62
    LOC_MASK = 0xFFFFFFFFFFFF
    PART_MASK = 0x3FFF

    def __init__(self, index: Tensor, part_ids: Optional[Tensor] = None) -> None:
        if part_ids is None:
            self._data = index.long()
        else:
            index = index.long()
            part_ids = part_ids.long().to(index.device)
            if index.is_cuda:
                self._data = ops.dist_pack(index, part_ids)
            else:
                self._data = (index & self.LOC_MASK) | ((part_ids & self.PART_MASK) << self.PART_SHIFT)

    def _unpack(self):
        if self._data.is_cuda:
            return ops.dist_unpack(self._data)
        d = self._data
        return d & self.LOC_MASK, (d >> self.PART_SHIFT) & self.PART_MASK, (d >> self.SHARED_BIT).to(torch.bool)

    @property
    def loc(self) -> Tensor:
        return self._unpack()[0]

    @property
    def part(self) -> Tensor:
        return self._unpack()[1]

    def set_shared(self, indx: Union[slice, Tensor]):
        self._data[indx] |= (1 << self.SHARED_BIT)

    @property
    def is_shared(self) -> Tensor:
        return self._unpack()[2]

    @property
    def dist(self) -> Tensor:
        return self._data

    @property
    def device(self):
        return self._data.device

    @property
    def shape(self):
        return self._data.shape

    def to(self, device):
        return DistRouteIndex(self._data.to(device))


class IDMapper:
    """Local / global / packed id conversion for one entity kind (nodes or edges)."""

    def __init__(self, loc_ids: Tensor, num_master: int, mode: str = 'identity', dist_mapper: Optional[Tensor] = None,
                 replica_table=None, offset: int = 0, global_num: int = 0):
        if mode not in ('identity', 'map', 'offset', 'dist_route_index'):
            raise ValueError(f"unknown id mode {mode!r}")
        self.loc_ids = loc_ids
        self._num_master = num_master
        self.mode = mode
        self.dist_mapper = dist_mapper
        self.offset = offset
        self._replica_table = replica_table
        self._global_num = global_num
        self._g2l_map: Optional[Tensor] = None
        if mode == 'map':
            self.build_g2l_map()

    @property
    def loc_nums(self):
        return self.loc_ids.size(0)

    @property
    def num_master(self):
        return self._num_master

    @property
    def global_nums(self):
        return self._global_num

    @property
    def replica_table(self):
        return self._replica_table

    @property
    def device(self):
        return self.loc_ids.device if self.loc_ids is not None else torch.device('cpu')

    def build_g2l_map(self):
        """Dense global -> local table filled with -1 (only mode 'map'); one-time set-up, not on the batch path."""
        if self.mode == 'map' and self.loc_ids is not None:
            self._g2l_map = torch.full((self.global_nums + 1,), -1, dtype=torch.long, device=self.device)
            self._g2l_map[self.loc_ids] = torch.arange(self.loc_ids.size(0), dtype=torch.long, device=self.device)

    def g2l_map(self, device=None) -> Optional[Tensor]:
        """The slot table on ``device`` (moved once and kept), for fusing the lookup into a gather/scatter."""
        if self._g2l_map is None:
            return None
        if device is not None and self._g2l_map.device != torch.device(device):
            self._g2l_map = self._g2l_map.to(device)
        return self._g2l_map

    def raw_ids(self, gids: Union[Tensor, DistRouteIndex], device=None) -> Tensor:
        """The id the slot computation starts from (low 48 bits for packed ids)."""
        raw = gids
        if isinstance(gids, DistRouteIndex):
            raw = gids.loc
        elif self.mode == 'dist_route_index' and isinstance(gids, Tensor):
            raw = DistRouteIndex(gids).loc
        if device is not None and isinstance(raw, Tensor) and raw.device != torch.device(device):
            raw = raw.to(device)
        return raw

    def to_local(self, gids: Union[Tensor, DistRouteIndex], device: torch.device = None) -> Tensor:
        if device is None:
            device = self.device
        raw = self.raw_ids(gids, device)
        if self.mode == 'offset':
            return raw - self.offset
        if self.mode == 'map':
            if self._g2l_map is None:
                raise RuntimeError("G2L Map not built! Call build_g2l_map() first.")
            m = self._g2l_map
            raw = raw.to(m.device)
            if m.is_cuda:
                return ops.gather_rows(m, raw)
            return m[raw]
        return raw

    def to_dist(self, local_idx: Tensor) -> Tensor:
        if self.dist_mapper is not None:
            return self.dist_mapper[local_idx.to(self.dist_mapper.device)].to(local_idx.device)
        return self.loc_ids.to(local_idx.device)[local_idx]

    def gid_to_dist_route_index(self, local_idx: Tensor) -> DistRouteIndex:
        assert self.dist_mapper is not None, "dist_mapper is required for DistRouteIndex conversion"
        return DistRouteIndex(self.dist_mapper[local_idx.to(self.dist_mapper.device)].to(local_idx.device))

    def get_master_part_by_dist(self, dist_idx: DistRouteIndex) -> Tensor:
        assert isinstance(dist_idx, DistRouteIndex), "dist_idx must be DistRouteIndex"
        return dist_idx.part

    def get_master_part_by_global(self, gid: Tensor) -> Tensor:
        d = self.dist_mapper[gid.to(self.dist_mapper.device)]
        return self.get_master_part_by_dist(DistRouteIndex(d.to(gid.device)))

    def is_master_by_local(self, local_idx: Tensor) -> Tensor:
        return (local_idx >= 0) & (local_idx < self._num_master)

    def is_remote_ids(self, global_idx: Tensor) -> Tensor:
        local_idx = global_idx if self.mode == 'identity' else self.to_local(global_idx, device=global_idx.device)
        return (local_idx < 0) | (local_idx >= self._num_master)

    def is_store_local(self, global_idx: Tensor) -> Tensor:
        local_idx = global_idx if self.mode == 'identity' else self.to_local(global_idx, device=global_idx.device)
        return local_idx >= 0


class PartitionState:
    def __init__(self, loc_ids: Tensor, num_master_nums: int, dist_nid_mapper: Optional[Tensor] = None,
                 node_mode: str = 'identity', node_replica_table=None, loc_eids: Optional[Tensor] = None,
                 num_master_edges: int = 0, dist_eid_mapper: Optional[Tensor] = None, edge_mode: str = 'identity',
                 edge_replica_table=None, num_nodes: int = 0, num_edges: int = 0):
        self.node_mapper = IDMapper(loc_ids=loc_ids, num_master=num_master_nums, mode=node_mode,
                                    dist_mapper=dist_nid_mapper, replica_table=node_replica_table, global_num=num_nodes)
        self.edge_mapper = None
        if loc_eids is not None:
            self.edge_mapper = IDMapper(loc_ids=loc_eids, num_master=num_master_edges, mode=edge_mode,
                                        dist_mapper=dist_eid_mapper, replica_table=edge_replica_table,
                                        global_num=num_edges)

    def build_g2l_maps(self):
        self.node_mapper.build_g2l_map()
        if self.edge_mapper:
            self.edge_mapper.build_g2l_map()

    def to_local_nid(self, gids, device: torch.device = None):
        return self.node_mapper.to_local(gids, device)

    def get_dist_nid(self, local_idx: Tensor):
        return self.node_mapper.to_dist(local_idx)

    def get_node_part_by_dist(self, global_idx: DistRouteIndex):
        return self.node_mapper.get_master_part_by_dist(global_idx)

    def is_master_node_by_local(self, local_idx: Tensor) -> Tensor:
        return self.node_mapper.is_master_by_local(local_idx)

    def is_master_node_by_global(self, gid: Tensor) -> Tensor:
        return self.is_master_node_by_local(self.to_local_nid(gid))

    def _check_edge(self):
        if self.edge_mapper is None:
            raise RuntimeError("Edge data not initialized in PartitionState")

    def to_local_eid(self, gids, device: torch.device = None):
        self._check_edge()
        return self.edge_mapper.to_local(gids, device)

    def get_dist_eid(self, local_idx: Tensor):
        self._check_edge()
        return self.edge_mapper.to_dist(local_idx)

    def get_edge_part_by_dist(self, global_idx: DistRouteIndex):
        self._check_edge()
        return self.edge_mapper.get_master_part_by_dist(global_idx)

    def is_master_edge_by_local(self, local_idx: Tensor) -> Tensor:
        self._check_edge()
        return self.edge_mapper.is_master_by_local(local_idx)
