"""Python graph API of the data path: temporal graph handle, asynchronous sampling, block assembly.

Mirrors starrygl/graph/graph.py of the reference (``NegSamplingSet`` :15-26, ``pyGraph`` :30-136, ``AsyncBlock``
:139-271, ``AsyncGraphBlob`` :274-293).  ``AsyncBlock.to_block`` returns plain index tensors (CSC ``indptr`` /
``indices`` plus the source-side ``nid`` / ``ts`` and edge-side ``eid`` / ``dt``) instead of DGL blocks, and builds them
from device-resident offsets without per-layer ``.item()`` read-backs.
"""
from typing import List, Optional

import torch

from ..lib import libstarrygl_comm as starrygl_ops
from ..utils.context import DistributedContext


class NegSamplingSet:
    def __init__(self, node_set):
        self.node_set = node_set

    def sample(self, num_samples: int, num_groups: int = 1) -> torch.Tensor:
        if isinstance(self.node_set, torch.Tensor):
            return self.node_set[torch.randint(0, len(self.node_set), (num_samples, num_groups),
                                               device=self.node_set.device)]
        raise TypeError("node_set must be a torch.Tensor")


class pyGraph:
    def __init__(self, src: torch.Tensor, dst: torch.Tensor, ts: torch.Tensor, node_num: int, chunk_size: int,
                 eid: torch.Tensor = None, chunk_mapper: Optional[torch.Tensor] = None,
                 weights: Optional[torch.Tensor] = None, add_inverse_edge: bool = False,
                 stream: Optional[torch.cuda.Stream] = None):
        ctx = DistributedContext.get_default_context()
        if eid is None:
            eid = torch.arange(src.size(0), dtype=torch.long, device=ctx.device)
        self.add_inverse_edge = add_inverse_edge
        self.g = starrygl_ops.from_edge_index(node_num, chunk_size, src.to(ctx.device), dst.to(ctx.device),
                                              ts.to(ctx.device), eid.to(ctx.device), chunk_mapper, stream, ctx.local_rank)

    def async_sample(self, time_start: int, time_end: int, chunk_list: torch.Tensor, policy: dict = {},
                     test_generate_kwargs: dict = {}, op: Optional[str] = None):
        """Queue one sampling task for the events in [time_start, time_end); results come back in FIFO order."""
        if not isinstance(chunk_list, torch.Tensor):
            raise TypeError("chunk_list must be a torch.Tensor")
        if not isinstance(policy, dict):
            raise TypeError("policy must be a dict")
        if not isinstance(test_generate_kwargs, dict):
            raise TypeError("test_generate_kwargs must be a dict")
        if op is not None and not isinstance(op, str):
            raise TypeError("op must be a str")
        ctx = DistributedContext.get_default_context()
        empty = torch.tensor([], dtype=torch.long, device=ctx.device)
        neg = test_generate_kwargs.get('test_generate_samples', empty)
        neg_ts = test_generate_kwargs.get('test_generate_samples_ts', empty)
        if policy['sample_type'] == 'cluster':
            return self.g.submit_query(time_start, time_end, chunk_list.to(ctx.device), neg.to(ctx.device),
                                       neg_ts.to(ctx.device), 'cluster', 1, 0, 0, 0, 0, op)
        if 'fanout' not in policy:
            raise ValueError("policy must contain 'fanout' for non-c sampling")
        if 'layers' not in policy:
            raise ValueError("policy must contain 'layers' for non-c sampling")
        return self.g.submit_query(time_start, time_end, chunk_list.to(ctx.device), neg.to(ctx.device),
                                   neg_ts.to(ctx.device), policy['sample_type'], policy['layers'], policy['fanout'],
                                   policy.get('allowed_offset', -1), policy.get('equal_root_time', False),
                                   policy.get('keep_root_time', False), op)

    def get_last_sample(self):
        return self.g.get()

    def slice_by_chunk_ts(self, chunk_list: torch.Tensor, time_begin: float, time_end: float):
        return self.g.slice_by_chunk_ts(chunk_list, time_begin, time_end)

    def sample_src_in_chunks_khop(self, roots, neg_roots, k: int, layers: int, allowed_offset: int = -1,
                                  equal_root_time: bool = False, keep_root_time: bool = False,
                                  sample_type: str = "recent"):
        return self.g.sample_src_in_chunks_khop(roots, neg_roots, k, layers, allowed_offset, equal_root_time,
                                                keep_root_time, sample_type)


class Block:
    """Message-flow block of one hop as plain tensors (CSC over the destination nodes)."""

    def __init__(self, indptr, indices, num_src, num_dst, srcdata, edata):
        self.indptr, self.indices = indptr, indices
        self.num_src_nodes, self.num_dst_nodes = num_src, num_dst
        self.srcdata, self.edata = srcdata, edata


class AsyncBlock:
    def __init__(self, graph: pyGraph, index: int):
        self.graph = graph
        self.index = index

    def value(self):
        return self.graph.get_last_sample()

    @staticmethod
    def to_block(root, neg_roots, neighbors, nid_mapper, self_loop=True, add_inverse_edge=False):
        """Per hop: destination nodes = source nodes of the previous hop (the roots' queries for hop 0); source nodes
        = [destinations (when ``self_loop``)] + the hop's neighbours in sampling order."""
        mfgs = []
        last_nodes = torch.repeat_interleave(root.roots, root.ts_ptr[1:] - root.ts_ptr[:-1]) if root.root_num else root.roots
        last_ts = root.ts
        if neg_roots is not None and neg_roots.root_num:
            last_nodes = torch.cat([last_nodes, neg_roots.roots])
            last_ts = torch.cat([last_ts, neg_roots.ts])
        for nb in neighbors:
            num_dst = nb.root_start_ptr.numel() - 1
            length = num_dst if self_loop else 0
            indptr = nb.root_start_ptr
            indices = torch.arange(nb.neighbor_num, device=indptr.device) + length
            eid = nb.neighbors_eid // 2 if add_inverse_edge else nb.neighbors_eid
            if self_loop:
                src_nid = torch.cat((last_nodes, nb.neighbors))
                src_ts = torch.cat((last_ts, nb.neighbors_ts))
            else:
                src_nid, src_ts = nb.neighbors, nb.neighbors_ts
            b = Block(indptr, indices, length + nb.neighbor_num, num_dst, {"nid": src_nid, "ts": src_ts},
                      {"eid": eid, "dt": nb.neighbors_dt})
            last_nodes, last_ts = nb.neighbors, nb.neighbors_ts   # the next hop queries exactly these
            mfgs.append(b)
        mfgs.reverse()
        return root, neg_roots, mfgs, nid_mapper


class AsyncGraphBlob:
    def __init__(self, graph: pyGraph, time_start: List[int], time_end: List[int], chunk_list: List[torch.Tensor],
                 policy: dict = {}, test_generate_kwargs: dict = {}):
        self.graph = []
        for i in range(len(time_start)):
            graph.async_sample(time_start[i], time_end[i], chunk_list[i], policy=policy,
                               test_generate_kwargs=test_generate_kwargs, op=('f' if i > 0 else 'r'))
            self.graph.append(AsyncBlock(graph, i))
