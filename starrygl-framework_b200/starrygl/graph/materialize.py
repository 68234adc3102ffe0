"""Materialised mini-batches: the per-slot files of the reference's offline pipeline, built on the GPU.

``MaterializedMultiLayerBuilder`` has the constructor and the ``build_aligned_batch`` signature of the reference's
class (prepare_sample.py:179-406).  One call builds, for one task slice of one partition, the list of per-layer
dictionaries -- layer 0: ``gids``, ``ts``, ``inv_map``, ``num_neg`` + the task tensors + ``comm_plan``; layer l+1:
``indptr``, ``indices``, ``eid``, ``edge_ts``, ``edge_dt``, ``gids``, ``ts`` -- and writes it with ``torch.save`` in the
layout the reference's loader reads (all tensors on the CPU, ``comm_plan`` = one ``CommPlan`` or ``None`` per layer
list).  Sampling, (node, ts) relabel, CSC and the route plans run through the library
(:func:`starrygl.graph.batch.build_batch_async`, ``sgl_plan_route``); the T-CSR is built once per partition.

Supported policy space = what the GPU sampler implements: continuous graphs (``graph_type == 'c'``), ``recent`` and
``uniform`` layers, ``end_offset`` 0 (strictly earlier edges) or 1 (edges at the query time included; integer
timestamps).  ``cluster`` / ``full`` layers and discrete graphs raise ``NotImplementedError``.  Negative destinations
of a ``'neg'`` task are drawn from a seeded torch generator (the reference draws from the unseeded global numpy state).
"""
from typing import List, Optional

import numpy as np
import torch

from .. import _C, ops
from ..cache.cache_route import CommPlan
from .batch import build_batch_async


def _dev_i64(x, dev):
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(np.ascontiguousarray(x))
    return x.to(dev, torch.int64).contiguous()


def prepare_distributed_metadata(node_parts, edge_index, num_parts: int, output_dir=None):
    """Partition book and replica table of a partitioned graph, in the reference's file layout
    (``prepare_distributed_metadata``, prepare_nparts_louvain.py:457-484).

    An event belongs to the partition of its destination.  ``partition_book[p]`` = the nodes partition p stores: the ones
    it owns (ascending id) followed by its halo -- sources of its events that another partition owns (ascending id).
    ``partition_book.pt`` holds ``(partition_book, node_parts, edge_parts)``, ``replica_table.pt`` the CSR over node id of
    every ``(rank, local slot)`` copy.  One-time set-up on whatever device the inputs live on; the files hold CPU tensors.
    Returns ``(partition_book, replica_table)``."""
    import os

    from ..cache.replica_table import build_replica_table
    node_parts = torch.as_tensor(node_parts, dtype=torch.int64)
    src, dst = (torch.as_tensor(x, dtype=torch.int64).to(node_parts.device) for x in edge_index)
    edge_parts = node_parts[dst]
    src_parts = node_parts[src]
    book = []
    for pid in range(int(num_parts)):
        owned = torch.nonzero(node_parts == pid, as_tuple=True)[0]
        halo = torch.unique(src[(edge_parts == pid) & (src_parts != pid)])
        book.append(torch.cat([owned, halo]).cpu())
    table = build_replica_table(node_parts.numel(), book, int(num_parts))
    if output_dir is not None:
        os.makedirs(output_dir, exist_ok=True)
        torch.save((book, node_parts.cpu(), edge_parts.cpu()), os.path.join(output_dir, "partition_book.pt"))
        torch.save(table, os.path.join(output_dir, "replica_table.pt"))
    return book, table


class MaterializedMultiLayerBuilder:
    def __init__(self, partition_data, num_nodes, node_parts, rep_table, pid, num_parts, device=None):
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if dev.type != "cuda":
            raise _C.SglError("MaterializedMultiLayerBuilder: the data path has no CPU implementation")
        self.device = dev
        src, dst, ts = (_dev_i64(partition_data[k], dev) for k in ("src", "dst", "ts"))
        eid = _dev_i64(partition_data["eid"], dev) if "eid" in partition_data else None
        if "cid" in partition_data and np.any(np.asarray(partition_data["cid"]) != 0):
            raise NotImplementedError("cluster ids: 'cluster' layers are not implemented on the GPU path")
        self.num_nodes = int(num_nodes)
        # rows keyed by the destination of an event, neighbour = its source, ascending time (prepare_sample.py:192-203)
        self.g = ops.tcsr_build(dst, src, ts, eid, self.num_nodes)
        self.node_parts = None if node_parts is None else _dev_i64(node_parts, dev)
        self.rep_table = None if rep_table is None else rep_table.to(dev)
        self.pid, self.num_parts = int(pid), int(num_parts)
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(0)

    # ---- route plan of one layer list (prepare_sample.py:266-310) ------------------------------------------------
    def _plan_async(self, layer_ids, d_n, status):
        if self.rep_table is None or self.node_parts is None or self.num_parts <= 1:
            return None
        cap = max(layer_ids.numel() * max(self.num_parts - 1, 1), 1)
        rt = self.rep_table
        return ops.plan_route(layer_ids, self.node_parts, self.pid, rt.indptr, rt.indices, rt.locs, self.num_parts, cap,
                              d_n=d_n, status=status)

    @staticmethod
    def _plan_finish(p) -> Optional[CommPlan]:
        if p is None:
            return None
        ranks, rows, locs, sizes, total = p
        n = int(total.item())
        if n == 0:
            return None
        return CommPlan(send_ranks=ranks[:n].cpu(), send_sizes=sizes.cpu(), send_indices=rows[:n].cpu(),
                        send_remote_indices=locs[:n].cpu())

    # ---- one slot ------------------------------------------------------------------------------------------------
    def build_aligned_batch(self, task_param, save_path, layer_configs, num_neg=1, global_dst_pool=None, cluster_ids=None,
                            seed: Optional[int] = None) -> List[dict]:
        task_type, task_nodes = task_param
        dev = self.device
        extra = {}
        if task_type == 'link':
            task_src, task_dst, task_ts, task_label, task_eid = task_nodes
            l0_nodes = torch.cat([_dev_i64(task_src, dev), _dev_i64(task_dst, dev)])
            t = _dev_i64(task_ts, dev)
            l0_ts = torch.cat([t, t])
            extra = {"task_ts": task_ts, "task_src": task_src, "task_dst": task_dst, "task_label": task_label,
                     "task_eid": task_eid}
        elif task_type == 'node':
            task_node, task_ts, task_label = task_nodes
            l0_nodes, l0_ts = _dev_i64(task_node, dev), _dev_i64(task_ts, dev)
            extra = {"task_node": task_node, "task_ts": task_ts, "task_label": task_label}
        elif task_type == 'neg':
            if num_neg <= 0 or global_dst_pool is None:
                raise ValueError("a 'neg' task needs num_neg > 0 and a destination pool")
            task_ts = task_nodes
            pool = torch.as_tensor(np.asarray(global_dst_pool), dtype=torch.int64)
            if seed is not None:
                self.gen.manual_seed(int(seed))
            pick = torch.randint(0, pool.numel(), (len(task_ts) * num_neg,), generator=self.gen)
            neg = pool[pick]
            l0_nodes = neg.to(dev)
            l0_ts = _dev_i64(task_ts, dev).repeat_interleave(num_neg)
            extra = {"task_nodes": neg, "task_ts": task_ts, "task_label": 'neg_set'}
        else:
            raise ValueError(f"Unsupported task type: {task_type}")

        meta = layer_configs.get('meta', {})
        if meta.get('graph_type', 'c') != 'c':
            raise NotImplementedError("discrete graphs (graph_type != 'c') are not implemented on the GPU path")
        end_offset = int(meta.get('end_offset', 0))
        if end_offset not in (0, 1):
            raise NotImplementedError("end_offset must be 0 (edges strictly before the query time) or 1 (inclusive)")
        kinds = {c['type'] for c in layer_configs['layer']}
        if not kinds <= {'recent', 'uniform'}:
            raise NotImplementedError(f"layer types {sorted(kinds - {'recent', 'uniform'})} are not implemented on the GPU path")
        if len(kinds) > 1:
            raise NotImplementedError("all layers of a batch use one policy")
        policy = kinds.pop() if kinds else 'recent'
        fanouts = [int(c['fanout']) for c in layer_configs['layer']]

        status = ops.StatusWord(dev)
        db = build_batch_async(self.g, l0_nodes, l0_ts, fanouts, policy, equal_root_time=bool(end_offset),
                               seed=0 if seed is None else int(seed), status=status)
        # plans of every layer list, enqueued behind the builder without a host round trip
        plans = [self._plan_async(db.layers[0]["gids"], db.counts[0], status)]
        for l in range(len(fanouts)):
            plans.append(self._plan_async(db.layers[l + 1]["gids"], db.counts[2 + 2 * l], status))
        layers = db.finish()                      # the one synchronisation of the slot
        routes = [self._plan_finish(p) for p in plans[:len(layers)]]
        if len(layers) >= 2 and layers[-1]["indptr"].numel() == 1:
            routes[-1] = None                     # the reference stops at an empty layer with no plan for it

        def host(x):
            if isinstance(x, np.ndarray):
                return torch.from_numpy(x)
            return x.cpu() if torch.is_tensor(x) else x
        final = [{k: host(v) for k, v in d.items()} for d in layers]
        final[0]["num_neg"] = num_neg
        final[0].update({k: host(v) for k, v in extra.items()})
        final[0]['comm_plan'] = routes
        if save_path is not None:
            torch.save(final, save_path)
        return final
