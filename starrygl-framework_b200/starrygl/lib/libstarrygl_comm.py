"""Python-visible surface of the native sampler module.

Same names and call signatures as the reference's pybind module ``libstarrygl_comm``
(csrc/srcs/starrygl/export.cu:20-254): ``from_edge_index``, ``CUDAGraph`` with ``submit_query`` / ``get`` /
``get_seeds_in_chunks`` / ``get_negative_root`` / ``sample_src_in_chunks_khop``, and the result types
``TemporalRoot``, ``NegativeRoot``, ``TemporalNeighbor``, ``TemporalResult``.  The work is done by libsgl_b200.so
through its C ABI; result attributes are the tensors the kernels wrote (no second device copy per attribute
read, unlike export.cu:28-185).

Semantics (where the reference's CUDA code is ill-defined, the CPU sampler's rule is used):
candidates of a query (node, t) are the node's out-edges with ts < t (ts <= t with ``equal_root_time``; and
ts >= t - allowed_offset when ``allowed_offset`` >= 0); "recent" keeps the last k in ascending time, "uniform"
k distinct ones in ascending position; ``neighbors_dt`` = ts - t as int64; hop l+1 queries every neighbour of
hop l at the time of the edge that reached it (or at the root's time with ``keep_root_time``).
"""
import queue
import threading
from typing import List, Optional

import torch

from .. import ops
from .. import _C


def _empty(dev):
    return torch.empty(0, dtype=torch.int64, device=dev)


class TemporalRoot:
    """Roots of a batch: ``roots[r]`` has query times ``ts[ts_ptr[r]:ts_ptr[r+1]]``; query q is backed by the events
    ``q_eid[q_ptr[q]:q_ptr[q+1]]``."""

    def __init__(self, roots, ts_ptr, ts, q_ptr=None, q_eid=None):
        dev = roots.device
        self.roots, self.ts_ptr, self.ts = roots, ts_ptr, ts
        self.q_ptr = q_ptr if q_ptr is not None else _empty(dev)
        self.q_eid = q_eid if q_eid is not None else _empty(dev)

    @property
    def root_num(self):
        return self.roots.numel()

    @property
    def root_ts_num(self):
        return self.ts.numel()

    def __repr__(self):
        return f"<TemporalRoot with {self.root_num} roots>"


class NegativeRoot:
    def __init__(self, roots, ts):
        self.roots, self.ts = roots, ts

    @property
    def root_num(self):
        return self.roots.numel()

    def __repr__(self):
        return f"<NegativeRoot with {self.root_num} roots>"


class TemporalNeighbor:
    """One hop: query q owns ``neighbors[root_start_ptr[q]:root_end_ptr[q]]`` (``root_start_ptr`` is the full
    exclusive prefix with one extra entry, ``root_end_ptr`` its shift by one)."""

    def __init__(self, hop: ops.Hop):
        n = hop.total()
        self.root_start_ptr = hop.offsets
        self.root_end_ptr = torch.cat([hop.offsets[1:], hop.offsets[-1:]])
        self.neighbors = hop.nbr[:n]
        self.neighbors_ts = hop.ts[:n]
        self.neighbors_eid = hop.eid[:n]
        self.neighbors_dt = hop.dt_i64[:n]
        self.neighbor_num = n

    @classmethod
    def from_arrays(cls, start_ptr, neighbors, neighbors_ts, neighbors_eid):
        """Layer given directly by its CSR arrays (``start_ptr`` with one extra entry)."""
        self = cls.__new__(cls)
        self.root_start_ptr = start_ptr
        self.root_end_ptr = torch.cat([start_ptr[1:], start_ptr[-1:]])
        self.neighbors, self.neighbors_ts, self.neighbors_eid = neighbors, neighbors_ts, neighbors_eid
        self.neighbors_dt = torch.zeros_like(neighbors_ts)
        self.neighbor_num = neighbors.numel()
        return self

    @property
    def start_ptr(self):   # name used by the reference's block builder (starrygl/graph/graph.py:174)
        return self.root_start_ptr

    def __repr__(self):
        return f"<TemporalNeighbor with {self.neighbor_num} neighbors>"


class TemporalResult:
    def __init__(self, roots: TemporalRoot, neg_roots: Optional[NegativeRoot] = None):
        self.roots = roots
        self.neg_roots = neg_roots
        self.neighbors_list: List[TemporalNeighbor] = []
        self.nodes_remapper_id = _empty(roots.roots.device)

    @property
    def neighbors(self):
        return self.neighbors_list

    def __repr__(self):
        return f"<TemporalResult with {len(self.neighbors_list)} neighbor layers>"


class CUDAGraph:
    """Temporal graph on one GPU + an asynchronous sampling worker (one thread, FIFO results)."""

    def __init__(self, g: ops.TCSR, ev, chunk_size, mapper, stream, rank):
        self.g = g
        self.ev = ev                      # events in time order: (src, ts, eid)
        self.chunk_size, self.mapper, self.rank = chunk_size, mapper, rank
        self.stream = stream
        self.status = ops.StatusWord(g.device)
        self.relabel = ops.NodeRelabeler(g.num_nodes, g.device)
        self._tasks = queue.Queue()
        self._results = queue.Queue()
        self._closed = False
        self._worker = threading.Thread(target=self._run, daemon=True)
        self._worker.start()

    # ---- synchronous entry points -----------------------------------------------------------------------
    def get_negative_root(self, negative_root: torch.Tensor, negative_time: torch.Tensor) -> NegativeRoot:
        return NegativeRoot(negative_root.to(self.g.device, torch.int64), negative_time.to(self.g.device, torch.int64))

    def get_seeds_in_chunks(self, chunks: torch.Tensor, time_begin: int, time_end: int,
                            using_full_timestamp: bool = False) -> TemporalRoot:
        if using_full_timestamp:
            raise NotImplementedError("dense per-timestep roots (using_full_timestamp) are not provided")
        with torch.cuda.stream(self.stream):
            r = ops.seeds_in_window(self.ev, self.g, chunks, self.mapper, int(time_begin), int(time_end),
                                    status=self.status)
        return TemporalRoot(*r)

    def sample_src_in_chunks_khop(self, postive_root: TemporalRoot, negative_root: Optional[NegativeRoot], k: int,
                                  layers: int, allowed_offset: int, equal_root_time: bool, keep_root_time: bool,
                                  sample_type: str) -> TemporalResult:
        if sample_type not in ("recent", "uniform"):
            raise RuntimeError("undefined sampling strategy")
        dev = self.g.device
        with torch.cuda.stream(self.stream):
            # one query per (root, timestamp) of the positive roots, then one per negative root
            reps = postive_root.ts_ptr[1:] - postive_root.ts_ptr[:-1] if postive_root.root_num else _empty(dev)
            q_nodes = torch.repeat_interleave(postive_root.roots, reps) if postive_root.root_num else _empty(dev)
            q_ts = postive_root.ts
            if negative_root is not None and negative_root.root_num:
                q_nodes = torch.cat([q_nodes, negative_root.roots])
                q_ts = torch.cat([q_ts, negative_root.ts])
            out = TemporalResult(postive_root, negative_root)
            tgt, tgt_ts, d_n = q_nodes.contiguous(), q_ts.contiguous(), None
            for l in range(int(layers)):
                hop = ops.sample_layer(self.g, tgt, tgt_ts, int(k), sample_type, d_n=d_n,
                                       equal_root_time=bool(equal_root_time), allowed_offset=int(allowed_offset),
                                       keep_root_time=bool(keep_root_time), rng_stream=l, want_dt_i64=True,
                                       status=self.status)
                nb = TemporalNeighbor(hop)     # reads the hop's size (one synchronisation per hop)
                out.neighbors_list.append(nb)
                tgt, tgt_ts, d_n = nb.neighbors, nb.neighbors_ts, None
            self.status.check("sample_src_in_chunks_khop")
        return out

    def slice_by_chunk_ts(self, chunks, time_begin, time_end, using_full_timestamp=False, stream=0) -> "TemporalResult":
        """Sub-graph of the chunks' nodes inside ``[time_begin, time_end)``: ``roots`` = the nodes that keep an edge with
        their distinct timestamps (``ts_ptr`` / ``ts``), one neighbour layer whose ``root_start_ptr`` has one entry per
        (node, timestamp) group (reference: csrc/include/starrygl/sample.cu.hpp:1189-1291)."""
        if using_full_timestamp:
            raise NotImplementedError("dense per-timestep groups (using_full_timestamp) are not provided")
        ev_ts = self.ev[1]
        with torch.cuda.stream(self.stream):
            lo, hi = ops.lower_bound(ev_ts, torch.tensor([int(time_begin), int(time_end)], dtype=torch.int64,
                                                         device=ev_ts.device)).tolist()
            nodes, node_ptr, group_ts, group_ptr, nbr, ts, eid = ops.slice_window(
                self.g, chunks, self.mapper, int(time_begin), int(time_end), max(hi - lo, 0), status=self.status)
        out = TemporalResult(TemporalRoot(nodes, node_ptr, group_ts))
        out.neighbors_list.append(TemporalNeighbor.from_arrays(group_ptr, nbr, ts, eid))
        return out

    def _remap(self, result: TemporalResult, reset: bool):
        """Node-level relabel: roots first, then every hop; local ids in ascending global id among the new ids."""
        if reset:
            self.relabel.reset()
        pieces = []
        loc, new_ids, d_new = self.relabel.insert(result.roots.roots, status=self.status)
        result.roots = TemporalRoot(loc, result.roots.ts_ptr, result.roots.ts, result.roots.q_ptr, result.roots.q_eid)
        pieces.append((new_ids, d_new))
        for nb in result.neighbors_list:
            loc, new_ids, d_new = self.relabel.insert(nb.neighbors, status=self.status)
            nb.neighbors = loc
            pieces.append((new_ids, d_new))
        counts = torch.cat([d for _, d in pieces]).tolist()
        result.nodes_remapper_id = torch.cat([ids[:c] for (ids, _), c in zip(pieces, counts)])

    # ---- asynchronous queue ----------------------------------------------------------------------------------
    def submit_query(self, time_start, time_end, chunk_list, test_generate_samples, test_generate_samples_ts,
                     sample_type, layers, fanout, allowed_offset, equal_root_time, keep_root_time, op) -> None:
        if self._closed:
            raise RuntimeError("graph is closed")
        fut = {"event": threading.Event(), "value": None, "error": None}
        neg = self.get_negative_root(test_generate_samples, test_generate_samples_ts)
        self._tasks.put((fut, (int(time_start), int(time_end), chunk_list, neg, sample_type, int(layers), int(fanout),
                               int(allowed_offset), bool(equal_root_time), bool(keep_root_time), op)))
        self._results.put(fut)

    def get(self) -> Optional[TemporalResult]:
        try:
            fut = self._results.get_nowait()
        except queue.Empty:
            return None
        fut["event"].wait()
        if fut["error"] is not None:
            raise fut["error"]
        return fut["value"]

    def _run(self):
        torch.cuda.set_device(self.g.device)
        while True:
            item = self._tasks.get()
            if item is None:
                return
            fut, (t0, t1, chunks, neg, stype, layers, fanout, off, eq, keep, op) = item
            try:
                if stype not in ("recent", "uniform"):
                    raise NotImplementedError("cluster slices are not part of the sampling data path")
                roots = self.get_seeds_in_chunks(chunks, t0, t1, False)
                res = self.sample_src_in_chunks_khop(roots, neg, fanout, layers, off, eq, keep, stype)
                with torch.cuda.stream(self.stream):
                    self._remap(res, op == "f")     # the reference restarts the numbering on "f"
                    self.status.check("submit_query")
                self.stream.synchronize()
                fut["value"] = res
            except BaseException as e:   # delivered to the caller of get()
                fut["error"] = e
            fut["event"].set()

    def close(self):
        if not self._closed:
            self._closed = True
            self._tasks.put(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def from_edge_index(n: int, chunk_size: int, src: torch.Tensor, dst: torch.Tensor, ts: torch.Tensor, eid: torch.Tensor,
                    mapper: Optional[torch.Tensor] = None, stream=0, rank: int = 0) -> CUDAGraph:
    """Build the time-sorted CSR (rows = source nodes, neighbours = destinations) on GPU ``rank``.

    ``stream`` is a ``torch.cuda.Stream``, a raw ``cudaStream_t`` value, or 0/None for a stream owned by the graph.
    Raises ``RuntimeError`` for non-CUDA / non-int64 inputs and for node ids outside [0, n).
    """
    for name, t in (("src", src), ("dst", dst), ("ts", ts), ("eid", eid)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(f"Graph construction failed: {name} must be a CUDA tensor")
        if t.dtype != torch.int64:
            raise RuntimeError(f"Graph construction failed: {name} must be int64")
    dev = src.device
    if isinstance(stream, torch.cuda.Stream):
        s = stream
    elif stream:
        s = torch.cuda.ExternalStream(int(stream), device=dev)
    else:
        s = torch.cuda.Stream(device=dev)
    if mapper is not None and mapper.numel():
        m = mapper.to(torch.int64).cpu()
        if bool((m[1:] < m[:-1]).any()):
            raise RuntimeError("Graph construction failed: chunk mapper must be non-decreasing in node id")
    s.wait_stream(torch.cuda.current_stream(dev))
    try:
        with torch.cuda.stream(s):
            g = ops.tcsr_build(src, dst, ts, eid, int(n))
            ev = ops.time_ordered_events(src, ts, eid)
    except _C.SglError as e:
        raise RuntimeError(f"Graph construction failed: {e}") from e
    return CUDAGraph(g, ev, chunk_size, mapper, s, rank)
