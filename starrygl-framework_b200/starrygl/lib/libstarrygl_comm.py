"""Python-visible surface of the native sampler module.

Same names and call signatures as the reference's pybind module ``libstarrygl_comm``
(csrc/srcs/starrygl/export.cu:20-254): ``from_edge_index``, ``CUDAGraph`` with ``submit_query`` / ``get`` /
``get_seeds_in_chunks`` / ``get_negative_root`` / ``sample_src_in_chunks_khop``, and the result types
``TemporalRoot``, ``NegativeRoot``, ``TemporalNeighbor``, ``TemporalResult``; plus the communicator and the sharded
feature table the same module exports (``create_nccl_id``, ``DistContext``,
csrc/include/starrygl/commContext.cu.hpp:259-268; ``init_p2p``, ``ShardTensorItem``, ``ShardTensor``,
csrc/include/starrygl/feature.cu.hpp:713-750).  The work is done by libsgl_b200.so
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
    exclusive prefix with one extra entry, ``root_end_ptr`` its shift by one).

    The hop's arrays are produced at capacity with their length on the device, so building the object costs no
    synchronisation.  Consumers that stay on the GPU use the capacity views (``hop``: ``nbr`` / ``ts`` / ``eid`` /
    ``dt_i64`` / ``offsets`` and the device count ``hop.d_total``).  The attributes of the reference's type (trimmed
    tensors, ``neighbor_num``) are cut to size on first use; all hops of a result are cut with ONE read-back of their
    counts (``TemporalResult.materialize``)."""

    def __init__(self, hop: ops.Hop, owner: "TemporalResult" = None, n_queries: Optional[int] = None):
        self.hop = hop
        self._owner = owner
        self._n = None                  # number of sampled neighbours, once known on the host
        self._nq = n_queries            # number of queries (None: known only once the previous hop has been cut)
        self._neighbors_override = None

    def _cut(self) -> int:
        if self._n is None:
            if self._owner is not None:
                self._owner.materialize()
            else:
                self._n = self.hop.total()
        return self._n

    @classmethod
    def from_arrays(cls, start_ptr, neighbors, neighbors_ts, neighbors_eid):
        """Layer given directly by its CSR arrays (``start_ptr`` with one extra entry)."""
        hop = ops.Hop(neighbors, None, neighbors_ts, None, neighbors_eid, start_ptr, neighbors.numel(), torch.zeros_like(neighbors_ts))
        self = cls(hop, None, start_ptr.numel() - 1)
        self._n = neighbors.numel()
        return self

    @property
    def neighbor_num(self) -> int:
        return self._cut()

    @property
    def root_start_ptr(self):
        self._cut()
        return self.hop.offsets if self._nq is None else self.hop.offsets[:self._nq + 1]

    @property
    def root_end_ptr(self):
        o = self.root_start_ptr
        return torch.cat([o[1:], o[-1:]])

    @property
    def neighbors(self):
        if self._neighbors_override is not None:
            return self._neighbors_override[:self._cut()]
        return self.hop.nbr[:self._cut()]

    @neighbors.setter
    def neighbors(self, value):
        self._neighbors_override = value

    @property
    def neighbors_ts(self):
        return self.hop.ts[:self._cut()]

    @property
    def neighbors_eid(self):
        return self.hop.eid[:self._cut()]

    @property
    def neighbors_dt(self):
        return self.hop.dt_i64[:self._cut()]

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
        self._remap_pieces = []          # (new global ids at capacity, device count) per relabelled list
        self._remapper = None
        self._status = None              # device status word of the graph that produced the result

    @property
    def neighbors(self):
        return self.neighbors_list

    def materialize(self):
        """The one read-back of a result: the sizes of every hop (and of every piece of the id map) in a single copy."""
        hops = [nb for nb in self.neighbors_list if nb._n is None]
        counts = [nb.hop.d_total for nb in hops] + [d for _, d in self._remap_pieces]
        if not counts:
            return
        if self._status is not None:     # the kernels' error bits ride along in the same copy
            counts = counts + [self._status.t.to(torch.int64)]
        host = torch.cat(counts).tolist()
        if self._status is not None:
            bits = int(host.pop())
            if bits:
                self._status.t.zero_()
                raise _C.SglError(f"sampling: device status {bits} ({_C.decode_status(bits)})")
        for nb, n in zip(hops, host):
            nb._n = int(n)
        prev = None
        for nb in self.neighbors_list:      # queries of hop l+1 = neighbours of hop l
            if nb._nq is None and prev is not None:
                nb._nq = prev._n
            prev = nb
        if self._remap_pieces:
            sizes = host[len(hops):]
            dev = self.roots.roots.device
            self._remapper = (torch.cat([ids[:int(c)] for (ids, _), c in zip(self._remap_pieces, sizes)])
                              if sizes else _empty(dev))
            self._remap_pieces = []

    @property
    def nodes_remapper_id(self):
        if self._remapper is None:
            if self._remap_pieces:
                self.materialize()
            else:
                self._remapper = _empty(self.roots.roots.device)
        return self._remapper

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
        with torch.cuda.stream(self.stream):
            roots, ts_ptr, ts, q_ptr, q_eid = ops.seeds_in_window(self.ev, self.g, chunks, self.mapper, int(time_begin),
                                                                  int(time_end), status=self.status)
            if using_full_timestamp:
                # every root gets all time steps of the window (snapshot graphs): time steps without an event own no event
                ts_ptr, ts, q_ptr = ops.densify_time_groups(ts_ptr, ts, q_ptr, int(time_begin), int(time_end))
        return TemporalRoot(roots, ts_ptr, ts, q_ptr, q_eid)

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
            out._status = self.status
            tgt, tgt_ts, d_n, n_q = q_nodes.contiguous(), q_ts.contiguous(), None, q_nodes.numel()
            for l in range(int(layers)):
                hop = ops.sample_layer(self.g, tgt, tgt_ts, int(k), sample_type, d_n=d_n,
                                       equal_root_time=bool(equal_root_time), allowed_offset=int(allowed_offset),
                                       keep_root_time=bool(keep_root_time), rng_stream=l, want_dt_i64=True,
                                       status=self.status)
                out.neighbors_list.append(TemporalNeighbor(hop, out, n_q))
                # the next hop queries this hop's neighbours: arrays at capacity, their number stays on the device
                tgt, tgt_ts, d_n, n_q = hop.nbr, hop.ts, hop.d_total, None
        return out

    def slice_by_chunk_ts(self, chunks, time_begin, time_end, using_full_timestamp=False, stream=0) -> "TemporalResult":
        """Sub-graph of the chunks' nodes inside ``[time_begin, time_end)``: ``roots`` = the nodes that keep an edge with
        their distinct timestamps (``ts_ptr`` / ``ts``), one neighbour layer whose ``root_start_ptr`` has one entry per
        (node, timestamp) group (reference: csrc/include/starrygl/sample.cu.hpp:1189-1291)."""
        ev_ts = self.ev[1]
        with torch.cuda.stream(self.stream):
            lo, hi = ops.lower_bound(ev_ts, torch.tensor([int(time_begin), int(time_end)], dtype=torch.int64,
                                                         device=ev_ts.device)).tolist()
            nodes, node_ptr, group_ts, group_ptr, nbr, ts, eid = ops.slice_window(
                self.g, chunks, self.mapper, int(time_begin), int(time_end), max(hi - lo, 0), status=self.status)
            if using_full_timestamp:
                node_ptr, group_ts, group_ptr = ops.densify_time_groups(node_ptr, group_ts, group_ptr, int(time_begin),
                                                                        int(time_end))
        out = TemporalResult(TemporalRoot(nodes, node_ptr, group_ts))
        out.neighbors_list.append(TemporalNeighbor.from_arrays(group_ptr, nbr, ts, eid))
        return out

    def _remap(self, result: TemporalResult, reset: bool):
        """Node-level relabel: roots first, then every hop; local ids in ascending global id among the new ids."""
        if reset:
            self.relabel.reset()
        pieces = result._remap_pieces
        loc, new_ids, d_new = self.relabel.insert(result.roots.roots, status=self.status)
        result.roots = TemporalRoot(loc, result.roots.ts_ptr, result.roots.ts, result.roots.q_ptr, result.roots.q_eid)
        pieces.append((new_ids, d_new))
        for nb in result.neighbors_list:      # capacity arrays + device counts: no read-back between the hops
            loc, new_ids, d_new = self.relabel.insert(nb.hop.nbr, d_n=nb.hop.d_total, status=self.status)
            nb.neighbors = loc
            pieces.append((new_ids, d_new))

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
                if stype in ("recent", "uniform"):
                    roots = self.get_seeds_in_chunks(chunks, t0, t1, False)
                    res = self.sample_src_in_chunks_khop(roots, neg, fanout, layers, off, eq, keep, stype)
                else:
                    # any other policy name is the "cluster" slice: the chunks' whole sub-graph inside the window, dense
                    # time steps (csrc/include/starrygl/sample.cu.hpp:1953-1961)
                    res = self.slice_by_chunk_ts(chunks, t0, t1, True)
                    res._status = self.status
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


# ---------------------------------------------------------------------------------------------------------------------
# communicator + sharded feature table
# ---------------------------------------------------------------------------------------------------------------------

def create_nccl_id() -> bytes:
    """Unique id of a new communicator, to be handed to every rank out of band (the reference puts it into the
    process group's store, starrygl/utils/context.py:111-117)."""
    import ctypes as C
    buf = C.create_string_buffer(128)
    _C.check(_C.lib().sgl_comm_unique_id(buf, 128))
    return buf.raw


class DistContext:
    """One rank of the library's own NCCL communicator: ``DistContext(rank, world_size, local_size, id)`` with
    ``rank()``, ``size()``, ``device()`` (csrc/include/starrygl/commContext.cu.hpp:11-60, :259-268).  The device of the
    rank is ``rank % local_size`` and is made current, as the reference's constructor does."""

    def __init__(self, rank: int, world_size: int, local_size: int, id: bytes):
        import ctypes as C
        if not (isinstance(id, (bytes, bytearray)) and len(id) >= 128):
            raise RuntimeError("DistContext: id must be the bytes create_nccl_id() returned")
        if local_size < 1 or not (0 <= rank < world_size):
            raise RuntimeError("DistContext: bad rank / size")
        self._rank, self._world, self._local = int(rank), int(world_size), int(local_size)
        self._device = self._rank % self._local
        torch.cuda.set_device(self._device)
        self.handle = C.c_void_p()
        _C.check(_C.lib().sgl_comm_init(C.byref(self.handle), self._rank, self._world, bytes(id)))
        from ..route.exchange import NativeComm
        NativeComm.adopt(self.handle, self._rank, self._world)     # the routes of this process use this communicator

    def rank(self) -> int:
        return self._rank

    def size(self) -> int:
        return self._world

    def device(self) -> int:
        return self._device


def init_p2p(devices: List[int]) -> int:
    """Enable peer access from the current GPU to the listed ones where the hardware allows it; returns how many of
    them are reachable.  With one process per GPU the mappings of other ranks' memory enable it when they are opened,
    so this matters only for a process that drives several GPUs."""
    import ctypes as C
    arr = (C.c_int * max(len(devices), 1))(*[int(d) for d in devices])
    ok = C.c_int(0)
    _C.check(_C.lib().sgl_init_p2p(arr, len(devices), C.byref(ok)))
    return ok.value


class ShardTensorItem:
    """Description of one shard that can travel between processes: owner rank and device, an inter-process handle of
    its memory, its shape and element size (csrc/include/starrygl/feature.cu.hpp:94-140)."""

    def __init__(self):
        self.rank, self.group, self.device = 0, 0, -1
        self.mem_handle, self.shape, self.element_size, self.dtype = b"", [], 4, "float32"

    def share_ipc(self):
        return (self.device, self.element_size, self.mem_handle, list(self.shape), self.rank, self.dtype)

    def from_ipc(self, ipc_data):
        self.device, self.element_size, self.mem_handle, shape = ipc_data[:4]
        self.shape = list(shape)
        if len(ipc_data) > 4:
            self.rank = int(ipc_data[4])
        if len(ipc_data) > 5:
            self.dtype = ipc_data[5]
        return self


class ShardTensor:
    """Row table sharded over the GPUs of one node; ``tensor[ids]`` with packed ids ``(partition << 48) | local row``
    returns the rows in the order of the ids (csrc/include/starrygl/feature.cu.hpp:142-422).

    Shard p belongs to rank p.  The owner appends its own CUDA tensor, every other rank appends the
    ``ShardTensorItem`` the owner published (``share_ipc``) and thereby maps the owner's memory.  The gather is ONE
    kernel that reads every row from its owner's memory over NVLink; the reference's plan -- split the ids by owner,
    send the ids, gather at the owner, send the rows back, scatter to the original order -- is what
    :meth:`gather_by_exchange` does for ranks without a mapping of each other's memory."""

    def __init__(self, device: int, context: Optional[DistContext] = None):
        self._device = int(device)
        self.context = context
        self._local = {}          # partition -> tensor owned here (kept alive)
        self._bases, self._rows = [], []
        self._opened = []
        self._row_shape, self._dtype = None, None
        self._tables = None

    # ---- building ------------------------------------------------------------------------------------------------
    def _check_layout(self, shape, dtype):
        if self._row_shape is None:
            self._row_shape, self._dtype = tuple(shape[1:]), dtype
        elif tuple(shape[1:]) != self._row_shape or dtype != self._dtype:
            raise RuntimeError("ShardTensor: all shards must have the same row shape and dtype")

    def append(self, item, target_device: Optional[int] = None):
        """Append the next partition's shard: a CUDA tensor of this process, or a ``ShardTensorItem`` of another."""
        import ctypes as C
        self._tables = None
        if isinstance(item, torch.Tensor):
            if not item.is_cuda or not item.is_contiguous():
                raise RuntimeError("ShardTensor.append: a local shard must be a contiguous CUDA tensor")
            self._check_layout(item.shape, item.dtype)
            self._local[len(self._bases)] = item
            self._bases.append(item.data_ptr())
            self._rows.append(int(item.shape[0]))
            return
        dtype = getattr(torch, item.dtype)
        self._check_layout(item.shape, dtype)
        ptr = C.c_void_p()
        _C.check(_C.lib().sgl_p2p_open(item.mem_handle, C.byref(ptr)))
        self._opened.append(ptr)
        self._bases.append(ptr.value)
        self._rows.append(int(item.shape[0]))

    def share_ipc(self) -> List[ShardTensorItem]:
        """Items for the shards this process owns (the memory must come from ``cudaMalloc``, i.e. be a whole torch
        allocation or one made with ``ShardTensor.alloc_shared``)."""
        out = []
        for part, t in self._local.items():
            it = ShardTensorItem()
            it.rank, it.device, it.shape, it.element_size = part, t.device.index, list(t.shape), t.element_size()
            it.dtype = str(t.dtype).replace("torch.", "")
            it.mem_handle = _ipc_handle(t)
            out.append(it)
        return out

    @classmethod
    def from_local(cls, local: torch.Tensor, context: Optional[DistContext] = None) -> "ShardTensor":
        """Collective convenience: every rank of the default process group passes its own shard (allocated with
        :func:`shared_empty`); the handles are exchanged through the group and every rank maps all shards."""
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        me = cls(local.device.index, context)
        mine = ShardTensorItem()
        mine.rank, mine.device, mine.shape, mine.element_size = rank, local.device.index, list(local.shape), local.element_size()
        mine.dtype = str(local.dtype).replace("torch.", "")
        mine.mem_handle = _ipc_handle(local)
        box = [None] * world
        dist.all_gather_object(box, mine.share_ipc())
        for p in range(world):
            me.append(local if p == rank else ShardTensorItem().from_ipc(box[p]))
        dist.barrier()
        return me

    # ---- queries ---------------------------------------------------------------------------------------------------
    def shape(self):
        return [sum(self._rows)] + list(self._row_shape or [])

    def size(self, dim: int) -> int:
        return self.shape()[dim]

    def numel(self) -> int:
        n = 1
        for d in self.shape():
            n *= d
        return n

    def stride(self, dim: int) -> int:
        s = 1
        for d in self.shape()[dim + 1:]:
            s *= d
        return s

    def device(self) -> int:
        return self._device

    def device_count(self) -> int:
        return len(self._bases)

    # ---- gather ------------------------------------------------------------------------------------------------------
    def _device_tables(self, dev):
        if self._tables is None:
            self._tables = (torch.tensor(self._bases, dtype=torch.int64, device=dev),
                            torch.tensor(self._rows, dtype=torch.int64, device=dev), ops.StatusWord(dev))
        return self._tables

    def __getitem__(self, indices: torch.Tensor) -> torch.Tensor:
        if not indices.is_cuda:
            raise RuntimeError("ShardTensor: the ids must be on the GPU")
        bases, rows, st = self._device_tables(indices.device)
        return ops.shard_gather(bases, rows, len(self._bases), self._row_shape, self._dtype, indices, status=st)

    def check(self):
        """Raise if a gather since the last check met an id outside its shard (one synchronisation)."""
        if self._tables is not None:
            self._tables[2].check("ShardTensor gather")

    def unregister(self):
        for p in self._opened:
            _C.lib().sgl_p2p_close(p)
        self._opened, self._bases, self._rows, self._local, self._tables = [], [], [], {}, None

    @staticmethod
    def gather_by_exchange(local: torch.Tensor, indices: torch.Tensor, group=None) -> torch.Tensor:
        """The same result without peer mappings, in the reference's five steps: ids ordered by owner, id exchange,
        gather at the owner, row exchange, rows put back in the order of ``indices``.  Collective over ``group``."""
        from ..route.exchange import exchange_rows
        from ..route.route import Route
        route, asked_rows, order = Route.all_to_all_ind2ptr(indices, group)
        mine = ops.gather_rows(local, asked_rows)                                   # what the others asked me for
        got = torch.empty((indices.numel(),) + tuple(local.shape[1:]), dtype=local.dtype, device=indices.device)
        exchange_rows(mine, route.recv_sizes, got, route.send_sizes, group).wait()  # rows arrive in owner order
        out = torch.empty_like(got)
        ops.scatter_rows(out, order, got)                                           # back to the order of the ids
        return out


def shared_empty(rows: int, row_shape, dtype=torch.float32):
    """A zero-filled CUDA tensor in memory of its own allocation, as inter-process handles need (a slice of torch's caching
    allocator cannot be exported on its own).  Returns the tensor; its memory is released with the tensor."""
    import ctypes as C
    n = int(rows)
    per = torch.empty(0, dtype=dtype).element_size()
    for d in row_shape:
        per *= int(d)
    nbytes = max(n * per, 256)
    base, handle = C.c_void_p(), C.create_string_buffer(64)
    _C.check(_C.lib().sgl_p2p_alloc(nbytes, C.byref(base), handle, 64))
    dev = torch.device("cuda", torch.cuda.current_device())
    t = _tensor_over(base.value, nbytes, dev).view(dtype)[: n * per // torch.empty(0, dtype=dtype).element_size()]
    t = t.view((n,) + tuple(int(d) for d in row_shape))
    _SHARED[t.data_ptr()] = (handle.raw, base)
    return t


_SHARED = {}   # data_ptr -> (ipc handle, base pointer) of tensors made by shared_empty


def _ipc_handle(t: torch.Tensor) -> bytes:
    hit = _SHARED.get(t.data_ptr())
    if hit is None:
        raise RuntimeError("ShardTensor: a shard that other processes map must be allocated with shared_empty()")
    return hit[0]


def _tensor_over(ptr: int, nbytes: int, dev) -> torch.Tensor:
    """uint8 tensor viewing foreign device memory through the CUDA array interface."""
    class _Mem:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
    return torch.as_tensor(_Mem(), device=dev)
