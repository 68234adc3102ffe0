"""Multi-hop mini-batch builder on the GPU: sampling, (node, ts)-pair dedup/relabel and per-hop CSC.

Produces the per-layer dictionaries of the reference's offline builder
(``MaterializedMultiLayerBuilder.build_aligned_batch``, prepare_sample.py:313-377) without its route
planning: layer 0 = sorted unique (id, ts) pairs of the roots + ``inv_map``; layer l+1 = CSC over the
previous list (``indptr``, ``indices``, ``eid``, ``edge_ts``, ``edge_dt``) + the merged sorted pair list
(``gids``, ``ts``).  All hops are enqueued on the current stream without an intermediate host
synchronisation: the number of edges a hop produced is handed to the next kernels as a device count.
``finish()`` performs the single synchronisation that is needed to give the tensors their final shapes.
"""
from typing import List, Optional, Sequence

import torch

from .. import ops


class DeviceBatch:
    """Un-trimmed result of :func:`build_batch_async` (all arrays at capacity, counts on the device)."""

    def __init__(self, g, layers, counts, status, fanouts, targets_first):
        self.g = g
        self.layers = layers          # list of dicts of capacity-sized tensors
        self.counts = counts          # list of device int64 scalars (1-element tensors), see finish()
        self.status = status
        self.fanouts = list(fanouts)
        self._targets_first = targets_first

    def finish(self) -> List[dict]:
        """One host synchronisation: read every count, check the device status word, trim the arrays."""
        host = self._host = torch.cat(self.counts).tolist()      # one read-back (synchronises the current stream)
        self.status.check("build_batch")
        n_list = host[0]
        out = [{"gids": self.layers[0]["gids"][:n_list], "ts": self.layers[0]["ts"][:n_list],
                "inv_map": self.layers[0]["inv_map"]}]
        prev_n = n_list
        for l in range(len(self.fanouts)):
            n_edges, n_next = host[1 + 2 * l], host[2 + 2 * l]
            L = self.layers[l + 1]
            if n_edges == 0 and not self._any_target_has_edges(l, out, prev_n):
                # the reference emits an empty layer and stops when no target has any edge at all
                # (prepare_sample.py:352-361)
                z = torch.zeros(0, dtype=torch.int64, device=self.g.device)
                out.append({"indptr": torch.zeros(1, dtype=torch.int64, device=self.g.device), "indices": z,
                            "eid": z, "edge_ts": z, "edge_dt": torch.zeros(0, dtype=torch.float32, device=self.g.device),
                            "gids": z, "ts": z})
                break
            out.append({"indptr": L["indptr"][:prev_n + 1], "indices": L["indices"][:n_edges], "eid": L["eid"][:n_edges],
                        "edge_ts": L["edge_ts"][:n_edges], "edge_dt": L["edge_dt"][:n_edges],
                        "gids": L["gids"][:n_next], "ts": L["ts"][:n_next]})
            prev_n = n_next
        return out

    def _any_target_has_edges(self, l, out, prev_n):
        tgt = out[0]["gids"] if l == 0 else self.layers[l]["raw_nbr"][:self._host[1 + 2 * (l - 1)]]
        if tgt.numel() == 0:
            return False
        deg = self.g.indptr[tgt + 1] - self.g.indptr[tgt]
        return bool((deg > 0).any().item())


def build_batch_async(g: ops.TCSR, roots: torch.Tensor, root_ts: torch.Tensor, fanouts: Sequence[int],
                      policy: str = "recent", *, ts_range: Optional[Sequence[int]] = None, equal_root_time=False,
                      allowed_offset=-1, seed=0, status: Optional[ops.StatusWord] = None,
                      side_streams: Optional[Sequence[torch.cuda.Stream]] = None) -> DeviceBatch:
    """Enqueue the whole batch construction on the current stream.

    ``ts_range`` = (lowest, highest) timestamp that can occur among the roots' query times; together with the
    graph's own timestamp range it fixes the width of the (id, ts) sort key.  When omitted it is read from
    ``root_ts`` (one extra synchronisation).

    ``side_streams`` (two streams): the independent chains of the construction run side by side -- hop l+1 samples the
    raw output of hop l, so the sampling of all hops proceeds while the relabel of the earlier hops is still sorting, and
    the CSC's sort (keyed by destination row and time) runs next to the relabel's sort; only its column indices need the
    relabel's result, and they are filled in with one gather at the end.  Everything is joined into the current stream
    before the function returns.  Captured into a CUDA graph this becomes a graph with parallel branches.
    """
    dev = g.device
    status = status or ops.StatusWord(dev)
    if ts_range is None:
        if root_ts.numel():
            lo, hi = root_ts.aminmax()
            ts_range = (int(lo.item()), int(hi.item()))
        else:
            ts_range = (g.ts_min, g.ts_max)
    ts_base = min(g.ts_min, int(ts_range[0]))
    ts_bits = ops.bits_for(max(g.ts_max, int(ts_range[1])) - ts_base)
    id_bits = ops.bits_for(g.num_nodes - 1)
    main = torch.cuda.current_stream(dev)
    s_sample, s_csc = (side_streams[0], side_streams[1]) if side_streams else (main, main)

    def after(stream_done, stream_wait):
        if stream_done is not stream_wait:
            ev = torch.cuda.Event()
            ev.record(stream_done)
            stream_wait.wait_event(ev)

    cur_id, cur_ts, inv0, _, d_cur = ops.unique_pairs(roots, root_ts, id_bits=id_bits, ts_bits=ts_bits, ts_base=ts_base,
                                                      status=status)
    layers = [{"gids": cur_id, "ts": cur_ts, "inv_map": inv0[:roots.numel()]}]
    counts = [d_cur]
    # the sampling chain: hop 0 queries the layer-0 list, hop l+1 one target per edge sampled by hop l at that edge's
    # timestamp (prepare_sample.py:345-346) -- no hop waits for a relabel but the first
    after(main, s_sample)
    hops = []
    tgt, tgt_ts, d_tgt = cur_id, cur_ts, d_cur
    with torch.cuda.stream(s_sample):
        for l, k in enumerate(fanouts):
            hop = ops.sample_layer(g, tgt, tgt_ts, k, policy, d_n=d_tgt, equal_root_time=equal_root_time,
                                   allowed_offset=allowed_offset, seed=seed, rng_stream=l, status=status)
            hops.append(hop)
            tgt, tgt_ts, d_tgt = hop.nbr, hop.ts, hop.d_total
    after(s_sample, main)
    if side_streams and len(hops) > 1:          # (a stream that joins a capture has to be joined back: only fork it for work)
        after(s_sample, s_csc)
    last_inv = None
    pending = []
    for l, hop in enumerate(hops):
        cap_cur = cur_id.numel()
        first = last_inv is None
        if not first and side_streams:
            # CSC of a later hop: its order does not depend on this hop's relabel -- sort it on the side with the edge
            # number as column index, translate the columns once the relabel is there
            after(main, s_csc)                      # last_inv / d_cur of the previous relabel
            with torch.cuda.stream(s_csc):
                iota = torch.arange(hop.capacity, dtype=torch.int64, device=dev)
                indptr, edge_no, e_ts, e_dt, e_eid = ops.build_csc(iota, hop.dst, last_inv, hop.ts, hop.dt, hop.eid, cap_cur,
                                                                   dst_bits=ops.bits_for(cap_cur), ts_bits=ts_bits,
                                                                   ts_base=ts_base, d_n_edges=hop.d_total, d_num_dst=d_cur,
                                                                   status=status)
        nxt_id, nxt_ts, _, nxt_inv, d_nxt = ops.unique_pairs(cur_id, cur_ts, hop.nbr, hop.ts, id_bits=id_bits,
                                                             ts_bits=ts_bits, ts_base=ts_base, d_n_a=d_cur,
                                                             d_n_b=hop.d_total, status=status)
        if first or not side_streams:
            indptr, idx, e_ts, e_dt, e_eid = ops.build_csc(nxt_inv, hop.dst, last_inv, hop.ts, hop.dt, hop.eid, cap_cur,
                                                           dst_bits=ops.bits_for(cap_cur), ts_bits=ts_bits, ts_base=ts_base,
                                                           d_n_edges=hop.d_total, d_num_dst=d_cur, presorted=first,
                                                           status=status)
        else:
            after(s_csc, main)
            idx = ops.gather_rows(nxt_inv, edge_no, d_n=hop.d_total, status=status)
        layers.append({"indptr": indptr, "indices": idx, "eid": e_eid, "edge_ts": e_ts, "edge_dt": e_dt,
                       "gids": nxt_id, "ts": nxt_ts, "raw_nbr": hop.nbr, "raw_ts": hop.ts, "inv": nxt_inv, "hop": hop})
        counts += [hop.d_total, d_nxt]
        cur_id, cur_ts, d_cur, last_inv = nxt_id, nxt_ts, d_nxt, nxt_inv
    return DeviceBatch(g, layers, counts, status, fanouts, None)


def build_batch(g, roots, root_ts, fanouts, policy="recent", **kw) -> List[dict]:
    """Synchronous form of :func:`build_batch_async`."""
    return build_batch_async(g, roots, root_ts, fanouts, policy, **kw).finish()


def batch_kernel_launches(num_nodes: int, num_roots: int, fanouts: Sequence[int], ts_span: int) -> int:
    """Kernels of this library that one mini-batch of :func:`build_batch_async` launches at the given capacities (pack,
    sort, head scan and emit of every relabel; count and fill of every hop; pack, sort and emit of every CSC after the
    first, which needs no sort).  Counted from the structure of the calls; the sorts' share comes from the library."""
    from .. import _C
    L = _C.lib()
    id_bits, ts_bits = ops.bits_for(num_nodes - 1), ops.bits_for(ts_span)
    total = 3 + L.sgl_radix_sort_launches(num_roots, id_bits + ts_bits)          # relabel of the roots
    cur, targets = num_roots, num_roots
    for l, k in enumerate(fanouts):
        edges = targets * k
        total += 2                                                               # count + fill
        total += 3 + L.sgl_radix_sort_launches(cur + edges, id_bits + ts_bits)   # merged list of the hop
        # CSC: a copy for the first hop; pack, sort, emit and the gather that fills in the column indices for the others
        total += 1 if l == 0 else 3 + L.sgl_radix_sort_launches(edges, ops.bits_for(cur) + ts_bits)
        cur, targets = cur + edges, edges
    return int(total)


class BatchGraph:
    """The whole multi-hop batch construction of :func:`build_batch_async` captured once as a CUDA graph for a fixed
    number of roots, and replayed per mini-batch: one launch instead of about a hundred small ones (the pipeline is a
    chain of short sort / scan / emit kernels, so at mini-batch sizes it is bound by launch overhead, not by the GPU).

    The result tensors are the same objects for every batch: consume (or copy) a result before the next ``run``.
    """

    def __init__(self, g: ops.TCSR, num_roots: int, fanouts: Sequence[int], policy: str = "recent", *,
                 ts_range: Sequence[int], equal_root_time=False, allowed_offset=-1, seed=0,
                 stream: Optional[torch.cuda.Stream] = None):
        from .. import _C
        dev = g.device
        self.g, self.num_roots = g, int(num_roots)
        self.stream = stream or torch.cuda.Stream(dev)
        self.roots = torch.zeros(self.num_roots, dtype=torch.int64, device=dev)
        self.root_ts = torch.full((self.num_roots,), int(ts_range[0]), dtype=torch.int64, device=dev)
        self.status = ops.StatusWord(dev)
        self._side = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
        kw = dict(ts_range=ts_range, equal_root_time=equal_root_time, allowed_offset=allowed_offset, seed=seed,
                  status=self.status, side_streams=self._side)
        # scratch used inside the graph must not be shared with eager calls: the capture gets its own workspace
        saved = _C.WORKSPACE
        _C.WORKSPACE = self._workspace = _C.Workspace()
        try:
            torch.cuda.synchronize(dev)
            with torch.cuda.stream(self.stream):
                build_batch_async(g, self.roots, self.root_ts, fanouts, policy, **kw)     # warm-up: sizes the scratch
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                self.batch = build_batch_async(g, self.roots, self.root_ts, fanouts, policy, **kw)
        finally:
            _C.WORKSPACE = saved
        self.stream.synchronize()
        self.kernel_launches = batch_kernel_launches(g.num_nodes, self.num_roots, fanouts, int(ts_range[1]) - min(g.ts_min, int(ts_range[0])))

    def run(self, roots: torch.Tensor, root_ts: torch.Tensor) -> DeviceBatch:
        """Enqueue one batch (exactly ``num_roots`` roots, already on the GPU); returns the un-trimmed device batch,
        whose ``finish()`` synchronises and trims."""
        if roots.numel() != self.num_roots:
            raise ValueError(f"this graph was captured for {self.num_roots} roots, got {roots.numel()}")
        with torch.cuda.stream(self.stream):
            self.roots.copy_(roots, non_blocking=True)
            self.root_ts.copy_(root_ts, non_blocking=True)
            self.graph.replay()
        return self.batch
