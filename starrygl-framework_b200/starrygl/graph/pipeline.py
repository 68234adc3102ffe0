"""Pre-bound sample -> gather pipeline for one mini-batch of roots.

The per-call work of :func:`starrygl.ops.sample_layer` / :func:`starrygl.ops.gather_rows` that does not depend
on the batch (output buffers, scratch, argument marshalling) is done once here, so that a step is a handful of
foreign calls: copy the roots in, sample one hop, gather the edge-feature rows of the sampled edges, and --
for callers whose consumer is on the host -- copy the block structure back.  It is what a prefetcher calls per
mini-batch (the reference's prefetcher/collator modules consume the sampler through ``AsyncBlock``,
starrygl/graph/graph.py:139-151, and read edge features as ``block.e_future``, starrygl/nn/model/tgn.py:161-162).

Buffers are reused from call to call: consume (or copy) a result before running the next batch on the same
pipeline object; use two objects for double buffering.
"""
import ctypes as C
from typing import Optional

import torch

from .. import _C, ops

I64 = torch.int64


class HostBlock:
    """Host views of one batch's block structure (``offsets``, ``nbr``, ``ts``, ``eid``, ``dt``), sliced out of the
    pipeline's pinned buffers on first use.  They alias those buffers: copy what must outlive the next batch."""

    _KEYS = ("offsets", "nbr", "ts", "eid", "dt")

    def __init__(self, pipe, n, tot):
        self._p, self._n, self._tot = pipe, n, tot

    def __getitem__(self, k):
        p, n, tot = self._p, self._n, self._tot
        o, cs = p._o, p._cs
        if k == "offsets":
            return p.h_blk[:n + 1]
        if k == "dt":
            return p.h_dt[:tot]
        if k in ("nbr", "ts", "eid"):
            b = o + ("nbr", "ts", "eid").index(k) * cs
            return p.h_blk[b:b + tot]
        raise KeyError(k)

    def keys(self):
        return self._KEYS

    def items(self):
        return [(k, self[k]) for k in self._KEYS]


class SampleGatherPipeline:
    def __init__(self, g: ops.TCSR, edge_feats: Optional[torch.Tensor], fanout: int, policy: str = "recent",
                 max_roots: int = 4096, *, equal_root_time=False, allowed_offset=-1, keep_root_time=False, seed=0,
                 gather_mode="auto", stream: Optional[torch.cuda.Stream] = None, export: str = "prefix"):
        if export not in ("prefix", "full"):
            raise _C.SglError("export must be 'prefix' (device-counted copy of the sampled edges) or 'full' (capacity)")
        self.export = export
        self.g, self.feats, self.k, self.max_roots = g, edge_feats, int(fanout), int(max_roots)
        dev = g.device
        self.dev = dev
        self.stream = stream or torch.cuda.current_stream(dev)
        self.L = _C.lib()
        cap = self.max_roots * self.k
        self.cap = cap
        # roots and query times of the current batch, contiguous ([2, max_roots]) so that one copy fills both
        self.roots_ts = torch.empty(2, self.max_roots, dtype=I64, device=dev)
        self.roots, self.root_ts = self.roots_ts[0], self.roots_ts[1]
        # one int64 block for the index outputs so that the block structure goes back to the host in ONE copy:
        # [offsets (max_roots+1) | nbr | ts | eid] each of capacity cap, then dt (float32) separately.  The target
        # slot of every edge (dst) stays on the device: on the host it is implied by the offsets.
        # (section starts are kept 16-byte aligned for the vectorised export copy: even element counts)
        o, cs = (self.max_roots + 2) & ~1, (cap + 1) & ~1
        self._o, self._cs = o, cs
        self.blk = torch.empty(o + 3 * cs, dtype=I64, device=dev)
        self.offsets = self.blk[:self.max_roots + 1]
        self.nbr, self.ts, self.eid = (self.blk[o + i * cs:o + i * cs + cap] for i in range(3))
        self.dst = torch.empty(cap, dtype=I64, device=dev)
        self.dt = torch.empty(cap, dtype=torch.float32, device=dev)
        self.done = torch.cuda.Event()
        self.status = ops.StatusWord(dev)
        self.ws = torch.empty(self.L.sgl_sample_ws_bytes(self.max_roots), dtype=torch.uint8, device=dev)
        self.out_feats = None
        if edge_feats is not None:
            self.out_feats = torch.empty((cap,) + tuple(edge_feats.shape[1:]), dtype=edge_feats.dtype, device=dev)
            self.row_bytes, self.src_pitch = ops._row_bytes(edge_feats)
        self.mode = _C.GATHER_MODE[gather_mode]
        self.args = dict(pol=_C.POLICY[policy], eq=int(bool(equal_root_time)), off=int(allowed_offset),
                         keep=int(bool(keep_root_time)), seed=int(seed) & (2 ** 64 - 1))
        # pinned host mirrors for callers with host buffers
        self.h_roots = torch.empty(self.max_roots, dtype=I64).pin_memory()
        self.h_root_ts = torch.empty(self.max_roots, dtype=I64).pin_memory()
        self.h_blk = torch.empty(self.blk.numel(), dtype=I64).pin_memory()
        self.h_dt = torch.empty(cap, dtype=torch.float32).pin_memory()
        # device-counted copy of the sampled edges (neighbour ids, timestamps, edge ids, dt) to the pinned mirrors
        v = C.c_void_p
        # (+ the offsets, copied whole: negative element size)
        self._exp_src = (v * 5)(self.nbr.data_ptr(), self.ts.data_ptr(), self.eid.data_ptr(), self.dt.data_ptr(),
                                self.offsets.data_ptr())
        self._exp_dst = (v * 5)(*[self.h_blk.data_ptr() + 8 * (o + i * cs) for i in range(3)], self.h_dt.data_ptr(),
                                self.h_blk.data_ptr())
        self._exp_elem = (C.c_int64 * 5)(8, 8, 8, 4, -8 * (self.max_roots + 1))
        self._exp_ok = all(p % 16 == 0 for p in list(self._exp_src) + list(self._exp_dst))
        self._h_blk_np, self._exec_host = self.h_blk.numpy(), None
        self.kernel_launches_per_step = 2 + (1 if edge_feats is not None else 0)
        self._g_dev = self._g_host = None
        # pre-converted argument list of the fused C call; per batch only the two input pointers and n change
        self._fused = None
        if edge_feats is not None:
            g_, a = g, self.args
            v = C.c_void_p
            self._a_roots, self._a_ts, self._a_n, self._a_rng = v(0), v(0), C.c_int64(0), C.c_uint32(0)
            self._fused = [v(g_.indptr.data_ptr()), v(g_.nbr.data_ptr()), v(g_.ts.data_ptr()), v(g_.eid.data_ptr()),
                           v(g_.fence.data_ptr() if g_.fence is not None else 0), C.c_int64(g_.num_nodes), self._a_roots, self._a_ts, self._a_n, C.c_int(self.k),
                           C.c_int(a["pol"]), C.c_int(a["eq"]), C.c_int64(a["off"]), C.c_int(a["keep"]),
                           C.c_uint64(a["seed"]), self._a_rng, v(self.nbr.data_ptr()), v(self.dst.data_ptr()),
                           v(self.ts.data_ptr()), v(self.dt.data_ptr()), v(self.eid.data_ptr()),
                           v(self.offsets.data_ptr()), v(edge_feats.data_ptr()), C.c_int64(edge_feats.shape[0]),
                           C.c_int64(self.row_bytes), C.c_int64(self.src_pitch), v(self.out_feats.data_ptr()),
                           C.c_int(self.mode), v(self.status.ptr()), v(self.ws.data_ptr()), C.c_size_t(self.ws.numel()),
                           v(self.stream.cuda_stream)]
            self._fn = self.L.sgl_sample_gather_fenced

    def run_device_ptr(self, roots_ptr: int, root_ts_ptr: int, n: int, rng_stream: int = 0):
        """:meth:`run_device` for callers that already hold raw device pointers: one foreign call per batch
        (sampling and gather are enqueued back to back by the library)."""
        if n > self.max_roots:
            raise _C.SglError(f"batch of {n} roots exceeds max_roots={self.max_roots}")
        self._a_roots.value, self._a_ts.value, self._a_n.value, self._a_rng.value = roots_ptr, root_ts_ptr, n, rng_stream
        rc = self._fn(*self._fused)
        if rc:
            _C.check(rc)

    # ---- CUDA graphs: one replay per batch instead of one foreign call per kernel -----------------------------
    def capture(self):
        """Capture the full-batch (``max_roots`` roots) step twice -- device inputs and host inputs -- as CUDA
        graphs on this pipeline's stream.  Afterwards :meth:`replay_device` / :meth:`submit_host` cost one
        graph launch per batch.  Call once, after the tables exist and before the timed loop."""
        n = self.max_roots
        self.roots.zero_()
        self.root_ts.zero_()
        torch.cuda.synchronize(self.dev)
        self.run_device(self.roots, self.root_ts)          # warm-up outside capture (lazy module loading etc.)
        self.stream.synchronize()
        self._g_dev = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._g_dev, stream=self.stream):
            self.run_device(self.roots, self.root_ts)
        self._g_host = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._g_host, stream=self.stream):
            self.roots.copy_(self.h_roots, non_blocking=True)
            self.root_ts.copy_(self.h_root_ts, non_blocking=True)
            self.run_device(self.roots, self.root_ts)
            self._export(n)
        self.stream.synchronize()
        return self

    def capture_native(self):
        """Record the full-batch device step (``sgl_sample_gather`` on this object's root buffers) with the library's
        own graph helpers; :meth:`replay_ptr` then costs one foreign call = one copy + one graph launch."""
        sp = self.stream.cuda_stream
        self.roots_ts.zero_()
        torch.cuda.synchronize(self.dev)
        self.run_device_ptr(self.roots.data_ptr(), self.root_ts.data_ptr(), self.max_roots)   # warm-up
        self.stream.synchronize()
        _C.check(self.L.sgl_graph_capture_begin(sp))
        try:
            self.run_device_ptr(self.roots.data_ptr(), self.root_ts.data_ptr(), self.max_roots)
        finally:
            ex = C.c_void_p()
            rc = self.L.sgl_graph_capture_end(sp, C.byref(ex))
        _C.check(rc)
        self._exec = ex
        v = C.c_void_p
        self._a_src = v(0)
        self._launch_args = [ex, self._a_src, v(self.roots_ts.data_ptr()), C.c_size_t(self.roots_ts.numel() * 8), v(sp)]
        self._launch = self.L.sgl_graph_launch
        self.stream.synchronize()
        return self

    def capture_native_host(self):
        """Record the full-batch host step -- ``sgl_sample_gather`` on this object's root buffers followed by the
        export of the block structure to the pinned mirrors -- with the library's graph helpers.
        :meth:`submit_host_ptr` then costs one foreign call: the copy of the roots from the caller's pinned buffer
        plus one graph launch."""
        if not (self._exp_ok and self.export == "prefix"):
            raise _C.SglError("capture_native_host needs the device-counted export (16-byte aligned buffers)")
        sp = self.stream.cuda_stream
        self.roots_ts.zero_()
        torch.cuda.synchronize(self.dev)
        self.run_device_ptr(self.roots.data_ptr(), self.root_ts.data_ptr(), self.max_roots)   # warm-up
        self._export(self.max_roots)
        self.stream.synchronize()
        _C.check(self.L.sgl_graph_capture_begin(sp))
        try:
            self.run_device_ptr(self.roots.data_ptr(), self.root_ts.data_ptr(), self.max_roots)
            self._export(self.max_roots)
        finally:
            ex = C.c_void_p()
            rc = self.L.sgl_graph_capture_end(sp, C.byref(ex))
        _C.check(rc)
        v = C.c_void_p
        self._exec_host, self._a_hsrc = ex, v(0)
        self._hlaunch_args = [ex, self._a_hsrc, v(self.roots_ts.data_ptr()), C.c_size_t(self.roots_ts.numel() * 8), v(sp)]
        self._launch = self.L.sgl_graph_launch
        self.stream.synchronize()
        return self

    def submit_host_ptr(self, roots_ts_host_ptr: int):
        """:meth:`submit_host` for a full batch whose roots and query times lie contiguously ([2, max_roots] int64) in
        PINNED host memory at the given address: H2D copy + the captured step, one foreign call."""
        self._n = self.max_roots
        self._a_hsrc.value = roots_ts_host_ptr
        rc = self._launch(*self._hlaunch_args)
        if rc:
            _C.check(rc)
        self.done.record(self.stream)

    def replay_ptr(self, roots_ts_ptr: int):
        """Run the captured step for a batch whose roots and query times lie contiguously ([2, max_roots] int64) at the
        given device (or pinned host) address."""
        self._a_src.value = roots_ts_ptr
        rc = self._launch(*self._launch_args)
        if rc:
            _C.check(rc)

    def replay_device(self, roots: torch.Tensor, root_ts: torch.Tensor):
        """Graph form of :meth:`run_device` for a full batch: copy the roots into the captured input buffers
        (device to device) and replay."""
        with torch.cuda.stream(self.stream):
            self.roots.copy_(roots, non_blocking=True)
            self.root_ts.copy_(root_ts, non_blocking=True)
            self._g_dev.replay()

    # ---- device-resident inputs ------------------------------------------------------------------------
    def run_device(self, roots: torch.Tensor, root_ts: torch.Tensor, rng_stream: int = 0, gather_events=None):
        """Sample + gather for roots already on the GPU.  Returns nothing: results are in ``self.offsets``,
        ``self.nbr`` ... ``self.out_feats`` (valid prefix = ``self.offsets[n]`` edges).  No synchronisation.
        ``gather_events`` = (start, end) CUDA events recorded around the gather launch (profiling hook)."""
        n = roots.numel()
        if n > self.max_roots:
            raise _C.SglError(f"batch of {n} roots exceeds max_roots={self.max_roots}")
        L, g, a, sp = self.L, self.g, self.args, self.stream.cuda_stream
        rc = L.sgl_sample_layer_fenced(g.indptr.data_ptr(), g.nbr.data_ptr(), g.ts.data_ptr(), g.eid.data_ptr(),
                                       None if g.fence is None else g.fence.data_ptr(), g.num_nodes,
                                       roots.data_ptr(), root_ts.data_ptr(), n, None, self.k, a["pol"], a["eq"], a["off"],
                                       a["keep"], a["seed"], rng_stream, self.nbr.data_ptr(), self.dst.data_ptr(),
                                       self.ts.data_ptr(), self.dt.data_ptr(), None, self.eid.data_ptr(),
                                       self.offsets.data_ptr(), self.status.ptr(), self.ws.data_ptr(), self.ws.numel(), sp)
        _C.check(rc)
        if self.feats is not None:
            if gather_events:
                gather_events[0].record(self.stream)
            d_total = self.offsets.data_ptr() + 8 * n
            rc = L.sgl_gather_rows(self.feats.data_ptr(), self.feats.shape[0], self.row_bytes, self.src_pitch,
                                   self.eid.data_ptr(), None, 0, n * self.k, d_total, self.out_feats.data_ptr(),
                                   self.row_bytes, None, None, self.mode, self.status.ptr(), sp)
            _C.check(rc)
            if gather_events:
                gather_events[1].record(self.stream)
        return n

    def sample_only(self, roots: torch.Tensor, root_ts: torch.Tensor, rng_stream: int = 0):
        """The hop without the feature gather (same buffers as :meth:`run_device`)."""
        n = roots.numel()
        if n > self.max_roots:
            raise _C.SglError(f"batch of {n} roots exceeds max_roots={self.max_roots}")
        L, g, a = self.L, self.g, self.args
        rc = L.sgl_sample_layer_fenced(g.indptr.data_ptr(), g.nbr.data_ptr(), g.ts.data_ptr(), g.eid.data_ptr(),
                                       None if g.fence is None else g.fence.data_ptr(), g.num_nodes,
                                       roots.data_ptr(), root_ts.data_ptr(), n, None, self.k, a["pol"], a["eq"], a["off"],
                                       a["keep"], a["seed"], rng_stream, self.nbr.data_ptr(), self.dst.data_ptr(),
                                       self.ts.data_ptr(), self.dt.data_ptr(), None, self.eid.data_ptr(),
                                       self.offsets.data_ptr(), self.status.ptr(), self.ws.data_ptr(), self.ws.numel(),
                                       self.stream.cuda_stream)
        _C.check(rc)

    def capture_sample_only(self):
        """Record the hop alone (full batch, this object's root buffers) as a graph; :meth:`replay_sample` then costs one
        copy + one graph launch -- for callers that gather later, and for timing the sampler without launch overhead."""
        sp = self.stream.cuda_stream
        self.roots_ts.zero_()
        torch.cuda.synchronize(self.dev)
        self.sample_only(self.roots, self.root_ts)
        self.stream.synchronize()
        _C.check(self.L.sgl_graph_capture_begin(sp))
        try:
            self.sample_only(self.roots, self.root_ts)
        finally:
            ex = C.c_void_p()
            rc = self.L.sgl_graph_capture_end(sp, C.byref(ex))
        _C.check(rc)
        v = C.c_void_p
        self._a_ssrc = v(0)
        self._slaunch_args = [ex, self._a_ssrc, v(self.roots_ts.data_ptr()), C.c_size_t(self.roots_ts.numel() * 8), v(sp)]
        self.stream.synchronize()
        return self

    def replay_sample(self, roots_ts_ptr: int):
        self._a_ssrc.value = roots_ts_ptr
        rc = self.L.sgl_graph_launch(*self._slaunch_args)
        if rc:
            _C.check(rc)

    # ---- host inputs / host results --------------------------------------------------------------------
    def submit_host(self, h_roots: torch.Tensor, h_root_ts: torch.Tensor, rng_stream: int = 0):
        """Enqueue one batch whose roots and query times are in (pinned) host tensors: H2D copy, sampling, gather,
        and the copy of the block structure (offsets, neighbour ids, timestamps, edge ids, dt) back to pinned host
        memory.  Returns immediately; :meth:`result` waits for it.  The gathered feature rows stay on the GPU
        (``self.out_feats``): their consumer is the model."""
        n = h_roots.numel()
        self._n = n
        if self._g_host is not None and n == self.max_roots and rng_stream == 0:
            # staged through this object's pinned buffers (their addresses are baked into the graph)
            self.h_roots.copy_(h_roots)
            self.h_root_ts.copy_(h_root_ts)
            with torch.cuda.stream(self.stream):
                self._g_host.replay()
                self.done.record(self.stream)
            return
        with torch.cuda.stream(self.stream):
            self.roots[:n].copy_(h_roots, non_blocking=True)
            self.root_ts[:n].copy_(h_root_ts, non_blocking=True)
            self.run_device(self.roots[:n], self.root_ts[:n], rng_stream)
            self._export(n)
            self.done.record(self.stream)

    def _export(self, n):
        """Block structure of the batch on this pipeline's stream -> pinned host mirrors: the offsets as one fixed-size
        copy, the per-edge arrays with a device-counted prefix copy (only the edges the batch really has cross PCIe,
        and the host never has to learn the count first)."""
        if self._exp_ok and self.export == "prefix":
            _C.check(self.L.sgl_copy_prefix(5, self._exp_src, self._exp_dst, self._exp_elem, self.offsets.data_ptr() + 8 * n,
                                            self.cap, self.stream.cuda_stream))
        else:   # whole-capacity copies (also when torch did not align the buffers to 16 bytes)
            self.h_blk.copy_(self.blk, non_blocking=True)
            self.h_dt.copy_(self.dt, non_blocking=True)

    def result(self):
        """(n_edges, dict of host views) of the batch submitted last; blocks until its copies have landed."""
        self.done.synchronize()
        tot = int(self._h_blk_np[self._n])
        return tot, HostBlock(self, self._n, tot)

    def run_host(self, h_roots: torch.Tensor, h_root_ts: torch.Tensor, rng_stream: int = 0):
        """Synchronous form: :meth:`submit_host` followed by :meth:`result`."""
        self.submit_host(h_roots, h_root_ts, rng_stream)
        return self.result()

    def h2d_bytes(self, n):
        return 16 * n

    def d2h_bytes(self, n_edges=None):
        """Bytes of one batch's result copy: the offsets plus 28 bytes per sampled edge (capacity when the count is
        not given)."""
        if n_edges is None or not self._exp_ok or self.export == "full":
            return self.blk.numel() * 8 + self.dt.numel() * 4
        return (self.max_roots + 1) * 8 + int(n_edges * 28)
