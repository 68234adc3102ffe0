"""Cache route over NVLink peer memory (single node): owner -> replica push of node rows without a collective
library call per step.

Same job as :class:`starrygl.cache.cache_route.CacheRoute` (reference: starrygl/cache/cache_route.py:211-277 +
starrygl/cache/NodeState.py:245-282), different transport: one kernel on the sender packs the rows
``[row | ts | slot]`` and stores them straight into the receivers' staging buffers (mapped with CUDA IPC); one
kernel on the receiver applies them to the node state.  Every rank must call :meth:`push` (and wait on the returned
future) for every step, in the same order -- an empty plan is fine.
"""
import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _C, ops
from .cache_route import CommPlan


class P2PFuture:
    def __init__(self, route, step, recv_arr, state):
        self.route, self.step, self.recv_arr, self.state = route, step, recv_arr, state
        self._done = False

    def wait(self):
        """Enqueue the receive kernel of this step on the current stream (it waits on the device, bounded, for the
        senders' rows) -- the point at which the remote writes become part of the stream's order."""
        if self._done:
            return
        self._done = True
        r, st = self.route, self.state
        has_ts = r.has_ts
        rc = r.L.sgl_p2p_route_recv(r.ctx, self.recv_arr, st._d_data.data_ptr(), st._d_data.shape[0], r.dim, int(has_ts),
                                    st._d_ts.data_ptr() if has_ts else None, self.step, r.status.ptr(), _C.stream_ptr())
        _C.check(rc)
        r._outstanding -= 1


class P2PCacheRoute:
    def __init__(self, dim: int, has_ts: bool = True, cap_rows: int = 16384, ring: int = 4,
                 device: Optional[torch.device] = None, wait_ms: int = -1, bulk_bytes: int = -1):
        """``wait_ms`` bounds every device-side wait (default 2 s); a pair's message of ``bulk_bytes`` and more travels
        as plain rows instead of tagged lines (default 2 MiB); every rank must pass the same values."""
        if not dist.is_initialized():
            raise RuntimeError("P2PCacheRoute needs an initialised process group (handles are exchanged through it)")
        self.L = _C.lib()
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.dim, self.has_ts, self.cap_rows, self.ring = int(dim), bool(has_ts), int(cap_rows), int(ring)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.pitch = ops.wire_pitch(self.dim + (1 if has_ts else 0), False)
        nbytes = self.L.sgl_p2p_buffer_bytes(self.world, self.ring, self.cap_rows, self.pitch)
        self.base = C.c_void_p()
        hbuf = C.create_string_buffer(64)
        _C.check(self.L.sgl_p2p_alloc(nbytes, C.byref(self.base), hbuf, 64))
        handles: List[bytes] = [None] * self.world
        dist.all_gather_object(handles, hbuf.raw)
        self.bases = (C.c_void_p * self.world)()
        self._opened = []
        for p in range(self.world):
            if p == self.rank:
                self.bases[p] = self.base.value
            else:
                ptr = C.c_void_p()
                _C.check(self.L.sgl_p2p_open(handles[p], C.byref(ptr)))
                self.bases[p] = ptr.value
                self._opened.append(ptr)
        self.ctx = C.c_void_p()
        _C.check(self.L.sgl_p2p_route_create(self.rank, self.world, self.ring, self.cap_rows, self.pitch, self.bases,
                                             C.byref(self.ctx)))
        _C.check(self.L.sgl_p2p_route_configure(self.ctx, int(wait_ms), int(bulk_bytes)))
        self.status = ops.StatusWord(self.device)
        self.step = 0
        self._outstanding = 0
        dist.barrier()        # every rank has mapped every buffer before the first store

    def recv_sizes(self, plan: CommPlan) -> List[int]:
        if plan.recv_sizes is None:
            if plan.send_sizes.numel() != self.world:
                raise ValueError(f"CommPlan.send_sizes has {plan.send_sizes.numel()} entries, the group has {self.world} ranks")
            from ..route.exchange import exchange_counts
            plan.recv_sizes = exchange_counts(plan.send_sizes.to(self.device))
        return plan.recv_sizes

    @torch.no_grad()
    def push(self, feats: torch.Tensor, plan: CommPlan, state, local_ts: Optional[torch.Tensor] = None) -> P2PFuture:
        """Send ``feats[plan.send_indices]`` (+ ``local_ts``) to the plan's ranks; ``state`` (a ``DistNodeState``) receives
        what the other ranks send here when the returned future is waited on."""
        if (local_ts is not None) != self.has_ts or feats.shape[1] != self.dim or feats.dtype != torch.float32:
            raise _C.SglError("P2PCacheRoute.push: row layout differs from the one the route was created for")
        if self._outstanding >= self.ring - 1:
            raise _C.SglError("P2PCacheRoute: too many steps in flight -- wait on earlier futures first")
        send_idx, remote, h_send, h_recv = self._bind(plan)
        feats = feats.contiguous()
        ts = None if local_ts is None else local_ts.contiguous()
        rc = self.L.sgl_p2p_route_send(self.ctx, feats.data_ptr(), feats.shape[0], self.dim,
                                       None if ts is None else ts.data_ptr(), send_idx.data_ptr(), remote.data_ptr(), h_send,
                                       self.step, self.status.ptr(), _C.stream_ptr())
        _C.check(rc)
        fut = P2PFuture(self, self.step, h_recv, state)
        fut._keep = (feats, ts)
        self.step += 1
        self._outstanding += 1
        return fut

    def _bind(self, plan: CommPlan):
        b = plan.__dict__.get("_p2p")
        if b is None:
            recv_list = self.recv_sizes(plan)
            b = plan.__dict__["_p2p"] = (plan.send_indices.to(self.device, torch.int64).contiguous(),
                                         plan.send_remote_indices.to(self.device, torch.int64).contiguous(),
                                         (C.c_int64 * self.world)(*plan.send_list()), (C.c_int64 * self.world)(*recv_list))
        return b

    def bind_step(self, feats: torch.Tensor, local_ts: Optional[torch.Tensor], plan: CommPlan, state, stream,
                  recv_stream=None):
        """Pre-convert every argument of ``push`` + ``wait`` for one (table, plan, state) combination and return a
        callable that runs the step (the step number is filled in per call).  With one stream the step is ONE foreign
        call; with a separate ``recv_stream`` the send kernels and the apply kernels form two independent chains
        (the apply kernel of a step only depends on the senders' tagged staging lines, not on this rank's stream order), which
        halves the per-step latency of the route."""
        send_idx, remote, h_send, h_recv = self._bind(plan)
        v = C.c_void_p
        step_a, step_b = C.c_uint64(0), C.c_uint64(0)
        f_ptr, n_rows, dim = v(feats.data_ptr()), C.c_int64(feats.shape[0]), C.c_int64(self.dim)
        ts_ptr = v(local_ts.data_ptr()) if local_ts is not None else None
        d_ptr, d_rows = v(state._d_data.data_ptr()), C.c_int64(state._d_data.shape[0])
        dts_ptr = v(state._d_ts.data_ptr()) if local_ts is not None else None
        st_ptr = v(self.status.ptr())
        keep = (feats, local_ts, send_idx, remote, state)
        if recv_stream is None:
            args = [self.ctx, f_ptr, n_rows, dim, ts_ptr, v(send_idx.data_ptr()), v(remote.data_ptr()), h_send, h_recv, d_ptr,
                    d_rows, dts_ptr, step_a, st_ptr, v(stream.cuda_stream)]
            fn = self.L.sgl_p2p_route_step

            def run(_keep=keep):
                step_a.value = self.step
                rc = fn(*args)
                if rc:
                    _C.check(rc)
                self.step += 1
            return run
        a_send = [self.ctx, f_ptr, n_rows, dim, ts_ptr, v(send_idx.data_ptr()), v(remote.data_ptr()), h_send, step_a, st_ptr,
                  v(stream.cuda_stream)]
        a_recv = [self.ctx, h_recv, d_ptr, d_rows, dim, C.c_int(1 if local_ts is not None else 0), dts_ptr, step_b, st_ptr,
                  v(recv_stream.cuda_stream)]
        f_send, f_recv = self.L.sgl_p2p_route_send, self.L.sgl_p2p_route_recv

        def run2(_keep=keep):
            step_a.value = step_b.value = self.step
            rc = f_send(*a_send) or f_recv(*a_recv)
            if rc:
                _C.check(rc)
            self.step += 1
        return run2

    # ---- plans that exist only on the device -------------------------------------------------------------------
    @torch.no_grad()
    def push_dev(self, feats: torch.Tensor, send_idx: torch.Tensor, remote_idx: torch.Tensor, d_send_sizes: torch.Tensor,
                 rows_hint: int, local_ts: Optional[torch.Tensor] = None, stream=None) -> int:
        """Send ``feats[send_idx[:sum(d_send_sizes)]]`` according to a plan whose sizes are device values
        (``ops.plan_route`` output): no host synchronisation, no count exchange.  ``rows_hint`` sizes the launch (the
        expected number of rows; any value is correct).  Returns the step number to pass to :meth:`apply_dev`."""
        if (local_ts is not None) != self.has_ts or feats.shape[1] != self.dim or feats.dtype != torch.float32:
            raise _C.SglError("P2PCacheRoute.push_dev: row layout differs from the one the route was created for")
        rc = self.L.sgl_p2p_route_send_dev(self.ctx, feats.data_ptr(), feats.shape[0], self.dim,
                                           None if local_ts is None else local_ts.data_ptr(), send_idx.data_ptr(),
                                           remote_idx.data_ptr(), d_send_sizes.data_ptr(), int(rows_hint), self.step,
                                           self.status.ptr(), _C.stream_ptr(stream))
        _C.check(rc)
        self.step += 1
        return self.step - 1

    @torch.no_grad()
    def apply_dev(self, step: int, state, rows_hint: int, stream=None):
        """Receive side of :meth:`push_dev`: applies what the other ranks pushed in ``step`` to ``state``; the row
        counts come from the senders."""
        rc = self.L.sgl_p2p_route_recv_dev(self.ctx, int(rows_hint), state._d_data.data_ptr(), state._d_data.shape[0], self.dim,
                                           int(self.has_ts), state._d_ts.data_ptr() if self.has_ts else None, int(step),
                                           self.status.ptr(), _C.stream_ptr(stream))
        _C.check(rc)

    def bind_dev(self, feats: torch.Tensor, send_idx: torch.Tensor, remote_idx: torch.Tensor, d_send_sizes: torch.Tensor,
                 rows_hint: int, local_ts: Optional[torch.Tensor], state, stream, apply_stream=None):
        """:meth:`push_dev` + :meth:`apply_dev` for buffers that stay the same from step to step (a captured step writes
        its plan and rows into fixed tensors): every argument is converted once; returns ``(send, apply)``, two
        callables without arguments that enqueue the step's send kernel on ``stream`` and its apply kernel on
        ``apply_stream`` (default: the same stream).  With two streams the pushes of a step can leave as soon as its rows
        exist, while the applies stay in step order with the caller's own table work."""
        if (local_ts is not None) != self.has_ts or feats.shape[1] != self.dim or feats.dtype != torch.float32:
            raise _C.SglError("P2PCacheRoute.bind_dev: row layout differs from the one the route was created for")
        v = C.c_void_p
        step_a, step_b = C.c_uint64(0), C.c_uint64(0)
        sp = v(stream.cuda_stream)
        a_send = [self.ctx, v(feats.data_ptr()), C.c_int64(feats.shape[0]), C.c_int64(self.dim),
                  v(local_ts.data_ptr()) if local_ts is not None else None, v(send_idx.data_ptr()), v(remote_idx.data_ptr()),
                  v(d_send_sizes.data_ptr()), C.c_int64(int(rows_hint)), step_a, v(self.status.ptr()), sp]
        a_recv = [self.ctx, C.c_int64(int(rows_hint)), v(state._d_data.data_ptr()), C.c_int64(state._d_data.shape[0]),
                  C.c_int64(self.dim), C.c_int(int(self.has_ts)), v(state._d_ts.data_ptr()) if self.has_ts else None, step_b,
                  v(self.status.ptr()), v(apply_stream.cuda_stream) if apply_stream is not None else sp]
        f_send, f_recv = self.L.sgl_p2p_route_send_dev, self.L.sgl_p2p_route_recv_dev
        keep = (feats, send_idx, remote_idx, d_send_sizes, local_ts, state)
        pending = []

        def send(_keep=keep):
            step_a.value = self.step
            rc = f_send(*a_send)
            if rc:
                _C.check(rc)
            pending.append(self.step)
            self.step += 1

        def apply():
            step_b.value = pending.pop(0)
            rc = f_recv(*a_recv)
            if rc:
                _C.check(rc)
        return send, apply

    # ---- life cycle ---------------------------------------------------------------------------------------------
    def close(self, collective: bool = True):
        """Release the context, the peer mappings and the staging buffer.  ``collective=False`` skips the barrier (for
        a process group that is already gone, e.g. inside ``__exit__`` after an error)."""
        if self.ctx:
            torch.cuda.synchronize(self.device)
            if collective and dist.is_initialized():
                dist.barrier()
            self.L.sgl_p2p_route_destroy(self.ctx)
            for p in self._opened:
                self.L.sgl_p2p_close(p)
            self.L.sgl_p2p_free(self.base)
            self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.close(collective=exc_type is None)
        return False
