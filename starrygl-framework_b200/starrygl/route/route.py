"""Halo exchange between graph partitions, differentiable.

Public surface of starrygl/route/route.py (``Route`` :21-354, ``RouteAgent`` :357-382, ``RouteContext`` :420-510,
``RouteSendFuncion`` / ``RouteRecvFunction`` :385-416): a route knows which of this rank's rows the other ranks want
(``send_index``, grouped by destination, ``send_sizes``) and how many rows arrive from each of them
(``recv_sizes``).

  halo   (forward of a plain route, backward of a reversed one)
         out = [ x ; rows received ]   where every rank sends x[send_index]
  fold   (forward of a reversed route, backward of a plain one)
         out = x[:n] with the tail x[n:] sent back to the owners and added onto x[send_index]

How it runs here: the pack is one gather kernel writing the send buffer, the exchange is one grouped send/recv enqueued
on the current stream by the library's own communicator and lands directly in the tail of the pre-allocated result
(CPU ranks: ``all_to_all_single``), and the fold accumulates ALL peers' rows in one kernel that adds the contributions
of a row in peer order -- the float32 sums equal those of a per-peer loop bit for bit.  The split-phase API
(``send`` now, ``recv`` later) hands a ticket tensor from one call to the other; both phases are nodes of the autograd
graph, so gradients flow through the exchange with the roles of the two operations swapped.
"""
import asyncio
from typing import List, Optional, Union

import torch
import torch.distributed as dist
from torch import Tensor

from .. import ops
from ..utils.partition_book import DistRouteIndex
from .exchange import exchange_counts, exchange_rows
from .timer import EventTimer


class Route:
    def __init__(self, send_sizes: List[int], recv_sizes: List[int], send_index: Optional[Tensor] = None,
                 group: Optional[dist.ProcessGroup] = None, task=None) -> None:
        self.send_sizes = send_sizes
        self.recv_sizes = recv_sizes
        self.send_index = send_index
        self.group = group
        self._per_device = {}          # device -> (send_index there, fold grouping there)

    # ---- sizes ---------------------------------------------------------------------------------------------------
    @property
    def send_len(self) -> int:
        return sum(self.send_sizes)

    @property
    def recv_len(self) -> int:
        return sum(self.recv_sizes)

    @classmethod
    def get_timer(cls) -> EventTimer:
        t = cls.__dict__.get("_timer_")
        if t is None:
            t = EventTimer()
            cls._timer_ = t
        return t

    # ---- the exchange ------------------------------------------------------------------------------------------------
    def forward(self, x: Tensor, reverse: bool = False, group=None) -> Tensor:
        return RouteAgent(self, reverse=reverse, group=group or self.group).forward(x)

    async def async_forward(self, x: Tensor, reverse: bool = False, group=None) -> Tensor:
        return await RouteAgent(self, reverse=reverse, group=group or self.group).async_forward(x)

    def send(self, x: Tensor, reverse: bool = False, group=None) -> Tensor:
        return RouteAgent(self, reverse=reverse, group=group or self.group).send(x)

    def recv(self, ctx: Tensor) -> Tensor:
        return RouteAgent.recv(ctx)

    # ---- placement / pickling ------------------------------------------------------------------------------------
    def _rebuilt(self, send_index):
        return type(self)(self.send_sizes, self.recv_sizes, send_index, self.group)

    def pin_memory(self, device=None):
        return self._rebuilt(self.send_index.pin_memory())

    def to(self, device=None, dtype=None, non_blocking=False, copy=False):
        return self._rebuilt(self.send_index.to(device=device, dtype=dtype, non_blocking=non_blocking, copy=copy))

    def __getstate__(self):
        return {"send_sizes": self.send_sizes, "recv_sizes": self.recv_sizes, "send_index": self.send_index}

    def __setstate__(self, state):
        self.__init__(state["send_sizes"], state["recv_sizes"], state["send_index"], None)

    def __repr__(self):
        return f"{type(self).__name__}(parts={len(self.send_sizes) if self.send_sizes else -1})"

    def _on(self, device):
        """(send_index, fold grouping) on ``device``, built on first use and kept."""
        hit = self._per_device.get(device)
        if hit is None:
            idx = self.send_index.to(device).contiguous()
            hit = self._per_device[device] = (idx, ops.route_groups(idx) if idx.is_cuda else None)
        return hit

    # ---- construction from packed (partition, local) ids ---------------------------------------------------------
    @classmethod
    def all_to_all_ind2ptr(cls, dist_index: Union[Tensor, DistRouteIndex], group=None):
        """Route that fetches the rows named by ``dist_index`` from their owners.  The ids are ordered by owner
        (stable), every owner learns which of its rows are wanted.  Returns ``(route, recv_ind, sort_idx)``:
        ``route.send_index`` = the wanted local rows in owner order (what THIS rank asks for), ``recv_ind`` = the local
        rows the other ranks ask this rank for, ``sort_idx`` = the permutation that ordered ``dist_index``."""
        if isinstance(dist_index, Tensor):
            dist_index = DistRouteIndex(dist_index)
        world = dist.get_world_size(group)
        owner = dist_index.part
        sort_idx = torch.argsort(owner, stable=True)
        wanted = dist_index.loc[sort_idx].contiguous()
        ask = torch.bincount(owner, minlength=world)
        asked = exchange_counts(ask, group)                      # rows every other rank wants from me
        ask = [int(v) for v in ask.tolist()]
        recv_ind = torch.empty(sum(asked), dtype=wanted.dtype, device=wanted.device)
        exchange_rows(wanted, ask, recv_ind, asked, group).wait()
        return cls(send_sizes=ask, recv_sizes=asked, send_index=wanted, group=group), recv_ind, sort_idx

    @classmethod
    async def all_to_all_ind2ptr_async(cls, dist_index, group=None):
        out = cls.all_to_all_ind2ptr(dist_index, group)
        await asyncio.sleep(0.0)
        return (*out, None)

    def prune(self, dst_m: Tensor, group=None):
        """Keep only the rows selected by the boolean mask ``dst_m`` over this rank's rows.  Returns the smaller route,
        the mask over [own rows ; halo rows] and the indices of the rows that remain in that concatenation."""
        if dst_m.dtype != torch.bool:
            raise AssertionError(f"dst_m must be a boolean tensor, but got {dst_m.dtype}")
        n = dst_m.numel()
        with torch.no_grad():
            src_m = self.forward(dst_m.float().unsqueeze(-1), group=group).squeeze(-1) != 0
        halo_kept = src_m[n:]
        keep_send = dst_m[self.send_index]
        send_bounds = torch.tensor([0] + list(self.send_sizes)).cumsum(0).tolist()
        recv_bounds = torch.tensor([0] + list(self.recv_sizes)).cumsum(0).tolist()
        send_sizes = [int(keep_send[a:b].sum()) for a, b in zip(send_bounds[:-1], send_bounds[1:])]
        recv_sizes = [int(halo_kept[a:b].sum()) for a, b in zip(recv_bounds[:-1], recv_bounds[1:])]
        route = type(self)(send_sizes, recv_sizes, self.send_index[keep_send], self.group)
        kept_halo = torch.nonzero(halo_kept).reshape(-1) + n
        return route, src_m, torch.cat([torch.arange(n, dtype=torch.long, device=dst_m.device), kept_halo])


class _InFlight:
    """One started exchange: the buffers it fills and what is left to do once the rows have arrived."""
    __slots__ = ("kind", "work", "result", "incoming", "route", "device")

    def __init__(self, kind, work, result, incoming, route, device):
        self.kind, self.work, self.result, self.incoming, self.route, self.device = kind, work, result, incoming, route, device

    def complete(self) -> Tensor:
        with Route.get_timer().record():
            self.work.wait()
        if self.kind == "fold":
            if self.result.dtype != torch.float32:
                raise RuntimeError("reverse route accumulates float32 rows")
            idx, groups = self.route._on(self.device)
            if groups is not None and self.result.is_cuda:
                ops.route_add_grouped(self.result, groups, self.incoming)
            else:                                  # CPU ranks of the host-logic tests: peer by peer
                s = 0
                for sz in self.route.send_sizes:
                    ops.route_add_rows(self.result, idx[s:s + sz], self.incoming[s:s + sz])
                    s += sz
        return self.result


def _start_halo(route: Route, x: Tensor, group) -> _InFlight:
    x = x.contiguous()
    n = x.size(0)
    idx, _ = route._on(x.device)
    out = torch.empty((n + route.recv_len,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    out[:n].copy_(x)
    outgoing = ops.gather_rows(x, idx)
    work = exchange_rows(outgoing, route.send_sizes, out[n:], route.recv_sizes, group)
    fl = _InFlight("halo", work, out, None, route, x.device)
    fl.incoming = outgoing           # keeps the send buffer alive until the exchange has been waited on
    return fl


def _start_fold(route: Route, x: Tensor, group) -> _InFlight:
    x = x.contiguous()
    n = x.size(0) - route.recv_len
    incoming = torch.empty((route.send_len,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    work = exchange_rows(x[n:], route.recv_sizes, incoming, route.send_sizes, group)
    # the accumulation must not touch the caller's tensor
    return _InFlight("fold", work, x[:n].clone(), incoming, route, x.device)


class RouteContext:
    """State of one split-phase exchange and of its gradient.  ``reverse`` selects fold instead of halo."""

    def __init__(self, route: Route, reverse: bool = False, group=None):
        self.route = route
        self.group = dist.GroupMember.WORLD if group is None else group
        self.reverse = reverse
        self.task: Optional[_InFlight] = None

    def _begin(self, x: Tensor, fold: bool):
        if self.task is not None:
            raise AssertionError("an exchange of this context is still in flight")
        start = _start_fold if fold else _start_halo
        with torch.no_grad():
            self.task = start(self.route, x.detach(), self.group)

    def _end(self) -> Tensor:
        if self.task is None:
            raise AssertionError("no exchange in flight")
        with torch.no_grad():
            out = self.task.complete()
        self.task = None
        return out

    def forward_send(self, x: Tensor):
        self._begin(x, fold=self.reverse)

    def forward_recv(self) -> Tensor:
        return self._end()

    def backward_send(self, g: Tensor):
        self._begin(g, fold=not self.reverse)

    def backward_recv(self) -> Tensor:
        return self._end()


class RouteSendFuncion(torch.autograd.Function):
    """Phase one: starts the exchange and returns the ticket (an empty tensor that carries the context)."""

    @staticmethod
    def forward(ctx, x: Tensor, route: Route, reverse: bool = False, group=None):
        rc = RouteContext(route, reverse=reverse, group=group)
        rc.forward_send(x)
        ticket = x.new_empty(0)
        ticket._route_context = rc
        ctx.rc = rc
        return ticket

    @staticmethod
    def backward(ctx, _ticket_grad):
        return ctx.rc.backward_recv(), None, None, None


class RouteRecvFunction(torch.autograd.Function):
    """Phase two: completes the exchange the ticket stands for; its gradient starts the opposite exchange."""

    @staticmethod
    def forward(ctx, ticket: Tensor):
        rc = getattr(ticket, "_route_context", None)
        if rc is None:
            raise RuntimeError("recv() needs the tensor that send() returned")
        ctx.rc = rc
        return rc.forward_recv()

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        ctx.rc.backward_send(grad_out)
        return grad_out.new_zeros(0)


class RouteAgent:
    def __init__(self, route: Route, reverse: bool = False, group=None) -> None:
        self.route, self.group, self.reverse = route, group, reverse

    def send(self, x: Tensor) -> Tensor:
        if self.route.send_index is None:
            raise RuntimeError("Empty route is unsupported for send")
        return RouteSendFuncion.apply(x, self.route, self.reverse, self.group)

    @staticmethod
    def recv(ctx: Tensor) -> Tensor:
        return RouteRecvFunction.apply(ctx)

    def forward(self, x: Tensor) -> Tensor:
        if self.route.send_index is None:
            return x
        return self.recv(self.send(x))

    async def async_forward(self, x: Tensor) -> Tensor:
        if self.route.send_index is None:
            return x
        ticket = self.send(x)
        await asyncio.sleep(0.0)
        return self.recv(ticket)
