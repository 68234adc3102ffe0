"""Halo exchange between graph partitions with autograd support.

Mirrors starrygl/route/route.py (``Route`` :21-354, ``RouteAgent`` :357-382, ``RouteSendFuncion`` /
``RouteRecvFunction`` :385-416, ``RouteContext`` :420-510).  Forward: every rank sends the rows
``x[send_index]`` (grouped by destination) and appends what it receives after its own rows.  Reverse /
backward: the appended tail travels back and is accumulated into ``x[send_index]`` peer segment by peer segment.
Pack is one gather kernel writing the send buffer; the receive lands directly in the tail of the pre-allocated
result (no ``torch.cat`` copy of the received rows); the reverse accumulation is one kernel per peer segment.
"""
import asyncio
from typing import List, Optional, Tuple, Union

import torch
import torch.autograd as autograd
import torch.distributed as dist
from torch import Tensor

from .. import ops
from ..utils.partition_book import DistRouteIndex
from .timer import EventTimer


class Route:
    def __init__(self, send_sizes: List[int], recv_sizes: List[int], send_index: Optional[Tensor] = None,
                 group: Optional[dist.ProcessGroup] = None, task=None) -> None:
        self.send_sizes = send_sizes
        self.recv_sizes = recv_sizes
        self.send_index = send_index
        self.group = group

    @classmethod
    def get_timer(cls) -> EventTimer:
        if not hasattr(cls, "_timer_"):
            setattr(cls, "_timer_", EventTimer())
        return getattr(cls, "_timer_")

    @property
    def send_len(self) -> int:
        return sum(self.send_sizes)

    @property
    def recv_len(self) -> int:
        return sum(self.recv_sizes)

    def forward(self, x: Tensor, reverse: bool = False, group=None) -> Tensor:
        group = self.group if group is None else group
        return RouteAgent(self, reverse=reverse, group=group).forward(x)

    async def async_forward(self, x: Tensor, reverse: bool = False, group=None) -> Tensor:
        group = self.group if group is None else group
        return await RouteAgent(self, reverse=reverse, group=group).async_forward(x)

    def send(self, x: Tensor, reverse: bool = False, group=None) -> Tensor:
        group = self.group if group is None else group
        return RouteAgent(self, reverse=reverse, group=group).send(x)

    def recv(self, ctx: Tensor) -> Tensor:
        return RouteAgent.recv(ctx)

    def pin_memory(self, device=None):
        return type(self)(send_index=self.send_index.pin_memory(), send_sizes=self.send_sizes,
                          recv_sizes=self.recv_sizes, group=self.group)

    def to(self, device=None, dtype=None, non_blocking=False, copy=False):
        return type(self)(send_index=self.send_index.to(device=device, dtype=dtype, non_blocking=non_blocking, copy=copy),
                          send_sizes=self.send_sizes, recv_sizes=self.recv_sizes, group=self.group)

    def __getstate__(self):
        return {"send_sizes": self.send_sizes, "recv_sizes": self.recv_sizes, "send_index": self.send_index}

    def __setstate__(self, state):
        self.send_sizes, self.recv_sizes, self.send_index = state["send_sizes"], state["recv_sizes"], state["send_index"]
        self.group = None

    def __repr__(self):
        p = len(self.send_sizes) if self.send_sizes else -1
        return f"{type(self).__name__}(parts={p})"

    @classmethod
    def all_to_all_ind2ptr(cls, dist_index: Union[Tensor, DistRouteIndex], group=None):
        """Build a route from packed (partition, local) ids: rows are sorted by owner partition (stable), the
        owners learn which of their rows are wanted.  Returns (route, recv_ind, sort_idx)."""
        if isinstance(dist_index, Tensor):
            dist_index = DistRouteIndex(dist_index)
        device = dist_index.device
        world_size = dist.get_world_size(group)
        part = dist_index.part
        sort_idx = torch.argsort(part, stable=True)
        sorted_loc = dist_index.loc[sort_idx]
        send_counts = torch.bincount(part, minlength=world_size)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        send_list, recv_list = send_counts.tolist(), recv_counts.tolist()
        recv_ind = torch.empty(sum(recv_list), dtype=sorted_loc.dtype, device=device)
        dist.all_to_all_single(recv_ind, sorted_loc, output_split_sizes=recv_list, input_split_sizes=send_list, group=group)
        route = cls(send_sizes=send_list, recv_sizes=recv_list, send_index=sorted_loc, group=group)
        return route, recv_ind, sort_idx

    @classmethod
    async def all_to_all_ind2ptr_async(cls, dist_index, group=None):
        route, recv_ind, sort_idx = cls.all_to_all_ind2ptr(dist_index, group)
        await asyncio.sleep(0.0)
        return route, recv_ind, sort_idx, None

    def prune(self, dst_m: Tensor, group=None):
        """Restrict the route to the rows selected by the boolean mask ``dst_m`` (and to what is still received)."""
        assert dst_m.dtype == torch.bool, f"dst_m must be a boolean tensor, but got {dst_m.dtype}"
        with torch.no_grad():
            src_m = self.forward(dst_m.float().unsqueeze(-1), group=group).squeeze(-1) != 0
        dst_ind = torch.arange(dst_m.numel(), dtype=torch.long, device=dst_m.device)
        src_ind = torch.arange(src_m.numel(), dtype=torch.long, device=src_m.device)
        send_index, send_sizes, recv_index, recv_sizes = [], [], [], []
        dst_s, src_s = 0, dst_m.numel()
        for i in range(len(self.send_sizes)):
            x = self.send_index[dst_s:dst_s + self.send_sizes[i]]
            x = x[dst_m[x]]
            send_index.append(x)
            send_sizes.append(x.numel())
            y = src_ind[src_s:src_s + self.recv_sizes[i]]
            y = y[src_m[y]]
            recv_index.append(y)
            recv_sizes.append(y.numel())
            dst_s += self.send_sizes[i]
            src_s += self.recv_sizes[i]
        route = type(self)(send_index=torch.cat(send_index, dim=0), send_sizes=send_sizes, recv_sizes=recv_sizes)
        route.group = self.group
        return route, src_m, torch.cat([dst_ind] + recv_index, dim=0)


class RouteAgent:
    def __init__(self, route: Route, reverse: bool = False, group=None) -> None:
        self.route, self.group, self.reverse = route, group, reverse

    def forward(self, x: Tensor) -> Tensor:
        if self.route.send_index is None:
            return x
        return self.recv(self.send(x))

    async def async_forward(self, x: Tensor) -> Tensor:
        if self.route.send_index is None:
            return x
        ctx = self.send(x)
        await asyncio.sleep(0.0)
        return self.recv(ctx)

    def send(self, x: Tensor) -> Tensor:
        if self.route.send_index is None:
            raise RuntimeError("Empty route is unsupported for send")
        return RouteSendFuncion.apply(x, self.route, self.reverse, self.group)

    @staticmethod
    def recv(ctx: Tensor) -> Tensor:
        return RouteRecvFunction.apply(ctx)


class RouteSendFuncion(autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, route: Route, reverse: bool = False, group=None):
        r_ctx = RouteContext(route, reverse=reverse, group=group)
        r_ctx.forward_send(x)
        ret = torch.empty(0, dtype=torch.float32, device="cpu")
        ret._r_ctx = r_ctx
        ctx.saved_r_ctx = r_ctx
        return ret

    @staticmethod
    def backward(ctx, _):
        return ctx.saved_r_ctx.backward_recv(), None, None, None


class RouteRecvFunction(autograd.Function):
    @staticmethod
    def forward(ctx, key: Tensor):
        r_ctx: RouteContext = key._r_ctx
        ctx.saved_r_ctx = r_ctx
        return r_ctx.forward_recv()

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        ctx.saved_r_ctx.backward_send(grad_output)
        return torch.empty(0, dtype=torch.float32, device="cpu")


class RouteContext:
    def __init__(self, route: Route, reverse: bool = False, group=None):
        self.route = route
        self.group = dist.GroupMember.WORLD if group is None else group
        self.reverse = reverse
        self.task: Union[Tensor, Tuple, None] = None

    def _send_impl(self, x: Tensor):
        x = x.contiguous()
        n = x.size(0)
        # result = [own rows | received rows]; the collective writes straight into the tail
        res = torch.empty(n + self.route.recv_len, *x.shape[1:], dtype=x.dtype, device=x.device)
        res[:n].copy_(x)
        y = ops.gather_rows(x, self.route.send_index.to(x.device))
        work = dist.all_to_all_single(res[n:], y, self.route.recv_sizes, self.route.send_sizes, group=self.group,
                                      async_op=True)
        return res, None, work

    def _send_post(self, res: Tensor, _, work):
        with Route.get_timer().record():
            work.wait()
        return res

    def _recv_impl(self, x: Tensor):
        x = x.contiguous()
        n = x.size(0) - self.route.recv_len
        head, tail = x[:n], x[n:]
        outs = torch.empty(self.route.send_len, *x.shape[1:], dtype=x.dtype, device=x.device)
        work = dist.all_to_all_single(outs, tail, self.route.send_sizes, self.route.recv_sizes, group=self.group,
                                      async_op=True)
        return head, outs, work

    def _recv_post(self, x: Tensor, outs: Tensor, work):
        with Route.get_timer().record():
            work.wait()
        if x.dtype != torch.float32:
            raise RuntimeError("reverse route accumulates float32 rows")
        idx = self.route.send_index.to(x.device)
        s = 0
        for sz in self.route.send_sizes:   # peer order = the reference's summation order
            ops.route_add_rows(x, idx[s:s + sz], outs[s:s + sz])
            s += sz
        return x

    @torch.no_grad()
    def forward_send(self, x: Tensor):
        assert self.task is None
        x = x.detach()
        self.task = self._recv_impl(x) if self.reverse else self._send_impl(x)

    @torch.no_grad()
    def forward_recv(self):
        assert not isinstance(self.task, Tensor)
        x = self._recv_post(*self.task) if self.reverse else self._send_post(*self.task)
        self.task = None
        return x

    @torch.no_grad()
    def backward_send(self, g: Tensor):
        assert self.task is None
        g = g.detach()
        self.task = self._send_impl(g) if self.reverse else self._recv_impl(g.clone())

    @torch.no_grad()
    def backward_recv(self):
        assert not isinstance(self.task, Tensor)
        g = self._send_post(*self.task) if self.reverse else self._recv_post(*self.task)
        self.task = None
        return g
