"""Process-group context: the thin part of the reference's ``DistributedContext`` the data path calls
(starrygl/utils/context.py:32-123 -- ``init``, ``get_default_context``, ``device``, ``local_rank``)."""
import os
from typing import Optional

import torch
import torch.distributed as dist


class DistributedContext:
    _default: Optional["DistributedContext"] = None

    def __init__(self, backend: str, device: torch.device, rank: int, world_size: int, local_rank: int):
        self.backend, self.device = backend, device
        self.rank, self.world_size, self.local_rank = rank, world_size, local_rank
        self.group = dist.GroupMember.WORLD if dist.is_initialized() else None
        self.cpu_group = None

    @classmethod
    def init(cls, backend: str = "nccl", use_cpu_group: bool = False) -> "DistributedContext":
        """One process per GPU.  RANK / WORLD_SIZE / LOCAL_RANK come from the launcher (torchrun);
        a single process without them gets a one-rank group."""
        rank = int(os.environ.get("RANK", os.environ.get("OMPI_COMM_WORLD_RANK", 0)))
        world = int(os.environ.get("WORLD_SIZE", os.environ.get("OMPI_COMM_WORLD_SIZE", 1)))
        local = int(os.environ.get("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", 0)))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend == "nccl":
            if not torch.cuda.is_available():
                raise RuntimeError("backend 'nccl' needs a CUDA device")
            torch.cuda.set_device(local)
            device = torch.device("cuda", local)
        else:
            device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
        if not dist.is_initialized():
            kw = {"device_id": device} if backend == "nccl" else {}
            dist.init_process_group(backend, rank=rank, world_size=world, **kw)
        ctx = cls(backend, device, rank, world, local)
        if use_cpu_group and backend != "gloo":
            ctx.cpu_group = dist.new_group(backend="gloo")
        cls._default = ctx
        return ctx

    @classmethod
    def get_default_context(cls) -> "DistributedContext":
        if cls._default is None:
            if torch.cuda.is_available():
                dev = torch.device("cuda", torch.cuda.current_device())
            else:
                dev = torch.device("cpu")
            r = dist.get_rank() if dist.is_initialized() else 0
            w = dist.get_world_size() if dist.is_initialized() else 1
            cls._default = cls("none", dev, r, w, dev.index or 0)
        return cls._default

    def barrier(self):
        if dist.is_initialized():
            dist.barrier()

    @classmethod
    def shutdown(cls):
        cls._default = None
        from ..cache.cache_route import CacheRouteManager, NativeComm
        NativeComm.shutdown()
        CacheRouteManager.reset()
        if dist.is_initialized():
            dist.destroy_process_group()
