"""Mini-batch prefetcher on the GPU: sampling + feature gather of the next batches run while the model consumes the
current one.

The reference's training scripts import a ``HostToDevicePrefetcher`` (``starrygl.data.prefetcher``, used at
test/test_offline.py:137-140 as ``HostToDevicePrefetcher(loader=..., device=..., ...)``) that is not part of the
reference tree; its job -- hide the data path behind the model -- is done here with ``depth`` pre-bound
:class:`~starrygl.graph.pipeline.SampleGatherPipeline` objects, each on its own stream.  ``loader`` yields the roots
of one mini-batch as ``(roots, query_times)`` int64 tensors (CUDA, or pinned host memory) of at most ``max_roots``
entries.  Iterating yields :class:`PrefetchedBatch` objects in loader order, already ordered into the consumer's
current stream; a batch's tensors alias the buffers of its pipeline object and may be read by kernels enqueued on that
stream until ``depth`` further batches have been requested.
"""
from collections import deque
from typing import Iterable, Optional

import torch

from .. import ops
from ..graph.pipeline import SampleGatherPipeline


class PrefetchedBatch:
    """Block structure and gathered edge-feature rows of one mini-batch (device tensors, capacity-sized; the valid
    prefix has ``offsets[n_roots]`` edges -- :meth:`num_edges` reads it, one synchronisation)."""

    def __init__(self, pipe: SampleGatherPipeline, n_roots: int, ready: torch.cuda.Event):
        self.pipe, self.n_roots, self.ready = pipe, n_roots, ready
        self.offsets, self.nbr, self.dst, self.ts, self.eid, self.dt = (pipe.offsets[:n_roots + 1], pipe.nbr, pipe.dst,
                                                                        pipe.ts, pipe.eid, pipe.dt)
        self.edge_feats = pipe.out_feats

    def wait(self, stream: Optional[torch.cuda.Stream] = None):
        """Make ``stream`` (default: the current one) wait for this batch -- no host blocking."""
        (stream or torch.cuda.current_stream()).wait_event(self.ready)
        return self

    def num_edges(self) -> int:
        self.ready.synchronize()
        return int(self.offsets[self.n_roots].item())


class HostToDevicePrefetcher:
    def __init__(self, loader: Iterable, g: ops.TCSR, edge_feats: Optional[torch.Tensor], fanout: int,
                 policy: str = "recent", max_roots: int = 4096, depth: int = 4, device=None, **sampler_options):
        self.loader, self.depth = loader, max(1, int(depth))
        self.streams = [torch.cuda.Stream(g.device) for _ in range(self.depth)]
        self.pipes = [SampleGatherPipeline(g, edge_feats, fanout, policy, max_roots, stream=s, **sampler_options)
                      for s in self.streams]
        self.events = [torch.cuda.Event() for _ in range(self.depth)]

    def _submit(self, slot, roots, root_ts):
        pipe, st = self.pipes[slot], self.streams[slot]
        # Orders the slot's reuse behind everything the consumer has enqueued so far on its stream: the work on the
        # batch that occupied this slot (handed out ``depth`` batches ago) and the kernels that produced ``roots``.
        # The batch submitted now is only needed ``depth`` requests later, so this does not stall the consumer.
        st.wait_stream(torch.cuda.current_stream())
        n = roots.numel()
        with torch.cuda.stream(st):
            if not roots.is_cuda:
                pipe.roots[:n].copy_(roots, non_blocking=True)
                pipe.root_ts[:n].copy_(root_ts, non_blocking=True)
                roots, root_ts = pipe.roots[:n], pipe.root_ts[:n]
            pipe.run_device(roots.contiguous(), root_ts.contiguous())
            self.events[slot].record(st)
        return PrefetchedBatch(pipe, n, self.events[slot])

    def __iter__(self):
        it = iter(self.loader)
        queue = deque()
        slot = 0
        for roots, root_ts in it:
            if len(queue) == self.depth:
                yield queue.popleft().wait()
            queue.append(self._submit(slot, roots, root_ts))
            slot = (slot + 1) % self.depth
        while queue:
            yield queue.popleft().wait()

    def check(self):
        for p in self.pipes:
            p.status.check("prefetcher")
