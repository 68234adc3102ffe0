"""Loader-side handling of materialised mini-batches: a dataset over slot files, a sampler that keeps the files of a slot
together, and the collator that merges several files into one batch.

The reference's training scripts import ``AtomicDataset``, ``SlotAwareSampler`` and ``collate_and_merge`` from
``starrygl.data.batches`` (test/test_offline.py:21, :118-140) but the module is not part of the reference tree; the
names and the call shapes used there (``AtomicDataset(...)[i]``, ``SlotAwareSampler`` as a ``DataLoader`` sampler,
``partial(collate_and_merge, world_size=...)`` as ``collate_fn``) are kept, the behaviour is defined here:

A file holds the list of per-layer dictionaries ``build_aligned_batch`` writes (layer 0: ``gids``, ``ts``, ``inv_map``,
task tensors, ``comm_plan`` = one plan or ``None`` per layer list; layer l+1: ``indptr``, ``indices``, ``eid``,
``edge_ts``, ``edge_dt``, ``gids``, ``ts``).  ``collate_and_merge`` puts the files of a batch side by side -- a block-
diagonal merge: every file keeps its own node lists (nothing is deduplicated across files, so every file's local
indices stay valid after a shift), the lists of a layer are concatenated in file order, ``inv_map`` / ``indices`` /
the plans' ``send_indices`` are shifted by the offset of their file's list, row pointers are chained, and the plans of
a layer are regrouped by destination rank (stable: file order inside a rank) with their sizes added up.  Pure index
arithmetic on the tensors as loaded (CPU); the result is moved to the GPU by the prefetcher in one copy per tensor.
"""
import glob
import os
import re
from typing import Dict, Iterator, List, Optional, Sequence

import torch
from torch.utils.data import Dataset, Sampler

from ..cache.cache_route import CommPlan


class AtomicDataset(Dataset):
    """The slot files of one partition directory (``slot_XXXX_sub_YYYY.pt``, prepare_nparts_louvain.py:444-451), ordered
    by (slot, sub); item i = the loaded list of layer dictionaries of file i."""

    _NAME = re.compile(r"slot_(\d+)_sub_(\d+)\.pt$")

    def __init__(self, root: str, files: Optional[Sequence[str]] = None):
        if files is None:
            files = glob.glob(os.path.join(root, "slot_*_sub_*.pt"))
        keyed = []
        for f in files:
            m = self._NAME.search(os.path.basename(f))
            if m:
                keyed.append((int(m.group(1)), int(m.group(2)), f))
        keyed.sort()
        self.files = [f for _, _, f in keyed]
        self.slots = [s for s, _, _ in keyed]

    def __len__(self):
        return len(self.files)

    def __getitem__(self, i):
        return torch.load(self.files[i], weights_only=False)


class SlotAwareSampler(Sampler):
    """Yields file indices slot by slot, in time order (slots are consecutive windows of the event stream, so training
    visits them in order); ``batch_slots`` consecutive slots form one batch when the sampler is used as a batch sampler
    through :meth:`batches`."""

    def __init__(self, dataset: AtomicDataset, batch_slots: int = 1):
        self.dataset, self.batch_slots = dataset, max(int(batch_slots), 1)

    def __iter__(self) -> Iterator[int]:
        return iter(range(len(self.dataset)))

    def __len__(self):
        return len(self.dataset)

    def batches(self) -> Iterator[List[int]]:
        cur, first = [], None
        for i, s in enumerate(self.dataset.slots):
            if first is None:
                first = s
            if s - first >= self.batch_slots:
                yield cur
                cur, first = [], s
            cur.append(i)
        if cur:
            yield cur


class MergedBatch:
    """Result of :func:`collate_and_merge`: ``layers`` (the merged per-layer dictionaries), ``routes`` (one merged
    ``CommPlan`` or ``None`` per layer list), ``roots`` (the task tensors of layer 0, concatenated) and ``file_ptr``
    (per layer: row offsets of every file's list inside the merged list)."""

    def __init__(self, layers, routes, roots, file_ptr):
        self.layers, self.routes, self.roots, self.file_ptr = layers, routes, roots, file_ptr

    def to(self, device, non_blocking=True):
        mv = lambda v: v.to(device, non_blocking=non_blocking) if torch.is_tensor(v) else v
        self.layers = [{k: mv(v) for k, v in d.items()} for d in self.layers]
        self.roots = {k: mv(v) for k, v in self.roots.items()}
        self.routes = [None if r is None else r.to(device, non_blocking) for r in self.routes]
        return self


def _merge_plans(plans: List[Optional[CommPlan]], offsets: List[int], world_size: int) -> Optional[CommPlan]:
    ranks, idx, rem = [], [], []
    for p, off in zip(plans, offsets):
        if p is None or p.send_indices.numel() == 0:
            continue
        if p.send_sizes.numel() != world_size:
            raise ValueError(f"a plan was built for {p.send_sizes.numel()} ranks, the batch is merged for {world_size}")
        ranks.append(p.send_ranks)
        idx.append(p.send_indices + off)
        rem.append(p.send_remote_indices)
    if not ranks:
        return None
    ranks, idx, rem = torch.cat(ranks), torch.cat(idx), torch.cat(rem)
    order = torch.argsort(ranks, stable=True)
    return CommPlan(send_ranks=ranks[order], send_sizes=torch.bincount(ranks, minlength=world_size), send_indices=idx[order],
                    send_remote_indices=rem[order])


def collate_and_merge(samples: List[List[dict]], world_size: int = 1) -> Optional[MergedBatch]:
    """Merge the files of one batch (see the module docstring).  Files may have different numbers of layers (a file
    whose sampling stopped early contributes empty blocks to the deeper layers)."""
    samples = [s for s in samples if s]
    if not samples:
        return None
    depth = max(len(s) for s in samples)
    i64 = torch.int64
    z = lambda dt=i64: torch.zeros(0, dtype=dt)
    layers, routes, file_ptr = [], [], []
    # row offset of every file's list, per layer
    list_len = [[(s[l]["gids"].numel() if l < len(s) else 0) for s in samples] for l in range(depth)]
    for l in range(depth):
        offs = [0]
        for n in list_len[l]:
            offs.append(offs[-1] + n)
        file_ptr.append(torch.tensor(offs, dtype=i64))
    # layer 0
    l0 = {"gids": torch.cat([s[0]["gids"] for s in samples]), "ts": torch.cat([s[0]["ts"] for s in samples]),
          "inv_map": torch.cat([s[0]["inv_map"] + int(file_ptr[0][f]) for f, s in enumerate(samples)])}
    layers.append(l0)
    roots: Dict[str, object] = {"num_neg": samples[0][0].get("num_neg", 0), "inv_map": l0["inv_map"]}
    for k in samples[0][0]:
        if k.startswith("task_"):
            vals = [s[0].get(k) for s in samples]
            if all(torch.is_tensor(v) for v in vals):
                roots[k] = torch.cat([v.reshape(-1) if v.dim() == 0 else v for v in vals])
            else:
                roots[k] = vals
    routes.append(_merge_plans([(s[0].get("comm_plan") or [None])[0] for s in samples], file_ptr[0][:-1].tolist(), world_size))
    # deeper layers
    for l in range(1, depth):
        ptr_parts, idx, eid, ets, edt, gid, ts = [], [], [], [], [], [], []
        e_off = 0
        for f, s in enumerate(samples):
            n_prev = list_len[l - 1][f]
            if l < len(s) and s[l]["indptr"].numel() == n_prev + 1:
                d = s[l]
                ptr_parts.append(d["indptr"][:-1] + e_off)
                idx.append(d["indices"] + int(file_ptr[l][f]))
                eid.append(d["eid"]), ets.append(d["edge_ts"]), edt.append(d["edge_dt"])
                gid.append(d["gids"]), ts.append(d["ts"])
                e_off += int(d["indices"].numel())
            else:                                   # this file has no (or an empty) layer l: rows without edges
                ptr_parts.append(torch.full((n_prev,), e_off, dtype=i64))
        ptr_parts.append(torch.tensor([e_off], dtype=i64))
        layers.append({"indptr": torch.cat(ptr_parts), "indices": torch.cat(idx) if idx else z(), "eid": torch.cat(eid) if eid else z(),
                       "edge_ts": torch.cat(ets) if ets else z(), "edge_dt": torch.cat(edt) if edt else z(torch.float32),
                       "gids": torch.cat(gid) if gid else z(), "ts": torch.cat(ts) if ts else z()})
        plans = []
        for s in samples:
            cp = s[0].get("comm_plan") or []
            plans.append(cp[l] if (l < len(cp) and l < len(s)) else None)
        routes.append(_merge_plans(plans, file_ptr[l][:-1].tolist(), world_size))
    return MergedBatch(layers, routes, roots, file_ptr)
