"""Generate the golden vectors in this folder from the reference implementation.

Run once, in a container where the reference checkout is available (path given by
``--reference``), and commit the resulting ``*.npz`` files.  The tests only read the
``*.npz`` files; they never import the reference.

What is pinned, and the reference code that produced it:

* ``sampler_*.npz``   -- ``MaterializedMultiLayerBuilder.__init__`` (T-CSR arrays) and
  ``_sample_layer`` / ``_jit_sample_kernel`` for the ``recent`` policy
  (prepare_sample.py:32-172, :179-203, :248-265).
* ``uniform_hist.npz`` -- position histogram of the ``uniform`` policy (prepare_sample.py:120-134),
  the distribution the chi-square test compares against.  This one file is statistical: the reference draws from
  unseeded generators, so a regenerated file differs in its counts (the test compares distributions, not bytes);
  every other file regenerates bit for bit.
* ``batch_*.npz``     -- ``build_aligned_batch`` per-layer dicts (prepare_sample.py:313-406)
  with route planning disabled (it needs ``torch_scatter``, which is absent).
* ``ids.npz``         -- ``DistRouteIndex`` packing, ``build_replica_table`` +
  ``CSRReplicaTable.lookup`` (starrygl/utils/partition_book.py:7-52,
  starrygl/cache/replica_table.py:16-82,178-215).
* ``route_2rank.npz`` -- ``CacheRoute.update_with_plan`` + ``HistoryLayerUpdater`` style write-back and
  ``Route.forward`` forward/backward over a 2-rank gloo group
  (starrygl/cache/cache_route.py:211-277, starrygl/route/route.py:427-466).
* ``plan.npz``        -- ``_compute_layer_route`` (prepare_sample.py:266-310) for every partition of a 4-way split.
* ``mail.npz``        -- ``mailbox.get_update_mail`` (starrygl/nn/memory/mailbox.py:56-84) on batches with distinct
  timestamps per node entry (``torch_scatter`` is absent: its ``scatter_max`` is a torch restatement, so the tie case
  stored beside them is defined by that restatement, not by the reference).
* ``slots.npz``       -- complete slot files of ``build_aligned_batch`` INCLUDING the per-layer ``comm_plan``
  (prepare_sample.py:313-406) for every partition of a 3-way split, read back from the ``.pt`` file the reference wrote.
* ``nodestate.npz``   -- ``DistNodeState.update`` / ``__getitem__`` with ``node_mode='map'``
  (starrygl/cache/NodeState.py:36-61, starrygl/utils/partition_book.py:98-133).
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _stub(name, **attrs):
    m = types.ModuleType(name)
    for k, v in attrs.items():
        setattr(m, k, v)
    sys.modules[name] = m
    return m


def load_prepare_sample(ref):
    _stub("torch_scatter")
    _stub("dgl")
    spec = importlib.util.spec_from_file_location("ref_prepare_sample", os.path.join(ref, "prepare_sample.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    import numba
    numba.set_num_threads(min(8, os.cpu_count() or 1))
    return mod


META = {'start_offset': -1, 'end_offset': 0, 'graph_type': 'c'}


def graph_tiny():
    src = np.array([1, 2, 3, 4, 5, 6, 0, 0], dtype=np.int64)
    dst = np.array([0, 0, 0, 0, 0, 0, 7, 7], dtype=np.int64)
    ts = np.array([10, 20, 20, 30, 40, 50, 25, 35], dtype=np.int64)
    return 8, src, dst, ts, np.arange(8, dtype=np.int64)


def graph_random(seed, n, m, tmax, shuffle):
    rng = np.random.default_rng(seed)
    # skewed degrees so that some rows are long and many are empty
    w = 1.0 / np.arange(1, n + 1) ** 1.1
    w /= w.sum()
    dst = rng.choice(n, size=m, p=w).astype(np.int64)
    src = rng.integers(0, n, m).astype(np.int64)
    ts = rng.integers(0, tmax, m).astype(np.int64)
    if not shuffle:
        ts = np.sort(ts)
    eid = rng.permutation(m).astype(np.int64)
    return n, src, dst, ts, eid


def gen_sampler(mod, out):
    B = mod.MaterializedMultiLayerBuilder
    cases = {
        "tiny": graph_tiny(),
        "rand_sorted": graph_random(1, 300, 6000, 5000, False),
        "rand_ties": graph_random(2, 64, 4000, 50, True),   # many equal timestamps, unsorted input
    }
    for name, (n, src, dst, ts, eid) in cases.items():
        b = B({'src': src, 'dst': dst, 'ts': ts, 'eid': eid}, n, None, None, 0, 1)
        rng = np.random.default_rng(7)
        rec = {"n": np.int64(n), "src": src, "dst": dst, "ts": ts, "eid": eid,
               "indptr": b.full_indptr, "s_src": b.sorted_src, "s_ts": b.sorted_ts, "s_eid": b.sorted_eid}
        if name == "tiny":
            q = np.array([0, 7, 3] * 6, dtype=np.int64)
            qt = np.repeat(np.array([5, 10, 20, 21, 30, 51], dtype=np.int64), 3)
        else:
            nq = 400
            q = rng.integers(0, n, nq).astype(np.int64)
            qt = rng.integers(0, int(ts.max()) + 3, nq).astype(np.int64)
        rec["q"], rec["qt"] = q, qt
        for k in (1, 3, 10):
            for end_offset in (0, 1):
                meta = dict(META, end_offset=end_offset)
                o = b._sample_layer(q, qt, k, 'recent', meta)
                tag = f"recent_k{k}_e{end_offset}"
                if o[0] is None:
                    o = (np.zeros(0, np.int64), np.zeros(0, np.int64), np.zeros(0, np.int64),
                         np.zeros(0, np.float32), np.zeros(0, np.int64))
                for nm, a in zip(("src", "dst", "ts", "dt", "eid"), o):
                    rec[f"{tag}_{nm}"] = a
        np.savez_compressed(os.path.join(out, f"sampler_{name}.npz"), **rec)

    # uniform policy: histogram of sampled positions for one row with 30 candidates, k = 10
    n = 4
    m = 30
    src = np.arange(m, dtype=np.int64) + 100
    dst = np.zeros(m, dtype=np.int64)
    ts = np.arange(m, dtype=np.int64)
    b = B({'src': src, 'dst': dst, 'ts': ts}, n, None, None, 0, 1)
    trials = 4000
    q = np.zeros(trials, dtype=np.int64)
    qt = np.full(trials, 1000, dtype=np.int64)
    o = b._sample_layer(q, qt, 10, 'uniform', META)
    hist = np.bincount(o[4], minlength=m).astype(np.int64)   # eid == position here
    per_root = np.bincount(o[1], minlength=trials)
    assert (per_root == 10).all()
    # ascending position inside each root, no repeats
    pos = o[4].reshape(trials, 10)
    assert (np.diff(pos, axis=1) > 0).all()
    np.savez_compressed(os.path.join(out, "uniform_hist.npz"), hist=hist, trials=np.int64(trials),
                        k=np.int64(10), cands=np.int64(m))


def gen_batches(mod, out):
    import torch
    B = mod.MaterializedMultiLayerBuilder
    B._compute_layer_route = lambda self, n, t: None
    cap = {}
    real_save = mod.torch.save               # ``mod.torch`` is the torch module itself: put it back when done
    mod.torch.save = lambda obj, path: cap.__setitem__('obj', obj)
    cases = {
        "tiny": (graph_tiny(), (np.array([1, 0]), np.array([0, 7]), np.array([30, 40])), [2, 2]),
        "rand": (graph_random(3, 200, 5000, 3000, False), None, [3, 2]),
        "rand_k10": (graph_random(4, 500, 20000, 100000, False), None, [10, 10]),
    }
    for name, (g, task, fanouts) in cases.items():
        n, src, dst, ts, eid = g
        b = B({'src': src, 'dst': dst, 'ts': ts, 'eid': eid}, n, None, None, 0, 1)
        if task is None:
            rng = np.random.default_rng(11)
            pick = np.sort(rng.choice(len(src), 40, replace=False))
            task = (src[pick], dst[pick], ts[pick])
        tsrc, tdst, tts = [np.asarray(a, dtype=np.int64) for a in task]
        cfg = {'meta': META, 'layer': [{'type': 'recent', 'fanout': f} for f in fanouts]}
        b.build_aligned_batch(('link', (tsrc, tdst, tts, np.ones_like(tsrc), np.arange(len(tsrc)))), "x", cfg, 1, None, None)
        rec = {"n": np.int64(n), "src": src, "dst": dst, "ts": ts, "eid": eid,
               "task_src": tsrc, "task_dst": tdst, "task_ts": tts, "fanouts": np.array(fanouts, dtype=np.int64),
               "num_layers": np.int64(len(cap['obj']))}
        for i, d in enumerate(cap['obj']):
            for k, v in d.items():
                if isinstance(v, torch.Tensor):
                    rec[f"L{i}_{k}"] = v.numpy()
        np.savez_compressed(os.path.join(out, f"batch_{name}.npz"), **rec)
    mod.torch.save = real_save


def _route_worker(rank, world, ref, port, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ref)
    het = _stub("dgl.heterograph", DGLBlock=object)
    _stub("dgl", heterograph=het)
    comm = _stub("starrygl.lib.libstarrygl_comm", DistContext=object, init_p2p=lambda *a: None)
    _stub("starrygl.lib", libstarrygl_comm=comm)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from starrygl.cache.cache_route import CommPlan, CacheRoute
    from starrygl.route.route import Route

    rng = np.random.default_rng(100 + rank)
    D = 5
    nloc = 12
    feats = torch.from_numpy(rng.standard_normal((nloc, D + 1)).astype(np.float32))
    # plan: rank 0 sends 3 rows to rank 1 and 1 row to itself; rank 1 sends 2 rows to rank 0
    if rank == 0:
        send_ranks = torch.tensor([0, 1, 1, 1])
        send_sizes = torch.tensor([1, 3])
        send_indices = torch.tensor([4, 0, 7, 7])
        send_remote = torch.tensor([9, 2, 5, 11])
    else:
        send_ranks = torch.tensor([0, 0])
        send_sizes = torch.tensor([2, 0])
        send_indices = torch.tensor([3, 10])
        send_remote = torch.tensor([1, 6])
    plan = CommPlan(send_ranks=send_ranks, send_sizes=send_sizes, send_indices=send_indices,
                    send_remote_indices=send_remote)
    data = torch.zeros(nloc, D)
    tsv = torch.zeros(nloc)

    def cb(idx, rows, mode):
        data[idx] = rows[:, :-1]
        tsv[idx] = rows[:, -1]
    futs = CacheRoute().update_with_plan(feats, plan, cb)
    for f in futs:
        f.wait()
    res = {"feats": feats.numpy(), "send_sizes": send_sizes.numpy(), "send_indices": send_indices.numpy(),
           "send_remote": send_remote.numpy(), "data": data.numpy(), "ts": tsv.numpy()}

    # Route forward / backward (halo exchange)
    if rank == 0:
        r = Route(send_sizes=[1, 2], recv_sizes=[1, 1], send_index=torch.tensor([2, 0, 3]))
    else:
        r = Route(send_sizes=[1, 2], recv_sizes=[2, 2], send_index=torch.tensor([1, 4, 1]))
    x = torch.from_numpy(rng.standard_normal((5, 3)).astype(np.float32)).requires_grad_()
    y = r.forward(x)
    w = torch.from_numpy(rng.standard_normal(tuple(y.shape)).astype(np.float32))
    (y * w).sum().backward()
    res.update({"r_send_sizes": np.array(r.send_sizes), "r_recv_sizes": np.array(r.recv_sizes),
                "r_send_index": r.send_index.numpy(), "x": x.detach().numpy(), "y": y.detach().numpy(),
                "w": w.numpy(), "gx": x.grad.numpy()})
    q.put((rank, res))
    dist.barrier()
    dist.destroy_process_group()


def gen_route(ref, out):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_route_worker, args=(r, world, ref, 29611, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join()
    rec = {}
    for r in range(world):
        for k, v in got[r].items():
            rec[f"r{r}_{k}"] = v
    np.savez_compressed(os.path.join(out, "route_2rank.npz"), **rec)


def gen_ids(ref, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ref)
    het = _stub("dgl.heterograph", DGLBlock=object)
    _stub("dgl", heterograph=het)
    comm = _stub("starrygl.lib.libstarrygl_comm", DistContext=object, init_p2p=lambda *a: None)
    _stub("starrygl.lib", libstarrygl_comm=comm)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = "29612"
    dist.init_process_group("gloo", rank=0, world_size=1)
    from starrygl.cache.replica_table import build_replica_table
    from starrygl.utils.partition_book import DistRouteIndex, PartitionState
    from starrygl.cache.NodeState import DistNodeState

    rng = np.random.default_rng(5)
    loc = torch.from_numpy(rng.integers(0, 2 ** 48, 64))
    part = torch.from_numpy(rng.integers(0, 2 ** 14, 64))
    d = DistRouteIndex(loc, part)
    shared_idx = torch.from_numpy(np.sort(rng.choice(64, 20, replace=False)))
    d.set_shared(shared_idx)
    rec = {"loc": loc.numpy(), "part": part.numpy(), "shared_idx": shared_idx.numpy(), "dist": d.dist.numpy(),
           "u_loc": d.loc.numpy(), "u_part": d.part.numpy(), "u_shared": d.is_shared.numpy()}

    N, P = 200, 4
    book = []
    for p in range(P):
        owned = np.arange(p * 50, (p + 1) * 50)
        halo = rng.choice(np.setdiff1d(np.arange(N), owned), 30, replace=False)
        book.append(torch.from_numpy(np.concatenate([owned, halo])))
        rec[f"book{p}"] = book[-1].numpy()
    rt = build_replica_table(N, book, P)
    rec.update({"rt_indptr": rt.indptr.numpy(), "rt_ranks": rt.indices.numpy(), "rt_locs": rt.locs.numpy()})
    ids = torch.from_numpy(rng.integers(0, N, 37))
    s, r, l = rt.lookup(ids)
    rec.update({"lk_ids": ids.numpy(), "lk_src": s.numpy(), "lk_ranks": r.numpy(), "lk_locs": l.numpy()})
    np.savez_compressed(os.path.join(out, "ids.npz"), **rec)

    # DistNodeState update / read
    loc_ids = torch.from_numpy(rng.permutation(100)[:40].astype(np.int64))
    ps = PartitionState(loc_ids=loc_ids, num_master_nums=25, node_mode='map', num_nodes=100)
    ns = DistNodeState(ps, 6, pinned=False)
    upd = torch.from_numpy(rng.permutation(100)[:50].astype(np.int64))     # some not stored locally
    vals = torch.from_numpy(rng.standard_normal((50, 6)).astype(np.float32))
    uts = torch.from_numpy(rng.integers(0, 1000, 50).astype(np.float32))
    ns.update(upd, vals, uts)
    rd = loc_ids[torch.from_numpy(rng.integers(0, 40, 33))]
    got, got_ts = ns[rd]
    np.savez_compressed(os.path.join(out, "nodestate.npz"), loc_ids=loc_ids.numpy(), num_nodes=np.int64(100),
                        upd=upd.numpy(), vals=vals.numpy(), uts=uts.numpy(), data=ns.data.numpy(), ts=ns.ts.numpy(),
                        rd=rd.numpy(), got=got.numpy(), got_ts=got_ts.numpy(),
                        is_master=ps.is_master_node_by_global(rd).numpy())
    dist.destroy_process_group()


def gen_plan(ref, out):
    """``_compute_layer_route`` (prepare_sample.py:266-310) on sorted unique (id, ts) layer lists.  ``torch_scatter`` is
    absent here, so its ``scatter_max`` is supplied as a torch restatement (max per group, index of the first
    maximum); on these inputs every (id, ts) pair is unique, so no tie can occur and the choice does not matter."""
    import torch
    sys.path.insert(0, ref)
    het = _stub("dgl.heterograph", DGLBlock=object)
    _stub("dgl", heterograph=het)
    comm = _stub("starrygl.lib.libstarrygl_comm", DistContext=object, init_p2p=lambda *a: None)
    _stub("starrygl.lib", libstarrygl_comm=comm)

    def scatter_max(src, index, dim=0):
        n = int(index.max()) + 1 if index.numel() else 0
        mx = torch.full((n,), torch.iinfo(src.dtype).min, dtype=src.dtype).scatter_reduce(0, index, src, "amax")
        is_max = src == mx[index]
        pos = torch.where(is_max, torch.arange(len(src)), torch.full((len(src),), len(src)))
        arg = torch.full((n,), len(src), dtype=torch.long).scatter_reduce(0, index, pos, "amin")
        return mx, arg
    _stub("torch_scatter", scatter_max=scatter_max)
    spec = importlib.util.spec_from_file_location("ref_prepare_sample2", os.path.join(ref, "prepare_sample.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    from starrygl.cache.cache_route import CommPlan
    from starrygl.cache.replica_table import build_replica_table
    mod.CommPlan = CommPlan
    rng = np.random.default_rng(21)
    N, P = 500, 4
    node_parts = torch.from_numpy(rng.integers(0, P, N))
    book = []
    for p in range(P):
        owned = torch.nonzero(node_parts == p)[:, 0].numpy()
        halo = rng.choice(np.setdiff1d(np.arange(N), owned), 120, replace=False)
        book.append(torch.from_numpy(np.concatenate([owned, halo])))
    rt = build_replica_table(N, book, P)
    rec = {"N": np.int64(N), "P": np.int64(P), "node_parts": node_parts.numpy(), "rt_indptr": rt.indptr.numpy(),
           "rt_ranks": rt.indices.numpy(), "rt_locs": rt.locs.numpy()}
    e = np.zeros(1, np.int64)
    for case in range(3):
        n_pairs = [400, 40, 1500][case]
        ids = rng.integers(0, N, n_pairs)
        ts = rng.integers(0, 1000, n_pairs)
        pairs = np.unique(np.stack([ids, ts], 1), axis=0)          # sorted by id, then ts
        for pid in range(P):
            b = mod.MaterializedMultiLayerBuilder({'src': e, 'dst': e, 'ts': e}, N, node_parts, rt, pid, P)
            plan = b._compute_layer_route(pairs[:, 0].copy(), pairs[:, 1].copy())
            tag = f"c{case}_p{pid}"
            rec[f"{tag}_ids"], rec[f"{tag}_ts"] = pairs[:, 0], pairs[:, 1]
            if plan is None:
                rec[f"{tag}_none"] = np.int64(1)
                continue
            rec[f"{tag}_send_ranks"] = plan.send_ranks.numpy()
            rec[f"{tag}_send_sizes"] = plan.send_sizes.numpy()
            rec[f"{tag}_send_indices"] = plan.send_indices.numpy()
            rec[f"{tag}_send_remote"] = plan.send_remote_indices.numpy()
    np.savez_compressed(os.path.join(out, "plan.npz"), **rec)


def gen_slots(ref, out):
    """``build_aligned_batch`` with route planning ON, written by the reference with ``torch.save`` and read back."""
    import tempfile
    import torch
    sys.path.insert(0, ref)
    het = _stub("dgl.heterograph", DGLBlock=object)
    _stub("dgl", heterograph=het)
    comm = _stub("starrygl.lib.libstarrygl_comm", DistContext=object, init_p2p=lambda *a: None)
    _stub("starrygl.lib", libstarrygl_comm=comm)

    def scatter_max(src, index, dim=0):
        n = int(index.max()) + 1 if index.numel() else 0
        mx = torch.full((n,), torch.iinfo(src.dtype).min, dtype=src.dtype).scatter_reduce(0, index, src, "amax")
        is_max = src == mx[index]
        pos = torch.where(is_max, torch.arange(len(src)), torch.full((len(src),), len(src)))
        arg = torch.full((n,), len(src), dtype=torch.long).scatter_reduce(0, index, pos, "amin")
        return mx, arg
    _stub("torch_scatter", scatter_max=scatter_max)
    spec = importlib.util.spec_from_file_location("ref_prepare_sample3", os.path.join(ref, "prepare_sample.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    from starrygl.cache.cache_route import CommPlan
    from starrygl.cache.replica_table import build_replica_table
    mod.CommPlan = CommPlan
    rng = np.random.default_rng(41)
    N, P, M = 300, 3, 6000
    node_parts = torch.from_numpy(rng.integers(0, P, N))
    book = []
    for p in range(P):
        owned = torch.nonzero(node_parts == p)[:, 0].numpy()
        halo = rng.choice(np.setdiff1d(np.arange(N), owned), 90, replace=False)
        book.append(torch.from_numpy(np.concatenate([owned, halo])))
    rt = build_replica_table(N, book, P)
    src, dst = rng.integers(0, N, M), rng.integers(0, N, M)
    ts = np.sort(rng.integers(0, 50000, M)).astype(np.int64)
    eid = rng.permutation(M).astype(np.int64)
    rec = {"N": np.int64(N), "P": np.int64(P), "node_parts": node_parts.numpy(), "rt_indptr": rt.indptr.numpy(),
           "rt_ranks": rt.indices.numpy(), "rt_locs": rt.locs.numpy(), "src": src, "dst": dst, "ts": ts, "eid": eid}
    pick = np.sort(rng.choice(M, 60, replace=False))
    cases = [("link", [3, 2], 0), ("node", [5], 1), ("link", [4, 4], 1)]
    rec["n_cases"] = np.int64(len(cases))
    for c, (kind, fanouts, end_offset) in enumerate(cases):
        cfg = {'meta': {'start_offset': -1, 'end_offset': end_offset, 'graph_type': 'c'},
               'layer': [{'type': 'recent', 'fanout': f} for f in fanouts]}
        if kind == "link":
            task = ('link', (src[pick], dst[pick], ts[pick], np.ones(len(pick), np.int64), eid[pick]))
        else:
            task = ('node', (dst[pick], ts[pick], np.zeros(len(pick), np.int64)))
        rec[f"c{c}_kind"], rec[f"c{c}_fanouts"], rec[f"c{c}_end_offset"] = np.array(kind), np.array(fanouts), np.int64(end_offset)
        rec[f"c{c}_pick"] = pick
        for pid in range(P):
            b = mod.MaterializedMultiLayerBuilder({'src': src, 'dst': dst, 'ts': ts, 'eid': eid}, N, node_parts, rt, pid, P)
            with tempfile.TemporaryDirectory() as d:
                path = os.path.join(d, "slot_0000_sub_0000.pt")
                b.build_aligned_batch(task, path, cfg, 1, None, None)
                data = torch.load(path, weights_only=False)
            tag = f"c{c}_p{pid}"
            rec[f"{tag}_num_layers"] = np.int64(len(data))
            for i, dct in enumerate(data):
                for k, v in dct.items():
                    if isinstance(v, torch.Tensor):
                        rec[f"{tag}_L{i}_{k}"] = v.numpy()
                    elif isinstance(v, (int, np.integer)):
                        rec[f"{tag}_L{i}_{k}"] = np.int64(v)
            plans = data[0]["comm_plan"]
            rec[f"{tag}_num_plans"] = np.int64(len(plans))
            for i, pl in enumerate(plans):
                if pl is None:
                    rec[f"{tag}_plan{i}_none"] = np.int64(1)
                    continue
                rec[f"{tag}_plan{i}_send_ranks"] = pl.send_ranks.numpy()
                rec[f"{tag}_plan{i}_send_sizes"] = pl.send_sizes.numpy()
                rec[f"{tag}_plan{i}_send_indices"] = pl.send_indices.numpy()
                rec[f"{tag}_plan{i}_send_remote"] = pl.send_remote_indices.numpy()
    np.savez_compressed(os.path.join(out, "slots.npz"), **rec)


def gen_mail(ref, out):
    """Runs the reference's ``mailbox.get_update_mail`` on CPU tensors."""
    import torch
    sys.path.insert(0, ref)

    def scatter_max(src, index, dim=0):
        n = int(index.max()) + 1 if index.numel() else 0
        mx = torch.full((n,), -float("inf"), dtype=src.dtype).scatter_reduce(0, index, src, "amax")
        is_max = src == mx[index]
        pos = torch.where(is_max, torch.arange(len(src)), torch.full((len(src),), len(src)))
        arg = torch.full((n,), len(src), dtype=torch.long).scatter_reduce(0, index, pos, "amin")
        return mx, arg
    _stub("torch_scatter", scatter_max=scatter_max)
    ctx = _stub("starrygl.utils.context", DistributedContext=object)
    _stub("starrygl.utils", context=ctx)
    _stub("starrygl", utils=sys.modules["starrygl.utils"])
    spec = importlib.util.spec_from_file_location("ref_mailbox", os.path.join(ref, "starrygl", "nn", "memory", "mailbox.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rng = np.random.default_rng(31)
    rec = {}
    for case, (n_nodes, B, D, E, ties, emb) in enumerate([(50, 40, 8, 5, False, 0), (2000, 300, 32, 172, False, 0),
                                                         (300, 200, 16, 0, False, 1), (300, 200, 16, 7, False, 2),
                                                         (30, 120, 4, 3, True, 0)]):
        mb = mod.mailbox(n_nodes, 1, D, E)
        half = n_nodes // 2
        src = rng.integers(0, half, B)
        dst = rng.integers(half, n_nodes, B)           # bipartite: an event never has the same node at both ends
        ts = rng.integers(0, 50, B) if ties else rng.permutation(100000)[:B]
        ts = np.sort(ts).astype(np.int64)
        mem_src = rng.standard_normal((B, D)).astype(np.float32)
        mem_dst = rng.standard_normal((B, D)).astype(np.float32)
        ef = rng.standard_normal((B, E)).astype(np.float32) if E else None
        embedding = rng.standard_normal((2 * B, D)).astype(np.float32) if emb else None
        kw = {}
        if emb:
            kw = dict(embedding=torch.from_numpy(embedding), use_src_emb=emb >= 1, use_dst_emb=emb >= 2)
        index, mail, mail_ts = mb.get_update_mail(torch.from_numpy(src), torch.from_numpy(dst), torch.from_numpy(ts),
                                                  torch.from_numpy(ef) if E else None, torch.from_numpy(mem_src),
                                                  torch.from_numpy(mem_dst), **kw)
        t = f"c{case}"
        rec.update({f"{t}_n_nodes": np.int64(n_nodes), f"{t}_src": src, f"{t}_dst": dst, f"{t}_ts": ts, f"{t}_mem_src": mem_src,
                    f"{t}_mem_dst": mem_dst, f"{t}_ties": np.int64(ties), f"{t}_emb": np.int64(emb),
                    f"{t}_index": index.numpy(), f"{t}_mail": mail.numpy(), f"{t}_mail_ts": mail_ts.numpy()})
        if E:
            rec[f"{t}_ef"] = ef
        if emb:
            rec[f"{t}_embedding"] = embedding
    rec["n_cases"] = np.int64(5)
    np.savez_compressed(os.path.join(out, "mail.npz"), **rec)
    for k in [k for k in sys.modules if k == "starrygl" or k.startswith("starrygl.")]:
        del sys.modules[k]


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", default="all")
    a = ap.parse_args()
    if a.only in ("all", "route"):
        gen_route(a.reference, HERE)
    if a.only in ("all", "sampler"):
        mod = load_prepare_sample(a.reference)
        gen_sampler(mod, HERE)
        gen_batches(mod, HERE)
    if a.only in ("all", "ids"):
        gen_ids(a.reference, HERE)
    if a.only in ("all", "plan"):
        gen_plan(a.reference, HERE)
    if a.only in ("all", "slots"):
        gen_slots(a.reference, HERE)
    if a.only in ("all", "mail"):
        gen_mail(a.reference, HERE)
    print("golden vectors written to", HERE)
