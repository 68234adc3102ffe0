"""Host-side logic of the route layer on two CPU ranks (gloo): split sizes, segment order, the fused wire
format, receive-count caching, autograd of the halo exchange, and a rank that fails.  The CUDA kernels are
replaced by CPU stand-ins (tests/route_fakes.py) -- this file checks the multi-rank control flow, the kernels
themselves are checked on the GPU against the same golden vectors."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _init(rank, world, port):
    for p in (ROOT, os.path.join(ROOT, "starrygl-framework_b200"), HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import route_fakes
    route_fakes.install()


def _worker_golden(rank, world, port, q):
    try:
        _init(rank, world, port)
        from starrygl.cache.cache_route import CacheRoute, CommPlan
        from starrygl.route.route import Route
        z = np.load(os.path.join(HERE, "golden", "route_2rank.npz"))
        t = lambda k: torch.from_numpy(z[f"r{rank}_{k}"])
        feats = t("feats")
        plan = CommPlan(send_ranks=torch.repeat_interleave(torch.arange(world), t("send_sizes")), send_sizes=t("send_sizes"),
                        send_indices=t("send_indices"), send_remote_indices=t("send_remote"))
        data, ts = torch.zeros_like(t("data")), torch.zeros_like(t("ts"))

        # (1) drop-in form: the caller concatenated [emb | ts] itself and brings a generic callback
        def cb(idx, rows, mode):
            assert mode == "cold"
            data[idx] = rows[:, :-1]
            ts[idx] = rows[:, -1]
        futs = CacheRoute().update_with_plan(feats, plan, cb)
        for f in futs:
            f.wait()
        ok1 = torch.equal(data, t("data")) and torch.equal(ts, t("ts"))
        assert plan.recv_sizes is not None            # cached: a second use of the plan exchanges no counts
        # (2) fused form: embedding and ts separate, receive side applied by the state object in one call
        data2, ts2 = torch.zeros_like(data), torch.zeros_like(ts)

        class State:
            def write_wire(self, wire, width):
                import route_fakes
                route_fakes.route_unpack(wire, width, data2, ts2)

        def cb2(idx, rows, mode):
            raise AssertionError("fused path must not call the generic callback")
        cb2.fused_state = State()
        for f in CacheRoute().update_with_plan(feats[:, :-1].contiguous(), plan, cb2, local_ts=feats[:, -1].contiguous()):
            f.wait()
        ok2 = torch.equal(data2, t("data")) and torch.equal(ts2, t("ts"))
        # (3) halo exchange forward + backward
        r = Route(send_sizes=t("r_send_sizes").tolist(), recv_sizes=t("r_recv_sizes").tolist(), send_index=t("r_send_index"))
        x = t("x").clone().requires_grad_()
        y = r.forward(x)
        (y * t("w")).sum().backward()
        ok3 = torch.equal(y.detach(), t("y")) and torch.allclose(x.grad, t("gx"), rtol=0, atol=0)
        # (4) empty plan on one rank still takes part in the collective
        e = CommPlan.empty(world) if rank == 0 else CommPlan(send_ranks=torch.tensor([0]), send_sizes=torch.tensor([1, 0]),
                                                              send_indices=torch.tensor([2]), send_remote_indices=torch.tensor([5]))
        got = {}

        def cb3(idx, rows, mode):
            got["idx"], got["rows"] = idx.clone(), rows.clone()
        for f in CacheRoute().update_with_plan(feats, e, cb3):
            f.wait()
        ok4 = (rank == 1 and not got) or (rank == 0 and got["idx"].tolist() == [5])
        # (5) a plan whose split array does not have one entry per rank is refused on the host, before any collective
        bad = CommPlan(send_ranks=torch.empty(0, dtype=torch.long), send_sizes=torch.empty(0, dtype=torch.long),
                       send_indices=torch.empty(0, dtype=torch.long), send_remote_indices=torch.empty(0, dtype=torch.long))
        try:
            CacheRoute().update_with_plan(feats, bad, cb3)
            ok4 = False
        except ValueError:
            pass
        # (6) distributed gather in the reference's five steps (ids by owner, id exchange, owner gather, row exchange,
        # original order) against the oracle's restatement
        from oracle import oracle_np as O
        from starrygl.lib.libstarrygl_comm import ShardTensor
        shards = [np.random.default_rng(40 + r).standard_normal((30 + 7 * r, 5)).astype(np.float32) for r in range(world)]
        rg = np.random.default_rng(60 + rank)
        part = rg.integers(0, world, 50)
        loc = np.array([rg.integers(0, shards[p].shape[0]) for p in part])
        ids = O.dist_pack(loc, part)
        got_rows = ShardTensor.gather_by_exchange(torch.from_numpy(shards[rank]), torch.from_numpy(ids))
        ok4 = ok4 and np.array_equal(got_rows.numpy(), O.shard_gather(shards, ids, rank))
        q.put((rank, ok1, ok2, ok3, ok4, None))
    except Exception as ex:  # pragma: no cover
        import traceback
        q.put((rank, False, False, False, False, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _spawn(fn, world=2, port=29641, timeout=120):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=fn, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=timeout) for _ in range(world)]
    for p in procs:
        p.join(timeout)
    return sorted(out)


def test_route_two_ranks_matches_reference():
    for rank, ok1, ok2, ok3, ok4, err in _spawn(_worker_golden):
        assert err is None, err
        assert ok1, f"rank {rank}: drop-in cache route differs from the reference"
        assert ok2, f"rank {rank}: fused cache route differs from the reference"
        assert ok3, f"rank {rank}: halo exchange forward/backward differs from the reference"
        assert ok4, f"rank {rank}: empty-plan exchange / plan validation / distributed gather"


def _worker_failure(rank, world, port, q):
    """Rank 1 raises before posting its collective; rank 0 must get an error from a short group timeout instead of
    waiting forever (failure is injected on the host, nothing faults)."""
    try:
        for p in (ROOT, os.path.join(ROOT, "starrygl-framework_b200"), HERE):
            if p not in sys.path:
                sys.path.insert(0, p)
        import datetime
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        import route_fakes
        route_fakes.install()
        from starrygl.cache.cache_route import CacheRoute, CommPlan
        dist.barrier()
        if rank == 1:
            q.put((rank, "left"))
            return
        plan = CommPlan(send_ranks=torch.tensor([1]), send_sizes=torch.tensor([0, 1]), send_indices=torch.tensor([0]),
                        send_remote_indices=torch.tensor([0]))
        try:
            for f in CacheRoute().update_with_plan(torch.zeros(2, 3), plan, lambda *a: None):
                f.wait()
            q.put((rank, "no error"))
        except Exception as ex:
            q.put((rank, "error: " + type(ex).__name__))
    except Exception as ex:  # pragma: no cover
        q.put((rank, "setup failed: " + repr(ex)))


def test_peer_that_never_joins_surfaces_as_error():
    res = dict(_spawn(_worker_failure, port=29642))
    assert res[1] == "left"
    assert res[0].startswith("error"), res[0]


def test_commplan_api():
    sys.path.insert(0, os.path.join(ROOT, "starrygl-framework_b200"))
    from starrygl.cache.cache_route import CommPlan
    e = CommPlan.empty(4)
    with pytest.raises(ValueError):
        CommPlan.empty(0)
    assert e.is_empty() and repr(e) == "CommPlan(Empty)" and e.send_sizes.tolist() == [0, 0, 0, 0]
    p = CommPlan(send_ranks=torch.tensor([0, 2, 2]), send_sizes=torch.tensor([1, 0, 2]), send_indices=torch.tensor([4, 5, 6]),
                 send_remote_indices=torch.tensor([1, 2, 3]))
    assert not p.is_empty() and "3 items -> 2 parts" in repr(p) and p.send_list() == [1, 0, 2]
