"""Cache route and halo route over NCCL on two GPUs (one process per GPU) against the reference's golden vectors.
Skipped on a single-GPU box; the same control flow is covered on CPU ranks in test_route_gloo.py."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _collect(q, procs, timeout=180):
    """Results of the two ranks; the children this test started are ended (by their own pids) whatever happens, so
    that a rank that waits for ever cannot keep its GPU after the test has failed."""
    try:
        return sorted(q.get(timeout=timeout) for _ in procs)
    finally:
        for p in procs:
            p.join(30)
            if p.is_alive():
                p.terminate()
                p.join(10)


def _worker(rank, world, port, q):
    try:
        import torch.distributed as dist
        for p in (ROOT, os.path.join(ROOT, "starrygl-framework_b200"), HERE):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", RANK=str(rank),
                          WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
        from starrygl.utils.context import DistributedContext
        ctx = DistributedContext.init("nccl")
        dev = ctx.device
        from starrygl.cache.cache_route import CacheRouteManager, CommPlan
        from starrygl.cache.NodeState import DistNodeState, HistoryLayerUpdater
        from starrygl.utils.partition_book import PartitionState
        from starrygl.route.route import Route
        z = np.load(os.path.join(HERE, "golden", "route_2rank.npz"))
        t = lambda k: torch.from_numpy(z[f"r{rank}_{k}"]).to(dev)
        feats = t("feats")
        n_loc, D = feats.shape[0], feats.shape[1] - 1
        plan = CommPlan(send_ranks=torch.repeat_interleave(torch.arange(world), torch.from_numpy(z[f"r{rank}_send_sizes"])),
                        send_sizes=torch.from_numpy(z[f"r{rank}_send_sizes"]), send_indices=t("send_indices"),
                        send_remote_indices=t("send_remote"))
        ps = PartitionState(loc_ids=torch.arange(n_loc, device=dev), num_master_nums=n_loc, node_mode='identity', num_nodes=n_loc)
        state = DistNodeState(ps, D, device=dev)
        upd = HistoryLayerUpdater([state])
        # owners write locally first (rows they send), then push; the golden state only holds the REMOTE writes,
        # so compare on the slots the reference wrote and check the local write separately
        emb, ets = feats[:, :D].contiguous(), feats[:, D].contiguous()
        own = torch.arange(n_loc, device=dev)
        futs = upd.update_embedding_and_broadcast(0, emb, ets, plan, own)
        for f in futs:
            f.wait()
        torch.cuda.synchronize()
        ref_d, ref_t = t("data"), t("ts")
        written = ref_d.abs().sum(1) > 0
        ok_remote = torch.equal(state.data[written], ref_d[written]) and torch.equal(state.ts[written], ref_t[written])
        ok_local = torch.equal(state.data[~written], emb[~written]) and torch.equal(state.ts[~written], ets[~written])
        state.status.check("route")
        r = Route(send_sizes=z[f"r{rank}_r_send_sizes"].tolist(), recv_sizes=z[f"r{rank}_r_recv_sizes"].tolist(),
                  send_index=t("r_send_index"))
        x = t("x").clone().requires_grad_()
        y = r.forward(x)
        (y * t("w")).sum().backward()
        ok_route = torch.equal(y.detach(), t("y")) and torch.equal(x.grad, t("gx"))
        q.put((rank, ok_remote, ok_local, ok_route, None))
        dist.barrier()
        DistributedContext.shutdown()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, False, False, False, traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_routes_on_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29651, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = _collect(q, procs)
    for rank, a, b, c, err in out:
        assert err is None, err
        assert a, f"rank {rank}: remote writes differ from the reference"
        assert b, f"rank {rank}: local writes"
        assert c, f"rank {rank}: halo route forward/backward differs from the reference"


def _worker_p2p(rank, world, port, q):
    try:
        import torch.distributed as dist
        for p in (ROOT, os.path.join(ROOT, "starrygl-framework_b200"), HERE):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", RANK=str(rank),
                          WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
        from starrygl.utils.context import DistributedContext
        ctx = DistributedContext.init("nccl")
        dev = ctx.device
        from starrygl.cache.cache_route import CommPlan
        from starrygl.cache.p2p_route import P2PCacheRoute
        from starrygl.cache.NodeState import DistNodeState
        from starrygl.utils.partition_book import PartitionState

        # (1) the reference's 2-rank case
        z = np.load(os.path.join(HERE, "golden", "route_2rank.npz"))
        t = lambda k: torch.from_numpy(z[f"r{rank}_{k}"]).to(dev)
        feats = t("feats")
        n_loc, D = feats.shape[0], feats.shape[1] - 1
        plan = CommPlan(send_ranks=torch.repeat_interleave(torch.arange(world), torch.from_numpy(z[f"r{rank}_send_sizes"])),
                        send_sizes=torch.from_numpy(z[f"r{rank}_send_sizes"]), send_indices=t("send_indices"),
                        send_remote_indices=t("send_remote"))
        ps = PartitionState(loc_ids=torch.arange(n_loc, device=dev), num_master_nums=n_loc, node_mode='identity', num_nodes=n_loc)
        state = DistNodeState(ps, D, device=dev)
        route = P2PCacheRoute(D, True, cap_rows=64, ring=4)
        route.push(feats[:, :D].contiguous(), plan, state, feats[:, D].contiguous()).wait()
        torch.cuda.synchronize()
        route.status.check("p2p route")
        ok_golden = torch.equal(state.data, t("data")) and torch.equal(state.ts, t("ts"))
        route.close()

        # (2) 40 steps through a ring of 4 with changing sizes (including empty ones); dim 100 -> 128-bit lanes.
        # Messages of 40 rows and more (16 KB) travel as plain rows + flag, smaller ones as tagged lines: both forms
        # and their mixture inside one step are exercised.
        D2, N, K = 100, 4096, 512
        route = P2PCacheRoute(D2, True, cap_rows=K, ring=4, bulk_bytes=16384)
        ps2 = PartitionState(loc_ids=torch.arange(N, device=dev), num_master_nums=N, node_mode='identity', num_nodes=N)
        state2 = DistNodeState(ps2, D2, device=dev)
        all_feats = [torch.randn(N, D2, generator=torch.Generator().manual_seed(50 + r)) for r in range(world)]
        all_ts = [torch.rand(N, generator=torch.Generator().manual_seed(70 + r)) for r in range(world)]
        my_f, my_t = all_feats[rank].to(dev), all_ts[rank].to(dev)
        ref_d, ref_t = torch.zeros(N, D2), torch.zeros(N)

        def plan_of(step, sender):
            g = torch.Generator().manual_seed(1000 * step + sender)
            sizes = torch.randint(0, K // 2, (world,), generator=g)
            if step % 7 == 3:
                sizes[:] = 0
            idx, slots = [], []
            for p in range(world):
                idx.append(torch.randint(0, N, (int(sizes[p]),), generator=g))
                # slots of different senders never collide inside a step: sender s owns [s*K, (s+1)*K)
                slots.append(torch.randperm(K, generator=g)[:int(sizes[p])] + sender * K)
            return sizes, torch.cat(idx), torch.cat(slots)

        pending = []
        for step in range(40):
            sizes, idx, slots = plan_of(step, rank)
            pl = CommPlan(send_ranks=torch.repeat_interleave(torch.arange(world), sizes), send_sizes=sizes, send_indices=idx,
                          send_remote_indices=slots)
            pl.recv_sizes = [int(plan_of(step, s)[0][rank]) for s in range(world)]
            pending.append(route.push(my_f, pl, state2, my_t))
            if len(pending) == 2:            # keep two steps in flight
                pending.pop(0).wait()
            for s in range(world):           # expected state, applied in step order
                sz, ix, sl = plan_of(step, s)
                off = int(sz[:rank].sum())
                seg = slice(off, off + int(sz[rank]))
                ref_d[sl[seg]] = all_feats[s][ix[seg]]
                ref_t[sl[seg]] = all_ts[s][ix[seg]]
        for f in pending:
            f.wait()
        torch.cuda.synchronize()
        route.status.check("p2p route ring")
        ok_ring = torch.equal(state2.data.cpu(), ref_d) and torch.equal(state2.ts.cpu(), ref_t)
        route.close()

        # (3) row widths whose slot words fall on every position of a 16-byte staging line, with and without timestamps
        for D3, has_ts in ((7, True), (6, True), (5, False), (8, False), (1, True)):
            route = P2PCacheRoute(D3, has_ts, cap_rows=K, ring=2)
            st3 = DistNodeState(ps2, D3, device=dev)
            f3 = [torch.randn(N, D3, generator=torch.Generator().manual_seed(90 + r + D3)) for r in range(world)]
            t3 = [torch.rand(N, generator=torch.Generator().manual_seed(95 + r + D3)) for r in range(world)]
            r_d, r_t = torch.zeros(N, D3), torch.zeros(N)
            for step in range(5):
                sizes, idx, slots = plan_of(step + 100 * D3, rank)
                pl = CommPlan(send_ranks=torch.repeat_interleave(torch.arange(world), sizes), send_sizes=sizes, send_indices=idx,
                              send_remote_indices=slots)
                pl.recv_sizes = [int(plan_of(step + 100 * D3, s)[0][rank]) for s in range(world)]
                route.push(f3[rank].to(dev), pl, st3, t3[rank].to(dev) if has_ts else None).wait()
                for s in range(world):
                    sz, ix, sl = plan_of(step + 100 * D3, s)
                    off = int(sz[:rank].sum())
                    seg = slice(off, off + int(sz[rank]))
                    r_d[sl[seg]] = f3[s][ix[seg]]
                    if has_ts:
                        r_t[sl[seg]] = t3[s][ix[seg]]
            torch.cuda.synchronize()
            route.status.check("p2p route widths")
            ok_ring = ok_ring and torch.equal(st3.data.cpu(), r_d) and torch.equal(st3.ts.cpu(), r_t)
            route.close()
        q.put((rank, ok_golden, ok_ring, True, None))
        dist.barrier()
        DistributedContext.shutdown()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, False, False, False, traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_p2p_cache_route_on_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_p2p, args=(r, 2, 29652, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = _collect(q, procs)
    for rank, a, b, _, err in out:
        assert err is None, err
        assert a, f"rank {rank}: peer-memory route differs from the reference's result"
        assert b, f"rank {rank}: 40 steps through the staging ring differ from the expected state"


def _worker_world1(rank, world, port, q):
    """A group of ONE NCCL rank: the native exchange (grouped send/recv to itself), the halo route with its gradient, the
    native cache route step, and the sharded table built through the process group -- the code paths of the two-GPU
    tests, on a box with a single GPU."""
    try:
        import torch.distributed as dist
        for p in (ROOT, os.path.join(ROOT, "starrygl-framework_b200"), HERE):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", RANK="0", WORLD_SIZE="1",
                          LOCAL_RANK="0")
        from oracle import oracle_np as O
        from starrygl.utils.context import DistributedContext
        ctx = DistributedContext.init("nccl")
        dev = ctx.device
        from starrygl.route.route import Route
        from starrygl.lib.libstarrygl_comm import ShardTensor, shared_empty
        from starrygl.utils.partition_book import DistRouteIndex
        g = torch.Generator().manual_seed(5)
        n, k, F = 40, 25, 12
        send_index = torch.randperm(n, generator=g)[:k]
        x_h = torch.randn(n, F, generator=g)
        w_h = torch.randn(n + k, F, generator=g)
        r = Route(send_sizes=[k], recv_sizes=[k], send_index=send_index.to(dev))
        x = x_h.clone().to(dev).requires_grad_()
        y = r.forward(x)
        (y * w_h.to(dev)).sum().backward()
        y_ref = O.route_forward([x_h.numpy()], [[k]], [[k]], [send_index.numpy()])[0]
        g_ref = O.route_reverse([w_h.numpy()], [[k]], [[k]], [send_index.numpy()])[0]
        ok_route = np.array_equal(y.detach().cpu().numpy(), y_ref) and np.array_equal(x.grad.cpu().numpy(), g_ref)
        # split-phase form and the reversed direction
        t = r.send(x_h.to(dev))
        ok_route = ok_route and np.array_equal(r.recv(t).cpu().numpy(), y_ref)
        ok_route = ok_route and np.array_equal(r.forward(w_h.to(dev), reverse=True).cpu().numpy(), g_ref)
        # ids -> route: every id is owned by partition 0 here
        ids = torch.randint(0, n, (60,), generator=g)
        route2, asked, order = Route.all_to_all_ind2ptr(DistRouteIndex(ids.to(dev), torch.zeros(60, dtype=torch.long, device=dev)))
        ok_ind = torch.equal(asked.cpu(), ids[order.cpu()]) and route2.send_sizes == [60] and route2.recv_sizes == [60]
        # sharded table through the group + the exchange form of the gather
        local = shared_empty(n, (F,))
        local.copy_(x_h)
        st = ShardTensor.from_local(local)
        got = st[ids.to(dev)]
        st.check()
        ok_shard = torch.equal(got.cpu(), x_h[ids])
        ok_shard = ok_shard and torch.equal(ShardTensor.gather_by_exchange(local, ids.to(dev)).cpu(), x_h[ids])
        st.unregister()
        q.put((rank, ok_route, ok_ind, ok_shard, None))
        dist.barrier()
        DistributedContext.shutdown()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, False, False, False, traceback.format_exc()))


def test_native_exchange_route_and_shard_tensor_in_a_group_of_one():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_world1, args=(0, 1, 29653, q))]
    procs[0].start()
    for rank, a, b, c, err in _collect(q, procs):
        assert err is None, err
        assert a, "halo route forward / backward / split phase / reverse differs from the oracle"
        assert b, "route built from packed ids"
        assert c, "sharded table gather (peer form or exchange form)"
