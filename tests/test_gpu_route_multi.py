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
    out = sorted(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(60)
    for rank, a, b, c, err in out:
        assert err is None, err
        assert a, f"rank {rank}: remote writes differ from the reference"
        assert b, f"rank {rank}: local writes"
        assert c, f"rank {rank}: halo route forward/backward differs from the reference"
