"""End-to-end TGN steps: the same model fed by (a) the CUDA data path and (b) the CPU oracle must produce the same
loss (tolerance 1e-4 relative, fp32) over several training steps, including the memory / mailbox write-back between
steps.  Graph shape follows the small reference configuration (bipartite, 9,000 + 1,000 nodes, 172-d edge features,
recent-10, one layer, memory dim 100, time dim 100, batch 200 with one negative destination per event, 160,000 events)."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, npy
from tgn_torch import TGN

pytestmark = pytest.mark.gpu
REL_TOL = 1e-4
DIM_MEM, DIM_EDGE, DIM_TIME, K, B = 100, 172, 100, 10, 200
FIRST = 80000          # index of the first training event: half of the stream is history


def make_data(seed=0, n_src=9000, n_dst=1000, m=160000):
    rng = np.random.default_rng(seed)
    zs = np.minimum(rng.zipf(1.2, m) - 1, n_src - 1)
    zd = np.minimum(rng.zipf(1.5, m) - 1, n_dst - 1)
    src = zs.astype(np.int64)
    dst = (n_src + zd).astype(np.int64)
    ts = np.sort(rng.integers(0, 2_600_000, m)).astype(np.int64)
    efeat = rng.standard_normal((m, DIM_EDGE)).astype(np.float32)
    # both directions, as the reference trains with inverse edges: rows keyed by the queried node
    key = np.concatenate([src, dst])
    nbr = np.concatenate([dst, src])
    tss = np.concatenate([ts, ts])
    eid = np.concatenate([np.arange(m), np.arange(m)]).astype(np.int64)
    return n_src + n_dst, src, dst, ts, efeat, key, nbr, tss, eid


class GpuPath:
    """Everything through the library: T-CSR, batch builder, node-state gathers, feature gather, state write-back."""

    def __init__(self, n, key, nbr, tss, eid, efeat):
        from starrygl import ops
        from starrygl.cache.NodeState import DistNodeState
        from starrygl.utils.partition_book import PartitionState
        self.ops = ops
        self.g = ops.tcsr_build(cu(key), cu(nbr), cu(tss), cu(eid), n)
        self.efeat = cu(efeat)
        ps = PartitionState(loc_ids=torch.arange(n, device="cuda"), num_master_nums=n, node_mode='identity', num_nodes=n)
        self.mem = DistNodeState(ps, DIM_MEM, device="cuda")
        self.mail = DistNodeState(ps, 2 * DIM_MEM + DIM_EDGE, device="cuda")

    def batch(self, roots, rts):
        from starrygl.graph.batch import build_batch
        L0, L1 = build_batch(self.g, cu(roots), cu(rts), [K], "recent", ts_range=(0, 2_600_000))
        out = {"inv_map": L0["inv_map"], "indptr": L1["indptr"], "indices": L1["indices"], "edge_dt": L1["edge_dt"],
               "efeat": self.ops.gather_rows(self.efeat, L1["eid"]), "gids0": L0["gids"]}
        for tag, gids in (("0", L0["gids"]), ("1", L1["gids"])):
            out["mem" + tag], out["mem_ts" + tag] = self.mem[gids]
            out["mail" + tag], out["mail_ts" + tag] = self.mail[gids]
        return out

    def write_back(self, nodes, new_mem, mem_ts, mails, mail_ts):
        self.mem.update(cu(nodes), new_mem, cu(mem_ts))
        self.mail.update(cu(nodes), mails, cu(mail_ts))


class OraclePath:
    """The same steps with the numpy oracle on the host; tensors are moved to the GPU only for the model."""

    def __init__(self, n, key, nbr, tss, eid, efeat):
        self.csr = O.tcsr_build(key, nbr, tss, eid, n)[:4]
        self.efeat = efeat
        self.g2l = np.arange(n + 1, dtype=np.int64)
        self.mem, self.mem_ts = np.zeros((n, DIM_MEM), np.float32), np.zeros(n, np.float32)
        self.mail, self.mail_ts = np.zeros((n, 2 * DIM_MEM + DIM_EDGE), np.float32), np.zeros(n, np.float32)

    def batch(self, roots, rts):
        L0, L1 = O.build_batch(*self.csr, roots, rts, [K])
        out = {"inv_map": cu(L0["inv_map"]), "indptr": cu(L1["indptr"]), "indices": cu(L1["indices"]),
               "edge_dt": cu(L1["edge_dt"]), "efeat": cu(O.gather_rows(self.efeat, L1["eid"])), "gids0": cu(L0["gids"])}
        for tag, gids in (("0", L0["gids"]), ("1", L1["gids"])):
            m, mt = O.state_read(self.mem, self.mem_ts, self.g2l, gids)
            ml, mlt = O.state_read(self.mail, self.mail_ts, self.g2l, gids)
            out["mem" + tag], out["mem_ts" + tag], out["mail" + tag], out["mail_ts" + tag] = cu(m), cu(mt), cu(ml), cu(mlt)
        return out

    def write_back(self, nodes, new_mem, mem_ts, mails, mail_ts):
        O.state_update(self.mem, self.mem_ts, self.g2l, nodes, npy(new_mem), mem_ts)
        O.state_update(self.mail, self.mail_ts, self.g2l, nodes, npy(mails), mail_ts)


def run(path_cls, steps=4):
    n, src, dst, ts, efeat, key, nbr, tss, eid = make_data()
    path = path_cls(n, key, nbr, tss, eid, efeat)
    torch.manual_seed(0)
    model = TGN(DIM_MEM, DIM_EDGE, DIM_TIME).cuda()
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    rng = np.random.default_rng(1)
    losses = []
    for s in range(steps):
        sl = slice(FIRST + s * B, FIRST + (s + 1) * B)
        e_src, e_dst, e_ts = src[sl], dst[sl], ts[sl]
        neg = (9000 + rng.integers(0, 1000, B)).astype(np.int64)
        roots = np.concatenate([e_src, e_dst, neg])
        rts = np.concatenate([e_ts, e_ts, e_ts])
        batch = path.batch(roots, rts)
        loss, x_dst = model(batch, B)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
        # write-back: updated memory of the batch's source and destination nodes (last event per node wins), and a
        # new mail [own memory | other end's memory | edge feature] stamped with the event time
        inv = batch["inv_map"]
        x = x_dst.detach()[inv]
        nodes_all = np.concatenate([e_src, e_dst])
        last = {int(v): i for i, v in enumerate(nodes_all)}          # later occurrences overwrite earlier ones
        pick = np.array(sorted(last.values()), dtype=np.int64)
        nodes = nodes_all[pick]
        own = x[:2 * B][cu(pick)]
        other = torch.cat([x[B:2 * B], x[:B]])[cu(pick)]
        ef = cu(efeat[np.arange(sl.start, sl.stop)][pick % B])
        mails = torch.cat([own, other, ef], 1).contiguous()
        t_ev = np.concatenate([e_ts, e_ts])[pick].astype(np.float32)
        path.write_back(nodes, own.contiguous(), t_ev, mails, t_ev)
    return losses


def test_tgn_loss_matches_between_cuda_path_and_oracle():
    """Two complete training runs.  The model's own scatter/index-add kernels use atomics, whose summation order changes
    from run to run and is amplified by training; deterministic algorithms are switched on so that the comparison sees
    the data path only."""
    import os
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    prev = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(True, warn_only=True)
    try:
        a = run(GpuPath)
        b = run(OraclePath)
    finally:
        torch.use_deterministic_algorithms(prev)
    assert len(a) == len(b) == 4
    for la, lb in zip(a, b):
        assert np.isfinite(la) and abs(la - lb) <= REL_TOL * abs(lb), (a, b)
    assert a[0] != a[-1]          # the model actually trains / the state actually changes


def test_tgn_inputs_and_state_are_bit_exact_in_lockstep():
    """Both data paths driven side by side with the same model outputs: every tensor handed to the model and the whole
    memory / mailbox state after every write-back must be identical, bit for bit."""
    n, src, dst, ts, efeat, key, nbr, tss, eid = make_data()
    G, Or = GpuPath(n, key, nbr, tss, eid, efeat), OraclePath(n, key, nbr, tss, eid, efeat)
    torch.manual_seed(0)
    model = TGN(DIM_MEM, DIM_EDGE, DIM_TIME).cuda()
    rng = np.random.default_rng(1)
    for s in range(4):
        sl = slice(FIRST + s * B, FIRST + (s + 1) * B)
        e_src, e_dst, e_ts = src[sl], dst[sl], ts[sl]
        neg = (9000 + rng.integers(0, 1000, B)).astype(np.int64)
        roots, rts = np.concatenate([e_src, e_dst, neg]), np.concatenate([e_ts, e_ts, e_ts])
        bg, bo = G.batch(roots, rts), Or.batch(roots, rts)
        for k in bo:
            assert torch.equal(bg[k], bo[k]), (s, k)
        with torch.no_grad():
            _, x_dst = model(bg, B)
        x = x_dst[bg["inv_map"]]
        nodes_all = np.concatenate([e_src, e_dst])
        pick = np.array(sorted({int(v): i for i, v in enumerate(nodes_all)}.values()), dtype=np.int64)
        own = x[:2 * B][cu(pick)].contiguous()
        other = torch.cat([x[B:2 * B], x[:B]])[cu(pick)]
        mails = torch.cat([own, other, cu(efeat[np.arange(sl.start, sl.stop)][pick % B])], 1).contiguous()
        t_ev = np.concatenate([e_ts, e_ts])[pick].astype(np.float32)
        G.write_back(nodes_all[pick], own, t_ev, mails, t_ev)
        Or.write_back(nodes_all[pick], own, t_ev, mails, t_ev)
        torch.cuda.synchronize()
        assert np.array_equal(npy(G.mem.data), Or.mem) and np.array_equal(npy(G.mem.ts), Or.mem_ts), s
        assert np.array_equal(npy(G.mail.data), Or.mail) and np.array_equal(npy(G.mail.ts), Or.mail_ts), s
