"""The reference-facing graph API (pyGraph / from_edge_index / submit_query / get) end to end on the GPU."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, npy

pytestmark = pytest.mark.gpu


def make_events(seed=0, n=400, m=20000, tmax=10000):
    rng = np.random.default_rng(seed)
    src = rng.integers(0, n, m).astype(np.int64)
    dst = rng.integers(0, n, m).astype(np.int64)
    ts = np.sort(rng.integers(0, tmax, m)).astype(np.int64)
    return n, src, dst, ts, np.arange(m, dtype=np.int64)


def ref_seeds(src, ts, eid, t0, t1, keep=None):
    sel = (ts >= t0) & (ts < t1)
    if keep is not None:
        sel &= keep[src]
    s, t, e = src[sel], ts[sel], eid[sel]
    order = np.lexsort((t, s))
    s, t, e = s[order], t[order], e[order]
    pairs = np.stack([s, t], 1)
    up, first = np.unique(pairs, axis=0, return_index=True) if len(s) else (np.zeros((0, 2), np.int64), np.zeros(0, np.int64))
    roots, rfirst = np.unique(up[:, 0], return_index=True) if len(up) else (np.zeros(0, np.int64), np.zeros(0, np.int64))
    return roots, np.append(rfirst, len(up)), up[:, 1], np.append(np.sort(first), len(s)), e


def test_seeds_and_async_sampling():
    from starrygl.graph.graph import pyGraph, AsyncGraphBlob, AsyncBlock
    n, src, dst, ts, eid = make_events()
    g = pyGraph(cu(src), cu(dst), cu(ts), n, 1, eid=cu(eid))
    # roots of a window
    r = g.g.get_seeds_in_chunks(torch.zeros(1, dtype=torch.int64).cuda(), 2000, 2300, False)
    roots, ts_ptr, rts, q_ptr, q_eid = ref_seeds(src, ts, eid, 2000, 2300)
    assert np.array_equal(npy(r.roots), roots) and np.array_equal(npy(r.ts_ptr), ts_ptr) and np.array_equal(npy(r.ts), rts)
    assert np.array_equal(npy(r.q_ptr), q_ptr) and np.array_equal(npy(r.q_eid), q_eid)
    empty = g.g.get_seeds_in_chunks(torch.zeros(1, dtype=torch.int64).cuda(), 20000, 20010, False)
    assert empty.root_num == 0 and npy(empty.ts_ptr).tolist() == [0]

    # queue three windows, results come back in order; check sampling + node-level relabel against the oracle
    indptr, nbr, tss, eids, _ = O.tcsr_build(src, dst, ts, eid, n)      # API keys rows by src, neighbour = dst
    policy = {"sample_type": "recent", "layers": 2, "fanout": 5, "allowed_offset": -1, "equal_root_time": False,
              "keep_root_time": False}
    starts, ends = [1000, 1100, 1200], [1100, 1200, 1300]
    neg = {"test_generate_samples": cu(np.array([3, 5, 7], np.int64)), "test_generate_samples_ts": cu(np.array([1500, 1500, 1500], np.int64))}
    blob = AsyncGraphBlob(g, starts, ends, [torch.zeros(1, dtype=torch.int64).cuda()] * 3, policy, neg)
    for t0, t1, blk in zip(starts, ends, blob.graph):
        res = blk.value()
        roots, ts_ptr, rts, q_ptr, q_eid = ref_seeds(src, ts, eid, t0, t1)
        qn = np.concatenate([np.repeat(roots, np.diff(ts_ptr)), [3, 5, 7]])
        qt = np.concatenate([rts, [1500, 1500, 1500]])
        h1 = O.sample_layer(indptr, nbr, tss, eids, qn, qt, 5)
        h2 = O.sample_layer(indptr, nbr, tss, eids, h1[0], h1[2], 5)
        loc, mapper = O.relabel_nodes([roots, h1[0], h2[0]])
        assert np.array_equal(npy(res.roots.roots), loc[0])
        for nb, h, l in zip(res.neighbors, (h1, h2), loc[1:]):
            assert np.array_equal(npy(nb.neighbors), l)
            assert np.array_equal(npy(nb.neighbors_ts), h[2]) and np.array_equal(npy(nb.neighbors_eid), h[4])
            assert np.array_equal(npy(nb.neighbors_dt), -(qt if h is h1 else h1[2])[h[1]] + h[2])
            assert np.array_equal(npy(nb.root_start_ptr), np.concatenate([[0], np.cumsum(h[5])]))
        # 'r' (first window) continues the numbering of the table, 'f' restarts it: every result carries its own new ids
        assert np.array_equal(npy(res.nodes_remapper_id), mapper)
        root, negr, mfgs, m = AsyncBlock.to_block(res.roots, res.neg_roots, res.neighbors, res.nodes_remapper_id)
        assert len(mfgs) == 2 and mfgs[-1].num_dst_nodes == len(qn)
        assert mfgs[-1].indptr.numel() == len(qn) + 1 and mfgs[-1].edata["eid"].numel() == len(h1[0])
    assert g.get_last_sample() is None
    g.g.close()


def test_bad_inputs_raise():
    from starrygl.lib import libstarrygl_comm as L
    n, src, dst, ts, eid = make_events(m=100)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        L.from_edge_index(n, 1, torch.from_numpy(src), cu(dst), cu(ts), cu(eid))
    with pytest.raises(RuntimeError, match="int64"):
        L.from_edge_index(n, 1, cu(src).int(), cu(dst), cu(ts), cu(eid))
    with pytest.raises(RuntimeError, match="outside"):
        L.from_edge_index(10, 1, cu(src), cu(dst), cu(ts), cu(eid))
    g = L.from_edge_index(n, 1, cu(src), cu(dst), cu(ts), cu(eid))
    with pytest.raises(RuntimeError, match="undefined sampling strategy"):
        g.sample_src_in_chunks_khop(g.get_seeds_in_chunks(torch.zeros(1, dtype=torch.int64).cuda(), 0, 10, False), None, 5, 1,
                                    -1, False, False, "nonsense")
    g.close()


def test_dense_time_steps_and_the_cluster_policy():
    """Snapshot graph (timestamps = small step numbers): ``using_full_timestamp`` gives every root / node ALL steps of the
    window, and any policy name other than recent / uniform queues that dense slice (the reference's cluster branch)."""
    from starrygl.lib import libstarrygl_comm as L
    n, src, dst, ts, eid = make_events(seed=5, n=60, m=3000, tmax=12)
    g = L.from_edge_index(n, 1, cu(src), cu(dst), cu(ts), cu(eid))
    chunk0 = torch.zeros(1, dtype=torch.int64).cuda()
    t0, t1 = 3, 9
    # roots
    r = g.get_seeds_in_chunks(chunk0, t0, t1, True)
    roots, ts_ptr, rts, q_ptr, q_eid = ref_seeds(src, ts, eid, t0, t1)
    d_ptr, d_ts, d_q = O.densify_time_groups(ts_ptr, rts, q_ptr, t0, t1)
    assert np.array_equal(npy(r.roots), roots) and np.array_equal(npy(r.ts_ptr), d_ptr) and np.array_equal(npy(r.ts), d_ts)
    assert np.array_equal(npy(r.q_ptr), d_q) and np.array_equal(npy(r.q_eid), q_eid)
    # brute force: the events behind (root, step) are exactly the root's events of that step
    qp = npy(r.q_ptr)
    for i in range(0, len(roots) * (t1 - t0), 7):
        u, t = roots[i // (t1 - t0)], t0 + i % (t1 - t0)
        assert sorted(npy(r.q_eid)[qp[i]:qp[i + 1]].tolist()) == sorted(eid[(src == u) & (ts == t)].tolist())
    # slice, directly and through the queue with the cluster policy
    indptr, s_nbr, s_ts, s_eid, _ = O.tcsr_build(src, dst, ts, eid, n)
    nodes, node_ptr, group_ts, group_ptr, k_nbr, k_ts, k_eid = O.slice_window(indptr, s_nbr, s_ts, s_eid, None, None, t0, t1)
    w_ptr, w_ts, w_g = O.densify_time_groups(node_ptr, group_ts, group_ptr, t0, t1)
    res = g.slice_by_chunk_ts(None, t0, t1, True)
    assert np.array_equal(npy(res.roots.roots), nodes) and np.array_equal(npy(res.roots.ts_ptr), w_ptr)
    assert np.array_equal(npy(res.roots.ts), w_ts) and np.array_equal(npy(res.neighbors[0].root_start_ptr), w_g)
    assert np.array_equal(npy(res.neighbors[0].neighbors_eid), k_eid)
    g.submit_query(t0, t1, chunk0, cu(np.zeros(0, np.int64)), cu(np.zeros(0, np.int64)), "cluster", 1, 0, 0, False, False, "f")
    q = g.get()
    assert np.array_equal(npy(q.neighbors[0].root_start_ptr), w_g) and np.array_equal(npy(q.neighbors[0].neighbors_eid), k_eid)
    loc, mapper = O.relabel_nodes([nodes, k_nbr])
    assert np.array_equal(npy(q.roots.roots), loc[0]) and np.array_equal(npy(q.neighbors[0].neighbors), loc[1])
    assert np.array_equal(npy(q.nodes_remapper_id), mapper)
    g.close()


def test_chunk_filter():
    from starrygl.lib import libstarrygl_comm as L
    n, src, dst, ts, eid = make_events(seed=2)
    mapper = torch.from_numpy((np.arange(n) // 100).astype(np.int64))          # 4 chunks of 100 nodes
    g = L.from_edge_index(n, 100, cu(src), cu(dst), cu(ts), cu(eid), mapper)
    r = g.get_seeds_in_chunks(torch.tensor([1, 3]).cuda(), 500, 900, False)
    keep = np.isin(np.arange(n) // 100, [1, 3])
    roots, ts_ptr, rts, q_ptr, q_eid = ref_seeds(src, ts, eid, 500, 900, keep)
    assert np.array_equal(npy(r.roots), roots) and np.array_equal(npy(r.ts_ptr), ts_ptr) and np.array_equal(npy(r.ts), rts)
    assert np.array_equal(npy(r.q_ptr), q_ptr) and np.array_equal(npy(r.q_eid), q_eid)
    g.close()


@pytest.mark.parametrize("chunks,t0,t1", [([1, 3], 500, 900), ([0, 1, 2, 3], 0, 10000), (None, 2000, 2001), ([2], 9000, 9000),
                                          ([0], -50, 20000)])
def test_slice_by_chunk_ts(chunks, t0, t1):
    """Chunk/time-window sub-graph (node -> distinct timestamps -> edges) against the oracle, through the graph API."""
    from starrygl.lib import libstarrygl_comm as L
    n, src, dst, ts, eid = make_events(seed=3, n=400, m=30000, tmax=3000)      # 10 events per timestamp: real groups
    src[:5000] = 7                                                             # one hub row spanning many ballots
    node_chunk = (np.arange(n) // 100).astype(np.int64)
    g = L.from_edge_index(n, 100, cu(src), cu(dst), cu(ts), cu(eid), torch.from_numpy(node_chunk))
    r = g.slice_by_chunk_ts(None if chunks is None else torch.tensor(chunks).cuda(), t0, t1)
    g.status.check("slice")
    indptr, s_nbr, s_ts, s_eid, _ = O.tcsr_build(src, dst, ts, eid, n)
    mask = None if chunks is None else np.isin(np.arange(4), chunks)
    nodes, node_ptr, group_ts, group_ptr, k_nbr, k_ts, k_eid = O.slice_window(indptr, s_nbr, s_ts, s_eid, node_chunk, mask, t0, t1)
    nb = r.neighbors[0]
    assert np.array_equal(npy(r.roots.roots), nodes) and np.array_equal(npy(r.roots.ts_ptr), node_ptr)
    assert np.array_equal(npy(r.roots.ts), group_ts) and np.array_equal(npy(nb.root_start_ptr), group_ptr)
    assert np.array_equal(npy(nb.neighbors), k_nbr) and np.array_equal(npy(nb.neighbors_ts), k_ts)
    assert np.array_equal(npy(nb.neighbors_eid), k_eid)
    # structure: groups partition the edges, one timestamp per group, ascending inside a node
    if len(k_ts):
        gp = npy(nb.root_start_ptr)
        assert all(len(set(k_ts[gp[i]:gp[i + 1]])) == 1 for i in range(0, len(gp) - 1, max(1, (len(gp) - 1) // 50)))
    g.close()


def test_slice_window_capacity_overflow_is_reported():
    from starrygl import _C, ops
    n, src, dst, ts, eid = make_events(seed=4, n=50, m=2000, tmax=100)
    g = ops.tcsr_build(cu(src), cu(dst), cu(ts), cu(eid), n)
    st = ops.StatusWord(g.device)
    with pytest.raises(_C.SglError):
        ops.slice_window(g, None, None, 0, 100, 10, status=st)
    out = ops.slice_window(g, None, None, 0, 100, 2000, status=st)
    assert out[4].numel() == 2000
