"""Multi-hop batch construction ((node, ts)-pair relabel + CSC) and the node-level relabel on the GPU."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, load, npy, build_graph

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", ["tiny", "rand", "rand_k10"])
def test_batch_matches_reference(case):
    from starrygl.graph.batch import build_batch
    z = load(f"batch_{case}.npz")
    g = build_graph(z)
    roots = np.concatenate([z["task_src"], z["task_dst"]])
    rts = np.concatenate([z["task_ts"], z["task_ts"]])
    out = build_batch(g, cu(roots), cu(rts), z["fanouts"].tolist(), "recent")
    assert len(out) == int(z["num_layers"])
    for i, d in enumerate(out):
        for k, v in d.items():
            ref = z[f"L{i}_{k}"]
            a = npy(v)
            assert a.dtype == ref.dtype and np.array_equal(a, ref), (i, k)


@pytest.mark.parametrize("policy", ["recent", "uniform"])
def test_batch_matches_oracle_two_hops(policy):
    from starrygl.graph.batch import build_batch
    rng = np.random.default_rng(4)
    n, m = 3000, 90000
    z = {"n": n, "dst": rng.integers(0, n, m).astype(np.int64), "src": rng.integers(0, n, m).astype(np.int64),
         "ts": np.sort(rng.integers(0, 10 ** 6, m)).astype(np.int64), "eid": np.arange(m, dtype=np.int64)}
    g = build_graph(z)
    indptr, nbr, ts, eid, _ = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], n)
    pick = rng.integers(0, m, 300)
    roots = np.concatenate([z["src"][pick], z["dst"][pick]])
    rts = np.concatenate([z["ts"][pick], z["ts"][pick]])
    pol = O.RECENT if policy == "recent" else O.UNIFORM
    ref = O.build_batch(indptr, nbr, ts, eid, roots, rts, [10, 10], pol, seed=5)
    out = build_batch(g, cu(roots), cu(rts), [10, 10], policy, seed=5, ts_range=(0, 10 ** 6))
    assert len(out) == len(ref)
    for i, (d, r) in enumerate(zip(out, ref)):
        for k in r:
            a = npy(d[k])
            assert a.dtype == r[k].dtype and np.array_equal(a, r[k]), (i, k)


def test_batch_edge_cases():
    from starrygl.graph.batch import build_batch
    z = load("batch_tiny.npz")
    g = build_graph(z)
    indptr, nbr, ts, eid, _ = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], 8)
    # roots without any edge at all: the reference emits one empty layer and stops
    for roots, rts in ((np.array([3, 4]), np.array([100, 100])), (np.array([0, 7]), np.array([5, 5])),
                       (np.array([0, 0, 0]), np.array([51, 51, 21]))):
        ref = O.build_batch(indptr, nbr, ts, eid, roots.astype(np.int64), rts.astype(np.int64), [2, 2])
        out = build_batch(g, cu(roots.astype(np.int64)), cu(rts.astype(np.int64)), [2, 2])
        assert len(out) == len(ref)
        for d, r in zip(out, ref):
            for k in r:
                assert np.array_equal(npy(d[k]), r[k]), (roots, k)


def test_unique_pairs_rejects_timestamps_outside_window():
    from starrygl import ops, _C
    st = ops.StatusWord(torch.device("cuda"))
    ops.unique_pairs(cu(np.array([1, 2], np.int64)), cu(np.array([5, 999], np.int64)), id_bits=4, ts_bits=4, ts_base=0,
                     status=st)
    with pytest.raises(_C.SglError, match="timestamp"):
        st.check("x")


def test_node_relabel_matches_oracle():
    from starrygl import ops
    rng = np.random.default_rng(8)
    n = 5000
    lists = [rng.integers(0, n, 400).astype(np.int64), rng.integers(0, n, 3000).astype(np.int64),
             rng.integers(0, n, 9000).astype(np.int64)]
    ref_local, ref_map = O.relabel_nodes(lists)
    rl = ops.NodeRelabeler(n, torch.device("cuda"))
    got_new = []
    for ids, r in zip(lists, ref_local):
        loc, new_ids, d_new = rl.insert(cu(ids))
        assert np.array_equal(npy(loc), r)
        got_new.append(npy(new_ids[:int(d_new.item())]))
    assert np.array_equal(np.concatenate(got_new), ref_map)
    # a new epoch restarts the numbering without clearing the tables
    rl.reset()
    loc, new_ids, d_new = rl.insert(cu(lists[0]))
    r2, m2 = O.relabel_nodes([lists[0]])
    assert np.array_equal(npy(loc), r2[0]) and np.array_equal(npy(new_ids[:int(d_new.item())]), m2)


def test_batch_graph_replay_matches_eager():
    """The CUDA-graph form of the batch builder gives the same layers as the call-by-call form, batch after batch."""
    from starrygl.graph.batch import BatchGraph, build_batch
    rng = np.random.default_rng(12)
    n, m = 2000, 60000
    z = {"n": n, "dst": rng.integers(0, n, m).astype(np.int64), "src": rng.integers(0, n, m).astype(np.int64),
         "ts": np.sort(rng.integers(0, 10 ** 5, m)).astype(np.int64), "eid": np.arange(m, dtype=np.int64)}
    g = build_graph(z)
    bg = BatchGraph(g, 256, [5, 5], "uniform", ts_range=(0, 10 ** 5), seed=9)
    for trial in range(3):
        pick = rng.integers(0, m, 256)
        roots, rts = cu(z["dst"][pick]), cu(z["ts"][pick])
        torch.cuda.synchronize()
        dev_batch = bg.run(roots, rts)
        with torch.cuda.stream(bg.stream):
            got = [{k: v.clone() for k, v in d.items()} for d in dev_batch.finish()]
        ref = build_batch(g, roots, rts, [5, 5], "uniform", ts_range=(0, 10 ** 5), seed=9)
        assert len(got) == len(ref)
        for d, r in zip(got, ref):
            for k in r:
                assert torch.equal(d[k], r[k]), (trial, k)
