"""Temporal sampling on the GPU: bit-exact against the reference's golden vectors and the oracle (recent),
bit-exact against the oracle's Philox restatement + distribution test against the reference (uniform)."""
import numpy as np
import pytest
import torch
from scipy import stats

from oracle import oracle_np as O
from gpu_util import cu, load, npy, build_graph

pytestmark = pytest.mark.gpu
NAMES = ("src", "dst", "ts", "dt", "eid")


def run(g, q, qt, k, policy="recent", **kw):
    from starrygl import ops
    st = ops.StatusWord(g.device)
    h = ops.sample_layer(g, cu(q), cu(qt), k, policy, status=st, **kw)
    n = h.total()
    st.check("sample")
    offs = npy(h.offsets)
    return [npy(x[:n]) for x in (h.nbr, h.dst, h.ts, h.dt, h.eid)], offs


@pytest.mark.parametrize("case", ["tiny", "rand_sorted", "rand_ties"])
def test_recent_matches_reference(case):
    z = load(f"sampler_{case}.npz")
    g = build_graph(z)
    for k in (1, 3, 10):
        for e in (0, 1):
            out, offs = run(g, z["q"], z["qt"], k, equal_root_time=bool(e))
            for nm, a in zip(NAMES, out):
                ref = z[f"recent_k{k}_e{e}_{nm}"]
                assert a.dtype == ref.dtype and np.array_equal(a, ref), (k, e, nm)
            assert offs[0] == 0 and offs[-1] == len(out[0]) and (np.diff(offs) >= 0).all()


def random_graph(seed, n, m, tmax, hub=0):
    rng = np.random.default_rng(seed)
    w = 1.0 / np.arange(1, n + 1) ** 1.3
    key = rng.choice(n, m, p=w / w.sum()).astype(np.int64)
    if hub:
        key[:hub] = 0
    nbr = rng.integers(0, n, m).astype(np.int64)
    ts = rng.integers(0, tmax, m).astype(np.int64)
    return {"n": n, "dst": key, "src": nbr, "ts": ts, "eid": rng.permutation(m).astype(np.int64)}


@pytest.mark.parametrize("policy", ["recent", "uniform"])
@pytest.mark.parametrize("k", [1, 7, 20, 32, 33, 48, 100])
def test_matches_oracle_with_hubs_and_options(policy, k):
    """Rows from empty to 60 000 edges (the multi-round warp search), every option of the policy dict."""
    z = random_graph(k, 500, 120000, 50000, hub=60000)
    g = build_graph(z)
    indptr, nbr, ts, eid, _ = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], z["n"])
    rng = np.random.default_rng(1)
    q = rng.integers(0, z["n"], 700).astype(np.int64)
    q[:50] = 0
    qt = rng.integers(-5, 50010, 700).astype(np.int64)
    pol = O.RECENT if policy == "recent" else O.UNIFORM
    for kw in ({}, {"equal_root_time": True}, {"allowed_offset": 400}, {"allowed_offset": 0, "equal_root_time": True},
               {"keep_root_time": True}):
        out, offs = run(g, q, qt, k, policy, seed=1234, rng_stream=3, **kw)
        ref = O.sample_layer(indptr, nbr, ts, eid, q, qt, k, pol, seed=1234, stream=3, **kw)
        for nm, a, r in zip(NAMES, out, ref[:5]):
            assert a.dtype == r.dtype and np.array_equal(a, r), (policy, k, kw, nm)
        assert np.array_equal(np.diff(offs), ref[5])


@pytest.mark.parametrize("policy", ["recent", "uniform"])
@pytest.mark.parametrize("n_q", [16384, 16385, 40000])
def test_large_launch_matches_oracle(policy, n_q):
    """Launches on both sides of the size where the searches switch from one warp per target to one lane per target
    (and the fill CTAs become a fraction of a count CTA): the C restatement of the oracle on the same queries."""
    from oracle import oracle_c as OC
    z = random_graph(11, 3000, 400000, 50000, hub=70000)
    g = build_graph(z)
    indptr, nbr, ts, eid, _ = OC.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], z["n"])
    rng = np.random.default_rng(n_q)
    q = rng.integers(0, z["n"], n_q).astype(np.int64)
    q[: n_q // 20] = 0                         # the hub row
    qt = rng.integers(-5, 50010, n_q).astype(np.int64)
    pol = O.RECENT if policy == "recent" else O.UNIFORM
    for k, kw in ((10, {}), (20, {"allowed_offset": 2000, "equal_root_time": True}), (40, {"keep_root_time": True})):
        out, offs = run(g, q, qt, k, policy, seed=77, rng_stream=1, **kw)
        ref = OC.sample_layer(indptr, nbr, ts, eid, q, qt, k, pol, seed=77, stream=1, **kw)
        for nm, a, r in zip(NAMES, out, ref[:5]):
            assert a.dtype == r.dtype and np.array_equal(a, r), (policy, k, kw, nm)
        assert np.array_equal(np.diff(offs), ref[5])


def test_edge_cases():
    z = random_graph(5, 40, 300, 100)
    g = build_graph(z)
    out, offs = run(g, np.zeros(0, np.int64), np.zeros(0, np.int64), 5)
    assert len(out[0]) == 0 and offs.tolist() == [0]
    # every query before the first event -> nothing sampled
    out, offs = run(g, np.arange(40, dtype=np.int64), np.full(40, -1, np.int64), 5)
    assert len(out[0]) == 0 and (offs == 0).all()
    # out-of-range node ids are reported through the status word
    from starrygl import ops, _C
    st = ops.StatusWord(g.device)
    ops.sample_layer(g, cu(np.array([3, 99], np.int64)), cu(np.array([50, 50], np.int64)), 5, status=st)
    with pytest.raises(_C.SglError, match="node id"):
        st.check("x")
    with pytest.raises(_C.SglError, match="uniform fanout"):
        ops.sample_layer(g, cu(np.array([3], np.int64)), cu(np.array([50], np.int64)), 513, "uniform")


def test_device_count_chaining():
    """A device-side count smaller than the launch capacity: only that many targets are sampled."""
    from starrygl import ops
    z = random_graph(9, 100, 5000, 1000)
    g = build_graph(z)
    indptr, nbr, ts, eid, _ = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], z["n"])
    rng = np.random.default_rng(2)
    q = rng.integers(0, 100, 300).astype(np.int64)
    qt = rng.integers(0, 1000, 300).astype(np.int64)
    d_n = torch.tensor([117], dtype=torch.int64, device="cuda")
    h = ops.sample_layer(g, cu(q), cu(qt), 6, d_n=d_n)
    ref = O.sample_layer(indptr, nbr, ts, eid, q[:117], qt[:117], 6)
    n = h.total()
    assert n == len(ref[0]) and np.array_equal(npy(h.nbr[:n]), ref[0]) and np.array_equal(npy(h.eid[:n]), ref[4])
    offs = npy(h.offsets)
    assert (offs[117:] == n).all()


def test_uniform_valid_and_distribution():
    """Every uniform sample is a distinct pre-query-time neighbour in ascending position, and the position
    histogram passes a chi-square test against the reference's histogram (golden) and the exact law."""
    zh = load("uniform_hist.npz")
    m, k, trials = int(zh["cands"]), int(zh["k"]), int(zh["trials"])
    z = {"n": 4, "dst": np.zeros(m, np.int64), "src": np.arange(m, dtype=np.int64) + 100, "ts": np.arange(m, dtype=np.int64),
         "eid": np.arange(m, dtype=np.int64)}
    g = build_graph(z)
    out, offs = run(g, np.zeros(trials, np.int64), np.full(trials, 1000, np.int64), k, "uniform", seed=77)
    assert (np.diff(offs) == k).all()
    pos = out[4].reshape(trials, k)
    assert (np.diff(pos, axis=1) > 0).all() and pos.min() >= 0 and pos.max() < m
    assert (out[2] < 1000).all()
    hist = np.bincount(out[4], minlength=m)
    exp = np.full(m, trials * k / m)
    assert stats.chisquare(hist, exp).pvalue > 1e-3
    assert stats.chi2_contingency(np.stack([hist, zh["hist"]]))[1] > 1e-3
    # different seeds / streams give different draws, same seed the same draws
    out2, _ = run(g, np.zeros(trials, np.int64), np.full(trials, 1000, np.int64), k, "uniform", seed=78)
    out3, _ = run(g, np.zeros(trials, np.int64), np.full(trials, 1000, np.int64), k, "uniform", seed=77)
    assert not np.array_equal(out[4], out2[4]) and np.array_equal(out[4], out3[4])


def test_large_batch_properties():
    """Full-size style batch (4096 roots, k = 20) on a power-law graph: size-independent properties."""
    from starrygl import ops
    rng = np.random.default_rng(0)
    n, m = 200000, 4000000
    deg_w = rng.pareto(1.1, n) + 1
    src = rng.choice(n, m, p=deg_w / deg_w.sum()).astype(np.int64)
    dst = rng.integers(0, n, m).astype(np.int64)
    ts = rng.integers(0, 10 ** 7, m).astype(np.int64)
    g = ops.tcsr_build(cu(src), cu(dst), cu(ts), None, n)
    pick = rng.integers(0, m, 4096)
    q, qt = src[pick], ts[pick]
    h = ops.sample_layer(g, cu(q), cu(qt), 20, "recent")
    tot = h.total()
    offs = npy(h.offsets)
    cnt = np.diff(offs)
    o_nbr, o_dst, o_ts, o_eid = (npy(x[:tot]) for x in (h.nbr, h.dst, h.ts, h.eid))
    assert cnt.max() <= 20 and (o_ts < qt[o_dst]).all()
    assert np.array_equal(src[o_eid], q[o_dst]) and np.array_equal(dst[o_eid], o_nbr) and np.array_equal(ts[o_eid], o_ts)
    # ascending time inside each target, and "most recent": nothing between the last sample and the query time is skipped
    same = o_dst[1:] == o_dst[:-1]
    assert (o_ts[1:][same] >= o_ts[:-1][same]).all()
    indptr = npy(g.indptr)
    ts_sorted = npy(g.ts)
    for i in rng.integers(0, 4096, 200):
        row = ts_sorted[indptr[q[i]]:indptr[q[i] + 1]]
        cut = np.searchsorted(row, qt[i], side="left")
        assert cnt[i] == min(cut, 20)
        assert np.array_equal(o_ts[offs[i]:offs[i + 1]], row[cut - cnt[i]:cut])


def test_fence_index_and_search_through_it():
    """The per-row search index (timestamp of the last edge of every 32-edge block) against numpy, and sampling with and
    without it: identical results -- it only changes which memory the time-range search reads."""
    from starrygl import ops
    z = random_graph(3, 300, 90000, 40000, hub=50000)
    key, nbr = z["dst"], z["src"]
    g = ops.tcsr_build(cu(key), cu(nbr), cu(z["ts"]), cu(z["eid"]), int(z["n"]))
    g0 = ops.tcsr_build(cu(key), cu(nbr), cu(z["ts"]), cu(z["eid"]), int(z["n"]), want_fence=False)
    assert g0.fence is None and g.fence is not None
    indptr, ts, fence = npy(g.indptr), npy(g.ts), npy(g.fence)
    assert len(fence) == (len(ts) >> 5) + int(z["n"]) + 1
    for r in range(int(z["n"])):
        s, e = indptr[r], indptr[r + 1]
        nb = (e - s + 31) // 32
        last = np.minimum(s + 32 * np.arange(nb) + 31, e - 1)
        assert np.array_equal(fence[(s >> 5) + r:(s >> 5) + r + nb], ts[last]), r
    rng = np.random.default_rng(5)
    for n_q in (700, 20000, 300000):          # one warp per target, and one lane per target
        q = rng.integers(0, z["n"], n_q).astype(np.int64)
        q[: n_q // 10] = 0                     # the hub row
        qt = rng.integers(-5, 40010, n_q).astype(np.int64)
        for kw in ({}, {"allowed_offset": 300, "equal_root_time": True}):
            for policy in ("recent", "uniform"):
                a = ops.sample_layer(g, cu(q), cu(qt), 10, policy, seed=9, **kw)
                b = ops.sample_layer(g0, cu(q), cu(qt), 10, policy, seed=9, **kw)
                n = a.total()
                assert n == b.total() and torch.equal(a.offsets, b.offsets)
                assert torch.equal(a.eid[:n], b.eid[:n]) and torch.equal(a.nbr[:n], b.nbr[:n]) and torch.equal(a.ts[:n], b.ts[:n])
