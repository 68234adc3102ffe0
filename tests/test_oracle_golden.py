"""The numpy oracle against vectors produced by running the reference (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
from scipy import stats

from oracle import oracle_np as O

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return np.load(os.path.join(G, name))


@pytest.mark.parametrize("case", ["tiny", "rand_sorted", "rand_ties"])
def test_tcsr_and_recent(case):
    z = load(f"sampler_{case}.npz")
    n = int(z["n"])
    # the reference keys rows by dst and returns src as the neighbour
    indptr, nbr, ts, eid, _ = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], n)
    assert np.array_equal(indptr, z["indptr"])
    assert np.array_equal(nbr, z["s_src"])
    assert np.array_equal(ts, z["s_ts"])
    assert np.array_equal(eid, z["s_eid"])
    for k in (1, 3, 10):
        for e in (0, 1):
            o = O.sample_layer(indptr, nbr, ts, eid, z["q"], z["qt"], k, O.RECENT, equal_root_time=bool(e))
            tag = f"recent_k{k}_e{e}"
            for nm, a in zip(("src", "dst", "ts", "dt", "eid"), o[:5]):
                ref = z[f"{tag}_{nm}"]
                assert a.dtype == ref.dtype, (tag, nm)
                assert np.array_equal(a, ref), (tag, nm)


def test_worked_example():
    z = load("sampler_tiny.npz")
    indptr, nbr, ts, eid, _ = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], 8)
    o = O.sample_layer(indptr, nbr, ts, eid, [0, 7, 3], [51, 51, 51], 3)
    assert o[0].tolist() == [4, 5, 6, 0, 0]
    assert o[1].tolist() == [0, 0, 0, 1, 1]
    assert o[2].tolist() == [30, 40, 50, 25, 35]
    assert o[3].tolist() == [21.0, 11.0, 1.0, 26.0, 16.0]
    assert o[4].tolist() == [3, 4, 5, 6, 7]
    o = O.sample_layer(indptr, nbr, ts, eid, [0, 7, 3], [10, 10, 10], 3)
    assert len(o[0]) == 0


@pytest.mark.parametrize("case", ["tiny", "rand", "rand_k10"])
def test_batch(case):
    z = load(f"batch_{case}.npz")
    n = int(z["n"])
    indptr, nbr, ts, eid, _ = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], n)
    roots = np.concatenate([z["task_src"], z["task_dst"]])
    rts = np.concatenate([z["task_ts"], z["task_ts"]])
    out = O.build_batch(indptr, nbr, ts, eid, roots, rts, z["fanouts"].tolist())
    assert len(out) == int(z["num_layers"])
    for i, d in enumerate(out):
        for k, v in d.items():
            ref = z[f"L{i}_{k}"]
            assert v.dtype == ref.dtype, (i, k, v.dtype, ref.dtype)
            assert np.array_equal(v, ref), (i, k)


def test_uniform_distribution_matches_reference():
    z = load("uniform_hist.npz")
    m, k, trials = int(z["cands"]), int(z["k"]), int(z["trials"])
    hist = np.zeros(m, np.int64)
    for i in range(trials):
        p = O.uniform_positions(m, k, seed=0, stream=0, slot=i)
        assert len(set(p)) == k and p == sorted(p) and 0 <= p[0] and p[-1] < m
        hist[p] += 1
    # both histograms against the exact law (every position equally likely) ...
    exp = np.full(m, trials * k / m)
    assert stats.chisquare(hist, exp).pvalue > 1e-3
    assert stats.chisquare(z["hist"], exp).pvalue > 1e-3
    # ... and against each other (homogeneity)
    assert stats.chi2_contingency(np.stack([hist, z["hist"]]))[1] > 1e-3


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10
    assert O.philox4x32_10((0, 0, 0, 0), (0, 0)) == (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)
    assert O.philox4x32_10((0xffffffff,) * 4, (0xffffffff, 0xffffffff)) == (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)
    assert O.philox4x32_10((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0)) == \
        (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)


def test_ids_and_replicas():
    z = load("ids.npz")
    sh = np.zeros(64, np.int64)
    sh[z["shared_idx"]] = 1
    d = O.dist_pack(z["loc"], z["part"], sh)
    assert np.array_equal(d, z["dist"])
    loc, part, shared = O.dist_unpack(z["dist"])
    assert np.array_equal(loc, z["u_loc"]) and np.array_equal(part, z["u_part"]) and np.array_equal(shared, z["u_shared"])
    book = [z[f"book{p}"] for p in range(4)]
    indptr, ranks, locs = O.build_replica_table(200, book)
    assert np.array_equal(indptr, z["rt_indptr"]) and np.array_equal(ranks, z["rt_ranks"]) and np.array_equal(locs, z["rt_locs"])
    s, r, l = O.replica_lookup(indptr, ranks, locs, z["lk_ids"])
    assert np.array_equal(s, z["lk_src"]) and np.array_equal(r, z["lk_ranks"]) and np.array_equal(l, z["lk_locs"])


def test_nodestate():
    z = load("nodestate.npz")
    g2l = O.build_g2l(z["loc_ids"], int(z["num_nodes"]))
    data = np.zeros_like(z["data"])
    ts = np.zeros_like(z["ts"])
    O.state_update(data, ts, g2l, z["upd"], z["vals"], z["uts"])
    assert np.array_equal(data, z["data"]) and np.array_equal(ts, z["ts"])
    got, gts = O.state_read(data, ts, g2l, z["rd"])
    assert np.array_equal(got, z["got"]) and np.array_equal(gts, z["got_ts"])
    loc = g2l[z["rd"]]
    assert np.array_equal((loc >= 0) & (loc < 25), z["is_master"])


def test_route_two_ranks():
    z = load("route_2rank.npz")
    P = 2
    feats = [z[f"r{r}_feats"] for r in range(P)]
    data = [np.zeros_like(z[f"r{r}_data"]) for r in range(P)]
    ts = [np.zeros_like(z[f"r{r}_ts"]) for r in range(P)]
    O.cache_route(feats, [z[f"r{r}_send_sizes"] for r in range(P)], [z[f"r{r}_send_indices"] for r in range(P)],
                  [z[f"r{r}_send_remote"] for r in range(P)], data, ts)
    for r in range(P):
        assert np.array_equal(data[r], z[f"r{r}_data"]) and np.array_equal(ts[r], z[f"r{r}_ts"])
    ss = [z[f"r{r}_r_send_sizes"] for r in range(P)]
    rs = [z[f"r{r}_r_recv_sizes"] for r in range(P)]
    si = [z[f"r{r}_r_send_index"] for r in range(P)]
    ys = O.route_forward([z[f"r{r}_x"] for r in range(P)], ss, rs, si)
    for r in range(P):
        assert np.array_equal(ys[r], z[f"r{r}_y"])
    # backward of sum(y*w) w.r.t. x = reverse route of w
    gx = O.route_reverse([z[f"r{r}_w"] for r in range(P)], ss, rs, si)
    for r in range(P):
        assert np.allclose(gx[r], z[f"r{r}_gx"], rtol=0, atol=0)


# ---- the C oracle (timed CPU baseline) against the numpy oracle and the golden vectors -------------------------

@pytest.mark.parametrize("case", ["tiny", "rand_sorted", "rand_ties"])
def test_c_oracle_matches_reference(case):
    from oracle import oracle_c as OC
    z = load(f"sampler_{case}.npz")
    n = int(z["n"])
    indptr, nbr, ts, eid, perm = OC.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], n)
    assert np.array_equal(indptr, z["indptr"]) and np.array_equal(nbr, z["s_src"])
    assert np.array_equal(ts, z["s_ts"]) and np.array_equal(eid, z["s_eid"])
    for k in (1, 3, 10):
        for e in (0, 1):
            o = OC.sample_layer(indptr, nbr, ts, eid, z["q"], z["qt"], k, 0, equal_root_time=bool(e))
            for nm, a in zip(("src", "dst", "ts", "dt", "eid"), o[:5]):
                assert np.array_equal(a, z[f"recent_k{k}_e{e}_{nm}"]), (k, e, nm)
    rng = np.random.default_rng(0)
    q = rng.integers(0, n, 300)
    qt = rng.integers(0, int(z["ts"].max()) + 2, 300)
    for kw in ({}, {"allowed_offset": 7}, {"keep_root_time": True, "equal_root_time": True}):
        a = OC.sample_layer(indptr, nbr, ts, eid, q, qt, 4, 1, seed=9, stream=2, **kw)
        b = O.sample_layer(indptr, nbr, ts, eid, q, qt, 4, O.UNIFORM, seed=9, stream=2, **kw)
        for x, y in zip(a, b):
            assert np.array_equal(x, y)


def test_c_oracle_gather():
    from oracle import oracle_c as OC
    rng = np.random.default_rng(1)
    table = rng.standard_normal((500, 43)).astype(np.float32)
    idx = rng.integers(-500, 500, 2000)
    assert np.array_equal(OC.gather_rows(table, idx), table[idx])
    hitmap = np.full(500, -1, np.int32)
    hot = rng.permutation(500)[:60]
    hitmap[hot] = np.arange(60, dtype=np.int32)
    ids = rng.integers(0, 500, 900)
    out, mp, mi = OC.cache_gather(table[hot].copy(), hitmap, table, ids)
    ref, hit, rp, ri = O.cache_gather(table[hot], hitmap, table, ids)
    assert np.array_equal(out, ref) and np.array_equal(mp, rp) and np.array_equal(mi, ri)


def plan_cases():
    z = load("plan.npz")
    for case in range(3):
        for pid in range(int(z["P"])):
            yield z, f"c{case}_p{pid}", pid


def same_plan_up_to_segment_order(got, z, tag):
    """Equal split sizes and, inside every destination-rank segment, the same multiset of (list row, receiver slot)."""
    if got is None:
        return f"{tag}_none" in z.files
    ranks, sizes, rows, locs = got
    if f"{tag}_none" in z.files or not np.array_equal(sizes, z[f"{tag}_send_sizes"]):
        return False
    if not np.array_equal(ranks, np.sort(z[f"{tag}_send_ranks"])):
        return False
    ref = sorted(zip(z[f"{tag}_send_ranks"].tolist(), z[f"{tag}_send_indices"].tolist(), z[f"{tag}_send_remote"].tolist()))
    return sorted(zip(ranks.tolist(), rows.tolist(), locs.tolist())) == ref


def test_route_plan_matches_reference():
    for z, tag, pid in plan_cases():
        got = O.compute_layer_route(z[f"{tag}_ids"], z[f"{tag}_ts"], z["node_parts"], pid, z["rt_indptr"], z["rt_ranks"],
                                    z["rt_locs"], int(z["P"]))
        assert same_plan_up_to_segment_order(got, z, tag), tag


def _mail_case(z, c):
    t = f"c{c}"
    ef = z[f"{t}_ef"] if f"{t}_ef" in z else None
    emb = int(z[f"{t}_emb"])
    kw = dict(embedding=z[f"{t}_embedding"], use_src_emb=emb >= 1, use_dst_emb=emb >= 2) if emb else {}
    return (z[f"{t}_src"], z[f"{t}_dst"], z[f"{t}_ts"], ef, z[f"{t}_mem_src"], z[f"{t}_mem_dst"]), kw


def test_mail_reduce_matches_reference():
    """``mailbox.get_update_mail`` run by the reference (the last case has equal timestamps inside a node's entries: its
    expected rows follow the first-occurrence rule of the scatter-max restatement used to generate it)."""
    z = load("mail.npz")
    for c in range(int(z["n_cases"])):
        args, kw = _mail_case(z, c)
        index, mail, mail_ts = O.get_update_mail(*args, **kw)
        assert np.array_equal(index, z[f"c{c}_index"]), c
        assert np.array_equal(mail_ts, z[f"c{c}_mail_ts"]), c
        assert np.array_equal(mail, z[f"c{c}_mail"]), c


def test_mailbox_write_ring():
    rng = np.random.default_rng(3)
    mb, mts, pos = np.zeros((10, 3, 4), np.float32), np.zeros((10, 3), np.float32), np.zeros(10, np.int64)
    for step in range(5):
        idx = rng.permutation(10)[:6]
        rows, ts = rng.standard_normal((6, 4)).astype(np.float32), rng.random(6).astype(np.float32)
        before = pos.copy()
        O.mailbox_write(mb, mts, pos, idx, rows, ts)
        assert np.array_equal(mb[idx, before[idx]], rows) and np.array_equal(mts[idx, before[idx]], ts)
        assert np.array_equal(pos[idx], (before[idx] + 1) % 3)


LAYER_KEYS = ("indptr", "indices", "eid", "edge_ts", "edge_dt", "gids", "ts")


def slot_cases():
    z = load("slots.npz")
    for c in range(int(z["n_cases"])):
        pick = z[f"c{c}_pick"]
        if str(z[f"c{c}_kind"]) == "link":
            roots, rts = np.concatenate([z["src"][pick], z["dst"][pick]]), np.concatenate([z["ts"][pick], z["ts"][pick]])
        else:
            roots, rts = z["dst"][pick], z["ts"][pick]
        for pid in range(int(z["P"])):
            yield z, c, pid, roots, rts


def test_slot_files_match_reference():
    """Whole slot files written by the reference's ``build_aligned_batch`` (route planning on): layer dictionaries and
    the per-layer plans, restated as oracle ``build_batch`` + ``compute_layer_route``."""
    for z, c, pid, roots, rts in slot_cases():
        csr = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], int(z["N"]))[:4]
        layers = O.build_batch(*csr, roots, rts, [int(f) for f in z[f"c{c}_fanouts"]],
                               equal_root_time=bool(int(z[f"c{c}_end_offset"])))
        tag = f"c{c}_p{pid}"
        assert len(layers) == int(z[f"{tag}_num_layers"]) == int(z[f"{tag}_num_plans"])
        for k in ("gids", "ts", "inv_map"):
            assert np.array_equal(layers[0][k], z[f"{tag}_L0_{k}"]), (tag, k)
        for i in range(1, len(layers)):
            for k in LAYER_KEYS:
                assert np.array_equal(layers[i][k], z[f"{tag}_L{i}_{k}"]), (tag, i, k)
        for i, L in enumerate(layers):
            got = O.compute_layer_route(L["gids"], L["ts"], z["node_parts"], pid, z["rt_indptr"], z["rt_ranks"], z["rt_locs"],
                                        int(z["P"]))
            assert same_plan_up_to_segment_order(got, z, f"{tag}_plan{i}"), (tag, i)


def test_slice_window_structure():
    """The chunk/time-window slice has no runnable reference (its kernels index the chunk table by block number); the
    oracle is checked against a brute-force enumeration on a small graph."""
    rng = np.random.default_rng(5)
    n, m = 30, 600
    src, dst = rng.integers(0, n, m), rng.integers(0, n, m)
    ts = rng.integers(0, 40, m).astype(np.int64)
    indptr, nbr, sts, eid, _ = O.tcsr_build(src, dst, ts, np.arange(m, dtype=np.int64), n)
    chunk = (np.arange(n) // 10).astype(np.int64)
    mask = np.array([1, 0, 1], bool)
    nodes, node_ptr, group_ts, group_ptr, k_nbr, k_ts, k_eid = O.slice_window(indptr, nbr, sts, eid, chunk, mask, 5, 25)
    want = {}
    for v in range(n):
        for e in range(indptr[v], indptr[v + 1]):
            if mask[chunk[v]] and mask[chunk[nbr[e]]] and 5 <= sts[e] < 25:
                want.setdefault(v, {}).setdefault(int(sts[e]), []).append((int(nbr[e]), int(eid[e])))
    assert nodes.tolist() == sorted(want)
    for u, v in enumerate(nodes):
        groups = range(node_ptr[u], node_ptr[u + 1])
        assert [int(group_ts[g]) for g in groups] == sorted(want[v])
        for g in groups:
            got = list(zip(k_nbr[group_ptr[g]:group_ptr[g + 1]].tolist(), k_eid[group_ptr[g]:group_ptr[g + 1]].tolist()))
            assert got == want[v][int(group_ts[g])]
