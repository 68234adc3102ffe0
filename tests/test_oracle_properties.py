"""Property checks of the numpy oracle against brute-force enumeration on small random inputs (hypothesis).  The oracle
is pinned to the reference by the golden vectors; these cases cover the corners the vectors do not reach (empty rows,
ties, windows, repeated nodes) and keep the oracle honest where the reference has no runnable code."""
import numpy as np
from hypothesis import given, settings, strategies as st

from oracle import oracle_np as O

SET = settings(max_examples=60, deadline=None)


def graph(draw, n_max=12, m_max=80, t_max=20):
    n = draw(st.integers(1, n_max))
    m = draw(st.integers(0, m_max))
    key = np.array(draw(st.lists(st.integers(0, n - 1), min_size=m, max_size=m)), np.int64)
    nbr = np.array(draw(st.lists(st.integers(0, n - 1), min_size=m, max_size=m)), np.int64)
    ts = np.array(draw(st.lists(st.integers(0, t_max), min_size=m, max_size=m)), np.int64)
    return n, key, nbr, ts, np.arange(m, dtype=np.int64)


@SET
@given(st.data())
def test_tcsr_is_the_stable_sort_by_row_then_time(data):
    n, key, nbr, ts, eid = graph(data.draw)
    indptr, s_nbr, s_ts, s_eid, perm = O.tcsr_build(key, nbr, ts, eid, n)
    order = sorted(range(len(key)), key=lambda j: (key[j], ts[j], j))
    assert s_eid.tolist() == order and s_nbr.tolist() == nbr[order].tolist() and s_ts.tolist() == ts[order].tolist()
    assert indptr.tolist() == [int((key < v).sum()) for v in range(n + 1)]


@SET
@given(st.data(), st.integers(1, 6), st.booleans(), st.sampled_from([-1, 0, 3]))
def test_recent_k_is_the_tail_of_the_candidates(data, k, inclusive, window):
    n, key, nbr, ts, eid = graph(data.draw)
    indptr, s_nbr, s_ts, s_eid, _ = O.tcsr_build(key, nbr, ts, eid, n)
    q = np.array(data.draw(st.lists(st.integers(0, n - 1), min_size=0, max_size=8)), np.int64)
    qt = np.array(data.draw(st.lists(st.integers(-1, 22), min_size=len(q), max_size=len(q))), np.int64)
    o_n, o_d, o_t, o_dt, o_e, counts = O.sample_layer(indptr, s_nbr, s_ts, s_eid, q, qt, k, O.RECENT, equal_root_time=inclusive,
                                                     allowed_offset=window)
    want_e, want_d = [], []
    for i, (v, t) in enumerate(zip(q, qt)):
        cand = [j for j in sorted(range(len(key)), key=lambda j: (ts[j], j)) if key[j] == v
                and (ts[j] <= t if inclusive else ts[j] < t) and (window < 0 or ts[j] >= t - window)]
        take = cand[-k:]
        want_e += take
        want_d += [i] * len(take)
        assert counts[i] == len(take)
    assert o_e.tolist() == want_e and o_d.tolist() == want_d
    assert o_n.tolist() == nbr[want_e].tolist() and o_t.tolist() == ts[want_e].tolist()
    assert np.array_equal(o_dt, (qt[want_d] - ts[want_e]).astype(np.float32))


@SET
@given(st.data(), st.integers(1, 5))
def test_uniform_k_takes_distinct_candidates_in_order(data, k):
    n, key, nbr, ts, eid = graph(data.draw)
    indptr, s_nbr, s_ts, s_eid, _ = O.tcsr_build(key, nbr, ts, eid, n)
    q = np.array(data.draw(st.lists(st.integers(0, n - 1), min_size=1, max_size=6)), np.int64)
    qt = np.array(data.draw(st.lists(st.integers(0, 22), min_size=len(q), max_size=len(q))), np.int64)
    o_n, o_d, o_t, o_dt, o_e, counts = O.sample_layer(indptr, s_nbr, s_ts, s_eid, q, qt, k, O.UNIFORM, seed=5)
    pos_of = {int(e): p for p, e in enumerate(s_eid)}
    off = 0
    for i, (v, t) in enumerate(zip(q, qt)):
        cand = int(((key == v) & (ts < t)).sum())
        assert counts[i] == min(cand, k)
        mine = o_e[off:off + counts[i]]
        off += counts[i]
        p = [pos_of[int(e)] for e in mine]
        assert p == sorted(set(p))                                   # distinct, ascending T-CSR position
        assert all(key[e] == v and ts[e] < t for e in mine)


@SET
@given(st.lists(st.tuples(st.integers(0, 6), st.integers(0, 5)), min_size=0, max_size=30),
       st.lists(st.tuples(st.integers(0, 6), st.integers(0, 5)), min_size=0, max_size=30))
def test_pair_relabel_is_sorted_unique_with_inverse(cur, raw):
    c = sorted(set(cur))
    cur_id, cur_ts = np.array([a for a, _ in c], np.int64), np.array([b for _, b in c], np.int64)
    raw_id, raw_ts = np.array([a for a, _ in raw], np.int64), np.array([b for _, b in raw], np.int64)
    u_id, u_ts, inv = O.merge_and_map(cur_id, cur_ts, raw_id, raw_ts)
    both = sorted(set(c) | set(raw))
    assert list(zip(u_id.tolist(), u_ts.tolist())) == both
    assert [both[j] for j in inv.tolist()] == raw


@SET
@given(st.data())
def test_mail_reduce_keeps_the_latest_entry_first_on_ties(data):
    b = data.draw(st.integers(0, 25))
    src = np.array(data.draw(st.lists(st.integers(0, 7), min_size=b, max_size=b)), np.int64)
    dst = np.array(data.draw(st.lists(st.integers(0, 7), min_size=b, max_size=b)), np.int64)
    ts = np.array(sorted(data.draw(st.lists(st.integers(0, 6), min_size=b, max_size=b))), np.int64)
    ms = np.arange(b * 2, dtype=np.float32).reshape(b, 2)
    md = -np.arange(b * 2, dtype=np.float32).reshape(b, 2) - 1
    index, mail, mail_ts = O.get_update_mail(src, dst, ts, None, ms, md)
    entries = [(int(v), float(t), j) for j, (v, t) in enumerate(zip(np.concatenate([src, dst]), np.concatenate([ts, ts])))]
    rows = np.concatenate([np.concatenate([ms, md], 1), np.concatenate([md, ms], 1)]) if b else np.zeros((0, 4), np.float32)
    want = {}
    for v, t, j in entries:
        if v not in want or t > want[v][0]:
            want[v] = (t, j)
    assert index.tolist() == sorted(want)
    for u, v in enumerate(index.tolist()):
        assert mail_ts[u] == want[v][0] and np.array_equal(mail[u], rows[want[v][1]])


@SET
@given(st.data())
def test_route_plan_sends_latest_row_of_owned_nodes_to_foreign_replicas(data):
    n, parts = 8, 3
    node_parts = np.array(data.draw(st.lists(st.integers(0, parts - 1), min_size=n, max_size=n)), np.int64)
    book = []
    for p in range(parts):
        owned = np.nonzero(node_parts == p)[0]
        halo = np.array(sorted(set(data.draw(st.lists(st.integers(0, n - 1), max_size=4))) - set(owned.tolist())), np.int64)
        book.append(np.concatenate([owned, halo]).astype(np.int64))
    indptr, ranks, locs = O.build_replica_table(n, book)
    pairs = sorted(set(data.draw(st.lists(st.tuples(st.integers(0, n - 1), st.integers(0, 9)), max_size=25))))
    ids, ts = np.array([a for a, _ in pairs], np.int64), np.array([b for _, b in pairs], np.int64)
    pid = data.draw(st.integers(0, parts - 1))
    got = O.compute_layer_route(ids, ts, node_parts, pid, indptr, ranks, locs, parts)
    want = []
    for v in sorted(set(ids.tolist())):
        if node_parts[v] != pid:
            continue
        row = max(j for j in range(len(ids)) if ids[j] == v)          # sorted by (id, ts): the last row is the latest
        for r in range(parts):
            if r != pid and v in book[r].tolist():
                want.append((r, row, book[r].tolist().index(v)))
    if not want:
        assert got is None
        return
    s_ranks, s_sizes, s_rows, s_locs = got
    assert sorted(zip(s_ranks.tolist(), s_rows.tolist(), s_locs.tolist())) == sorted(want)
    assert s_ranks.tolist() == sorted(s_ranks.tolist())
    assert s_sizes.tolist() == [sum(1 for w in want if w[0] == r) for r in range(parts)]
