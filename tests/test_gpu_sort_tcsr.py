"""Radix sort and T-CSR build on the GPU against numpy / the oracle / the reference's golden vectors."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, load, npy, build_graph

pytestmark = pytest.mark.gpu


# Sizes on both sides of the mini-batch path's limits (one tile of 8,192 keys: all passes in one kernel; up to 64 tiles:
# one kernel per pass of up to 11 bits; above: three kernels per pass of 8 or 9 bits) and key widths that need
# 1 to 6 passes there.
@pytest.mark.parametrize("n,bits", [(0, 64), (1, 64), (33, 8), (4096, 16), (4097, 40), (100003, 64), (1 << 20, 24),
                                    (5000, 9), (70001, 17), (12345, 27), (300000, 44), (9999, 63), (40, 1),
                                    (8192, 44), (8193, 44), (8191, 11), (16384, 12), (454656, 44), (454656, 43),
                                    (524288, 33), (524289, 44), (200000, 22), (65536, 55), (3 * 8192 + 1, 5)])
def test_radix_sort_stable(n, bits):
    from starrygl import ops
    rng = np.random.default_rng(n + bits)
    hi = (1 << bits) if bits < 64 else (1 << 63)
    keys = rng.integers(0, hi, n, dtype=np.int64) if n else np.zeros(0, np.int64)
    if n > 10:
        keys[: n // 2] = keys[n // 2: n // 2 * 2]   # many duplicates -> stability matters
    vals = np.arange(n, dtype=np.int32)
    k, v = ops.radix_sort_pairs(cu(keys), cu(vals), bits)
    order = np.argsort(keys.astype(np.uint64), kind="stable")
    assert np.array_equal(npy(k), keys[order])
    assert np.array_equal(npy(v), vals[order])


@pytest.mark.parametrize("case", ["tiny", "rand_sorted", "rand_ties"])
def test_tcsr_matches_reference(case):
    z = load(f"sampler_{case}.npz")
    g = build_graph(z)
    assert np.array_equal(npy(g.indptr), z["indptr"])
    assert np.array_equal(npy(g.nbr), z["s_src"])
    assert np.array_equal(npy(g.ts), z["s_ts"])
    assert np.array_equal(npy(g.eid), z["s_eid"])
    assert g.ts_min == int(z["ts"].min()) and g.ts_max == int(z["ts"].max())
    _, _, _, _, order = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], int(z["n"]))
    assert np.array_equal(npy(g.perm), order)


@pytest.mark.parametrize("n,m,tmax", [(1, 50, 10), (1000, 0, 10), (5, 7, 1), (20000, 300000, 10 ** 7),
                                      (300, 70000, 3), (50, 2000, 2 ** 62)])
def test_tcsr_matches_oracle(n, m, tmax):
    from starrygl import ops
    rng = np.random.default_rng(m + n)
    key = rng.integers(0, n, m).astype(np.int64)
    nbr = rng.integers(0, n, m).astype(np.int64)
    ts = rng.integers(-tmax, tmax, m).astype(np.int64) if tmax < 2 ** 40 else rng.integers(-tmax, tmax, m, dtype=np.int64)
    g = ops.tcsr_build(cu(key), cu(nbr), cu(ts), None, n, want_perm=True)
    indptr, o_nbr, o_ts, o_eid, order = O.tcsr_build(key, nbr, ts, np.arange(m, dtype=np.int64), n)
    assert np.array_equal(npy(g.indptr), indptr)
    assert np.array_equal(npy(g.nbr), o_nbr) and np.array_equal(npy(g.ts), o_ts) and np.array_equal(npy(g.eid), o_eid)
    assert np.array_equal(npy(g.perm), order)


def test_tcsr_two_round_sort_for_wide_keys():
    """node bits + timestamp bits > 64 takes the timestamp-then-node path."""
    from starrygl import ops
    rng = np.random.default_rng(3)
    n, m = 1 << 20, 5000
    key = rng.integers(0, n, m).astype(np.int64)
    ts = rng.integers(-2 ** 62, 2 ** 62, m, dtype=np.int64)
    ts[:100] = ts[100:200]
    g = ops.tcsr_build(cu(key), cu(key), cu(ts), None, n, want_perm=True)
    _, _, o_ts, o_eid, order = O.tcsr_build(key, key, ts, np.arange(m, dtype=np.int64), n)
    assert np.array_equal(npy(g.perm), order) and np.array_equal(npy(g.ts), o_ts)


def test_tcsr_rejects_out_of_range_ids():
    from starrygl import ops, _C
    key = cu(np.array([0, 5, 2], dtype=np.int64))
    with pytest.raises(_C.SglError, match="outside"):
        ops.tcsr_build(key, key, key, None, 5)
    with pytest.raises(_C.SglError):
        ops.tcsr_build(cu(np.array([-1], dtype=np.int64)), key[:1], key[:1], None, 5)
