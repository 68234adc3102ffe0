"""Row gather / scatter / cache kernels: bit-exact against numpy indexing and the reference's golden vectors."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, load, npy

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["auto", "vec", "bulk"])
@pytest.mark.parametrize("rows,dim,dtype,n", [(1000, 172, torch.float32, 5000), (1000, 128, torch.float32, 4097),
                                              (777, 128, torch.bfloat16, 3000), (50, 100, torch.float32, 1),
                                              (64, 4, torch.float32, 100), (3000, 256, torch.float32, 70000),
                                              (400, 1280, torch.float32, 2000), (300, 1116, torch.float32, 1500)])
def test_gather_rows(mode, rows, dim, dtype, n):
    from starrygl import ops
    if mode == "bulk" and dim * 4 > 4096:
        pytest.skip("rows above 4 KB do not fit two to a pipeline stage: 'auto' routes them to the 128-bit lanes")
    g = torch.Generator().manual_seed(rows + dim)
    table = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    idx = torch.randint(0, rows, (n,), generator=g).cuda()
    st = ops.StatusWord(table.device)
    out = ops.gather_rows(table, idx, mode=mode, status=st)
    st.check("gather")
    assert torch.equal(out, table[idx])


def test_gather_rows_unaligned_rows_use_narrow_lanes():
    from starrygl import ops, _C
    table = torch.randn(500, 186).cuda()        # 744-byte rows: not a multiple of 16
    idx = torch.randint(0, 500, (2000,)).cuda()
    assert torch.equal(ops.gather_rows(table, idx), table[idx])
    with pytest.raises(_C.SglError):
        ops.gather_rows(table, idx, mode="bulk")
    t1 = torch.arange(1000, dtype=torch.int64).cuda() * 3      # 1-D tables (8-byte rows)
    assert torch.equal(ops.gather_rows(t1, idx), t1[idx])


def test_wide_rows_in_auto_mode_and_explicit_bulk_refusal():
    """Rows of 5,120 bytes (1280 x fp32) and the 4,464-byte rows of a three-slot mailbox with 1,024 and more ids: the
    automatic mode must pick a kernel that takes them; only an explicitly requested bulk mode may refuse."""
    from starrygl import ops, _C
    from starrygl.nn.memory.mailbox import mailbox as MailBox
    table = torch.randn(300, 1280).cuda()
    idx = torch.randint(0, 300, (4096,)).cuda()
    assert torch.equal(ops.gather_rows(table, idx, mode="auto"), table[idx])
    with pytest.raises(_C.SglError, match="too large for bulk"):
        ops.gather_rows(table, idx, mode="bulk")
    mb = MailBox(500, 3, 100, 172, device=torch.device("cuda"))
    mb.mailbox.copy_(torch.randn_like(mb.mailbox))
    mb.mailbox_ts.copy_(torch.rand_like(mb.mailbox_ts))
    ids = torch.randint(0, 500, (2048,)).cuda()
    rows, ts = mb.get_message(ids)
    assert torch.equal(rows, mb.mailbox[ids]) and torch.equal(ts, mb.mailbox_ts[ids])


def test_gather_negative_wrap_map_and_status():
    from starrygl import ops, _C
    table = torch.randn(100, 8).cuda()
    idx = torch.tensor([-1, 0, -100, 99]).cuda()
    assert torch.equal(ops.gather_rows(table, idx), table[idx])        # negative rows count from the end
    st = ops.StatusWord(table.device)
    ops.gather_rows(table, torch.tensor([100]).cuda(), status=st)
    with pytest.raises(_C.SglError, match="row index"):
        st.check("x")
    empty = ops.gather_rows(table, torch.zeros(0, dtype=torch.int64).cuda())
    assert empty.shape == (0, 8)


def test_node_state_matches_reference():
    """DistNodeState.update / __getitem__ against vectors produced by the reference classes."""
    from starrygl.cache.NodeState import DistNodeState
    from starrygl.utils.partition_book import PartitionState
    z = load("nodestate.npz")
    for dev in ("cuda", "cpu"):      # "cpu" = pinned host memory addressed by the kernels
        ps = PartitionState(loc_ids=torch.from_numpy(z["loc_ids"]).to("cuda" if dev == "cuda" else "cpu"),
                            num_master_nums=25, node_mode='map', num_nodes=int(z["num_nodes"]))
        ns = DistNodeState(ps, 6, device=dev)
        ns.update(cu(z["upd"]), cu(z["vals"]), cu(z["uts"]))
        torch.cuda.synchronize()
        assert np.array_equal(npy(ns.data), z["data"]) and np.array_equal(npy(ns.ts), z["ts"])
        got, gts = ns[cu(z["rd"])]
        assert np.array_equal(npy(got), z["got"]) and np.array_equal(npy(gts), z["got_ts"])
        assert np.array_equal(npy(ps.is_master_node_by_global(cu(z["rd"]) if dev == "cuda" else torch.from_numpy(z["rd"]))),
                              z["is_master"])
        ns.status.check("node state")


@pytest.mark.parametrize("dtype,dim", [(torch.float32, 128), (torch.bfloat16, 128), (torch.float32, 186)])
def test_cache_gather(dtype, dim):
    from starrygl import ops
    rng = np.random.default_rng(dim)
    N, C, n = 20000, 2000, 30000
    backing = torch.randn(N, dim).to(dtype).cuda()
    perm = rng.permutation(N)
    hot = perm[:C]
    hitmap = np.full(N, -1, np.int32)
    hitmap[hot] = np.arange(C, dtype=np.int32)
    cache = backing[cu(hot)].clone()
    ranks = np.minimum(rng.zipf(1.1, n) - 1, N - 1)
    ids = perm[ranks].astype(np.int64)
    st = ops.StatusWord(backing.device)
    out, miss_pos, miss_ids, counts = ops.cache_gather(cache, cu(hitmap), backing, cu(ids), status=st)
    hits, misses = counts.tolist()
    st.check("cache")
    ref_out, hit, ref_pos, ref_ids = O.cache_gather(npy(cache.view(torch.int16) if dtype == torch.bfloat16 else cache),
                                                    hitmap, npy(backing.view(torch.int16) if dtype == torch.bfloat16 else backing), ids)
    got = npy(out.view(torch.int16) if dtype == torch.bfloat16 else out)
    assert np.array_equal(got, ref_out)
    assert hits == int(hit.sum()) and misses == len(ref_pos)
    assert np.array_equal(npy(miss_pos[:misses]), ref_pos) and np.array_equal(npy(miss_ids[:misses]), ref_ids)
    # without a backing store the miss rows are left for the caller (miss list tells which)
    out2, mp2, mi2, c2 = ops.cache_gather(cache, cu(hitmap), None, cu(ids))
    assert c2.tolist() == [hits, misses]
    assert torch.equal(out2[cu(hit)], out[cu(hit)])


def test_scatter_and_wire_format():
    from starrygl import ops
    rng = np.random.default_rng(1)
    N, D, S = 500, 100, 300
    feats = torch.randn(N, D).cuda()
    ts = torch.rand(N).cuda()
    send_idx = cu(rng.integers(0, N, S).astype(np.int64))
    remote = cu(rng.permutation(N)[:S].astype(np.int64))
    wire = ops.route_pack(feats, ts, send_idx, remote_idx=remote)
    assert wire.shape == (S, ops.wire_pitch(D, True)) and ops.wire_pitch(D, True) % 4 == 0
    assert torch.equal(wire[:, :D], feats[send_idx]) and torch.equal(wire[:, D], ts[send_idx])
    assert torch.equal(ops.wire_slots(wire, D + 1), remote)
    data, tst = torch.zeros(N, D).cuda(), torch.zeros(N).cuda()
    ops.route_unpack(wire, D + 1, data, tst)
    ref_d, ref_t = torch.zeros(N, D).cuda(), torch.zeros(N).cuda()
    ref_d[remote] = feats[send_idx]
    ref_t[remote] = ts[send_idx]
    assert torch.equal(data, ref_d) and torch.equal(tst, ref_t)
    # odd dimension: narrow-lane path, same format
    f7 = torch.randn(N, 7).cuda()
    w7 = ops.route_pack(f7, ts, send_idx, remote_idx=remote)
    assert w7.shape[1] == 12 and torch.equal(w7[:, :7], f7[send_idx]) and torch.equal(w7[:, 7], ts[send_idx])
    d7, t7 = torch.zeros(N, 7).cuda(), torch.zeros(N).cuda()
    ops.route_unpack(w7, 8, d7, t7)
    r7 = torch.zeros(N, 7).cuda()
    r7[remote] = f7[send_idx]
    assert torch.equal(d7, r7) and torch.equal(t7, ref_t)
    # plain pack (no ts, no slots) = x[send_index]
    assert torch.equal(ops.route_pack(feats, None, send_idx), feats[send_idx])
    # scatter with a trailing timestamp column and ids that are not stored locally (slot -1 is skipped)
    packed = torch.cat([feats[:50], ts[:50, None]], 1).contiguous()
    slots = torch.arange(50).cuda() * 2
    slots[::5] = -1
    d2, t2 = torch.zeros(N, D).cuda(), torch.zeros(N).cuda()
    ops.scatter_rows(d2, slots, packed, ts_table=t2, split_last_col=True)
    keep = slots >= 0
    r_d, r_t = torch.zeros(N, D).cuda(), torch.zeros(N).cuda()
    r_d[slots[keep]] = feats[:50][keep]
    r_t[slots[keep]] = ts[:50][keep]
    assert torch.equal(d2, r_d) and torch.equal(t2, r_t)
    # reverse-route accumulate
    x = torch.randn(N, 16).cuda()
    x0 = x.clone()
    seg = cu(rng.permutation(N)[:120].astype(np.int64))
    outs = torch.randn(120, 16).cuda()
    ops.route_add_rows(x, seg, outs)
    x0[seg] += outs
    assert torch.equal(x, x0)


def test_ids_and_replica_lookup_match_reference():
    from starrygl import ops
    from starrygl.utils.partition_book import DistRouteIndex
    from starrygl.cache.replica_table import build_replica_table
    z = load("ids.npz")
    d = DistRouteIndex(cu(z["loc"]), cu(z["part"]))
    d.set_shared(cu(z["shared_idx"]))
    assert np.array_equal(npy(d.dist), z["dist"])
    assert np.array_equal(npy(d.loc), z["u_loc"]) and np.array_equal(npy(d.part), z["u_part"])
    assert np.array_equal(npy(d.is_shared), z["u_shared"])
    neg = cu(np.array([-1, -2 ** 62, 2 ** 62 + 5], np.int64))      # sign bit set: shared reads as true, like the reference
    loc, part, sh = ops.dist_unpack(neg)
    rl, rp, rs = O.dist_unpack(npy(neg))
    assert np.array_equal(npy(loc), rl) and np.array_equal(npy(part), rp) and np.array_equal(npy(sh), rs)
    rt = build_replica_table(200, [torch.from_numpy(z[f"book{p}"]) for p in range(4)], 4)
    assert np.array_equal(npy(rt.indptr), z["rt_indptr"]) and np.array_equal(npy(rt.indices), z["rt_ranks"])
    s, r, l = rt.to("cuda").lookup(cu(z["lk_ids"]))
    assert np.array_equal(npy(s), z["lk_src"]) and np.array_equal(npy(r), z["lk_ranks"]) and np.array_equal(npy(l), z["lk_locs"])


def test_route_plan_matches_reference():
    """compute_layer_route on the GPU against plans produced by the reference's _compute_layer_route."""
    from starrygl.cache.cache_route import compute_layer_route
    from starrygl.cache.replica_table import CSRReplicaTable
    z = load("plan.npz")
    P = int(z["P"])
    rt = CSRReplicaTable(cu(z["rt_indptr"]), cu(z["rt_ranks"]), cu(z["rt_locs"]))
    parts = cu(z["node_parts"])
    for case in range(3):
        for pid in range(P):
            tag = f"c{case}_p{pid}"
            plan = compute_layer_route(cu(z[f"{tag}_ids"]), parts, pid, rt, P)
            ref = O.compute_layer_route(z[f"{tag}_ids"], z[f"{tag}_ts"], z["node_parts"], pid, z["rt_indptr"], z["rt_ranks"],
                                        z["rt_locs"], P)
            if ref is None:
                assert plan is None and f"{tag}_none" in z.files
                continue
            # bit-exact against the oracle (same stable order) ...
            assert np.array_equal(npy(plan.send_ranks), ref[0]) and np.array_equal(npy(plan.send_sizes), ref[1])
            assert np.array_equal(npy(plan.send_indices), ref[2]) and np.array_equal(npy(plan.send_remote_indices), ref[3])
            # ... and, per destination segment, the same (row, slot) multiset as the reference's own plan
            assert np.array_equal(npy(plan.send_sizes), z[f"{tag}_send_sizes"])
            got = sorted(zip(npy(plan.send_ranks).tolist(), npy(plan.send_indices).tolist(), npy(plan.send_remote_indices).tolist()))
            want = sorted(zip(z[f"{tag}_send_ranks"].tolist(), z[f"{tag}_send_indices"].tolist(), z[f"{tag}_send_remote"].tolist()))
            assert got == want, tag
