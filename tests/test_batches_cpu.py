"""collate_and_merge / AtomicDataset / SlotAwareSampler on the host: merging slot files is pure index arithmetic, checked
here against the files it merged (every file must be recoverable from the merged batch)."""
import os

import numpy as np
import torch

from oracle import oracle_np as O


def _file(seed, world):
    rng = np.random.default_rng(seed)
    n, m = 60, 1500
    src, dst = rng.integers(0, n, m), rng.integers(0, n, m)
    ts = np.sort(rng.integers(0, 500, m))
    indptr, nbr, tss, eid, _ = O.tcsr_build(dst, src, ts, np.arange(m), n)
    q = rng.integers(0, n, 20 + seed)
    qt = rng.integers(100, 500, 20 + seed)
    layers = [{k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in d.items()}
              for d in O.build_batch(indptr, nbr, tss, eid, q, qt, [3, 2])]
    from starrygl.cache.cache_route import CommPlan
    plans = []
    for d in layers:
        k = int(d["gids"].numel())
        rows = torch.from_numpy(rng.permutation(k)[: k // 2])
        ranks = torch.sort(torch.from_numpy(rng.integers(0, world, rows.numel()))).values
        plans.append(CommPlan(send_ranks=ranks, send_sizes=torch.bincount(ranks, minlength=world), send_indices=rows,
                              send_remote_indices=rows + 1000 * seed))
    plans[1] = None if seed % 2 else plans[1]
    layers[0]["comm_plan"] = plans
    layers[0]["num_neg"] = 1
    layers[0]["task_src"] = torch.from_numpy(q)
    layers[0]["task_ts"] = torch.from_numpy(qt)
    return layers


def test_collate_and_merge_keeps_every_file_recoverable(tmp_path):
    from starrygl.data.batches import AtomicDataset, SlotAwareSampler, collate_and_merge
    world = 3
    files = [_file(s, world) for s in (1, 2, 3)]
    files[2] = files[2][:2]                               # a file whose sampling stopped after one hop
    for i, f in enumerate(files):
        torch.save(f, os.path.join(tmp_path, f"slot_{i // 2:04d}_sub_{i % 2:04d}.pt"))
    ds = AtomicDataset(str(tmp_path))
    assert len(ds) == 3 and ds.slots == [0, 0, 1]
    assert list(SlotAwareSampler(ds, 1).batches()) == [[0, 1], [2]] and list(SlotAwareSampler(ds, 2).batches()) == [[0, 1, 2]]
    mb = collate_and_merge([ds[i] for i in range(3)], world_size=world)
    assert len(mb.layers) == 3 and len(mb.routes) == 3
    for f, orig in enumerate(files):
        a0, b0 = mb.file_ptr[0][f], mb.file_ptr[0][f + 1]
        assert torch.equal(mb.layers[0]["gids"][a0:b0], orig[0]["gids"]) and torch.equal(mb.layers[0]["ts"][a0:b0], orig[0]["ts"])
    # inv_map still finds every root's (id, ts) pair
    inv, roots, rts = mb.layers[0]["inv_map"], torch.cat([f[0]["task_src"] for f in files]), torch.cat([f[0]["task_ts"] for f in files])
    assert torch.equal(mb.layers[0]["gids"][inv], roots) and torch.equal(mb.layers[0]["ts"][inv], rts)
    assert torch.equal(mb.roots["task_src"], roots)
    for l in (1, 2):
        L = mb.layers[l]
        assert L["indptr"].numel() == mb.layers[l - 1]["gids"].numel() + 1 and int(L["indptr"][-1]) == L["indices"].numel()
        for f, orig in enumerate(files):
            r0, r1 = int(mb.file_ptr[l - 1][f]), int(mb.file_ptr[l - 1][f + 1])
            e0, e1 = int(L["indptr"][r0]), int(L["indptr"][r1])
            if l < len(orig):
                d = orig[l]
                assert torch.equal(L["indptr"][r0:r1 + 1] - e0, d["indptr"]) and torch.equal(L["eid"][e0:e1], d["eid"])
                assert torch.equal(L["gids"][L["indices"][e0:e1]], d["gids"][d["indices"]])     # same neighbours after the shift
                assert torch.equal(L["ts"][L["indices"][e0:e1]], d["ts"][d["indices"]])
            else:
                assert e0 == e1
    # plans: grouped by rank, sizes added, indices shifted into the merged lists
    for l in range(3):
        plans = [(f[0]["comm_plan"][l] if l < len(f[0]["comm_plan"]) and l < len(f) else None) for f in files]
        r = mb.routes[l]
        want = sum(p.send_sizes for p in plans if p is not None)
        assert torch.equal(r.send_sizes, want) and torch.equal(r.send_ranks, torch.sort(r.send_ranks).values)
        got = sorted(zip(r.send_ranks.tolist(), r.send_indices.tolist(), r.send_remote_indices.tolist()))
        exp = sorted((int(a), int(b) + int(mb.file_ptr[l][f]), int(c)) for f, p in enumerate(plans) if p is not None
                     for a, b, c in zip(p.send_ranks, p.send_indices, p.send_remote_indices))
        assert got == exp
    assert collate_and_merge([], world) is None


def test_partition_book_and_replica_table_files(tmp_path):
    """Owned nodes first, then the halo (remote sources of the partition's events); the replica table lists every copy;
    the two files load back with the reference's layout."""
    from starrygl.graph.materialize import prepare_distributed_metadata
    rng = np.random.default_rng(0)
    n, m, P = 50, 400, 3
    parts = rng.integers(0, P, n)
    src, dst = rng.integers(0, n, m), rng.integers(0, n, m)
    book, table = prepare_distributed_metadata(torch.from_numpy(parts), (torch.from_numpy(src), torch.from_numpy(dst)), P, str(tmp_path))
    for p in range(P):
        owned = np.nonzero(parts == p)[0]
        halo = np.unique(src[(parts[dst] == p) & (parts[src] != p)])
        assert np.array_equal(book[p].numpy(), np.concatenate([owned, halo]))
    indptr, ranks, locs = O.build_replica_table(n, [b.numpy() for b in book])
    assert np.array_equal(table.indptr.numpy(), indptr) and np.array_equal(table.indices.numpy(), ranks)
    assert np.array_equal(table.locs.numpy(), locs)
    b2, np2, ep2 = torch.load(os.path.join(tmp_path, "partition_book.pt"), weights_only=False)
    assert all(torch.equal(a, b) for a, b in zip(b2, book)) and np.array_equal(np2.numpy(), parts)
    assert np.array_equal(ep2.numpy(), parts[dst])
    t2 = torch.load(os.path.join(tmp_path, "replica_table.pt"), weights_only=False)
    assert torch.equal(t2.indptr, table.indptr) and torch.equal(t2.locs, table.locs)
