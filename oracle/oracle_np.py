"""CPU oracle (numpy) for the per-mini-batch data path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain numpy, the algorithm of the reference's CPU path so that the CUDA
kernels can be checked against it.  Only the tests, the smoke check and the benchmark's CPU-baseline
leg may import it; nothing in the shipped package does.

Parity pin: every function here is checked in ``tests/test_oracle_golden.py`` against vectors produced
by running the reference itself (``tests/golden/make_golden.py``).

Reference locations restated (paths inside the reference project):

* T-CSR order                      prepare_sample.py:192-203
* temporal sampling                prepare_sample.py:32-172 (continuous graph branch), :248-265
  optional window flags            csrc/include/starrygl/sample.cu.hpp:706-734, :783-827
* (node, ts) pair relabel + CSC    prepare_sample.py:205-246, :313-377
* node-level relabel               csrc/include/starrygl/sample.cu.hpp:1766-1852
* id packing                       starrygl/utils/partition_book.py:7-52
* id -> slot map, master test      starrygl/utils/partition_book.py:98-133, :160-168
* node state read / write          starrygl/cache/NodeState.py:36-61
* chunk-cache hit / miss split     starrygl/cache/NodeState.py:152-194 (commented design)
* replica lookup                   starrygl/cache/replica_table.py:16-82, :178-215
* cache route                      starrygl/cache/cache_route.py:211-277, starrygl/cache/NodeState.py:245-282
* halo route                       starrygl/route/route.py:427-466
* distributed gather (intent)      csrc/include/starrygl/feature.cu.hpp:298-422 (parity unpinned: the reference
                                   code cannot run; this restates the steps its comments and calls name)
* mailbox update                   starrygl/nn/memory/mailbox.py:41-84
"""
import numpy as np

I64 = np.int64

# ----------------------------------------------------------------------------------------------
# T-CSR
# ----------------------------------------------------------------------------------------------


def tcsr_build(key, nbr, ts, eid, num_nodes):
    """Rows keyed by ``key`` in ascending node id; inside a row ascending ``ts``; ties keep input order.

    prepare_sample.py:192-203 -- ``np.lexsort((ts, dst))`` is stable, row pointer = cumsum of counts.
    Returns (indptr[num_nodes+1], nbr_sorted, ts_sorted, eid_sorted, perm).
    """
    key = np.asarray(key, I64)
    order = np.lexsort((np.asarray(ts, I64), key))
    indptr = np.zeros(num_nodes + 1, I64)
    valid = key[(key >= 0) & (key < num_nodes)]
    np.add.at(indptr, valid + 1, 1)
    np.cumsum(indptr, out=indptr)
    return indptr, np.asarray(nbr, I64)[order], np.asarray(ts, I64)[order], np.asarray(eid, I64)[order], order


# ----------------------------------------------------------------------------------------------
# Philox4x32-10 (the counter-based generator of the uniform policy; published algorithm:
# Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11)
# ----------------------------------------------------------------------------------------------

_PH_M0, _PH_M1 = 0xD2511F53, 0xCD9E8D57
_PH_W0, _PH_W1 = 0x9E3779B9, 0xBB67AE85
_M32 = 0xFFFFFFFF


def philox4x32_10(ctr, key):
    c0, c1, c2, c3 = ctr
    k0, k1 = key
    for _ in range(10):
        p0 = _PH_M0 * c0
        p1 = _PH_M1 * c2
        hi0, lo0 = (p0 >> 32) & _M32, p0 & _M32
        hi1, lo1 = (p1 >> 32) & _M32, p1 & _M32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _M32, lo1, (hi0 ^ c3 ^ k1) & _M32, lo0
        k0 = (k0 + _PH_W0) & _M32
        k1 = (k1 + _PH_W1) & _M32
    return c0, c1, c2, c3


def uniform_positions(n_cand, k, seed, stream, slot):
    """k distinct positions of [0, n_cand), ascending -- Floyd's subset algorithm driven by Philox.

    Draw j (j = 0..k-1) uses counter (slot_lo, slot_hi, j, stream), key (seed_lo, seed_hi) and the
    first two output words as one 64-bit integer u; t = u mod (n_cand - k + j + 1).  If t is already
    chosen the value n_cand - k + j is taken instead.  Every k-subset is equally likely (the distribution of
    ``np.random.choice(cut, k, replace=False)`` followed by ``sort``, prepare_sample.py:124-125).
    """
    chosen = []
    for j in range(k):
        bound = n_cand - k + j + 1
        o = philox4x32_10((slot & _M32, (slot >> 32) & _M32, j, stream & _M32), (seed & _M32, (seed >> 32) & _M32))
        u = o[0] | (o[1] << 32)
        t = u % bound
        chosen.append(bound - 1 if t in chosen else t)
    return sorted(chosen)


# ----------------------------------------------------------------------------------------------
# temporal neighbour sampling
# ----------------------------------------------------------------------------------------------

RECENT, UNIFORM = 0, 1


def sample_layer(indptr, nbr, ts, eid, targets, target_ts, fanout, policy=RECENT, *, equal_root_time=False,
                 allowed_offset=-1, keep_root_time=False, seed=0, stream=0):
    """One hop.  prepare_sample.py:32-172 (continuous branch) / :248-265.

    For target i (node ``targets[i]``, query time ``t = target_ts[i]``): candidates are the row's
    edges with ``ts < t`` (``ts <= t`` with equal_root_time; additionally ``ts >= t - allowed_offset``
    when allowed_offset >= 0).  recent: the last min(k, cand) in ascending time.  uniform: all if
    cand <= k else k distinct positions, ascending.  Returns (nbr, dst_slot, ts, dt float32 = t - ts, eid)
    concatenated over targets in target order, plus the per-target counts.
    """
    targets = np.asarray(targets, I64)
    target_ts = np.asarray(target_ts, I64)
    o_n, o_d, o_t, o_dt, o_e = [], [], [], [], []
    counts = np.zeros(len(targets), I64)
    for i in range(len(targets)):
        s, e = int(indptr[targets[i]]), int(indptr[targets[i] + 1])
        t = int(target_ts[i])
        row = ts[s:e]
        cut = int(np.searchsorted(row, t + (1 if equal_root_time else 0), side="left"))
        lo = int(np.searchsorted(row, t - allowed_offset, side="left")) if allowed_offset >= 0 else 0
        lo = min(lo, cut)
        cand = cut - lo
        if cand <= 0:
            continue
        if policy == RECENT:
            pos = np.arange(max(lo, cut - fanout), cut)
        elif cand <= fanout:
            pos = np.arange(lo, cut)
        else:
            pos = lo + np.array(uniform_positions(cand, fanout, seed, stream, i), I64)
        idx = s + pos
        counts[i] = len(idx)
        o_n.append(nbr[idx])
        o_d.append(np.full(len(idx), i, I64))
        o_t.append(np.full(len(idx), t, I64) if keep_root_time else ts[idx])
        o_dt.append((t - ts[idx]).astype(np.float32))
        o_e.append(eid[idx])

    def cat(parts, dt):
        return np.concatenate(parts).astype(dt) if parts else np.zeros(0, dt)
    return cat(o_n, I64), cat(o_d, I64), cat(o_t, I64), cat(o_dt, np.float32), cat(o_e, I64), counts


# ----------------------------------------------------------------------------------------------
# relabel: (node, ts) pairs (batch dictionaries) and node level (pybind result type)
# ----------------------------------------------------------------------------------------------


def _pairs(ids, ts):
    a = np.empty(len(ids), dtype=[("id", I64), ("ts", I64)])
    a["id"], a["ts"] = ids, ts
    return a


def unique_pairs(ids, ts):
    """prepare_sample.py:205-213 -- sorted unique (id, ts) pairs and the rank of every input item."""
    u, inv = np.unique(_pairs(ids, ts), return_inverse=True)
    return u["id"].copy(), u["ts"].copy(), inv.astype(I64)


def merge_and_map(cur_ids, cur_ts, raw_ids, raw_ts):
    """prepare_sample.py:231-246 -- sorted unique union; rank of each raw item in it."""
    raw = _pairs(raw_ids, raw_ts)
    u = np.unique(np.concatenate([_pairs(cur_ids, cur_ts), raw]))
    return u["id"].copy(), u["ts"].copy(), np.searchsorted(u, raw).astype(I64)


def build_csc(src_local, dst_local, ts, dt, eid, num_dst):
    """prepare_sample.py:215-229 -- stable order by (dst_local, ts); indptr over the previous list."""
    if len(src_local) == 0:
        return np.zeros(num_dst + 1, I64), np.zeros(0, I64), np.zeros(0, I64), np.zeros(0, np.float32), np.zeros(0, I64)
    perm = np.lexsort((ts, dst_local))
    indptr = np.zeros(num_dst + 1, I64)
    d = dst_local[perm]
    np.add.at(indptr, d[d < num_dst] + 1, 1)
    np.cumsum(indptr, out=indptr)
    return indptr, src_local[perm], ts[perm], dt[perm], eid[perm]


def build_batch(indptr, nbr, ts, eid, roots, root_ts, fanouts, policy=RECENT, **kw):
    """prepare_sample.py:313-377 without route planning: list of per-layer dicts.

    Layer 0: unique (id, ts) pairs of the roots + inv_map.  Layer l+1: targets are the current unique list
    (l = 0) or one target per sampled edge of the previous hop (l > 0) at that edge's timestamp.
    """
    cur_id, cur_ts, inv0 = unique_pairs(roots, root_ts)
    out = [{"gids": cur_id, "ts": cur_ts, "inv_map": inv0}]
    last_inv = None
    for l, k in enumerate(fanouts):
        tgt = cur_id if l == 0 else cur_id[last_inv]
        tgt_t = cur_ts if l == 0 else cur_ts[last_inv]
        r_n, r_d, r_t, r_dt, r_e, _ = sample_layer(indptr, nbr, ts, eid, tgt, tgt_t, k, policy, stream=l, **kw)
        if len(r_n) == 0 and not ((indptr[tgt + 1] - indptr[tgt]) > 0).any():
            # the reference stops here when no target has any edge (prepare_sample.py:352-361)
            out.append({"indptr": np.zeros(1, I64), "indices": np.zeros(0, I64), "eid": np.zeros(0, I64),
                        "edge_ts": np.zeros(0, I64), "edge_dt": np.zeros(0, np.float32),
                        "gids": np.zeros(0, I64), "ts": np.zeros(0, I64)})
            break
        d_map = last_inv[r_d] if last_inv is not None else r_d
        n_id, n_ts, n_inv = merge_and_map(cur_id, cur_ts, r_n, r_t)
        ptr, idx, b_ts, b_dt, b_e = build_csc(n_inv, d_map, r_t, r_dt, r_e, len(cur_id))
        out.append({"indptr": ptr, "indices": idx, "eid": b_e, "edge_ts": b_ts, "edge_dt": b_dt,
                    "gids": n_id, "ts": n_ts})
        cur_id, cur_ts, last_inv = n_id, n_ts, n_inv
    return out


def relabel_nodes(id_lists):
    """Node-level relabel of csrc/include/starrygl/sample.cu.hpp:1766-1852.

    ``id_lists`` = [roots, layer-1 neighbours, layer-2 neighbours, ...].  Local ids are handed out list by
    list; inside a list the not-yet-seen ids get consecutive numbers in ascending global id.  Returns
    (list of local-id arrays, nodes_remapper_id) with nodes_remapper_id[local] = global.
    """
    seen = {}
    order = []
    out = []
    for ids in id_lists:
        new = sorted(set(int(x) for x in ids if int(x) not in seen))
        for g in new:
            seen[g] = len(order)
            order.append(g)
        out.append(np.array([seen[int(x)] for x in ids], I64))
    return out, np.array(order, I64)


# ----------------------------------------------------------------------------------------------
# ids, gather, cache
# ----------------------------------------------------------------------------------------------

LOC_MASK = (1 << 48) - 1
PART_MASK = 0x3FFF


def dist_pack(loc, part, shared=None):
    """starrygl/utils/partition_book.py:19-37."""
    d = (np.asarray(loc, I64) & LOC_MASK) | ((np.asarray(part, I64) & PART_MASK) << 48)
    if shared is not None:
        d = d | (np.asarray(shared, I64) << 62)
    return d


def dist_unpack(d):
    """starrygl/utils/partition_book.py:28-41 -> (loc, part, is_shared)."""
    d = np.asarray(d, I64)
    return d & LOC_MASK, (d >> 48) & PART_MASK, (d >> 62).astype(bool)


def build_g2l(loc_ids, global_num):
    """starrygl/utils/partition_book.py:98-104."""
    m = np.full(global_num + 1, -1, I64)
    m[loc_ids] = np.arange(len(loc_ids), dtype=I64)
    return m


def gather_rows(table, idx):
    return table[idx]


def state_read(data, ts, g2l, gids):
    """starrygl/cache/NodeState.py:36-44 with IDMapper mode 'map'."""
    loc = g2l[gids]
    return data[loc], ts[loc]


def state_update(data, ts, g2l, gids, values, new_ts):
    """starrygl/cache/NodeState.py:46-61: rows whose id is not stored locally (slot < 0) are skipped."""
    loc = g2l[gids]
    m = loc >= 0
    data[loc[m]] = values[m]
    if new_ts is not None:
        ts[loc[m]] = new_ts[m]


def cache_gather(cache_rows, hitmap, backing, ids):
    """Hit/miss split of the GPU-cache design in starrygl/cache/NodeState.py:152-194.

    slot = hitmap[id]; slot >= 0 -> row from ``cache_rows[slot]``, else from ``backing[id]``.  Returns
    (rows, hit_mask, miss_pos ascending, miss_ids).
    """
    slot = hitmap[ids]
    hit = slot >= 0
    out = np.empty((len(ids), backing.shape[1]), backing.dtype)
    out[hit] = cache_rows[slot[hit]]
    miss_pos = np.nonzero(~hit)[0].astype(I64)
    out[miss_pos] = backing[ids[miss_pos]]
    return out, hit, miss_pos, ids[miss_pos]


def build_replica_table(num_nodes, partition_book):
    """starrygl/cache/replica_table.py:178-215 -- CSR over node id of (rank, loc), sorted by (node, rank, loc)."""
    trip = []
    for p, nodes in enumerate(partition_book):
        nodes = np.asarray(nodes, I64)
        trip.append(np.stack([nodes, np.full(len(nodes), p, I64), np.arange(len(nodes), dtype=I64)]))
    allp = np.concatenate(trip, axis=1) if trip else np.zeros((3, 0), I64)
    u = np.unique(allp, axis=1)
    indptr = np.zeros(num_nodes + 1, I64)
    indptr[1:] = np.cumsum(np.bincount(u[0], minlength=num_nodes))
    return indptr, u[1].copy(), u[2].copy()


def replica_lookup(indptr, ranks, locs, ids):
    """starrygl/cache/replica_table.py:16-82 -> (src_indices, target_ranks, target_locs)."""
    s, e = indptr[ids], indptr[ids + 1]
    ln = e - s
    src = np.repeat(np.arange(len(ids), dtype=I64), ln)
    base = np.repeat(s, ln)
    inner = np.arange(ln.sum(), dtype=I64) - np.repeat(np.cumsum(ln) - ln, ln)
    g = base + inner
    return src, ranks[g], locs[g]


# ----------------------------------------------------------------------------------------------
# route (all ranks simulated in one process)
# ----------------------------------------------------------------------------------------------


def cache_route(feats, send_sizes, send_indices, send_remote, data, ts):
    """starrygl/cache/cache_route.py:211-277 + starrygl/cache/NodeState.py:269-274, all ranks at once.

    ``feats[r]`` [n_r, D+1]; ``send_sizes[r]`` [P]; ``send_indices[r]`` / ``send_remote[r]`` [S_r] grouped by
    destination rank.  Receiver q gets the segments of senders 0..P-1 in rank order and writes
    ``data[q][idx] = row[:-1]``, ``ts[q][idx] = row[-1]``.  Returns per receiver (recv_idx, recv_rows).
    """
    P = len(feats)
    offs = [np.concatenate([[0], np.cumsum(send_sizes[r])]) for r in range(P)]
    got = []
    for q in range(P):
        idx, rows = [], []
        for r in range(P):
            a, b = int(offs[r][q]), int(offs[r][q + 1])
            idx.append(np.asarray(send_remote[r][a:b], I64))
            rows.append(feats[r][np.asarray(send_indices[r][a:b], I64)])
        idx = np.concatenate(idx)
        rows = np.concatenate(rows) if len(idx) else np.zeros((0, feats[q].shape[1]), feats[q].dtype)
        if len(idx):
            data[q][idx] = rows[:, :-1]
            ts[q][idx] = rows[:, -1]
        got.append((idx, rows))
    return got


def route_forward(xs, send_sizes, recv_sizes, send_index):
    """starrygl/route/route.py:427-442 on every rank: ``cat([x, a2a(x[send_index])])``."""
    P = len(xs)
    offs = [np.concatenate([[0], np.cumsum(send_sizes[r])]).astype(int) for r in range(P)]
    ys = []
    for q in range(P):
        parts = [xs[q]]
        for r in range(P):
            seg = send_index[r][offs[r][q]:offs[r][q + 1]]
            assert len(seg) == recv_sizes[q][r]
            parts.append(xs[r][seg])
        ys.append(np.concatenate(parts))
    return ys


def route_reverse(gs, send_sizes, recv_sizes, send_index):
    """starrygl/route/route.py:444-466 on every rank: the halo tail goes back to its owners and is
    added into ``x[send_index[seg]]`` peer segment by peer segment (duplicates inside one segment keep
    the last write of ``x[idx] += v``, exactly as torch advanced indexing does)."""
    P = len(gs)
    roffs = [np.concatenate([[0], np.cumsum(recv_sizes[r])]).astype(int) for r in range(P)]
    soffs = [np.concatenate([[0], np.cumsum(send_sizes[r])]).astype(int) for r in range(P)]
    outs = []
    for r in range(P):
        n = len(gs[r]) - int(np.sum(recv_sizes[r]))
        x = gs[r][:n].copy()
        for q in range(P):   # what q received from r comes back to r
            tail = gs[q][len(gs[q]) - int(np.sum(recv_sizes[q])):]
            back = tail[roffs[q][r]:roffs[q][r + 1]]
            seg = send_index[r][soffs[r][q]:soffs[r][q + 1]]
            x[seg] += back
        outs.append(x)
    return outs


# ----------------------------------------------------------------------------------------------
# route plan of one layer
# ----------------------------------------------------------------------------------------------


def shard_gather(shards, dist_idx, me=0):
    """Distributed row gather as rank ``me`` would run it, step by step as ShardTensor::operator[] lays it out
    (csrc/include/starrygl/feature.cu.hpp:298-422): split the packed ids by owner partition (copy_if per partition, in
    partition order :353-357), send every owner its list of local rows (:367), the owner gathers them from its shard
    (tensor_gather :377-380), the rows travel back (:387) and are scattered to the positions the ids came from
    (:389-392).  ``shards[p]`` = rows owned by partition p; ``dist_idx`` = (part << 48) | loc."""
    dist_idx = np.asarray(dist_idx, I64)
    part = (dist_idx >> 48) & 0x3FFF
    loc = dist_idx & ((1 << 48) - 1)
    out = np.empty((len(dist_idx),) + shards[0].shape[1:], shards[0].dtype)
    for p in range(len(shards)):
        pos = np.nonzero(part == p)[0]          # original positions of the ids partition p owns, ascending
        asked = loc[pos]                        # id message to owner p
        rows = shards[p][asked]                 # owner-side gather, row message back
        out[pos] = rows                         # scatter to the original order
    return out


def compute_layer_route(layer_ids, layer_ts, node_parts, pid, rep_indptr, rep_ranks, rep_locs, num_parts):
    """prepare_sample.py:266-310.  For every distinct node id of the layer list: the list row with the latest timestamp
    (first such row on ties); nodes this partition owns are sent to every OTHER rank holding a replica.  Returns
    (send_ranks, send_sizes[num_parts], send_indices = list row, send_remote_indices = slot on the receiver), grouped by
    rank in ascending list-row order (the reference's order inside a rank segment is unspecified: unstable argsort),
    or None when nothing is sent."""
    layer_ids = np.asarray(layer_ids, I64)
    layer_ts = np.asarray(layer_ts, I64)
    if len(layer_ids) == 0:
        return None
    uniq, inv = np.unique(layer_ids, return_inverse=True)
    arg = np.full(len(uniq), -1, I64)
    best = np.full(len(uniq), np.iinfo(np.int64).min, I64)
    for i in range(len(layer_ids)):
        if layer_ts[i] > best[inv[i]]:
            best[inv[i]], arg[inv[i]] = layer_ts[i], i
    mine = np.asarray(node_parts)[uniq] == pid
    q_ids, q_rows = uniq[mine], arg[mine]
    if len(q_ids) == 0:
        return None
    src, ranks, locs = replica_lookup(rep_indptr, rep_ranks, rep_locs, q_ids)
    keep = ranks != pid
    src, ranks, locs = src[keep], ranks[keep], locs[keep]
    if len(ranks) == 0:
        return None
    rows = q_rows[src]
    order = np.lexsort((rows, ranks))          # by rank, then list row (stable, ascending)
    sizes = np.bincount(ranks, minlength=num_parts).astype(I64)
    return ranks[order], sizes, rows[order], locs[order]


# ----------------------------------------------------------------------------------------------
# mailbox update
# ----------------------------------------------------------------------------------------------


def scatter_max_first(values, groups, n_groups):
    """Per group the maximum and the position of its FIRST occurrence (the sequential strict-greater update of a CPU
    scatter-max; the reference calls ``torch_scatter.scatter_max``, whose GPU kernel leaves ties unordered)."""
    best = np.full(n_groups, -np.inf, dtype=np.float64)
    arg = np.full(n_groups, -1, dtype=I64)
    for j in range(len(values)):
        g = groups[j]
        if arg[g] < 0 or values[j] > best[g]:
            best[g], arg[g] = values[j], j
    return arg


def get_update_mail(src, dst, ts, edge_feats, mem_src, mem_dst, embedding=None, use_src_emb=False, use_dst_emb=False):
    """starrygl/nn/memory/mailbox.py:56-84: index = cat(src, dst); one mail row per entry
    ``[own | other | edge feature]``; timestamps cat(ts, ts) as fp32; per distinct node (ascending) the entry with the
    largest timestamp.  Returns (index, mail, mail_ts)."""
    src, dst = np.asarray(src, I64), np.asarray(dst, I64)
    n = len(src)
    emb_src = emb_dst = None
    if embedding is not None:
        emb_src, emb_dst = embedding[:n], embedding[n:]
    src_mail = np.concatenate([emb_src if use_src_emb else mem_src, emb_dst if use_dst_emb else mem_dst], 1)
    dst_mail = np.concatenate([emb_dst if use_src_emb else mem_dst, emb_src if use_dst_emb else mem_src], 1)
    if edge_feats is not None:
        src_mail = np.concatenate([src_mail, edge_feats], 1)
        dst_mail = np.concatenate([dst_mail, edge_feats], 1)
    mail = np.concatenate([src_mail, dst_mail], 0).astype(np.float32)
    mail_ts = np.concatenate([ts, ts]).astype(np.float32)
    index = np.concatenate([src, dst])
    uniq, inv = np.unique(index, return_inverse=True)
    arg = scatter_max_first(mail_ts, inv.reshape(-1), len(uniq))
    return uniq.astype(I64), mail[arg], mail_ts[arg]


def reduce_max_rows(index, rows, ts):
    """Head of mailbox.set_mailbox_local with Reduce_Op == 'max' (starrygl/nn/memory/mailbox.py:41-47)."""
    index = np.asarray(index, I64)
    ts32 = np.asarray(ts).astype(np.float32)
    uniq, inv = np.unique(index, return_inverse=True)
    arg = scatter_max_first(ts32, inv.reshape(-1), len(uniq))
    return uniq.astype(I64), rows[arg], ts32[arg]


def mailbox_write(mailbox, mailbox_ts, next_pos, index, rows, ts):
    """starrygl/nn/memory/mailbox.py:49-54 (in place): slot = next_mail_pos[index]; the position advances modulo the
    slot count when there is more than one slot."""
    index = np.asarray(index, I64)
    slots = mailbox.shape[1]
    p = next_pos[index]
    mailbox_ts[index, p] = np.asarray(ts).astype(np.float32)
    mailbox[index, p] = rows
    if slots > 1:
        next_pos[index] = (p + 1) % slots


# ----------------------------------------------------------------------------------------------
# chunk / time-window slice
# ----------------------------------------------------------------------------------------------


def slice_window(indptr, nbr, ts, eid, node_chunk, chunk_mask, t_begin, t_end):
    """Intended result of Graph::slice_by_chunk_ts (csrc/include/starrygl/sample.cu.hpp:1189-1291): edges whose two
    end nodes lie in selected chunks and whose timestamp lies in [t_begin, t_end), as node -> distinct timestamps ->
    edges.  Returns (nodes, node_ptr, group_ts, group_ptr, nbr, ts, eid)."""
    n = len(indptr) - 1
    src = np.repeat(np.arange(n, dtype=I64), np.diff(indptr))
    sel_node = np.ones(n, bool) if chunk_mask is None else np.asarray(chunk_mask, bool)[
        node_chunk if node_chunk is not None else np.zeros(n, I64)]
    keep = sel_node[src] & sel_node[nbr] & (ts >= t_begin) & (ts < t_end)
    k_src, k_nbr, k_ts, k_eid = src[keep], nbr[keep], ts[keep], eid[keep]
    e = len(k_src)
    if e == 0:
        z = np.zeros(0, I64)
        return z, np.zeros(1, I64), z, np.zeros(1, I64), z, z, z
    head = np.ones(e, bool)
    head[1:] = (k_src[1:] != k_src[:-1]) | (k_ts[1:] != k_ts[:-1])
    group_start = np.nonzero(head)[0].astype(I64)
    g_src, g_ts = k_src[group_start], k_ts[group_start]
    node_head = np.ones(len(g_src), bool)
    node_head[1:] = g_src[1:] != g_src[:-1]
    node_start = np.nonzero(node_head)[0].astype(I64)
    return (g_src[node_start], np.append(node_start, len(g_src)).astype(I64), g_ts, np.append(group_start, e).astype(I64),
            k_nbr, k_ts, k_eid)


def densify_time_groups(node_ptr, group_ts, group_ptr, t_begin, t_end):
    """The dense form the reference builds when ``use_full_timestamps`` is set (csrc/include/starrygl/sample.cu.hpp:
    454-483 for the slice, :667-683 for the roots; parity unpinned -- those kernels cannot run): every node gets all time
    steps ``t_begin .. t_end-1``; the group of (node, t) holds the node's edges with timestamp t, so its start is the
    first edge of the node with timestamp >= t.  Returns (node_ptr[U+1], ts[U*T], group_ptr[U*T+1])."""
    U, T = len(node_ptr) - 1, int(t_end - t_begin)
    o_ts = np.tile(np.arange(t_begin, t_end, dtype=I64), U)
    o_ptr = np.zeros(U * T + 1, I64)
    for u in range(U):
        a, b = int(node_ptr[u]), int(node_ptr[u + 1])
        for j in range(T):
            g = a + int(np.searchsorted(group_ts[a:b], t_begin + j, side="left"))
            o_ptr[u * T + j] = group_ptr[g]
    o_ptr[U * T] = group_ptr[node_ptr[U]] if U else 0
    return np.arange(U + 1, dtype=I64) * T, o_ts, o_ptr
