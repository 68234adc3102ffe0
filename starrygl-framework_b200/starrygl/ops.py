"""Tensor-level wrappers over the C ABI (one function per entry point of include/sgl_b200.h).

All tensors are CUDA tensors; outputs are allocated with torch (device memory plumbing only) and handed to
the kernels as raw pointers.  Functions run on the current torch CUDA stream and do not synchronise unless
the docstring says so.
"""
import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _C

I64 = torch.int64


def _i64(t):
    if t.dtype != I64:
        raise _C.SglError(f"expected int64 tensor, got {t.dtype}")
    return t.contiguous()


def bits_for(v: int) -> int:
    return max(int(v), 0).bit_length()


class StatusWord:
    """Device int32 the kernels OR error bits into; ``check()`` reads it back (one synchronisation)."""

    def __init__(self, device):
        self.t = torch.zeros(1, dtype=torch.int32, device=device)

    def ptr(self):
        return self.t.data_ptr()

    def check(self, what=""):
        v = int(self.t.item())
        if v:
            self.t.zero_()
            raise _C.SglError(f"{what}: device status {v} ({_C.decode_status(v)})")


# --------------------------------------------------------------------------------------------------------------
# sort / T-CSR
# --------------------------------------------------------------------------------------------------------------

def radix_sort_pairs(keys: torch.Tensor, vals: torch.Tensor, num_bits: int = 64):
    """Stable sort of uint64 keys (stored as int64 bit patterns) with int32 payload; returns sorted copies."""
    L = _C.lib()
    n = keys.numel()
    k0, v0 = keys.clone().contiguous(), vals.clone().contiguous()
    k1, v1 = torch.empty_like(k0), torch.empty_like(v0)
    _, wp, wn = _C.workspace(L.sgl_radix_sort_ws_bytes(n), keys.device)
    alt = C.c_int(0)
    _C.check(L.sgl_radix_sort_u64_u32(_C.ptr(k0), _C.ptr(v0), _C.ptr(k1), _C.ptr(v1), n, num_bits, C.byref(alt), wp, wn,
                                      _C.stream_ptr()))
    return (k1, v1) if alt.value else (k0, v0)


@dataclass
class TCSR:
    """Time-sorted CSR: row r = edges of node r in ascending timestamp (ties in input order)."""
    num_nodes: int
    indptr: torch.Tensor
    nbr: torch.Tensor
    ts: torch.Tensor
    eid: torch.Tensor
    perm: Optional[torch.Tensor]
    ts_min: int
    ts_max: int
    fence: Optional[torch.Tensor] = None    # timestamp of the last edge of every 32-edge block of a row (search index)

    @property
    def num_edges(self):
        return self.nbr.numel()

    @property
    def device(self):
        return self.indptr.device


def tcsr_build(key, nbr, ts, eid, num_nodes: int, want_perm: bool = False, want_fence: bool = True) -> TCSR:
    """Build the T-CSR keyed by ``key`` (and, unless ``want_fence`` is off, the search index the sampler walks before it
    touches a row).  Synchronises the stream once.  Raises on out-of-range keys."""
    L = _C.lib()
    key, nbr, ts = _i64(key), _i64(nbr), _i64(ts)
    eid = None if eid is None else _i64(eid)
    m = key.numel()
    if not (nbr.numel() == m and ts.numel() == m and (eid is None or eid.numel() == m)):
        raise _C.SglError("tcsr_build: edge arrays differ in length")
    dev = key.device
    indptr = torch.empty(num_nodes + 1, dtype=I64, device=dev)
    o_nbr, o_ts, o_eid = (torch.empty(m, dtype=I64, device=dev) for _ in range(3))
    perm = torch.empty(m, dtype=I64, device=dev) if want_perm else None
    rng = (C.c_int64 * 2)(0, 0)
    _, wp, wn = _C.workspace(L.sgl_tcsr_build_ws_bytes(num_nodes, m), dev)
    _C.check(L.sgl_tcsr_build(num_nodes, m, _C.ptr(key), _C.ptr(nbr), _C.ptr(ts), _C.ptr(eid), _C.ptr(indptr),
                              _C.ptr(o_nbr), _C.ptr(o_ts), _C.ptr(o_eid), _C.ptr(perm), rng, wp, wn, _C.stream_ptr()))
    fence = None
    if want_fence and m and num_nodes:
        fence = torch.empty(L.sgl_tcsr_fence_len(num_nodes, m), dtype=I64, device=dev)
        _C.check(L.sgl_tcsr_fence(_C.ptr(indptr), _C.ptr(o_ts), num_nodes, m, _C.ptr(fence), _C.stream_ptr()))
    return TCSR(num_nodes, indptr, o_nbr, o_ts, o_eid, perm, int(rng[0]), int(rng[1]), fence)


# --------------------------------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------------------------------

@dataclass
class Hop:
    """Compact result of one hop; valid entries are [0, offsets[-1]) -- the arrays have capacity n_targets*fanout."""
    nbr: torch.Tensor
    dst: torch.Tensor
    ts: torch.Tensor
    dt: torch.Tensor
    eid: torch.Tensor
    offsets: torch.Tensor      # [n_targets + 1]
    capacity: int
    dt_i64: Optional[torch.Tensor] = None   # ts - t (int64), only when asked for

    @property
    def d_total(self):
        """Device int64 view of the number of sampled edges."""
        return self.offsets[-1:]

    def total(self) -> int:
        """Number of sampled edges (synchronises)."""
        return int(self.offsets[-1].item())

    def trimmed(self):
        n = self.total()
        return Hop(self.nbr[:n], self.dst[:n], self.ts[:n], self.dt[:n], self.eid[:n], self.offsets, n,
                   None if self.dt_i64 is None else self.dt_i64[:n])


def sample_layer(g: TCSR, targets, target_ts, fanout: int, policy="recent", *, d_n=None, equal_root_time=False,
                 allowed_offset=-1, keep_root_time=False, seed=0, rng_stream=0, want_dt_i64=False,
                 status: Optional[StatusWord] = None) -> Hop:
    L = _C.lib()
    targets, target_ts = _i64(targets), _i64(target_ts)
    n = targets.numel()
    if target_ts.numel() != n:
        raise _C.SglError("sample_layer: targets and target_ts differ in length")
    dev = g.device
    cap = max(n * fanout, 1)
    o_nbr, o_dst, o_ts, o_eid = (torch.empty(cap, dtype=I64, device=dev) for _ in range(4))
    o_dt = torch.empty(cap, dtype=torch.float32, device=dev)
    offs = torch.empty(n + 1, dtype=I64, device=dev)
    o_dti = torch.empty(cap, dtype=I64, device=dev) if want_dt_i64 else None
    pol = _C.POLICY[policy] if isinstance(policy, str) else int(policy)
    _, wp, wn = _C.workspace(L.sgl_sample_ws_bytes(n), dev)
    _C.check(L.sgl_sample_layer_fenced(_C.ptr(g.indptr), _C.ptr(g.nbr), _C.ptr(g.ts), _C.ptr(g.eid), _C.ptr(g.fence), g.num_nodes,
                                _C.ptr(targets), _C.ptr(target_ts), n, _C.ptr(d_n), int(fanout), pol,
                                int(bool(equal_root_time)), int(allowed_offset), int(bool(keep_root_time)),
                                int(seed) & (2 ** 64 - 1), int(rng_stream) & 0xFFFFFFFF, _C.ptr(o_nbr), _C.ptr(o_dst),
                                _C.ptr(o_ts), _C.ptr(o_dt), _C.ptr(o_dti), _C.ptr(o_eid), _C.ptr(offs),
                                status.ptr() if status else None, wp, wn, _C.stream_ptr()))
    return Hop(o_nbr, o_dst, o_ts, o_dt, o_eid, offs, cap, o_dti)


# --------------------------------------------------------------------------------------------------------------
# roots of a time window
# --------------------------------------------------------------------------------------------------------------

def time_ordered_events(src, ts, eid):
    """(src, ts, eid) in ascending time, ties in input order -- the index the time-window root extraction slices.
    One-time set-up; already ordered input (the usual case for event streams) is used as is."""
    src, ts, eid = _i64(src), _i64(ts), _i64(eid)
    if ts.numel() < 2 or bool((ts[1:] >= ts[:-1]).all().item()):
        return src, ts, eid
    g = tcsr_build(torch.zeros_like(src), src, ts, eid, 1)
    return g.nbr, g.ts, g.eid


def lower_bound(sorted_vals, values):
    L = _C.lib()
    values = _i64(values)
    out = torch.empty_like(values)
    _C.check(L.sgl_lower_bound_i64(_C.ptr(sorted_vals), sorted_vals.numel(), _C.ptr(values), values.numel(),
                                   _C.ptr(out), _C.stream_ptr()))
    return out


def seeds_in_window(ev, g: TCSR, chunks, node_chunk, t_begin: int, t_end: int, *, status: Optional[StatusWord] = None):
    """Roots of the events with t_begin <= ts < t_end whose source node is in one of ``chunks``.
    Returns (roots, ts_ptr, ts, q_ptr, q_eid) trimmed to size (two small read-backs: window bounds, counts)."""
    L = _C.lib()
    ev_src, ev_ts, ev_eid = ev
    dev = ev_src.device
    lo, hi = lower_bound(ev_ts, torch.tensor([t_begin, t_end], dtype=I64, device=dev)).tolist()
    n = max(hi - lo, 0)
    chunk_mask = None
    num_chunks = 0
    d_node_chunk = None
    if node_chunk is not None and node_chunk.numel() and chunks is not None:
        if not hasattr(g, "_node_chunk_dev"):
            g._node_chunk_dev = node_chunk.to(dev, I64).contiguous()
            g._num_chunks = int(node_chunk.max().item()) + 1
        d_node_chunk, num_chunks = g._node_chunk_dev, g._num_chunks
        chunk_mask = torch.zeros(num_chunks, dtype=torch.uint8, device=dev)
        chunk_mask[chunks.to(dev, I64)] = 1
    roots, tsv, q_eid = (torch.empty(max(n, 1), dtype=I64, device=dev) for _ in range(3))
    ts_ptr, q_ptr = (torch.empty(n + 1, dtype=I64, device=dev) for _ in range(2))
    counts = torch.zeros(3, dtype=I64, device=dev)
    id_bits = bits_for(g.num_nodes - 1)
    ts_bits = bits_for(g.ts_max - g.ts_min)
    _, wp, wn = _C.workspace(L.sgl_seeds_ws_bytes(n), dev)
    sl = slice(lo, lo + n)
    _C.check(L.sgl_seeds_in_window(_C.ptr(ev_src[sl]) if n else None, _C.ptr(ev_ts[sl]) if n else None,
                                   _C.ptr(ev_eid[sl]) if n else None, n, _C.ptr(d_node_chunk), _C.ptr(chunk_mask),
                                   num_chunks, g.num_nodes, id_bits, ts_bits, g.ts_min, _C.ptr(roots), _C.ptr(ts_ptr),
                                   _C.ptr(tsv), _C.ptr(q_ptr), _C.ptr(q_eid), _C.ptr(counts),
                                   status.ptr() if status else None, wp, wn, _C.stream_ptr()))
    n_roots, n_pairs, n_ev = counts.tolist()
    return roots[:n_roots], ts_ptr[:n_roots + 1], tsv[:n_pairs], q_ptr[:n_pairs + 1], q_eid[:n_ev]


def slice_window(g: TCSR, chunks, node_chunk, t_begin: int, t_end: int, cap_edges: int, *,
                 status: Optional[StatusWord] = None):
    """Two-level CSR of the edges with ``t_begin <= ts < t_end`` whose two end nodes lie in ``chunks`` (see
    ``sgl_slice_window``; ``chunks`` None = every chunk).  Returns (nodes, node_ptr, group_ts, group_ptr, nbr, ts, eid)
    trimmed to size (one read-back of the three counts).  ``cap_edges`` bounds the kept edges, e.g. the number of events
    in the window."""
    L = _C.lib()
    dev = g.device
    chunk_mask, d_node_chunk, num_chunks = None, None, 0
    if chunks is not None and node_chunk is not None and node_chunk.numel():
        if not hasattr(g, "_node_chunk_dev"):
            g._node_chunk_dev = node_chunk.to(dev, I64).contiguous()
            g._num_chunks = int(node_chunk.max().item()) + 1
        d_node_chunk, num_chunks = g._node_chunk_dev, g._num_chunks
        chunk_mask = torch.zeros(num_chunks, dtype=torch.uint8, device=dev)
        chunk_mask[chunks.to(dev, I64)] = 1
    n, cap = g.num_nodes, max(int(cap_edges), 1)
    nodes, node_ptr = torch.empty(max(n, 1), dtype=I64, device=dev), torch.empty(n + 1, dtype=I64, device=dev)
    group_ts, nbr, ts, eid = (torch.empty(cap, dtype=I64, device=dev) for _ in range(4))
    group_ptr = torch.empty(cap + 1, dtype=I64, device=dev)
    counts = torch.zeros(3, dtype=I64, device=dev)
    _, wp, wn = _C.workspace(L.sgl_slice_window_ws_bytes(n), dev)
    _C.check(L.sgl_slice_window(_C.ptr(g.indptr), _C.ptr(g.nbr), _C.ptr(g.ts), _C.ptr(g.eid), n, _C.ptr(d_node_chunk),
                                _C.ptr(chunk_mask), num_chunks, int(t_begin), int(t_end), int(cap_edges), _C.ptr(nodes),
                                _C.ptr(node_ptr), _C.ptr(group_ts), _C.ptr(group_ptr), _C.ptr(nbr), _C.ptr(ts), _C.ptr(eid),
                                _C.ptr(counts), status.ptr() if status else None, wp, wn, _C.stream_ptr()))
    u, gcnt, e = counts.tolist()
    if status is not None:
        status.check("slice_window")
    return nodes[:u], node_ptr[:u + 1], group_ts[:gcnt], group_ptr[:gcnt + 1], nbr[:e], ts[:e], eid[:e]


def densify_time_groups(node_ptr, group_ts, group_ptr, t_begin: int, t_end: int):
    """Dense per-time-step groups out of sparse ones (see ``sgl_densify_time_groups``).  Returns
    (node_ptr[U+1], ts[U*T], group_ptr[U*T+1])."""
    L = _C.lib()
    U, T = node_ptr.numel() - 1, int(t_end) - int(t_begin)
    dev = node_ptr.device
    o_node = torch.empty(U + 1, dtype=I64, device=dev)
    o_ts = torch.empty(max(U * T, 1), dtype=I64, device=dev)
    o_ptr = torch.empty(U * T + 1, dtype=I64, device=dev)
    _C.check(L.sgl_densify_time_groups(_C.ptr(_i64(node_ptr)), _C.ptr(_i64(group_ts)) if group_ts.numel() else None,
                                       _C.ptr(_i64(group_ptr)), U, None, int(t_begin), int(t_end), _C.ptr(o_node), _C.ptr(o_ts),
                                       _C.ptr(o_ptr), _C.stream_ptr()))
    return o_node, o_ts[:U * T], o_ptr


# --------------------------------------------------------------------------------------------------------------
# relabel
# --------------------------------------------------------------------------------------------------------------

def unique_pairs(a_id, a_ts, b_id=None, b_ts=None, *, id_bits, ts_bits, ts_base, d_n_a=None, d_n_b=None,
                 status: Optional[StatusWord] = None):
    """Sorted unique (id, ts) union of segments A and B.  Returns (out_id, out_ts, inv_a, inv_b, d_n_unique);
    out arrays have capacity len(A)+len(B); the valid prefix length is the device scalar d_n_unique."""
    L = _C.lib()
    a_id, a_ts = _i64(a_id), _i64(a_ts)
    na = a_id.numel()
    nb = 0 if b_id is None else b_id.numel()
    if b_id is not None:
        b_id, b_ts = _i64(b_id), _i64(b_ts)
    dev = a_id.device
    n = na + nb
    out_id = torch.empty(max(n, 1), dtype=I64, device=dev)
    out_ts = torch.empty(max(n, 1), dtype=I64, device=dev)
    inv_a = torch.empty(max(na, 1), dtype=I64, device=dev)
    inv_b = torch.empty(max(nb, 1), dtype=I64, device=dev) if nb else None
    d_nu = torch.zeros(1, dtype=I64, device=dev)
    _, wp, wn = _C.workspace(L.sgl_unique_pairs_ws_bytes(n), dev)
    _C.check(L.sgl_unique_pairs(_C.ptr(a_id), _C.ptr(a_ts), na, _C.ptr(d_n_a), _C.ptr(b_id), _C.ptr(b_ts), nb,
                                _C.ptr(d_n_b), int(id_bits), int(ts_bits), int(ts_base), _C.ptr(out_id), _C.ptr(out_ts),
                                _C.ptr(inv_a), _C.ptr(inv_b), _C.ptr(d_nu), status.ptr() if status else None, wp, wn,
                                _C.stream_ptr()))
    return out_id, out_ts, inv_a, inv_b, d_nu


def build_csc(src_local, dst, dst_map, ts, dt, eid, num_dst: int, *, dst_bits, ts_bits, ts_base, d_n_edges=None,
              d_num_dst=None, presorted: bool = False, status: Optional[StatusWord] = None):
    """CSC of one hop, stable (dst_local, ts) order.  Returns (indptr[num_dst+1], indices, ts, dt, eid).
    ``presorted``: the edges already are in that order (first hop: target i is row i) -- no sort."""
    L = _C.lib()
    n = src_local.numel()
    dev = src_local.device
    indptr = torch.empty(num_dst + 1, dtype=I64, device=dev)
    o_idx, o_ts, o_eid = (torch.empty(max(n, 1), dtype=I64, device=dev) for _ in range(3))
    o_dt = torch.empty(max(n, 1), dtype=torch.float32, device=dev)
    _, wp, wn = _C.workspace(L.sgl_build_csc_ws_bytes(n, num_dst), dev)
    _C.check(L.sgl_build_csc(_C.ptr(src_local), _C.ptr(dst), _C.ptr(dst_map), _C.ptr(ts), _C.ptr(dt), _C.ptr(eid), n,
                             _C.ptr(d_n_edges), num_dst, _C.ptr(d_num_dst), int(dst_bits), int(ts_bits), int(ts_base),
                             _C.ptr(indptr), _C.ptr(o_idx), _C.ptr(o_ts), _C.ptr(o_dt), _C.ptr(o_eid), int(bool(presorted)),
                             status.ptr() if status else None, wp, wn, _C.stream_ptr()))
    return indptr, o_idx, o_ts, o_dt, o_eid


class NodeRelabeler:
    """Node-level relabel state (csrc/include/starrygl/sample.cu.hpp:1752-1854): a per-node local-id table and an
    epoch mask; ``reset()`` starts a new numbering without clearing the tables."""

    def __init__(self, num_nodes: int, device):
        self.num_nodes = num_nodes
        self.mapper = torch.zeros(num_nodes, dtype=I64, device=device)
        self.mask = torch.zeros(num_nodes, dtype=I64, device=device)
        self.epoch = 1
        self.next_local = torch.zeros(1, dtype=I64, device=device)

    def reset(self):
        self.epoch += 1
        self.next_local.zero_()

    def insert(self, ids, d_n=None, status: Optional[StatusWord] = None):
        """Returns (local ids of ``ids``, new global ids in local-id order [capacity len(ids)], device count of new ids)."""
        L = _C.lib()
        ids = _i64(ids)
        n = ids.numel()
        dev = ids.device
        out_local = torch.empty(max(n, 1), dtype=I64, device=dev)
        new_ids = torch.empty(max(n, 1), dtype=I64, device=dev)
        d_new = torch.zeros(1, dtype=I64, device=dev)
        _, wp, wn = _C.workspace(L.sgl_relabel_nodes_ws_bytes(n), dev)
        _C.check(L.sgl_relabel_nodes(_C.ptr(ids), n, _C.ptr(d_n), self.num_nodes, _C.ptr(self.mapper), _C.ptr(self.mask),
                                     self.epoch, _C.ptr(self.next_local), _C.ptr(out_local), _C.ptr(new_ids),
                                     _C.ptr(d_new), status.ptr() if status else None, wp, wn, _C.stream_ptr()))
        return out_local[:n], new_ids, d_new


# --------------------------------------------------------------------------------------------------------------
# gather / scatter / cache
# --------------------------------------------------------------------------------------------------------------

def _row_bytes(t):
    if t.dim() == 1:
        return t.element_size(), t.element_size()
    if t.stride(-1) != 1 and t.shape[-1] > 1:
        raise _C.SglError("rows must be contiguous")
    inner = 1
    for s in t.shape[1:]:
        inner *= s
    return inner * t.element_size(), t.stride(0) * t.element_size()


def gather_rows(table, idx, *, map=None, d_n=None, ts_table=None, mode="auto", out=None,
                status: Optional[StatusWord] = None):
    """out[i] = table[row(i)] (row(i) = map[idx[i]] when map is given; negative rows count from the end).
    With ts_table also returns ts_table[row(i)]."""
    L = _C.lib()
    idx = _i64(idx)
    n = idx.numel()
    row_bytes, src_pitch = _row_bytes(table)
    if out is None:
        out = torch.empty((n,) + tuple(table.shape[1:]), dtype=table.dtype, device=idx.device)
    _, dst_pitch = _row_bytes(out) if n else (row_bytes, row_bytes)
    out_ts = torch.empty(n, dtype=torch.float32, device=idx.device) if ts_table is not None else None
    _C.check(L.sgl_gather_rows(_C.ptr(table) if table.numel() else None, table.shape[0], row_bytes, src_pitch,
                               _C.ptr(idx), _C.ptr(map), 0 if map is None else map.numel(), n, _C.ptr(d_n),
                               out.data_ptr() if out.numel() else None, dst_pitch, _C.ptr(ts_table), _C.ptr(out_ts),
                               _C.GATHER_MODE[mode], status.ptr() if status else None, _C.stream_ptr()))
    return (out, out_ts) if ts_table is not None else out


def scatter_rows(table, idx, rows, *, map=None, d_n=None, ts_table=None, ts=None, split_last_col=False,
                 status: Optional[StatusWord] = None):
    """table[row(i)] = rows[i] for row(i) >= 0; optionally ts_table[row(i)] = ts[i] (or the trailing column)."""
    L = _C.lib()
    idx = _i64(idx)
    n = idx.numel()
    row_bytes, dst_pitch = _row_bytes(table)
    _, src_pitch = _row_bytes(rows) if n else (0, row_bytes + (4 if split_last_col else 0))
    _C.check(L.sgl_scatter_rows(_C.ptr(table) if table.numel() else None, table.shape[0], row_bytes, dst_pitch,
                                _C.ptr(idx), _C.ptr(map), 0 if map is None else map.numel(), n, _C.ptr(d_n),
                                rows.data_ptr() if rows.numel() else None, src_pitch, _C.ptr(ts_table), _C.ptr(ts),
                                int(bool(split_last_col)), status.ptr() if status else None, _C.stream_ptr()))


def cache_gather(cache_rows, hitmap, backing, ids, *, status: Optional[StatusWord] = None):
    """Gather through the device cache.  Returns (out, miss_pos, miss_ids, counts) where counts = [hits, misses]
    (device int64) and the miss lists have capacity len(ids)."""
    L = _C.lib()
    ids = _i64(ids)
    n = ids.numel()
    if hitmap.dtype != torch.int32:
        raise _C.SglError("hitmap must be int32")
    row_bytes, pitch = _row_bytes(cache_rows)
    if pitch != row_bytes or (backing is not None and _row_bytes(backing) != (row_bytes, row_bytes)):
        raise _C.SglError("cache and backing rows must be dense and of equal size")
    dev = ids.device
    out = torch.empty((n,) + tuple(cache_rows.shape[1:]), dtype=cache_rows.dtype, device=dev)
    miss_pos = torch.empty(max(n, 1), dtype=I64, device=dev)
    miss_ids = torch.empty(max(n, 1), dtype=I64, device=dev)
    counts = torch.zeros(2, dtype=I64, device=dev)
    _, wp, wn = _C.workspace(L.sgl_cache_gather_ws_bytes(n), dev)
    _C.check(L.sgl_cache_gather(_C.ptr(cache_rows), cache_rows.shape[0], _C.ptr(hitmap), hitmap.numel(),
                                _C.ptr(backing), row_bytes, _C.ptr(ids), n,
                                out.data_ptr() if n else None, _C.ptr(miss_pos), _C.ptr(miss_ids), _C.ptr(counts),
                                status.ptr() if status else None, wp, wn, _C.stream_ptr()))
    return out, miss_pos, miss_ids, counts


# --------------------------------------------------------------------------------------------------------------
# route helpers, ids
# --------------------------------------------------------------------------------------------------------------

def wire_pitch(dim: int, has_ts: bool, has_slot: bool = True) -> int:
    """Floats per wire row: payload, and with slots two slot words plus zero padding to a multiple of four."""
    w = dim + (1 if has_ts else 0)
    return (w + 2 + 3) // 4 * 4 if has_slot else w


def route_pack(feats, ts, send_idx, *, remote_idx=None, status: Optional[StatusWord] = None):
    """Send buffer rows ``[feats[send_idx[i]] | ts[send_idx[i]] | remote_idx[i] as two 32-bit words]`` (float32);
    the timestamp column and the slot words are present only when ``ts`` / ``remote_idx`` are given."""
    L = _C.lib()
    send_idx = _i64(send_idx)
    if feats.dtype != torch.float32 or feats.dim() != 2 or not feats.is_contiguous():
        raise _C.SglError("route_pack: feats must be a contiguous float32 matrix")
    if ts is not None:
        ts = ts.to(torch.float32).contiguous()
    n, d = send_idx.numel(), feats.shape[1]
    packed = torch.empty(n, wire_pitch(d, ts is not None, remote_idx is not None), dtype=torch.float32,
                         device=send_idx.device)
    _C.check(L.sgl_route_pack(_C.ptr(feats), feats.shape[0], d, _C.ptr(ts), _C.ptr(send_idx),
                              None if remote_idx is None else _C.ptr(_i64(remote_idx)), n,
                              packed.data_ptr() if n else None, status.ptr() if status else None, _C.stream_ptr()))
    return packed


def route_unpack(wire, width: int, data, ts_table=None, *, status: Optional[StatusWord] = None):
    """Receiver side of :func:`route_pack` rows carrying their slot: data[slot] = row[:dim], ts_table[slot] = row[dim]."""
    L = _C.lib()
    n = wire.shape[0]
    if n == 0:
        return
    if wire.dtype != torch.float32 or not wire.is_contiguous() or wire.shape[1] != wire_pitch(width, False):
        raise _C.SglError("route_unpack: wire rows must be contiguous float32 with the pitch of wire_pitch()")
    _C.check(L.sgl_route_unpack(_C.ptr(wire), n, width, _C.ptr(data), data.shape[0], data.shape[1], _C.ptr(ts_table),
                                status.ptr() if status else None, _C.stream_ptr()))


def wire_slots(wire, width: int):
    """The int64 write slots carried in the last two 32-bit words of every wire row."""
    return wire[:, width:width + 2].contiguous().view(torch.int64).reshape(-1)


def route_add_rows(x, send_idx, outs, *, status: Optional[StatusWord] = None):
    """x[send_idx[j]] += outs[j] for one peer segment (indices unique inside the segment)."""
    L = _C.lib()
    send_idx = _i64(send_idx)
    n = send_idx.numel()
    if n == 0:
        return
    x2 = x.view(x.shape[0], -1)
    _C.check(L.sgl_route_add_rows(_C.ptr(x2), x2.shape[0], x2.shape[1], _C.ptr(send_idx), _C.ptr(outs.contiguous()), n,
                                  status.ptr() if status else None, _C.stream_ptr()))


def route_groups(send_index):
    """Grouping of a route's ``send_index`` by destination row for :func:`route_add_grouped` (built once per route):
    ``(rows[U], row_ptr[U+1], pos[S])`` -- the distinct rows, and for each the positions in ``send_index`` that name it,
    ascending (= peer order).  A stable sort by row; the small amount of bookkeeping around it is torch."""
    send_index = _i64(send_index)
    n = send_index.numel()
    dev = send_index.device
    if n == 0:
        z = torch.zeros(0, dtype=I64, device=dev)
        return z, torch.zeros(1, dtype=I64, device=dev), z
    if (send_index < 0).any():
        raise _C.SglError("route_groups: negative rows are not supported in a route's send_index")
    keys, pos = radix_sort_pairs(send_index, torch.arange(n, dtype=torch.int32, device=dev),
                                 num_bits=bits_for(int(send_index.max().item())))
    rows, counts = torch.unique_consecutive(keys, return_counts=True)
    row_ptr = torch.zeros(rows.numel() + 1, dtype=I64, device=dev)
    row_ptr[1:] = torch.cumsum(counts, 0)
    return rows.contiguous(), row_ptr, pos.to(I64).contiguous()


def route_add_grouped(x, groups, outs, *, status: Optional[StatusWord] = None):
    """``x[rows[u]] += outs[pos[j]]`` for every group, contributions added in ascending position: all peer segments of
    the reverse route in one launch, same float32 result as the per-peer loop."""
    L = _C.lib()
    rows, row_ptr, pos = groups
    if rows.numel() == 0:
        return
    if x.dtype != torch.float32 or outs.dtype != torch.float32:
        raise _C.SglError("route_add_grouped accumulates float32 rows")
    x2, o2 = x.view(x.shape[0], -1), outs.contiguous().view(outs.shape[0], -1)
    _C.check(L.sgl_route_add_grouped(_C.ptr(x2), x2.shape[0], x2.shape[1], _C.ptr(rows), _C.ptr(row_ptr), _C.ptr(pos),
                                     rows.numel(), _C.ptr(o2), o2.shape[0], status.ptr() if status else None, _C.stream_ptr()))


def shard_gather(d_bases, d_shard_rows, world: int, row_shape, dtype, dist_idx, *, d_n=None,
                 status: Optional[StatusWord] = None):
    """Rows of a table sharded over the GPUs of one node, read from their owners' memory (see ``sgl_shard_gather``).
    ``d_bases`` / ``d_shard_rows``: device int64 arrays of the shards' base addresses and row counts."""
    L = _C.lib()
    dist_idx = _i64(dist_idx)
    n = dist_idx.numel()
    out = torch.empty((n,) + tuple(row_shape), dtype=dtype, device=dist_idx.device)
    row_bytes = out.element_size()
    for d in row_shape:
        row_bytes *= int(d)
    _C.check(L.sgl_shard_gather(_C.ptr(d_bases), _C.ptr(d_shard_rows), int(world), row_bytes, _C.ptr(dist_idx), n, _C.ptr(d_n),
                                out.data_ptr() if n else None, status.ptr() if status else None, _C.stream_ptr()))
    return out


def dist_pack(loc, part, shared=None):
    L = _C.lib()
    loc, part = _i64(loc), _i64(part)
    out = torch.empty_like(loc)
    sh = None if shared is None else shared.to(torch.uint8).contiguous()
    _C.check(L.sgl_dist_pack(_C.ptr(loc), _C.ptr(part), _C.ptr(sh), loc.numel(), _C.ptr(out), _C.stream_ptr()))
    return out


def dist_unpack(dist):
    L = _C.lib()
    dist = _i64(dist)
    loc, part = torch.empty_like(dist), torch.empty_like(dist)
    sh = torch.empty(dist.numel(), dtype=torch.uint8, device=dist.device)
    _C.check(L.sgl_dist_unpack(_C.ptr(dist), dist.numel(), _C.ptr(loc), _C.ptr(part), _C.ptr(sh), _C.stream_ptr()))
    return loc, part, sh.view(dist.shape).bool()


def replica_lookup(indptr, ranks, locs, ids, cap: int, *, status: Optional[StatusWord] = None):
    """Returns (src, rank, loc, offsets); the three lists have capacity ``cap``, valid length offsets[-1]."""
    L = _C.lib()
    ids = _i64(ids)
    n = ids.numel()
    dev = ids.device
    src, rk, lc = (torch.empty(max(cap, 1), dtype=I64, device=dev) for _ in range(3))
    offs = torch.empty(n + 1, dtype=I64, device=dev)
    _, wp, wn = _C.workspace(L.sgl_replica_lookup_ws_bytes(n), dev)
    _C.check(L.sgl_replica_lookup(_C.ptr(indptr), _C.ptr(ranks), _C.ptr(locs), indptr.numel() - 1, _C.ptr(ids), n, cap,
                                  _C.ptr(src), _C.ptr(rk), _C.ptr(lc), _C.ptr(offs), status.ptr() if status else None,
                                  wp, wn, _C.stream_ptr()))
    return src, rk, lc, offs


def plan_route(layer_ids, node_parts, pid: int, rep_indptr, rep_ranks, rep_locs, num_parts: int, cap: int, *, d_n=None,
               status: Optional[StatusWord] = None):
    """Route plan of one layer (see ``sgl_plan_route``).  Returns (ranks, rows, locs, send_sizes[num_parts], d_total);
    the three lists have capacity ``cap``, valid length ``d_total`` (device scalar)."""
    L = _C.lib()
    layer_ids = _i64(layer_ids)
    n = layer_ids.numel()
    dev = layer_ids.device
    ranks, rows, locs = (torch.empty(max(cap, 1), dtype=I64, device=dev) for _ in range(3))
    sizes = torch.zeros(num_parts, dtype=I64, device=dev)
    total = torch.zeros(1, dtype=I64, device=dev)
    _, wp, wn = _C.workspace(L.sgl_plan_route_ws_bytes(n, cap), dev)
    _C.check(L.sgl_plan_route(_C.ptr(layer_ids), n, _C.ptr(d_n), _C.ptr(_i64(node_parts)), node_parts.numel(), int(pid),
                              _C.ptr(rep_indptr), _C.ptr(rep_ranks), _C.ptr(rep_locs), int(num_parts), int(cap), _C.ptr(ranks),
                              _C.ptr(rows), _C.ptr(locs), _C.ptr(sizes), _C.ptr(total), status.ptr() if status else None, wp, wn,
                              _C.stream_ptr()))
    return ranks, rows, locs, sizes, total


# --------------------------------------------------------------------------------------------------------------
# mailbox update
# --------------------------------------------------------------------------------------------------------------

def mail_reduce(ids_a, ids_b, ts, num_nodes: int, segments=(), *, want_pos: bool = False,
                status: Optional[StatusWord] = None):
    """Latest message per node (see ``sgl_mail_reduce``).  ``ids_a`` / ``ids_b``: int64 node ids of the two entry lists
    (``ids_b`` may be None); ``ts``: int64 or fp32, one value per entry or one per event; ``segments``: list of
    ``(table_a, table_b)`` fp32 row tables whose rows are concatenated into the mail of the winning entry.
    Returns ``(index, mail, mail_ts, pos, d_num_unique)`` with capacity ``len(ids_a) + len(ids_b)``; the valid
    length is the device scalar ``d_num_unique`` (no synchronisation here).  ``mail`` is None without segments."""
    L = _C.lib()
    ids_a = _i64(ids_a)
    dev = ids_a.device
    n_a = ids_a.numel()
    ids_b = _i64(ids_b) if ids_b is not None else None
    n_b = ids_b.numel() if ids_b is not None else 0
    n = n_a + n_b
    if ts.dtype not in (torch.int64, torch.float32):
        raise _C.SglError(f"mail_reduce: timestamps must be int64 or float32, got {ts.dtype}")
    ts = ts.contiguous()
    segs = []
    for ta, tb in segments:
        ta = ta.contiguous()
        tb = ta if tb is None else tb.contiguous()
        if ta.dtype != torch.float32 or tb.dtype != torch.float32 or ta.dim() != 2 or tb.shape[1:] != ta.shape[1:]:
            raise _C.SglError("mail_reduce: segments are pairs of fp32 [rows, dim] tables of equal width")
        if ta.shape[0] < n_a or (n_b and tb.shape[0] < n_b):
            raise _C.SglError("mail_reduce: a segment table has fewer rows than its entry list")
        segs.append((ta, tb))
    width = sum(int(a.shape[1]) for a, _ in segs)
    cap = max(n, 1)
    index = torch.empty(cap, dtype=I64, device=dev)
    pos = torch.empty(cap, dtype=I64, device=dev) if want_pos else None
    out_ts = torch.empty(cap, dtype=torch.float32, device=dev)
    mail = torch.empty((cap, width), dtype=torch.float32, device=dev) if segs else None
    d_u = torch.zeros(1, dtype=I64, device=dev)
    k = len(segs)
    arr_a = (C.c_void_p * max(k, 1))(*[a.data_ptr() for a, _ in segs])
    arr_b = (C.c_void_p * max(k, 1))(*[b.data_ptr() for _, b in segs])
    arr_d = (C.c_int64 * max(k, 1))(*[int(a.shape[1]) for a, _ in segs])
    _, wp, wn = _C.workspace(L.sgl_mail_reduce_ws_bytes(n), dev)
    _C.check(L.sgl_mail_reduce(_C.ptr(ids_a), n_a, _C.ptr(ids_b) if n_b else None, n_b, int(num_nodes), _C.ptr(ts), ts.numel(),
                               1 if ts.dtype == torch.int64 else 0, k, C.cast(arr_a, C.c_void_p), C.cast(arr_b, C.c_void_p),
                               C.cast(arr_d, C.c_void_p), _C.ptr(index), _C.ptr(pos) if want_pos else None, _C.ptr(out_ts),
                               _C.ptr(mail) if mail is not None else None, _C.ptr(d_u), status.ptr() if status else None,
                               wp, wn, _C.stream_ptr()))
    return index, mail, out_ts, pos, d_u


def mailbox_write(index, mail, mail_ts, mailbox, mailbox_ts, next_mail_pos, *, d_n=None, advance: bool = True,
                  status: Optional[StatusWord] = None):
    """``mailbox[index, next_mail_pos[index]] = mail`` (+ timestamps, + ring position), see ``sgl_mailbox_write``.
    ``index`` must hold distinct nodes.  With ``d_n`` (device int64) only the first ``*d_n`` rows are written."""
    L = _C.lib()
    index = _i64(index)
    if mailbox.dim() != 3 or not mailbox.is_contiguous() or not mailbox_ts.is_contiguous():
        raise _C.SglError("mailbox_write: mailbox must be a contiguous [nodes, slots, width] tensor")
    nodes, slots, width = mailbox.shape
    if mail.dim() != 2 or mail.shape[1] != width or mail.dtype != torch.float32 or mail_ts.dtype != torch.float32:
        raise _C.SglError("mailbox_write: mail rows must be fp32 of the mailbox's width")
    if next_mail_pos is not None:
        next_mail_pos = _i64(next_mail_pos)
    n = min(index.numel(), mail.shape[0])
    _C.check(L.sgl_mailbox_write(_C.ptr(index), n, _C.ptr(d_n), _C.ptr(mail.contiguous()), _C.ptr(mail_ts.contiguous()), width,
                                 _C.ptr(mailbox), _C.ptr(mailbox_ts), _C.ptr(next_mail_pos) if next_mail_pos is not None else None,
                                 nodes, slots, 1 if advance else 0, status.ptr() if status else None, _C.stream_ptr()))
