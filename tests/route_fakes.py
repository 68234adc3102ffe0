"""CPU stand-ins for the CUDA data-movement calls, used ONLY by the multi-rank host-logic tests (gloo ranks have
no GPU).  They restate the kernels' contracts with torch indexing; the shipped package never imports this file."""
import torch


def gather_rows(table, idx, *, map=None, d_n=None, ts_table=None, mode="auto", out=None, status=None):
    rows = idx if map is None else map[idx]
    res = table[rows]
    return (res, ts_table[rows]) if ts_table is not None else res


def route_pack(feats, ts, send_idx, *, remote_idx=None, status=None):
    cols = [feats[send_idx]]
    if ts is not None:
        cols.append(ts[send_idx].reshape(-1, 1).float())
    if remote_idx is not None:
        cols.append(remote_idx.contiguous().view(torch.float32).reshape(-1, 2))
        w = sum(c.shape[1] for c in cols)
        cols.append(torch.zeros(len(send_idx), (w + 3) // 4 * 4 - w))
    return torch.cat(cols, 1).contiguous()


def route_unpack(wire, width, data, ts_table=None, *, status=None):
    slots = wire[:, width:width + 2].contiguous().view(torch.int64).reshape(-1)
    d = data.shape[1]
    data[slots] = wire[:, :d]
    if ts_table is not None:
        ts_table[slots] = wire[:, d]


def route_add_rows(x, send_idx, outs, *, status=None):
    x[send_idx] += outs


def scatter_rows(table, idx, rows, *, map=None, d_n=None, ts_table=None, ts=None, split_last_col=False, status=None):
    r = idx if map is None else map[idx]
    keep = r >= 0
    d = table.shape[1]
    table[r[keep]] = rows[keep][:, :d]
    if ts_table is not None:
        ts_table[r[keep]] = rows[keep][:, d] if split_last_col else ts[keep]


def install(monkeypatch_or_module=None):
    from starrygl import ops
    for name in ("gather_rows", "route_pack", "route_unpack", "route_add_rows", "scatter_rows"):
        setattr(ops, name, globals()[name])
