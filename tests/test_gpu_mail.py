"""Mailbox update on the GPU (latest message per node, row assembly, mailbox write) against the oracle and against the
vectors produced by the reference's ``mailbox.get_update_mail``."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, npy
from test_oracle_golden import _mail_case, load

pytestmark = pytest.mark.gpu


def _mb(n_nodes, slots, d, e):
    from starrygl.nn.memory.mailbox import mailbox
    return mailbox(n_nodes, slots, d, e, device="cuda")


def test_get_update_mail_matches_reference_vectors():
    z = load("mail.npz")
    for c in range(int(z["n_cases"])):
        (src, dst, ts, ef, ms, md), kw = _mail_case(z, c)
        mb = _mb(int(z[f"c{c}_n_nodes"]), 1, ms.shape[1], 0 if ef is None else ef.shape[1])
        if kw:
            kw = dict(kw, embedding=cu(kw["embedding"]))
        index, mail, mail_ts = mb.get_update_mail(cu(src), cu(dst), cu(ts), None if ef is None else cu(ef), cu(ms), cu(md), **kw)
        mb.status.check("mail")
        assert np.array_equal(npy(index), z[f"c{c}_index"]), c
        assert np.array_equal(npy(mail_ts), z[f"c{c}_mail_ts"]), c
        assert np.array_equal(npy(mail), z[f"c{c}_mail"]), c


@pytest.mark.parametrize("n_nodes,B,D,E,fp_ts", [(1, 5, 3, 0, False), (1000, 4000, 100, 172, False), (1 << 20, 20000, 32, 16, True),
                                                  (70000, 1, 1, 1, False)])
def test_get_update_mail_random(n_nodes, B, D, E, fp_ts):
    rng = np.random.default_rng(B + D)
    src = rng.integers(0, n_nodes, B)
    dst = rng.integers(0, n_nodes, B)                     # self loops and repeated nodes allowed: ties are exercised
    ts = np.sort(rng.integers(0, max(B // 4, 2), B)).astype(np.int64)
    if fp_ts:
        ts = (ts.astype(np.float32) * np.float32(0.37) - np.float32(100.0)).astype(np.float32)   # negative and fractional
    ms, md = rng.standard_normal((B, D)).astype(np.float32), rng.standard_normal((B, D)).astype(np.float32)
    ef = rng.standard_normal((B, E)).astype(np.float32) if E else None
    mb = _mb(n_nodes, 1, D, E)
    index, mail, mail_ts = mb.get_update_mail(cu(src), cu(dst), cu(ts), None if ef is None else cu(ef), cu(ms), cu(md))
    mb.status.check("mail")
    o_index, o_mail, o_ts = O.get_update_mail(src, dst, ts, ef, ms, md)
    assert np.array_equal(npy(index), o_index)
    assert np.array_equal(npy(mail_ts), o_ts)
    assert np.array_equal(npy(mail), o_mail)


def test_empty_batch_and_bad_node():
    from starrygl import _C
    mb = _mb(10, 1, 4, 0)
    e = torch.zeros(0, dtype=torch.int64, device="cuda")
    index, mail, mail_ts = mb.get_update_mail(e, e, e, None, torch.zeros(0, 4, device="cuda"), torch.zeros(0, 4, device="cuda"))
    assert index.numel() == 0 and mail.shape == (0, 8) and mail_ts.numel() == 0
    one = torch.tensor([3], device="cuda")
    bad = torch.tensor([10], device="cuda")
    mb.get_update_mail(one, bad, one, None, torch.zeros(1, 4, device="cuda"), torch.zeros(1, 4, device="cuda"))
    with pytest.raises(_C.SglError):
        mb.status.check("mail")


@pytest.mark.parametrize("slots", [1, 3])
def test_mailbox_steps_match_oracle(slots):
    """Several update steps: reduce -> write -> ring position, state compared after every step; then the read side."""
    rng = np.random.default_rng(slots)
    n_nodes, B, D, E = 500, 300, 8, 6
    W = 2 * D + E
    mb = _mb(n_nodes, slots, D, E)
    r_mb, r_ts, r_pos = np.zeros((n_nodes, slots, W), np.float32), np.zeros((n_nodes, slots), np.float32), np.zeros(n_nodes, np.int64)
    for step in range(6):
        src, dst = rng.integers(0, n_nodes, B), rng.integers(0, n_nodes, B)
        ts = np.sort(rng.integers(1000 * step, 1000 * (step + 1), B)).astype(np.int64)
        ms, md = rng.standard_normal((B, D)).astype(np.float32), rng.standard_normal((B, D)).astype(np.float32)
        ef = rng.standard_normal((B, E)).astype(np.float32)
        if step % 2 == 0:    # synchronous form
            index, mail, mail_ts = mb.get_update_mail(cu(src), cu(dst), cu(ts), cu(ef), cu(ms), cu(md))
            mb.update_mailbox(index, mail, mail_ts)
        else:                # no host synchronisation between the reduce and the write
            index, mail, mail_ts, d_n = mb.get_update_mail_async(cu(src), cu(dst), cu(ts), cu(ef), cu(ms), cu(md))
            mb.update_mailbox(index, mail, mail_ts, d_n=d_n)
        o_index, o_mail, o_ts = O.get_update_mail(src, dst, ts, ef, ms, md)
        O.mailbox_write(r_mb, r_ts, r_pos, o_index, o_mail, o_ts)
        mb.status.check("mailbox")
        assert np.array_equal(npy(mb.mailbox), r_mb) and np.array_equal(npy(mb.mailbox_ts), r_ts), step
        assert np.array_equal(npy(mb.next_mail_pos), r_pos), step
    idx = rng.integers(0, n_nodes, 64)
    rows, ts = mb.get_message(cu(idx))
    assert np.array_equal(npy(rows), r_mb[idx]) and np.array_equal(npy(ts), r_ts[idx])


def test_set_mailbox_local_with_max_reduce():
    rng = np.random.default_rng(9)
    n_nodes, n, W = 200, 1000, 20
    mb = _mb(n_nodes, 2, 5, 10)
    index = rng.integers(0, n_nodes, n)
    rows, ts = rng.standard_normal((n, W)).astype(np.float32), rng.integers(0, 300, n).astype(np.float32)
    mb.set_mailbox_local(cu(index), cu(rows), cu(ts), Reduce_Op='max')
    mb.status.check("mailbox")
    r_mb, r_ts, r_pos = np.zeros((n_nodes, 2, W), np.float32), np.zeros((n_nodes, 2), np.float32), np.zeros(n_nodes, np.int64)
    O.mailbox_write(r_mb, r_ts, r_pos, *O.reduce_max_rows(index, rows, ts))
    assert np.array_equal(npy(mb.mailbox), r_mb) and np.array_equal(npy(mb.mailbox_ts), r_ts)
    assert np.array_equal(npy(mb.next_mail_pos), r_pos)
