"""Failure handling of the peer-memory route on ONE GPU (world size 1, the rank is its own peer): an apply kernel whose
rows never arrive gives up after its (shortened) bound, reports SGL_DEV_TIMEOUT through the status word, publishes
nothing -- and the process keeps working: a fresh route context moves rows normally afterwards.  Nothing here hangs or
faults the GPU: the wait that runs out is the kernel's own bounded poll."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DIM, ROWS, SLOTS = 8, 5, 100


def make_ctx(L, _C, wait_ms=-1, bulk_bytes=-1, dim=DIM):
    pitch = L.sgl_wire_pitch(dim, 1, 1)
    nbytes = L.sgl_p2p_buffer_bytes(1, 2, 64, pitch)
    base, handle = C.c_void_p(), C.create_string_buffer(64)
    _C.check(L.sgl_p2p_alloc(nbytes, C.byref(base), handle, 64))
    bases = (C.c_void_p * 1)(base.value)
    ctx = C.c_void_p()
    _C.check(L.sgl_p2p_route_create(0, 1, 2, 64, pitch, bases, C.byref(ctx)))
    _C.check(L.sgl_p2p_route_configure(ctx, wait_ms, bulk_bytes))
    return ctx, base


def test_apply_gives_up_with_a_status_and_the_context_stays_usable():
    from starrygl import _C, ops
    L = _C.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    data, ts = torch.zeros(SLOTS, DIM, device=dev), torch.zeros(SLOTS, device=dev)
    status = ops.StatusWord(dev)
    n_rows = (C.c_int64 * 1)(ROWS)
    sp = _C.stream_ptr()

    # (1) nothing was sent for step 0: the wait for the sender's word runs out
    ctx, base = make_ctx(L, _C, wait_ms=200)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _C.check(L.sgl_p2p_route_recv(ctx, n_rows, data.data_ptr(), SLOTS, DIM, 1, ts.data_ptr(), 0, status.ptr(), sp))
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.15 < waited < 10.0, waited
    with pytest.raises(_C.SglError, match="(?i)timeout|wait"):
        status.check("apply without rows")
    assert not data.any() and not ts.any()                      # nothing was applied
    _C.check(L.sgl_p2p_route_destroy(ctx))
    _C.check(L.sgl_p2p_free(base))

    # (2) same process, fresh context: send + apply of real rows
    ctx, base = make_ctx(L, _C)
    feats = torch.randn(50, DIM, device=dev)
    fts = torch.rand(50, device=dev)
    send_idx = torch.tensor([3, 7, 7, 49, 0], device=dev)
    slots = torch.tensor([10, 11, 99, 0, 42], device=dev)
    _C.check(L.sgl_p2p_route_send(ctx, feats.data_ptr(), 50, DIM, fts.data_ptr(), send_idx.data_ptr(), slots.data_ptr(), n_rows,
                                  0, status.ptr(), sp))
    _C.check(L.sgl_p2p_route_recv(ctx, n_rows, data.data_ptr(), SLOTS, DIM, 1, ts.data_ptr(), 0, status.ptr(), sp))
    torch.cuda.synchronize()
    status.check("send + apply")
    want_d, want_t = np.zeros((SLOTS, DIM), np.float32), np.zeros(SLOTS, np.float32)
    want_d[slots.cpu().numpy()] = feats.cpu().numpy()[send_idx.cpu().numpy()]
    want_t[slots.cpu().numpy()] = fts.cpu().numpy()[send_idx.cpu().numpy()]
    assert np.array_equal(data.cpu().numpy(), want_d) and np.array_equal(ts.cpu().numpy(), want_t)
    _C.check(L.sgl_p2p_route_destroy(ctx))
    _C.check(L.sgl_p2p_free(base))


@pytest.mark.parametrize("dim", [8, 100])
@pytest.mark.parametrize("bulk_bytes", [1, 1000000000])
@pytest.mark.parametrize("counts_on", ["host", "device"])
def test_world1_roundtrip_plain_rows_and_tagged_lines(bulk_bytes, dim, counts_on):
    """Both wire forms of a pair's message (plain rows + completion word for large messages, tagged lines for small
    ones), 4-byte and 128-bit row lanes (dim 8 / dim 100), several steps through a ring of 2, rank 0 sending to itself;
    with the row counts named by the host, and with counts that exist only in device memory (the receiver then learns
    them from the sender's word)."""
    from starrygl import _C, ops
    L = _C.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    ctx, base = make_ctx(L, _C, bulk_bytes=bulk_bytes, dim=dim)
    data, ts = torch.zeros(SLOTS, dim, device=dev), torch.zeros(SLOTS, device=dev)
    want_d, want_t = np.zeros((SLOTS, dim), np.float32), np.zeros(SLOTS, np.float32)
    status = ops.StatusWord(dev)
    sp = _C.stream_ptr()
    g = torch.Generator().manual_seed(bulk_bytes % 97 + dim)
    keep = []
    for step in range(7):
        n = int(torch.randint(0, 40, (1,), generator=g))
        feats = torch.randn(50, dim, generator=g).to(dev)
        fts = torch.rand(50, generator=g).to(dev)
        send_idx = torch.randint(0, 50, (n,), generator=g).to(dev)
        slots = torch.randperm(SLOTS, generator=g)[:n].to(dev)
        if counts_on == "host":
            rows = (C.c_int64 * 1)(n)
            _C.check(L.sgl_p2p_route_send(ctx, feats.data_ptr(), 50, dim, fts.data_ptr(), send_idx.data_ptr(), slots.data_ptr(),
                                          rows, step, status.ptr(), sp))
            _C.check(L.sgl_p2p_route_recv(ctx, rows, data.data_ptr(), SLOTS, dim, 1, ts.data_ptr(), step, status.ptr(), sp))
        else:
            # a device-built plan keeps its index arrays at capacity; only the count varies
            d_rows = torch.tensor([n], dtype=torch.int64, device=dev)
            idx_cap, slot_cap = torch.zeros(64, dtype=torch.int64, device=dev), torch.zeros(64, dtype=torch.int64, device=dev)
            idx_cap[:n], slot_cap[:n] = send_idx, slots
            keep.append((idx_cap, slot_cap))
            _C.check(L.sgl_p2p_route_send_dev(ctx, feats.data_ptr(), 50, dim, fts.data_ptr(), idx_cap.data_ptr(),
                                              slot_cap.data_ptr(), d_rows.data_ptr(), 64, step, status.ptr(), sp))
            _C.check(L.sgl_p2p_route_recv_dev(ctx, 64, data.data_ptr(), SLOTS, dim, 1, ts.data_ptr(), step, status.ptr(), sp))
            keep.append(d_rows)
        keep.append((feats, fts, send_idx, slots))
        want_d[slots.cpu().numpy()] = feats.cpu().numpy()[send_idx.cpu().numpy()]
        want_t[slots.cpu().numpy()] = fts.cpu().numpy()[send_idx.cpu().numpy()]
    torch.cuda.synchronize()
    status.check("world-1 route")
    assert np.array_equal(data.cpu().numpy(), want_d) and np.array_equal(ts.cpu().numpy(), want_t)
    _C.check(L.sgl_p2p_route_destroy(ctx))
    _C.check(L.sgl_p2p_free(base))


def test_world1_count_mismatch_and_overflow_are_reported():
    """A receiver that was told a different row count than the sender pushed, and a device-side count above the staging
    capacity, both end in a status bit -- not in a wait or a wrong write."""
    from starrygl import _C, ops
    L = _C.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    ctx, base = make_ctx(L, _C)
    data, ts = torch.zeros(SLOTS, DIM, device=dev), torch.zeros(SLOTS, device=dev)
    status = ops.StatusWord(dev)
    sp = _C.stream_ptr()
    feats, fts = torch.randn(50, DIM, device=dev), torch.rand(50, device=dev)
    send_idx = torch.arange(5, device=dev)
    slots = torch.arange(5, device=dev)
    _C.check(L.sgl_p2p_route_send(ctx, feats.data_ptr(), 50, DIM, fts.data_ptr(), send_idx.data_ptr(), slots.data_ptr(),
                                  (C.c_int64 * 1)(5), 0, status.ptr(), sp))
    _C.check(L.sgl_p2p_route_recv(ctx, (C.c_int64 * 1)(4), data.data_ptr(), SLOTS, DIM, 1, ts.data_ptr(), 0, status.ptr(), sp))
    torch.cuda.synchronize()
    with pytest.raises(_C.SglError, match="(?i)different number of rows"):
        status.check("mismatch")
    # capacity of the context is 64 rows per pair: a device count of 1000 is cut to 64 and flagged
    big_idx = torch.zeros(1000, dtype=torch.int64, device=dev)
    big_slots = torch.arange(1000, device=dev) % SLOTS
    d_rows = torch.tensor([1000], dtype=torch.int64, device=dev)
    _C.check(L.sgl_p2p_route_send_dev(ctx, feats.data_ptr(), 50, DIM, fts.data_ptr(), big_idx.data_ptr(), big_slots.data_ptr(),
                                      d_rows.data_ptr(), 1000, 1, status.ptr(), sp))
    _C.check(L.sgl_p2p_route_recv_dev(ctx, 64, data.data_ptr(), SLOTS, DIM, 1, ts.data_ptr(), 1, status.ptr(), sp))
    torch.cuda.synchronize()
    with pytest.raises(_C.SglError, match="(?i)capacity"):
        status.check("overflow")
    assert torch.equal(data[:64], feats[0].expand(64, DIM))
    _C.check(L.sgl_p2p_route_destroy(ctx))
    _C.check(L.sgl_p2p_free(base))


def test_send_without_credit_gives_up_and_publishes_nothing():
    """Ring flow control: a step may reuse a ring slot only after the receiver has acknowledged the step that used it last.
    With a ring of 2 and no apply in between, the third send finds no acknowledgement: its one-warp credit kernel gives up
    after the (shortened) bound, the status word carries the timeout, and the send kernel behind it stores nothing -- the
    two steps that were sent are applied intact afterwards."""
    from starrygl import _C, ops
    L = _C.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    ctx, base = make_ctx(L, _C, wait_ms=200)
    data, ts = torch.zeros(SLOTS, DIM, device=dev), torch.zeros(SLOTS, device=dev)
    status = ops.StatusWord(dev)
    sp = _C.stream_ptr()
    n_rows = (C.c_int64 * 1)(ROWS)
    g = torch.Generator().manual_seed(11)
    sent = []
    for step in range(3):
        feats = torch.randn(50, DIM, generator=g).to(dev)
        fts = torch.rand(50, generator=g).to(dev)
        send_idx = torch.randint(0, 50, (ROWS,), generator=g).to(dev)
        slots = (torch.randperm(30, generator=g)[:ROWS] + 30 * step).to(dev)        # disjoint slots per step
        sent.append((feats, fts, send_idx, slots))
        _C.check(L.sgl_p2p_route_send(ctx, feats.data_ptr(), 50, DIM, fts.data_ptr(), send_idx.data_ptr(), slots.data_ptr(), n_rows,
                                      step, status.ptr(), sp))
        torch.cuda.synchronize()
        if step < 2:
            status.check(f"send of step {step}")
    with pytest.raises(_C.SglError, match="(?i)timeout|wait"):
        status.check("third send without an acknowledgement")
    status2 = ops.StatusWord(dev)
    for step in range(2):
        _C.check(L.sgl_p2p_route_recv(ctx, n_rows, data.data_ptr(), SLOTS, DIM, 1, ts.data_ptr(), step, status2.ptr(), sp))
    torch.cuda.synchronize()
    status2.check("apply of the two steps that were sent")
    want_d, want_t = torch.zeros(SLOTS, DIM, device=dev), torch.zeros(SLOTS, device=dev)
    for feats, fts, send_idx, slots in sent[:2]:
        want_d[slots] = feats[send_idx]
        want_t[slots] = fts[send_idx]
    assert torch.equal(data, want_d) and torch.equal(ts, want_t)      # step 2's rows (slots 60..89) never arrived
    _C.check(L.sgl_p2p_route_destroy(ctx))
    _C.check(L.sgl_p2p_free(base))
