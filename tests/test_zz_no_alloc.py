"""The sampling entry point that needs no scratch from the caller (``sgl_sample_layer_static``).

It exists for hosts that cannot allocate device memory when a batch arrives -- a sampler thread beside a running
training loop (a cudaMalloc would stall all of the GPU's streams), or a process whose HBM is owned by another
framework's pool.  This test calls it through the C ABI, twice in a row (the second call finds the built-in scratch
full of the first call's data), and requires the outputs to be identical to those of ``sgl_sample_layer`` with a
caller-provided workspace.  It also checks the size limit.  Collected last on purpose: a run that stops at the first
failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _graph(seed, n=3000, m=200000):
    from starrygl import ops
    rng = np.random.default_rng(seed)
    w = 1.0 / np.arange(1, n + 1) ** 1.2
    key = torch.from_numpy(rng.choice(n, m, p=w / w.sum()).astype(np.int64)).cuda()
    nbr = torch.from_numpy(rng.integers(0, n, m).astype(np.int64)).cuda()
    ts = torch.from_numpy(rng.integers(0, 100000, m).astype(np.int64)).cuda()
    return ops.tcsr_build(key, nbr, ts, None, n), rng


def _call_static(L, g, q, qt, k, policy, seed):
    n = q.numel()
    cap = max(n * k, 1)
    dev = q.device
    o_nbr, o_dst, o_ts, o_eid = (torch.full((cap,), -7, dtype=torch.int64, device=dev) for _ in range(4))
    o_dt = torch.full((cap,), -7.0, dtype=torch.float32, device=dev)
    offs = torch.full((n + 1,), -7, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = L.sgl_sample_layer_static(g.indptr.data_ptr(), g.nbr.data_ptr(), g.ts.data_ptr(), g.eid.data_ptr(), g.num_nodes,
                                   q.data_ptr(), qt.data_ptr(), n, k, policy, 0, -1, 0, seed, 0, o_nbr.data_ptr(),
                                   o_dst.data_ptr(), o_ts.data_ptr(), o_dt.data_ptr(), o_eid.data_ptr(), offs.data_ptr(),
                                   status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, (o_nbr, o_dst, o_ts, o_dt, o_eid, offs), status


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from starrygl import _C, ops
    L = _C.lib()
    g, rng = _graph(0)
    for call, (nq, k, policy) in enumerate([(5000, 20, "recent"), (777, 10, "uniform")]):   # two calls in a row
        q = torch.from_numpy(rng.integers(0, g.num_nodes, nq).astype(np.int64)).cuda()
        qt = torch.from_numpy(rng.integers(0, 100001, nq).astype(np.int64)).cuda()
        rc, out, status = _call_static(L, g, q, qt, k, _C.POLICY[policy], seed=11)
        assert rc == 0, L.sgl_last_error()
        ref = ops.sample_layer(g, q, qt, k, policy, seed=11)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        tot = int(ref.offsets[-1].item())
        assert tot > 0 and torch.equal(out[5], ref.offsets), f"call {call}: offsets differ"
        for name, a, b in zip(("nbr", "dst", "ts", "dt", "eid"), out[:5], (ref.nbr, ref.dst, ref.ts, ref.dt, ref.eid)):
            assert torch.equal(a[:tot], b[:tot]), f"call {call}: {name} differs"   # bit-exact, as in the other tests
        # and against the CPU oracle directly
        from oracle import oracle_np as O
        cpu = lambda t: t.cpu().numpy()
        want = O.sample_layer(cpu(g.indptr), cpu(g.nbr), cpu(g.ts), cpu(g.eid), cpu(q), cpu(qt), k,
                              O.RECENT if policy == "recent" else O.UNIFORM, seed=11)
        for name, a, w in zip(("nbr", "dst", "ts", "dt", "eid"), out[:5], want[:5]):
            assert np.array_equal(cpu(a[:tot]), w), f"call {call}: {name} differs from the oracle"


def test_static_scratch_entry_point_rejects_oversized_batches():
    from starrygl import _C
    L = _C.lib()
    g, _ = _graph(1, n=100, m=1000)
    n = 65536 + 1
    q = torch.zeros(n, dtype=torch.int64, device="cuda")
    rc, _, _ = _call_static(L, g, q, q, 1, 0, seed=0)
    assert rc == -1
    msg = L.sgl_last_error().decode()
    assert "65536" in msg and "exceed" in msg
    # an empty batch is fine and writes the single offset
    e = torch.zeros(0, dtype=torch.int64, device="cuda")
    rc, out, _ = _call_static(L, g, e, e, 3, 0, seed=0)
    torch.cuda.synchronize()
    assert rc == 0 and out[5].tolist() == [0]
