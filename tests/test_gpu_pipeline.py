"""The pre-bound sample -> gather step (``SampleGatherPipeline``): every way of driving it -- device tensors, raw
pointers, torch CUDA graphs, the library's own graph helpers, pinned host buffers with the device-counted result copy
-- must give the oracle's block structure and feature rows, bit for bit."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, npy, build_graph
from test_gpu_sampler import random_graph

pytestmark = pytest.mark.gpu
K, B, DIM = 7, 512, 44            # 176-byte rows


@pytest.fixture(scope="module")
def world():
    z = random_graph(5, 3000, 200000, 100000, hub=20000)
    g = build_graph(z)
    csr = O.tcsr_build(z["dst"], z["src"], z["ts"], z["eid"], z["n"])[:4]
    rng = np.random.default_rng(2)
    feats = rng.standard_normal((200000, DIM)).astype(np.float32)
    batches = []
    for b in range(5):
        q = rng.integers(0, z["n"], B).astype(np.int64)
        q[:20] = 0
        qt = rng.integers(0, 100000, B).astype(np.int64)
        batches.append((q, qt, O.sample_layer(*csr, q, qt, K, O.RECENT)))
    return g, cu(feats), feats, batches


def check_device(pipe, feats_np, ref, n=B):
    src, dst, ts, dt, eid, counts = ref[:6]
    tot = len(src)
    offs = npy(pipe.offsets[:n + 1])
    assert offs[0] == 0 and np.array_equal(np.diff(offs), counts) and offs[-1] == tot
    assert np.array_equal(npy(pipe.nbr[:tot]), src) and np.array_equal(npy(pipe.ts[:tot]), ts)
    assert np.array_equal(npy(pipe.eid[:tot]), eid) and np.array_equal(npy(pipe.dt[:tot]), dt)
    assert np.array_equal(npy(pipe.dst[:tot]), dst)
    assert np.array_equal(npy(pipe.out_feats[:tot]), feats_np[eid])


def check_host(res, ref, n=B):
    tot, views = res
    src, dst, ts, dt, eid, counts = ref[:6]
    assert tot == len(src)
    assert np.array_equal(np.diff(views["offsets"].numpy()), counts) and len(views["offsets"]) == n + 1
    for k, r in (("nbr", src), ("ts", ts), ("eid", eid), ("dt", dt)):
        assert np.array_equal(views[k].numpy(), r), k


def make(world, **kw):
    from starrygl.graph.pipeline import SampleGatherPipeline
    g, feats, _, _ = world
    return SampleGatherPipeline(g, feats, K, "recent", B, stream=torch.cuda.Stream(), **kw)


def test_device_paths(world):
    _, _, feats_np, batches = world
    pipe = make(world)
    for q, qt, ref in batches[:2]:
        pipe.run_device(cu(q), cu(qt))
        pipe.stream.synchronize()
        check_device(pipe, feats_np, ref)
    q, qt, ref = batches[2]
    dq, dqt = cu(q), cu(qt)
    pipe.run_device_ptr(dq.data_ptr(), dqt.data_ptr(), B)
    pipe.stream.synchronize()
    check_device(pipe, feats_np, ref)
    # a short batch through the same object
    pipe.run_device(dq[:100], dqt[:100])
    pipe.stream.synchronize()
    assert int(pipe.offsets[100].item()) == int(np.sum(ref[5][:100]))
    pipe.status.check("pipeline")


def test_graph_replays(world):
    _, _, feats_np, batches = world
    pipe = make(world).capture().capture_native()
    for i, (q, qt, ref) in enumerate(batches):
        both = torch.stack([cu(q), cu(qt)]).contiguous()
        if i % 2:
            pipe.replay_device(both[0], both[1])
        else:
            pipe.replay_ptr(both.data_ptr())
        pipe.stream.synchronize()
        check_device(pipe, feats_np, ref)
    pipe.status.check("pipeline")


@pytest.mark.parametrize("export", ["prefix", "full"])
def test_host_paths(world, export):
    _, _, feats_np, batches = world
    pipe = make(world, export=export)
    pin = lambda a: torch.from_numpy(a).pin_memory()
    q, qt, ref = batches[0]
    check_host(pipe.run_host(pin(q), pin(qt)), ref)                    # call by call
    check_device(pipe, feats_np, ref)
    check_host(pipe.run_host(pin(q[:33]), pin(qt[:33])), [r[:int(np.sum(ref[5][:33]))] for r in ref[:5]] + [ref[5][:33]], 33)
    pipe.capture()
    for q, qt, ref in batches[1:3]:                                    # torch graph with the copies inside
        check_host(pipe.run_host(pin(q), pin(qt)), ref)
    if export == "prefix":
        pipe.capture_native_host()
        for q, qt, ref in batches[3:]:                                 # library graph: one foreign call per batch
            both = torch.from_numpy(np.stack([q, qt])).pin_memory()
            pipe.submit_host_ptr(both.data_ptr())
            check_host(pipe.result(), ref)
            check_device(pipe, feats_np, ref)
    pipe.status.check("pipeline")


def test_copy_prefix_edges():
    """Device-counted copy: counts 0, odd byte tails, clamping to the capacity, whole-array entries."""
    import ctypes as C
    from starrygl import _C
    L = _C.lib()
    a = torch.arange(1000, dtype=torch.int64, device="cuda")
    b = torch.arange(1000, dtype=torch.float32, device="cuda")
    c = torch.arange(64, dtype=torch.uint8, device="cuda")
    for cnt in (0, 1, 3, 999, 1000, 5000):
        oa, ob = torch.full((1000,), -1, dtype=torch.int64).pin_memory(), torch.full((1000,), -1.0).pin_memory()
        oc = torch.zeros(64, dtype=torch.uint8).pin_memory()
        d = torch.tensor([cnt], device="cuda")
        v = C.c_void_p
        src, dst = (v * 3)(a.data_ptr(), b.data_ptr(), c.data_ptr()), (v * 3)(oa.data_ptr(), ob.data_ptr(), oc.data_ptr())
        _C.check(L.sgl_copy_prefix(3, src, dst, (C.c_int64 * 3)(8, 4, -37), d.data_ptr(), 1000, _C.stream_ptr()))
        torch.cuda.synchronize()
        m = min(cnt, 1000)
        assert torch.equal(oa[:m], a[:m].cpu()) and (oa[m:] == -1).all()
        assert torch.equal(ob[:m], b[:m].cpu()) and (ob[m:] == -1).all()
        assert torch.equal(oc[:37], c[:37].cpu()) and (oc[37:] == 0).all()


def test_prefetcher_yields_every_batch_in_order(world):
    """Batches from a loader (device tensors and pinned host tensors mixed) through 3 pipeline slots; a consumer kernel
    per batch copies what it reads, the copies are checked after the loop (so a slot overwritten too early would show)."""
    from starrygl.data.prefetcher import HostToDevicePrefetcher
    g, feats, feats_np, batches = world

    def loader():
        for i in range(12):
            q, qt, _ = batches[i % len(batches)]
            if i % 2:
                yield torch.from_numpy(q).pin_memory(), torch.from_numpy(qt).pin_memory()
            else:
                yield cu(q), cu(qt)
    pf = HostToDevicePrefetcher(loader(), g, feats, K, "recent", B, depth=3)
    kept = []
    for b in pf:
        kept.append((b.offsets.clone(), b.nbr.clone(), b.eid.clone(), b.dt.clone(), b.edge_feats.clone()))
    torch.cuda.synchronize()
    pf.check()
    assert len(kept) == 12
    for i, (offs, nbr, eid, dt, ef) in enumerate(kept):
        src, dst, ts, rdt, reid, counts = batches[i % len(batches)][2][:6]
        tot = len(src)
        assert np.array_equal(np.diff(npy(offs)), counts)
        assert np.array_equal(npy(nbr[:tot]), src) and np.array_equal(npy(eid[:tot]), reid) and np.array_equal(npy(dt[:tot]), rdt)
        assert np.array_equal(npy(ef[:tot]), feats_np[reid])
