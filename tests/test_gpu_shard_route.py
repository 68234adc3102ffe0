"""One-GPU checks of the communicator surface, the sharded-table gather and the reverse-route accumulate:
``create_nccl_id`` / ``DistContext`` / ``init_p2p``, ``ShardTensor[...]`` against the oracle's restatement of the
reference's distributed gather, and the one-launch accumulate over all peers against the per-peer loop (bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O
from gpu_util import cu, npy

pytestmark = pytest.mark.gpu


def test_dist_context_world_of_one_and_init_p2p():
    from starrygl.lib import libstarrygl_comm as M
    dev = torch.cuda.current_device()
    cid = M.create_nccl_id()
    assert isinstance(cid, bytes) and len(cid) == 128
    ctx = M.DistContext(0, 1, torch.cuda.device_count(), cid)
    assert (ctx.rank(), ctx.size(), ctx.device()) == (0, 1, 0)
    assert M.init_p2p([dev]) == 1
    with pytest.raises(RuntimeError):
        M.DistContext(0, 1, 1, b"short")
    torch.cuda.set_device(dev)
    from starrygl.route.exchange import NativeComm
    NativeComm.shutdown()


@pytest.mark.parametrize("dim,dtype", [(128, torch.float32), (172, torch.float32), (186, torch.float32), (128, torch.bfloat16)])
def test_shard_tensor_gather_matches_the_oracle(dim, dtype):
    """Three shards of different sizes (all on this GPU -- the kernel only sees base addresses), packed ids in random
    order with repeats: rows come back in the order of the ids."""
    from starrygl.lib.libstarrygl_comm import ShardTensor
    rng = np.random.default_rng(dim)
    sizes = [700, 1, 1300]
    shards = [torch.randn(n, dim, generator=torch.Generator().manual_seed(n)).to(dtype).cuda() for n in sizes]
    st = ShardTensor(torch.cuda.current_device())
    for s in shards:
        st.append(s)
    assert st.shape() == [2001, dim] and st.device_count() == 3 and st.size(0) == 2001 and st.stride(0) == dim
    assert st.numel() == 2001 * dim
    part = rng.integers(0, 3, 5000)
    loc = np.array([rng.integers(0, sizes[p]) for p in part])
    ids = O.dist_pack(loc, part)
    got = st[cu(ids)]
    st.check()
    want = O.shard_gather([npy(s.view(torch.int16) if dtype == torch.bfloat16 else s) for s in shards], ids)
    assert np.array_equal(npy(got.view(torch.int16) if dtype == torch.bfloat16 else got), want)
    # an id past the end of its shard is reported, not read
    from starrygl import _C
    st[cu(O.dist_pack(np.array([1]), np.array([1])))]
    with pytest.raises(_C.SglError, match="row index"):
        st.check()
    assert st[cu(np.zeros(0, np.int64))].shape == (0, dim)


@pytest.mark.parametrize("dim", [1, 7, 100, 128])
def test_reverse_route_accumulate_equals_the_per_peer_loop(dim):
    """Rows of x hit by several peers: the grouped kernel adds them in peer order, as the loop over peers does."""
    from starrygl import ops
    g = torch.Generator().manual_seed(dim)
    n_rows, sizes = 300, [120, 0, 250, 77]
    idx = torch.cat([torch.randperm(n_rows, generator=g)[:s] for s in sizes]).cuda()   # unique inside a peer segment
    outs = torch.randn(sum(sizes), dim, generator=g).cuda()
    x = torch.randn(n_rows, dim, generator=g).cuda()
    ref = x.clone()
    s = 0
    for sz in sizes:                      # the reference's loop: x[idx[s:s+sz]] += outs[s:s+sz]
        ref[idx[s:s + sz]] += outs[s:s + sz]
        s += sz
    got = x.clone()
    st = ops.StatusWord(x.device)
    ops.route_add_grouped(got, ops.route_groups(idx), outs, status=st)
    st.check("grouped add")
    assert torch.equal(got, ref)
    # and the per-segment kernel agrees too
    got2 = x.clone()
    s = 0
    for sz in sizes:
        ops.route_add_rows(got2, idx[s:s + sz], outs[s:s + sz])
        s += sz
    assert torch.equal(got2, ref)
