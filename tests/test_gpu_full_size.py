"""Largest configuration of the baseline (16.8 M nodes, 190 M events, 186 x fp32 edge rows, uniform [10, 10] over
32 x 4,000 events) at FULL size, checked through size-independent properties computed on the GPU with torch (the CPU
oracle would take minutes here): T-CSR invariants, sampling counts / time bounds / membership, and the 744-byte row
gather (the row width that is not a multiple of 16 bytes).  Inputs are seeded synthetic stand-ins of that shape."""
import pytest
import torch

pytestmark = pytest.mark.gpu
N, M, K, ROOTS = 16_800_000, 190_000_000, 10, 128_000


def test_full_size_tcsr_sampling_and_gather():
    from starrygl import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    free, _ = torch.cuda.mem_get_info(dev)
    if free < 60 * 2 ** 30:
        pytest.skip("needs 60 GB of free device memory")
    gen = torch.Generator(device=dev).manual_seed(5)
    # bursty timestamps: events cluster around 2,000 burst centres in [0, 2.5e6)
    centres = torch.randint(0, 2_500_000, (2000,), device=dev, generator=gen)
    ts = (centres[torch.randint(0, 2000, (M,), device=dev, generator=gen)]
          + torch.randint(0, 4000, (M,), device=dev, generator=gen)).clamp_(0, 2_499_999)
    src = (torch.rand(M, device=dev, generator=gen).pow_(3.0) * N).long().clamp_(0, N - 1)     # skewed degrees
    dst = torch.randint(0, N, (M,), device=dev, generator=gen)

    g = ops.tcsr_build(src, dst, ts, None, N, want_perm=True)
    torch.cuda.synchronize()
    indptr, perm = g.indptr, g.perm
    # ---- T-CSR invariants ----
    assert int(indptr[0]) == 0 and int(indptr[-1]) == M and bool((indptr[1:] >= indptr[:-1]).all())
    assert bool(torch.equal(indptr[1:] - indptr[:-1], torch.bincount(src, minlength=N)))
    row_of = torch.repeat_interleave(torch.arange(N, device=dev), indptr[1:] - indptr[:-1])
    assert bool(torch.equal(src[perm], row_of))                                   # every edge sits in its source's row
    assert bool(torch.equal(g.nbr, dst[perm])) and bool(torch.equal(g.ts, ts[perm])) and bool(torch.equal(g.eid, perm))
    inner = row_of[1:] == row_of[:-1]
    assert bool((g.ts[1:][inner] >= g.ts[:-1][inner]).all())                      # ascending time inside a row
    tie = inner & (g.ts[1:] == g.ts[:-1])
    assert bool((perm[1:][tie] > perm[:-1][tie]).all())                           # ties keep input order (stable)
    assert int(perm.sum()) == M * (M - 1) // 2                                    # a permutation of the input
    del row_of, inner, tie

    # ---- one mega-batch of roots, uniform-10 and recent-10 ----
    pick = torch.randint(0, M, (ROOTS,), device=dev, generator=gen)
    q, qt = src[pick].contiguous(), ts[pick].contiguous()
    lo, hi = indptr[q], indptr[q + 1]
    # candidates of root i = edges of its row with ts < qt[i]: count them with a segmented search
    pos = torch.searchsorted(g.ts + (torch.repeat_interleave(torch.arange(N, device=dev), indptr[1:] - indptr[:-1]) << 22),
                             qt + (q << 22))
    cand = pos - lo
    assert bool((cand >= 0).all()) and bool((pos <= hi).all())
    for policy in ("recent", "uniform"):
        st = ops.StatusWord(dev)
        h = ops.sample_layer(g, q, qt, K, policy, seed=11, status=st)
        tot = h.total()
        st.check(policy)
        cnt = h.offsets[1:ROOTS + 1] - h.offsets[:ROOTS]
        assert bool(torch.equal(cnt, cand.clamp(max=K)))
        o_dst, o_eid, o_ts, o_nbr = h.dst[:tot], h.eid[:tot], h.ts[:tot], h.nbr[:tot]
        assert bool(torch.equal(src[o_eid], q[o_dst])) and bool(torch.equal(dst[o_eid], o_nbr)) and bool(torch.equal(ts[o_eid], o_ts))
        assert bool((o_ts < qt[o_dst]).all())
        if policy == "recent":   # the k latest candidates: positions pos - cnt .. pos of the row
            first = torch.repeat_interleave(pos - cnt, cnt)
            rank = torch.arange(tot, device=dev) - torch.repeat_interleave(h.offsets[:ROOTS], cnt)
            assert bool(torch.equal(o_eid, g.eid[first + rank]))
        else:                    # k distinct candidates in ascending position
            same = o_dst[1:] == o_dst[:-1]
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(M, device=dev)
            p = inv[o_eid]                                       # position of every sample in the T-CSR
            assert bool((p[1:][same] > p[:-1][same]).all())
            del inv, p
    del pos, cand

    # ---- 186 x fp32 rows (744 bytes: 4-byte lanes), table sample of 4 M rows ----
    table = torch.randn(4_000_000, 186, device=dev, generator=gen)
    idx = (h.eid[:tot] % 4_000_000).contiguous()
    out = ops.gather_rows(table, idx)
    assert bool(torch.equal(out, table[idx]))
