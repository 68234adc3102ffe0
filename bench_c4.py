"""Multi-GPU arm of bench.py: the partitioned TGN data path (BASELINE configs[3]) on N ranks of one box.

Synthetic stand-in for the distributed configuration: a planted-community temporal graph with ONE community per rank
(312,500 nodes and 12.5 M events per rank -- 2.5 M nodes / 100 M events at 8 ranks; weak scaling), 80 % of an event's
sources inside the destination's community, the rest uniform over the other communities; partition = community; an
event belongs to the partition of its destination.  Every rank stores its owned nodes followed by the halo (remote
sources it has seen) and samples from its own events only (both directions of an event are rows of its T-CSR).

One step per rank = one batch of 4,000 events = 12,000 root queries (source, destination, negative destination):

  A1  (id, ts) relabel of the roots -> the layer-0 list              sgl_unique_pairs
  A2  most-recent-10 sampling of the 12,000 roots                      sgl_sample_layer
  A3  gather of node memory (100 x fp32 + ts) for roots and sampled neighbours, of the roots' mails (372 x fp32 + ts)
      through the global -> local slot map                             sgl_gather_rows
  A4  stand-in for the model: new memory / mail rows for the layer-0 list, a pure function of (node id, step)
  A5  local write of those rows                                        sgl_scatter_rows
  A6  route plan of the step, built on the device from the layer-0 list, the partition book and the replica table
                                                                       sgl_plan_route
  R   owners push the fresh memory rows and mails to every rank that holds a replica, over NVLink peer memory, with the
      plan's sizes read from device memory (no host synchronisation, no count exchange); the receivers apply them
                                                                       sgl_p2p_route_send_dev / sgl_p2p_route_recv_dev

A1, A2 and A6 touch no table and run ahead on their own streams (NBUF sets of buffers take turns).  A3, A4, the applies of
R and A5 form one chain in step order; the pushes of R leave as soon as A4 is done.  A step's received rows are written when
the next step updates the tables, after that step's reads -- the reference's order (starrygl/cache/NodeState.py:269-274) --
so A3 of step s+1 reads what A5 of step s and R of step s-1 wrote.  After the timed loop every rank recomputes, from the seeds alone, which step wrote every one of its rows last (its own batches and every
peer's) and compares its whole memory and mail tables with that expectation bit for bit.
"""
import statistics
import time

import torch
import torch.distributed as dist

N_PER = 312_500           # nodes per partition
E_PER = 12_500_000        # events per partition
T_MAX = 10_000_000
P_INTRA = 0.8
EVENTS = 4000             # events per rank and step
FANOUT = 10
MEM_DIM = 100
MAIL_DIM = 2 * MEM_DIM + 172
NUM_BATCHES = 64
NBUF = 4                  # steps in preparation at a time (sets of step buffers; measured at N = 2: 2 -> 0.212, 3 -> 0.181,
                          # 4 -> 0.168, 6 -> 0.168, 8 -> 0.186 ms per step)


def make_partition(rank, world, dev, n_per=N_PER, e_per=E_PER):
    """Events of partition ``rank`` (seeded by the rank alone, so that any rank can regenerate any partition)."""
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    base = rank * n_per
    dst = base + torch.randint(0, n_per, (e_per,), device=dev, generator=gen)
    src = base + torch.randint(0, n_per, (e_per,), device=dev, generator=gen)
    cross = torch.rand(e_per, device=dev, generator=gen) >= P_INTRA
    far = torch.randint(0, max(world - 1, 1) * n_per, (e_per,), device=dev, generator=gen)
    far = far + (far >= base) * n_per                      # skip the own id range
    if world > 1:
        src = torch.where(cross, far, src)
    ts = torch.sort(torch.randint(0, T_MAX, (e_per,), device=dev, generator=gen)).values
    neg = base + torch.randint(0, n_per, (NUM_BATCHES, EVENTS), device=dev, generator=gen)
    return src, dst, ts, neg


def batches_of(src, dst, ts, neg):
    """[NUM_BATCHES, 12000] roots and query times (views of one [NUM_BATCHES, 2, 12000] block, so that a batch is one
    contiguous copy): the last NUM_BATCHES * EVENTS events in time order."""
    e = src.numel()
    lo = e - NUM_BATCHES * EVENTS
    s, d, t = (x[lo:].view(NUM_BATCHES, EVENTS) for x in (src, dst, ts))
    both = torch.stack([torch.cat([s, d, neg], 1), torch.cat([t, t, t], 1)], 1).contiguous()
    return both[:, 0], both[:, 1]


def model_base(ids, step_t):
    """((131 v + 7 s) mod 65536) as fp32: what the stand-in model's rows of node v at step s start with."""
    return (torch.add(ids * 131, step_t, alpha=7) % 65536).to(torch.float32)


def model_rows(ids, step_t, dim, base=None, cols=None):
    """Stand-in for the model's output for the layer list: row of node v at step s = ((131 v + 7 s) mod 65536) + j, j the
    column -- small integers, exact in fp32, and a function of (v, s) only, so that the state every rank must hold can
    be recomputed from the seeds."""
    if base is None:
        base = model_base(ids, step_t)
    if cols is None:
        cols = torch.arange(dim, device=ids.device, dtype=torch.float32)
    return base.unsqueeze(1) + cols


class Partition:
    """Everything rank ``rank`` holds: T-CSR of its events, node memory and mail tables (owned rows, then halo rows), the
    global -> local slot map, the partition book and the replica table of the nodes it owns."""

    def __init__(self, rank, world, dev, n_per=N_PER, e_per=E_PER):
        from starrygl import ops
        from starrygl.cache.NodeState import DistNodeState
        from starrygl.cache.replica_table import CSRReplicaTable
        from starrygl.utils.partition_book import PartitionState
        self.rank, self.world, self.dev, self.n_per = rank, world, dev, n_per
        n_glob = world * n_per
        src, dst, ts, neg = make_partition(rank, world, dev, n_per, e_per)
        self.roots, self.root_ts = batches_of(src, dst, ts, neg)
        eid = torch.arange(e_per, device=dev)
        self.g = ops.tcsr_build(torch.cat([dst, src]), torch.cat([src, dst]), torch.cat([ts, ts]), torch.cat([eid, eid]), n_glob)
        base = rank * n_per
        remote = src[(src < base) | (src >= base + n_per)]
        halo = torch.unique(remote) if remote.numel() else remote
        del src, dst, ts, eid, remote
        self.loc_ids = torch.cat([torch.arange(base, base + n_per, device=dev), halo])
        ps = PartitionState(loc_ids=self.loc_ids, num_master_nums=n_per, node_mode='map', num_nodes=n_glob)
        self.mem = DistNodeState(ps, MEM_DIM, device=dev)
        self.mail = DistNodeState(ps, MAIL_DIM, device=dev)
        self.g2l = ps.node_mapper.g2l_map(dev)
        self.node_parts = torch.arange(n_glob, device=dev) // n_per
        # replica table of the nodes owned here: which other ranks hold them as halo, and in which slot
        n_halo = torch.tensor([halo.numel()], device=dev)
        if world > 1:
            counts = [torch.zeros_like(n_halo) for _ in range(world)]
            dist.all_gather(counts, n_halo)
            counts = [int(c.item()) for c in counts]
            pad = torch.zeros(max(max(counts), 1), dtype=torch.int64, device=dev)
            pad[:halo.numel()] = halo
            box = [torch.empty_like(pad) for _ in range(world)]
            dist.all_gather(box, pad)
        else:
            counts, box = [0], [halo]
        self.halo_counts = counts
        node, rk, lc = [], [], []
        for q in range(world):
            if q == rank:
                continue
            h = box[q][:counts[q]]
            mine = (h >= base) & (h < base + n_per)
            node.append(h[mine])
            rk.append(torch.full((int(mine.sum()),), q, dtype=torch.int64, device=dev))
            lc.append(torch.nonzero(mine).reshape(-1) + n_per)          # slot on q: after q's owned rows, halo order
        node = torch.cat(node) if node else torch.zeros(0, dtype=torch.int64, device=dev)
        rk = torch.cat(rk) if rk else node.clone()
        lc = torch.cat(lc) if lc else node.clone()
        order = torch.argsort(node * world + rk)
        indptr = torch.zeros(n_glob + 1, dtype=torch.int64, device=dev)
        indptr[1:] = torch.cumsum(torch.bincount(node, minlength=n_glob), 0)
        pad1 = torch.zeros(1, dtype=torch.int64, device=dev)      # keeps the arrays non-empty on a single partition
        self.rep = CSRReplicaTable(indptr, torch.cat([rk[order], pad1]), torch.cat([lc[order], pad1]))
        self.max_rep = int((indptr[1:] - indptr[:-1]).max().item()) if node.numel() else 0


class Step:
    """The device work of one step, captured once as three CUDA graphs over static buffers: what touches no node table
    and can be prefetched (A1, A2, A6), the table reads with the model stand-in behind them (A3, A4), and the local writes
    (A5).  Several such objects take turns (``shared`` = the first one: step counter, row counter and status word are
    common): while the tables serve step s, the next objects already prepare the steps after it in their own buffers."""

    def __init__(self, part: Partition, use_graphs=True, shared: "Step" = None):
        from starrygl import _C, ops
        self.p, self.ops = part, ops
        dev = part.dev
        self.n_roots = 3 * EVENTS
        self.in_rt = torch.zeros(2, self.n_roots, dtype=torch.int64, device=dev)      # roots and query times of the batch
        self.in_roots, self.in_ts = self.in_rt[0], self.in_rt[1]
        self.batches = part.roots._base                                              # [NUM_BATCHES, 2, n_roots]
        self.in_rt.copy_(self.batches[0])
        if shared is None:
            self.step_t = torch.zeros(1, dtype=torch.int64, device=dev)      # number of the step being built
            self.rows_sent = torch.zeros(1, dtype=torch.int64, device=dev)   # rows this rank pushed so far (one table)
            self.status = ops.StatusWord(dev)
        else:
            self.step_t, self.rows_sent, self.status = shared.step_t, shared.rows_sent, shared.status
        self.id_bits = ops.bits_for(part.g.num_nodes - 1)
        self.ts_bits = ops.bits_for(T_MAX)
        self.plan_cap = self.n_roots * max(part.world - 1, 1)
        self.stream = torch.cuda.Stream(dev)
        self.side = [torch.cuda.Stream(dev) for _ in range(3)]           # branches inside the captured graphs
        self.c131 = torch.tensor([131], dtype=torch.int64, device=dev)
        self.cols_mem = torch.arange(MEM_DIM, device=dev, dtype=torch.float32)
        self.cols_mail = torch.arange(MAIL_DIM, device=dev, dtype=torch.float32)
        self.use_graphs = use_graphs
        self.kernel_launches = None
        self.h_out = None               # pinned host mirrors of a batch's block structure (host-buffer form of the step)
        if not use_graphs:
            return
        saved = _C.WORKSPACE
        _C.WORKSPACE = self._ws = _C.Workspace()
        try:
            with torch.cuda.stream(self.stream):
                self._prepare()
                self._read()
                self._model()
                self._write()
            self.stream.synchronize()
            self.step_t.zero_()
            self.rows_sent.zero_()
            part.mem.reset(), part.mail.reset()
            self.g1, self.g2, self.g2m, self.g3 = (torch.cuda.CUDAGraph() for _ in range(4))
            with torch.cuda.graph(self.g1, stream=self.stream):
                self._prepare()
            with torch.cuda.graph(self.g2, stream=self.stream):
                self._read()
            with torch.cuda.graph(self.g2m, stream=self.stream):
                self._model()
            with torch.cuda.graph(self.g3, stream=self.stream):
                self._write()
        finally:
            _C.WORKSPACE = saved
        self.stream.synchronize()
        # kernels of this library per step: relabel of the roots (pack, sort, head scan, emit), the hop (2), three gathers,
        # two scatters, the plan (count, expand, sort, emit); the stand-in model's element-wise kernels are torch's
        L = _C.lib()
        self.kernel_launches = (3 + L.sgl_radix_sort_launches(self.n_roots, self.id_bits + self.ts_bits) + 2 + 3 + 2 +
                                3 + L.sgl_radix_sort_launches(self.plan_cap, ops.bits_for(part.world - 1)))
        self.step_t.zero_()
        self.rows_sent.zero_()
        part.mem.reset(), part.mail.reset()

    def _prepare(self):
        """What a prefetcher can do ahead of the model, because it touches no node table: A1 relabel of the roots, then A6,
        the route plan from the layer-0 list; next to them A2, the hop."""
        ops, p = self.ops, self.p
        st = self.status
        cur, s1 = torch.cuda.current_stream(), self.side[0]
        s1.wait_stream(cur)
        with torch.cuda.stream(s1):
            self.hop = ops.sample_layer(p.g, self.in_roots, self.in_ts, FANOUT, "recent", status=st)
        self.u_id, self.u_ts, self.inv, _, self.d_n0 = ops.unique_pairs(self.in_roots, self.in_ts, id_bits=self.id_bits,
                                                                        ts_bits=self.ts_bits, ts_base=0, status=st)
        (self.pl_ranks, self.pl_rows, self.pl_locs, self.pl_sizes, self.pl_total) = ops.plan_route(
            self.u_id, p.node_parts, p.rank, p.rep.indptr, p.rep.indices, p.rep.locs, p.world, self.plan_cap, d_n=self.d_n0,
            status=st)
        cur.wait_stream(s1)

    def _read(self):
        """A3, the three gathers side by side."""
        ops, p = self.ops, self.p
        st = self.status
        cur, s1, s2 = torch.cuda.current_stream(), self.side[1], self.side[2]
        s1.wait_stream(cur)
        s2.wait_stream(cur)
        with torch.cuda.stream(s1):
            self.m_nbrs, self.m_nbrs_ts = ops.gather_rows(p.mem.data, self.hop.nbr, map=p.g2l, d_n=self.hop.d_total,
                                                          ts_table=p.mem.ts, status=st)
        with torch.cuda.stream(s2):
            self.mails, self.mails_ts = ops.gather_rows(p.mail.data, self.in_roots, map=p.g2l, ts_table=p.mail.ts, status=st)
        self.m_roots, self.m_roots_ts = ops.gather_rows(p.mem.data, self.in_roots, map=p.g2l, ts_table=p.mem.ts, status=st)
        cur.wait_stream(s1)
        cur.wait_stream(s2)

    def _model(self):
        """A4: the stand-in model's rows (a real model computes them from what A3 gathered, so the caller places this behind
        A3), and the step counters.  It touches no table, so it can run next to the applies of the step before."""
        cur, s1, s2 = torch.cuda.current_stream(), self.side[1], self.side[2]
        # (the stand-in costs kernel launches, not bandwidth: keep its chain short -- the counters go on a side branch)
        s2.wait_stream(cur)
        with torch.cuda.stream(s2):
            self.new_ts = self.step_t.to(torch.float32).expand(self.u_id.numel()).contiguous()
            self.rows_sent += self.pl_total
        step7 = self.step_t * 7
        base = torch.remainder(torch.addcmul(step7, self.u_id, self.c131), 65536, out=torch.empty_like(self.u_id, dtype=torch.float32))
        s1.wait_stream(cur)
        with torch.cuda.stream(s1):
            self.new_mail = model_rows(None, None, MAIL_DIM, base, self.cols_mail)
        self.new_mem = model_rows(None, None, MEM_DIM, base, self.cols_mem)
        cur.wait_stream(s2)
        self.step_t += 1
        cur.wait_stream(s1)

    def _write(self):
        """A5: the two local writes side by side (they replace rows A3 read)."""
        ops, p = self.ops, self.p
        st = self.status
        cur, s1 = torch.cuda.current_stream(), self.side[1]
        s1.wait_stream(cur)
        with torch.cuda.stream(s1):
            ops.scatter_rows(p.mail.data, self.u_id, self.new_mail, map=p.g2l, d_n=self.d_n0, ts_table=p.mail.ts, ts=self.new_ts,
                             status=st)
        ops.scatter_rows(p.mem.data, self.u_id, self.new_mem, map=p.g2l, d_n=self.d_n0, ts_table=p.mem.ts, ts=self.new_ts, status=st)
        cur.wait_stream(s1)

    # The methods below enqueue on the CURRENT stream, which the caller sets to ``self.stream`` once for a whole loop
    # (a stream context manager per call costs more host time than the calls themselves).
    def sample(self, b):
        self.in_rt.copy_(self.batches[b], non_blocking=True)
        self.g1.replay() if self.use_graphs else self._prepare()

    def sample_from_host(self, h_batch):
        """A1-A2 for a batch whose roots and query times ([2, n_roots]) are in PINNED host memory (the copy is asynchronous:
        the caller keeps the tensor untouched until the step has run)."""
        self.in_rt.copy_(h_batch, non_blocking=True)
        self.g1.replay() if self.use_graphs else self._prepare()

    def export_to_host(self):
        """Block structure of the batch (offsets, neighbour ids, timestamps, edge ids, dt) -> pinned host memory; the
        gathered rows stay on the GPU for the model."""
        hop = self.hop
        if self.h_out is None:
            self.h_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (hop.offsets, hop.nbr, hop.ts, hop.eid, hop.dt)]
        for h, t in zip(self.h_out, (hop.offsets, hop.nbr, hop.ts, hop.eid, hop.dt)):
            h.copy_(t, non_blocking=True)
        return sum(h.numel() * h.element_size() for h in self.h_out)

    def read_tables(self):
        self.g2.replay() if self.use_graphs else self._read()

    def model(self):
        self.g2m.replay() if self.use_graphs else self._model()

    def write_tables(self):
        self.g3.replay() if self.use_graphs else self._write()


def _expected_last_step(rank, world, dev, n_steps_total, routed_from, my_part):
    """For every global node id: the last step whose write reached rank ``rank``'s copy (-1 = never written).
    Local writes: every node of the rank's own layer-0 list, at every step.  Pushes: nodes OWNED by the peer that appear in
    the peer's layer-0 list, from step ``routed_from`` on, if this rank holds a replica."""
    n_glob = world * my_part.n_per
    last = torch.full((n_glob,), -1, dtype=torch.int64, device=dev)

    def apply(roots, first_step, only_range=None):
        # batches are cycled: batch b is used at steps b, b + NUM_BATCHES, ...; visit them in the order of their last use
        order = []
        for b in range(NUM_BATCHES):
            if b >= n_steps_total:
                continue
            s_last = b + ((n_steps_total - 1 - b) // NUM_BATCHES) * NUM_BATCHES
            if s_last >= first_step:
                order.append((s_last, b))
        for s_last, b in sorted(order):
            ids = roots[b]
            if only_range is not None:
                ids = ids[(ids >= only_range[0]) & (ids < only_range[1])]
            last[ids] = torch.maximum(last[ids], torch.full_like(ids, s_last))
    apply(my_part.roots, 0)
    for q in range(world):
        if q == rank:
            continue
        src, dst, ts, neg = make_partition(q, world, dev, my_part.n_per, my_part.g.num_edges // 2)
        roots_q, _ = batches_of(src, dst, ts, neg)
        del src, dst, ts, neg
        apply(roots_q, routed_from, (q * my_part.n_per, (q + 1) * my_part.n_per))
    return last


def check_state(part, n_steps_total, routed_from):
    """Whole memory and mail tables of this rank against the expectation (chunked); returns (ok, rows written, text that
    describes the first difference)."""
    dev = part.dev
    last = _expected_last_step(part.rank, part.world, dev, n_steps_total, routed_from, part)
    loc_last = last[part.loc_ids]                      # nodes without a local slot cannot be written here
    bad, why = 0, ""
    for name, state, dim in (("memory", part.mem, MEM_DIM), ("mail", part.mail, MAIL_DIM)):
        for a in range(0, part.loc_ids.numel(), 200_000):
            ids, ls = part.loc_ids[a:a + 200_000], loc_last[a:a + 200_000]
            want = model_rows(ids, ls.clamp_min(0), dim) * (ls >= 0).unsqueeze(1)
            want_ts = ls.clamp_min(0).to(torch.float32) * (ls >= 0)
            diff = (state.data[a:a + 200_000] != want).any(1) | (state.ts[a:a + 200_000] != want_ts)
            n_bad = int(diff.sum().item())
            if n_bad and not why:
                j = int(torch.nonzero(diff)[0].item())
                why = (f"{name} table: {n_bad} rows differ in slots [{a}, {a + ids.numel()}); first: slot {a + j} node {int(ids[j])} "
                       f"expected last write at step {int(ls[j])}, table holds ts {float(state.ts[a + j])} row[0] {float(state.data[a + j, 0])} "
                       f"(want {float(want[j, 0])})")
            bad += n_bad
    return bad == 0, int((loc_last >= 0).sum().item()), why


def run(args, rank, world, dev, clocks, peak_info, n_per=N_PER, e_per=E_PER):
    from starrygl.cache.p2p_route import P2PCacheRoute
    K, W = args.steps, max(args.warmup, 3)
    part = Partition(rank, world, dev, n_per, e_per)
    step = Step(part)
    steps = [step] + [Step(part, shared=step) for _ in range(NBUF - 1)]      # the next steps are prepared while the tables serve step s
    rows_hint = 3 * EVENTS * max(1, min(world - 1, 5))
    cap_rows = max(16384, 3 * EVENTS)
    mem_route = P2PCacheRoute(MEM_DIM, True, cap_rows=cap_rows, ring=4)
    mail_route = P2PCacheRoute(MAIL_DIM, True, cap_rows=cap_rows, ring=4)
    hi_prio = min(torch.cuda.Stream.priority_range())    # the table chain is the critical one: its CTAs are placed first
    r_streams = [torch.cuda.Stream(dev) for _ in range(2)]                  # the pushes: memory rows and mails side by side
    t_stream = torch.cuda.Stream(dev, priority=hi_prio)  # everything that touches the node tables, in step order
    t_side = torch.cuda.Stream(dev, priority=hi_prio)    # the mail table's applies, next to the memory table's
    m_stream = torch.cuda.Stream(dev, priority=hi_prio)  # the model stand-in: behind a step's gathers, next to the applies
    g_done = [torch.cuda.Event() for _ in range(NBUF)]   # a step's gathers have finished
    fork, join = torch.cuda.Event(), torch.cuda.Event()
    p_done = [torch.cuda.Event() for _ in range(NBUF)]   # a step's layer-0 list, hop and route plan exist
    m_done = [torch.cuda.Event() for _ in range(NBUF)]   # ... its fresh rows exist (A4)
    t_done = [torch.cuda.Event() for _ in range(NBUF)]   # ... its table reads and local writes have finished
    s_done = [[torch.cuda.Event() for _ in range(2)] for _ in range(NBUF)]   # ... its pushes have left its buffers
    n_done = [0]                     # steps issued so far (the device's step counter follows)
    marks, marking = [], [False]

    def mark(s, what, stream):
        if marking[0]:
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            marks.append((s, what, e))

    h_batches = step.batches.cpu().pin_memory()                     # the host-buffer form starts here
    d2h = [0]
    routes = []
    for st in steps:
        routes.append(mem_route.bind_dev(st.new_mem, st.pl_rows, st.pl_locs, st.pl_sizes, rows_hint, st.new_ts, part.mem,
                                         r_streams[0], t_stream)
                      + mail_route.bind_dev(st.new_mail, st.pl_rows, st.pl_locs, st.pl_sizes, rows_hint, st.new_ts, part.mail,
                                            r_streams[1], t_side))

    owed = []                        # bound applies of the step whose pushes have not been applied here yet

    def apply_owed():
        while owed:                  # the two tables' applies side by side (each is a short, latency-bound kernel)
            s_prev, apply_mem, apply_mail = owed.pop(0)
            fork.record(t_stream)
            t_side.wait_event(fork)
            apply_mail()
            join.record(t_side)
            apply_mem()
            t_stream.wait_event(join)
            mark(s_prev, "apply<", t_stream)

    def one_step(routed, host=False):
        # Two chains.  (1) On the step object's own stream: relabel, hop, plan -- nothing of it touches the tables, so
        # it runs ahead by up to NBUF - 1 steps.  (2) On t_stream, in step order: the gathers of step s, then the rows the
        # peers pushed in step s-1 (next to them, on its own stream, the model stand-in of step s, which needs the gathered
        # rows but no table), then the local writes of step s.  That is the reference's order: a
        # step's received rows are written when the NEXT update is called (starrygl/cache/NodeState.py:269-274: the
        # future of the previous update is waited on first), so a step reads the local writes of the step before it and
        # the remote rows of the step before that, and the transfer of step s has the whole of step s+1's reads to land.
        # The pushes leave on their own streams as soon as the fresh rows exist.
        s = n_done[0]
        i = s % NBUF
        st = steps[i]
        torch.cuda.set_stream(st.stream)
        if s >= NBUF:
            st.stream.wait_event(t_done[i])                           # step s - NBUF used the same buffers
            if routed:
                st.stream.wait_event(s_done[i][0])
                st.stream.wait_event(s_done[i][1])
        mark(s, "prepare>", st.stream)
        if host:
            st.sample_from_host(h_batches[s % NUM_BATCHES])
        else:
            st.sample(s % NUM_BATCHES)
        p_done[i].record(st.stream)
        mark(s, "prepare<", st.stream)
        if host:
            d2h[0] = st.export_to_host()
        torch.cuda.set_stream(t_stream)
        t_stream.wait_event(p_done[i])
        mark(s, "read>", t_stream)
        st.read_tables()
        g_done[i].record(t_stream)
        mark(s, "read<", t_stream)
        torch.cuda.set_stream(m_stream)
        m_stream.wait_event(g_done[i])
        st.model()
        m_done[i].record(m_stream)
        mark(s, "model<", m_stream)
        torch.cuda.set_stream(t_stream)
        if routed:
            send_mem, apply_mem, send_mail, apply_mail = routes[i]
            for r in r_streams:
                r.wait_event(m_done[i])
            send_mail(), send_mem()
            for j, r in enumerate(r_streams):
                s_done[i][j].record(r)
            mark(s, "push mem<", r_streams[0])
            mark(s, "push mail<", r_streams[1])
            apply_owed()                                              # the pushes of step s-1, next to the model of step s
            owed.append((s, apply_mem, apply_mail))
        t_stream.wait_event(m_done[i])
        st.write_tables()
        t_done[i].record(t_stream)
        mark(s, "write<", t_stream)
        n_done[0] += 1

    def print_marks():
        import sys
        torch.cuda.synchronize(dev)
        t0 = marks[0][2]
        for s, what, e in marks:
            print(f"timeline rank {rank} step {s:4d} {what:11s} {t0.elapsed_time(e):9.4f} ms", file=sys.stderr)
        marks.clear()

    def timed(n_steps, routed, host=False):
        torch.cuda.synchronize(dev)
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        main = torch.cuda.current_stream(dev)
        e0.record(main)
        for st in steps:
            st.stream.wait_stream(main)
        for r in r_streams:
            r.wait_stream(main)
        t_stream.wait_stream(main)
        t_side.wait_stream(main)
        m_stream.wait_stream(main)
        t0 = time.perf_counter()
        for _ in range(n_steps):
            one_step(routed, host)
        apply_owed()                 # the last step's pushes are applied inside the region that sent them
        torch.cuda.set_stream(main)
        t_issue = time.perf_counter() - t0
        for st in steps:
            main.wait_stream(st.stream)
        for r in r_streams:
            main.wait_stream(r)
        main.wait_stream(t_stream)
        main.wait_stream(t_side)
        main.wait_stream(m_stream)
        e1.record(main)
        torch.cuda.synchronize(dev)
        wall = time.perf_counter() - t0
        t = torch.tensor([e0.elapsed_time(e1), wall * 1e3], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0].item()), t_issue, float(t[1].item())

    # same workload on one partition without the exchange (what a rank does when nothing has to be pushed)
    timed(W, False)
    reps = max(3, min(10, 400 // max(K, 1)))
    local_ms = statistics.median([timed(K, False)[0] for _ in range(reps)])
    routed_from = n_done[0]
    # the partitioned step with the route
    timed(W, True)
    if clocks is not None:
        clocks.start()
    rows0 = int(step.rows_sent.item())
    regions = [timed(K, True) for _ in range(reps)]
    rows1 = int(step.rows_sent.item())
    # end to end: roots from host memory every step, block structure back to pinned host memory every step (wall clock)
    timed(W, True, host=True)
    e2e_ms = statistics.median([timed(K, True, host=True)[2] for _ in range(reps)])
    clk = clocks.stop() if clocks is not None else None
    if getattr(args, "timeline", False):             # one more routed region with an event after every stage, printed by rank 0
        marking[0] = True
        timed(4 * NBUF, True)
        marking[0] = False
        print_marks()
    ms = statistics.median([r[0] for r in regions])
    t_issue = statistics.median([r[1] for r in regions])
    for st, what in ((step.status, "step"), (mem_route.status, "memory route"), (mail_route.status, "mail route"),
                     (part.mem._status(), "memory table"), (part.mail._status(), "mail table")):
        st.check(f"bench ({what})")
    ok, written, why = check_state(part, n_done[0], routed_from)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) != 1:
        raise SystemExit(f"rank {rank}: node state differs from the expectation recomputed from the seeds ({why or 'on another rank'})")
    edges = int(steps[(n_done[0] - 1) % NBUF].hop.total())
    # the two captured chains of a step, each replayed alone (after the state check: these replays advance the step counter)
    chain_ms = {}
    if step.use_graphs:
        for name, g in (("prepare", step.g1), ("gathers", step.g2), ("model_stand_in", step.g2m), ("write", step.g3)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(step.stream):
                for _ in range(5):
                    g.replay()
                e0.record()
                for _ in range(50):
                    g.replay()
                e1.record()
            torch.cuda.synchronize(dev)
            chain_ms[name] = e0.elapsed_time(e1) / 50
    rows_per_step = (rows1 - rows0) / (reps * K)
    rt = torch.tensor([rows_per_step], dtype=torch.float64, device=dev)
    dist.all_reduce(rt, op=dist.ReduceOp.MAX)
    rows_per_step = float(rt.item())
    mem_route.close(), mail_route.close()
    if rank != 0:
        return None
    peak, peak_kind = peak_info
    wire = (mem_route.pitch + mail_route.pitch) * 4
    payload = (MEM_DIM + 1 + MAIL_DIM + 1) * 4
    n_roots = 3 * EVENTS
    gather_bytes = (n_roots + edges) * (2 * MEM_DIM * 4 + 4 + 8 + 8) + n_roots * (2 * MAIL_DIM * 4 + 4 + 8 + 8)
    step_ms, local_step_ms = ms / K, local_ms / K
    route_gbps = rows_per_step * payload / step_ms / 1e6
    return {"metric": "sampled+gathered events/sec", "value": world * n_roots * K / (ms / 1e3), "unit": "events/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": {"workload": "8xB200 distributed TGN data path (BASELINE configs[3]): planted-community graph, one partition "
                                   "per rank, recent-10, memory dim 100, 4,000 events per rank and step, owner -> replica route of "
                                   "memory rows and mails with plans built on the device every step",
                       "graph": f"{world * n_per} nodes, {world * e_per} events, {int(P_INTRA * 100)} % intra-partition, both "
                                "directions of an event sampled, int64 ids, ts U[0,1e7)",
                       "events_per_rank_and_step": EVENTS, "event": "one root query (4,000 interactions = 12,000 of them: source, "
                                                                     "destination, negative destination)",
                       "policy": f"recent-{FANOUT}, 1 hop", "memory_row": f"{MEM_DIM} x fp32 + ts", "mail_row": f"{MAIL_DIM} x fp32 + ts",
                       "l2": "node tables (0.1-1 GB memory, 0.5-2.7 GB mails) and the 25 M-edge adjacency exceed L2; 64 distinct batches",
                       "parallelism": f"{world} partitions, one process per GPU; peer-memory route, device-built plans",
                       "timing": f"median of {reps} repeats of the K-step region (CUDA events, max over ranks)"},
            "interactions_per_s": world * EVENTS * K / (ms / 1e3),
            "e2e": {"value": world * n_roots * K / (e2e_ms / 1e3), "unit": "events/s", "h2d_bytes_per_step": 16 * n_roots,
                    "d2h_bytes_per_step": d2h[0],
                    "note": "per step: roots and query times from host memory (staged through a pinned buffer), the step with its "
                            "route, the block structure (offsets, neighbour ids, timestamps, edge ids, dt) to pinned host memory; "
                            "wall clock around the K-step loop and a device synchronisation, max over ranks"},
            "same_workload_one_partition": {"ms_per_step": local_step_ms, "events_per_s_per_gpu": n_roots / local_step_ms * 1e3,
                                            "weak_scaling_efficiency_vs_it": local_step_ms / step_ms,
                                            "note": "the same step on one partition without the exchange, measured in this run; "
                                                    "the N = 1 line of this benchmark is a different workload (sampler microbenchmark)"},
            "host_issue_ms_per_step": t_issue * 1e3 / K,
            "chains_alone_ms": dict(chain_ms, note="each captured graph replayed back to back on rank 0: 'prepare' = relabel, hop, "
                                    "plan (runs ahead, several steps in flight); 'gathers', 'model_stand_in' and 'write' = local "
                                    "writes follow each other in step order"),
            "route": {"rows_per_rank_and_step": rows_per_step, "replicas_per_owned_node_max": part.max_rep,
                      "payload_bytes_per_rank_and_step": rows_per_step * payload, "wire_bytes_per_rank_and_step": rows_per_step * wire,
                      "GBps_per_direction_over_the_step": route_gbps, "frac_of_900": route_gbps / 900, "frac_of_770_measured_peer_copy": route_gbps / 770,
                      "note": "bytes a rank pushes per step / step time: a lower bound of the link rate while the route runs "
                              "(the step also samples, gathers and plans)"},
            "e2e_check": {"routed_state_equals_expectation_on_every_rank": True, "rows_written_on_rank0": written,
                          "steps_checked": n_done[0]},
            "roofline": {"bound": "hbm", "kernel": "gather_rows (node memory + mails through the slot map)", "unit": "GB/s",
                         "bytes_per_step": gather_bytes, "achieved_over_the_step": gather_bytes / local_step_ms / 1e6, "peak": peak,
                         "frac": gather_bytes / local_step_ms / 1e6 / peak, "peak_source": peak_kind,
                         "note": "algorithmic gather bytes of a step over the whole one-partition step time (sampling, relabel, "
                                 "plan included): a lower bound for the gather kernels"},
            # + the route's kernels: credit + send and gate + apply, for each of the two tables
            "gpu_launches": (None if step.kernel_launches is None else (step.kernel_launches + 8) * K * reps),
            "kernel_launches_per_step": (None if step.kernel_launches is None else step.kernel_launches + 8),
            "edges_per_step": edges, "clocks": clk}
