#!/usr/bin/env python
"""Benchmark of the per-mini-batch data path (temporal sampling + feature gather [+ route]) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step = one mini-batch of 4,096 roots on a synthetic temporal graph of 1 M nodes / 50 M edges (out-degree
power law, alpha 2.1; int64 ids; timestamps uniform in [0, 1e7)): most-recent-20 sampling of every root before
its query time, then the gather of the sampled edges' feature rows (172 x fp32) from a table that is much
larger than L2.  An "event" is one root query.  Prints ONE JSON line (rank 0).

  value      events/s with the batch's roots already in HBM (CUDA-event time of K steps, max over ranks)
  e2e        the same through the host-facing call: pinned host roots -> H2D -> sample -> gather -> block
             structure back to pinned host memory (the gathered rows stay on the GPU for the model)
  roofline   the dominant kernel (the edge-feature gather): algorithmic bytes / its CUDA-event time
  cpu_baseline  the CPU oracle (C/OpenMP restatement of the reference's CPU sampler + row gather) on the
             host cores, on a bounded sample of the same batches
With --gpus N > 1 (under torchrun) every rank owns one partition of equal size (weak scaling) and every step
additionally pushes node-memory rows (100 x fp32 + ts) to the other partitions through the cache route.

Side measurements (their own one-line JSON, not the benchmark line): ``--tcsr-only`` times the T-CSR construction of
the benchmark graph; ``--route-bw-rows R`` (N > 1) times the route alone with R rows per rank and step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "starrygl-framework_b200"))
sys.path.insert(0, ROOT)

# more hardware work queues than the default 8: the benchmark drives up to 10 streams per GPU, and streams that share a
# queue serialise behind each other's kernels (must be set before CUDA is initialised)
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

import numpy as np
import torch

NUM_NODES = 1_000_000
NUM_EDGES = 50_000_000
BATCH = 4096
FANOUT = 20
EDGE_DIM = 172
MEM_DIM = 100
TS_MAX = 10_000_000
NUM_BATCHES = 64          # distinct pre-generated batches cycled through the steps
STREAMS = 6
ROUTE = "p2p"
GRAPHS = True
# DRAM bytes per gathered row measured with ncu on the small case (profiles/gather_bulk_kernel_172xfp32_small_case.txt:
# 57.1 MB for 65,160 rows); roofline.traffic scales it by the rows of a full-size launch
GATHER_TRAFFIC_BYTES_PER_ROW = 876.0
ROUTE_ROWS = 800          # rows per step a partition pushes to its peers (20 % cut edges of a 4,096-root batch)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)).get("hbm_gbs", 6650.0), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def make_graph(dev, seed):
    """Seeded synthetic stand-in for the sampler microbenchmark graph (generated on the GPU)."""
    gen = torch.Generator(device=dev).manual_seed(seed)
    u = torch.rand(NUM_NODES, device=dev, generator=gen).clamp_min_(1e-9)
    w = u.pow(-1.0 / 1.1).double()                      # Pareto tail index 1.1 <=> degree pdf exponent 2.1
    cdf = torch.cumsum(w, 0)
    cdf /= cdf[-1].clone()
    src = torch.searchsorted(cdf, torch.rand(NUM_EDGES, device=dev, dtype=torch.double, generator=gen)).clamp_max_(NUM_NODES - 1)
    dst = torch.randint(0, NUM_NODES, (NUM_EDGES,), device=dev, generator=gen)
    ts = (torch.rand(NUM_EDGES, device=dev, dtype=torch.double, generator=gen) * TS_MAX).long()
    return src, dst, ts, gen


def make_batches(src, ts, gen, dev):
    pick = torch.randint(0, NUM_EDGES, (NUM_BATCHES, BATCH), device=dev, generator=gen)
    # [batch, 2, BATCH]: roots and query times of one batch are contiguous; query time = the drawn edge's own timestamp
    both = torch.stack([src[pick], ts[pick]], 1).contiguous()
    return both[:, 0], both[:, 1]


def run_reference(args, rank, out_stream):
    """The reference's CPU path (its C/OpenMP restatement: the reference is numba/Python and cannot travel) on
    the host cores, same batches, bounded sample."""
    if rank != 0:
        return
    from oracle import oracle_c as OC
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else None
    out = cpu_baseline_measure(dev, steps=args.steps, warmup=args.warmup, budget_s=60.0)
    line = {"metric": "sampled+gathered events/sec", "value": out["value"], "unit": "events/s", "n_gpus": args.gpus,
            "steps": out["steps"], "warmup": args.warmup, "ms_per_step": out["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic", "impl": "reference",
            "config": workload_config(1), "cpu_baseline": out["cpu_baseline"],
            "e2e": {"value": out["value"], "unit": "events/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), file=out_stream, flush=True)


def workload_config(n_gpus):
    return {"workload": "1xB200 sampler microbench + sampled edge-feature gather (BASELINE configs[1] graph, configs[2] rows)",
            "graph": f"{NUM_NODES} nodes, {NUM_EDGES} edges, out-degree power law alpha 2.1, int64 ids, ts U[0,1e7)",
            "batch_roots": BATCH, "policy": f"recent-{FANOUT}, 1 hop", "edge_feat": f"{EDGE_DIM} x fp32",
            "edge_feat_rows": NUM_EDGES, "event": "one root query (a link-prediction interaction = three of them: source, destination, negative destination)",
            "l2": "inputs larger than L2: 64 distinct batches over a 34 GB feature table and a 1.2 GB adjacency",
            "batches_in_flight": STREAMS, "parallelism": f"{n_gpus} partition(s), one process per GPU" +
                           (f", cache route ({ROUTE}) of {ROUTE_ROWS} memory rows per step" if n_gpus > 1 else "")}


def _time_ms(fn, stream, iters, warm=3):
    for _ in range(warm):
        fn()
    stream.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(iters):
        fn()
    b.record(stream)
    stream.synchronize()
    return a.elapsed_time(b) / iters


def secondary_measurements(g, dev, peak):
    """The other single-GPU configurations of the baseline, reported next to the headline (not part of `value`):
    uniform [10,10] two-hop batches with (node, ts) dedup/relabel on the same graph, and the node-feature gather through a
    10 % GPU cache (10 M x 128 table, 200,000 ids per batch drawn Zipf(1.1) over a seeded permutation), fp32 and bf16."""
    from starrygl import ops
    from starrygl.graph.batch import build_batch_async
    out = {}
    cur = torch.cuda.current_stream(dev)
    gen = torch.Generator(device=dev).manual_seed(7)
    # ---- uniform [10,10] + relabel --------------------------------------------------------------------------------
    m = g.num_edges
    picks = [torch.randint(0, m, (BATCH,), device=dev, generator=gen) for _ in range(8)]
    # roots = source node of a drawn edge; the row of a node lists its edges, so a drawn position identifies (node, ts)
    node_of_edge = torch.repeat_interleave(torch.arange(g.num_nodes, device=dev), g.indptr[1:] - g.indptr[:-1])
    batches = [(node_of_edge[p].contiguous(), g.ts[p].contiguous()) for p in picks]
    del node_of_edge
    it = [0]

    def two_hop():
        q, qt = batches[it[0] % 8]
        it[0] += 1
        return build_batch_async(g, q, qt, [10, 10], "uniform", ts_range=(0, TS_MAX), seed=0)
    ms_eager = _time_ms(two_hop, cur, 20)
    from starrygl.graph.batch import BatchGraph
    bg = BatchGraph(g, BATCH, [10, 10], "uniform", ts_range=(0, TS_MAX), seed=0)

    def two_hop_graph():
        q, qt = batches[it[0] % 8]
        it[0] += 1
        return bg.run(q, qt)
    bg.stream.wait_stream(cur)
    ms = _time_ms(two_hop_graph, bg.stream, 50)
    with torch.cuda.stream(bg.stream):
        layers = two_hop_graph().finish()
    # the chain is latency-bound: with several batches in flight (one captured builder per stream, as a prefetcher
    # runs them) the GPU overlaps their short kernels
    FLY = 4
    bgs = [bg] + [BatchGraph(g, BATCH, [10, 10], "uniform", ts_range=(0, TS_MAX), seed=0) for _ in range(FLY - 1)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    reps = 80
    for timed in (False, True):
        if timed:
            e0.record(cur)
            for b_ in bgs:
                b_.stream.wait_stream(cur)
        for i in range(reps if timed else 8):
            q, qt = batches[i % 8]
            bgs[i % FLY].run(q, qt)
        for b_ in bgs:
            cur.wait_stream(b_.stream)
        if timed:
            e1.record(cur)
        torch.cuda.synchronize(dev)
    ms_fly = e0.elapsed_time(e1) / reps
    for b_ in bgs:
        b_.status.check("two-hop builder")
    del bgs
    out["uniform_10_10_relabel"] = {"ms_per_batch": ms, "ms_per_batch_without_cuda_graph": ms_eager,
                                    "ms_per_batch_4_in_flight": ms_fly, "events_per_s_4_in_flight": BATCH / ms_fly * 1e3,
                                    "events_per_s": BATCH / ms * 1e3, "roots": BATCH,
                                    "unique_pairs_per_layer": [int(d["gids"].numel()) for d in layers],
                                    "edges_per_layer": [int(d["indices"].numel()) for d in layers[1:]],
                                    "note": "sampling + (node, ts) dedup/relabel + CSC per hop: a chain of ~100 short kernels, replayed "
                                            "as one CUDA graph per batch"}
    # ---- node features through the cache ---------------------------------------------------------------------------
    N, D, IDS = 10_000_000, 128, 200_000
    perm = torch.randperm(N, device=dev, generator=gen)
    C_ = N // 10
    hitmap = torch.full((N,), -1, dtype=torch.int32, device=dev)
    hitmap[perm[:C_]] = torch.arange(C_, dtype=torch.int32, device=dev)
    rng = np.random.default_rng(0)
    ids = [perm[torch.from_numpy(np.minimum(rng.zipf(1.1, IDS) - 1, N - 1)).to(dev)].contiguous() for _ in range(8)]
    for name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        table = torch.empty(N, D, dtype=dt, device=dev)
        for s_ in range(0, N, 2_000_000):
            table[s_:s_ + 2_000_000].normal_(generator=gen)
        cache = table[perm[:C_]].contiguous()
        it[0] = 0

        def cg():
            r = ops.cache_gather(cache, hitmap, table, ids[it[0] % 8])
            it[0] += 1
            return r
        ms = _time_ms(cg, cur, 30)
        hits, misses = cg()[3].tolist()
        rb = D * table.element_size()
        alg = IDS * (2 * rb + 8 + 4) + misses * 16
        out[f"cache_gather_{name}"] = {"ms_per_batch": ms, "ids": IDS, "hit_rate": hits / IDS, "misses_compacted": misses,
                                       "algorithmic_bytes": alg, "achieved_GBps": alg / ms / 1e6,
                                       "frac_of_peak": alg / ms / 1e6 / peak}
        del table, cache
    return out


def route_bandwidth(args, rank, world, dev, out_stream):
    """Side measurement (not the benchmark line): the cache route alone at a message size where NVLink bandwidth, not
    latency, bounds it.  Every rank pushes ``--route-bw-rows`` rows of 100 x fp32 + ts per step, split evenly over the
    other ranks, through (a) the peer-memory kernels and (b) the grouped NCCL send/recv path.  GB/s = payload bytes a
    rank sends per step / step time (device time, max over ranks); every rank receives as much as it sends."""
    import torch.distributed as dist
    from starrygl.cache.cache_route import CacheRoute, CommPlan
    from starrygl.cache.p2p_route import P2PCacheRoute
    from starrygl.cache.NodeState import DistNodeState
    from starrygl.utils.partition_book import PartitionState
    N, D, rows = 2_000_000, MEM_DIM, int(args.route_bw_rows)
    per = rows // (world - 1)
    ranks = torch.cat([torch.full((per,), p, dtype=torch.long) for p in range(world) if p != rank])
    sizes = torch.bincount(ranks, minlength=world)
    g = torch.Generator().manual_seed(rank)
    plan = CommPlan(ranks, sizes, torch.randint(0, N, (ranks.numel(),), generator=g),
                    torch.randperm(N, generator=g)[:ranks.numel()]).to(dev)
    mem, mts = torch.randn(N, D, device=dev), torch.rand(N, device=dev)
    ps = PartitionState(loc_ids=torch.arange(N, device=dev), num_master_nums=N, node_mode='identity', num_nodes=N)
    state = DistNodeState(ps, D, device=dev)
    payload = ranks.numel() * (D + 1) * 4
    K = 50
    res = {"rows_per_step": int(ranks.numel()), "payload_MB_per_rank_and_step": payload / 1e6, "peers": world - 1}

    def timed(step_fn, streams):
        for _ in range(5):
            step_fn()
        torch.cuda.synchronize(dev)
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(streams[0])
        for st in streams[1:]:
            st.wait_stream(streams[0])
        for _ in range(K):
            step_fn()
        for st in streams[1:]:
            streams[0].wait_stream(st)
        e1.record(streams[0])
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / K], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    st_a, st_b = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    p2p = P2PCacheRoute(D, True, cap_rows=max(1024, per), ring=4)
    step = p2p.bind_step(mem, mts, plan, state, st_a, st_b)
    ms = timed(step, [st_a, st_b])
    p2p.status.check("route bandwidth (peer memory)")
    res["p2p"] = {"ms_per_step": ms, "GBps_per_direction": payload / ms / 1e6}
    p2p.close()

    cr = CacheRoute()

    def cb(idx, rows_, mode):
        state.write_packed(idx, rows_)
    cb.fused_state = state
    cr._exchange_counts(plan, dev)

    def nccl_step():
        with torch.cuda.stream(st_a):
            for f in cr.update_with_plan(mem, plan, cb, local_ts=mts):
                f.wait()
    ms = timed(nccl_step, [st_a])
    res["nccl"] = {"ms_per_step": ms, "GBps_per_direction": payload / ms / 1e6}
    if rank == 0:
        print(json.dumps({"route_bandwidth": res, "n_gpus": world, "nvlink_peak_GBps_per_direction": 900,
                          "measured_peer_copy_GBps": 770}), file=out_stream, flush=True)


def cpu_baseline_measure(dev, steps, warmup, budget_s):
    """Times the C oracle on the same graph and batches.  The graph is generated with the same seeded generator
    (on the GPU when there is one, and copied to the host); the feature table is a 1 M-row host sample
    (edge id modulo 1 M) because 34 GB of host rows are not needed to time a row gather."""
    from oracle import oracle_c as OC
    gdev = dev if dev is not None else torch.device("cpu")
    if dev is None:
        raise RuntimeError("the benchmark graph is generated on the GPU")
    src, dst, ts, gen = make_graph(gdev, 0)
    b_roots, b_ts = make_batches(src, ts, gen, gdev)
    src_h, dst_h, ts_h = src.cpu().numpy(), dst.cpu().numpy(), ts.cpu().numpy()
    del src, dst, ts
    torch.cuda.empty_cache()
    cores = os.cpu_count() or 1
    OC.set_threads(cores)
    t0 = time.perf_counter()
    indptr, nbr, tss, eid, _ = OC.tcsr_build(src_h, dst_h, ts_h, None, NUM_NODES)
    build_s = time.perf_counter() - t0
    del src_h, dst_h
    rows_h = 1_000_000
    feats = np.random.default_rng(0).standard_normal((rows_h, EDGE_DIM), dtype=np.float32)
    roots_h, rts_h = b_roots.cpu().numpy(), b_ts.cpu().numpy()
    out_rows = np.empty((BATCH * FANOUT, EDGE_DIM), np.float32)

    def step(i):
        o = OC.sample_layer(indptr, nbr, tss, eid, roots_h[i % NUM_BATCHES], rts_h[i % NUM_BATCHES], FANOUT, 0, trim=False)
        tot = int(o[5][-1])
        OC.gather_rows(feats, o[4][:tot] % rows_h, out_rows)
        return tot
    for i in range(max(warmup, 3)):
        step(i)
    n_done, t0 = 0, time.perf_counter()
    while n_done < max(steps, 1) * 50 and time.perf_counter() - t0 < min(budget_s, 20.0):
        step(n_done)
        n_done += 1
    dt = time.perf_counter() - t0
    val = n_done * BATCH / dt
    return {"value": val, "steps": n_done, "ms_per_step": dt / n_done * 1e3,
            "cpu_baseline": {"value": val, "unit": "events/s", "cores": cores, "kind": "port",
                             "sample": f"{n_done} of the benchmark's batches (recent-{FANOUT} sampling on the full 50 M-edge graph + gather "
                                       f"of the sampled rows from a {rows_h}-row host table), C/OpenMP restatement of the reference's numba "
                                       f"sampler; T-CSR build on the host took {build_s:.1f} s"}}


def _protect_stdout():
    """Libraries may print banners to stdout (NCCL does with NCCL_DEBUG=VERSION); the JSON line must stay alone
    there.  File descriptor 1 is pointed at stderr and the original is returned for the final print."""
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    return os.fdopen(saved, "w")


def main():
    global NUM_NODES, NUM_EDGES, STREAMS, GRAPHS, ROUTE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the uniform two-hop and cache-gather measurements")
    ap.add_argument("--gather-mode", default="auto")
    ap.add_argument("--streams", type=int, default=6, help="mini-batches in flight (one pipeline object + stream each)")
    ap.add_argument("--graph-value", action="store_true",
                    help="replay a CUDA graph per step in the device-resident loop too (default: one fused C call per step; "
                         "the host-buffer loop always replays a graph that includes its copies)")
    ap.add_argument("--route", default="p2p", choices=["p2p", "nccl", "none"],
                    help="transport of the cache route at N > 1: peer-memory kernels (default) or grouped NCCL send/recv")
    ap.add_argument("--e2e-mode", default="native", choices=["native", "torch"],
                    help="host-buffer step as one library call (copy + captured graph) or as a torch CUDA-graph replay")
    ap.add_argument("--e2e-export", default="prefix", choices=["prefix", "full"],
                    help="result copy to the host: device-counted prefix (exact bytes) or whole-capacity copies")
    ap.add_argument("--no-numa-bind", action="store_true", help="N > 1: do not bind the rank to the CPUs of its GPU's NUMA node")
    ap.add_argument("--row-align", type=int, default=0, help="pad the feature table's rows in HBM to this many bytes (0 = dense)")
    ap.add_argument("--route-bw-rows", type=int, default=0,
                    help="N > 1: measure the route alone with this many rows per rank and step (bandwidth-bound sizes) and exit")
    ap.add_argument("--tcsr-only", action="store_true", help="time the T-CSR construction of the benchmark graph and exit")
    ap.add_argument("--no-step-graph", action="store_true",
                    help="issue sample+gather as one fused foreign call (three kernel launches) instead of one graph launch")
    ap.add_argument("--num-nodes", type=int, default=NUM_NODES, help="smaller graphs are for profiler captures only")
    ap.add_argument("--num-edges", type=int, default=NUM_EDGES)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    out_stream = _protect_stdout()
    ROUTE = args.route
    NUM_NODES, NUM_EDGES, STREAMS, GRAPHS = args.num_nodes, args.num_edges, max(1, args.streams), True
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference(args, rank, out_stream)

    import torch.distributed as dist
    from starrygl import ops, _C
    from starrygl.graph.pipeline import SampleGatherPipeline
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    multi = world > 1
    from starrygl.utils.affinity import bind_to_gpu_numa_node
    host_info = bind_to_gpu_numa_node(local) if (multi and not args.no_numa_bind) else {"numa_node": None, "cpus": len(os.sched_getaffinity(0))}
    if multi:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    if args.route_bw_rows > 0:
        if not multi:
            raise SystemExit("--route-bw-rows needs at least two ranks")
        return route_bandwidth(args, rank, world, dev, out_stream)

    # ---- set-up (untimed): graph, T-CSR, feature table, batches -------------------------------------------
    src, dst, ts, gen = make_graph(dev, seed=rank)
    if args.tcsr_only:
        # side measurement (not the benchmark line): T-CSR construction of the benchmark graph, CUDA-event timed
        ops.tcsr_build(src, dst, ts, None, NUM_NODES)
        e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0_.record()
        for _ in range(reps):
            ops.tcsr_build(src, dst, ts, None, NUM_NODES)
        e1_.record()
        torch.cuda.synchronize(dev)
        ms_ = e0_.elapsed_time(e1_) / reps
        alg_ = NUM_EDGES * 56 + (NUM_NODES + 1) * 8 + 6 * 2 * NUM_EDGES * 12
        if rank == 0:
            print(json.dumps({"tcsr_build_ms": ms_, "edges": NUM_EDGES, "nodes": NUM_NODES, "algorithmic_bytes": alg_,
                              "algorithmic_GBps": alg_ / ms_ / 1e6}), file=out_stream, flush=True)
        return
    g = ops.tcsr_build(src, dst, ts, None, NUM_NODES)
    b_roots, b_ts = make_batches(src, ts, gen, dev)
    del src, dst, ts
    # rows padded in HBM to a multiple of --row-align bytes (0 = dense): a 688-byte row that starts on a 64-byte boundary
    # touches 11 DRAM atoms instead of 11-12 and 22 sectors instead of 22-23
    pitch_f = EDGE_DIM if args.row_align <= 0 else ((EDGE_DIM * 4 + args.row_align - 1) // args.row_align) * args.row_align // 4
    feats = torch.empty(NUM_EDGES, pitch_f, dtype=torch.float32, device=dev)[:, :EDGE_DIM]
    for s in range(0, NUM_EDGES, 5_000_000):
        feats[s:s + 5_000_000].normal_(generator=gen)
    h_both = b_roots._base.cpu().pin_memory()           # [batch, 2, BATCH]: one contiguous host block per batch
    h_roots, h_ts = h_both[:, 0], h_both[:, 1]
    h_ptrs = [h_both[b].data_ptr() for b in range(NUM_BATCHES)]

    S = max(1, args.streams)
    streams = [torch.cuda.Stream(dev) for _ in range(S)]
    pipes = [SampleGatherPipeline(g, feats, FANOUT, "recent", BATCH, gather_mode=args.gather_mode, stream=st,
                                  export=args.e2e_export) for st in streams]
    pipe, stream = pipes[0], streams[0]
    use_graph = args.graph_value
    for p_ in pipes:
        p_.capture()
        if not args.no_step_graph:
            p_.capture_native()
        if args.e2e_mode == "native":
            p_.capture_native_host()
    main_stream = torch.cuda.Stream(dev)
    route_stream = torch.cuda.Stream(dev, priority=-1)     # its few CTAs must not queue behind the persistent gather CTAs
    route_recv_stream = torch.cuda.Stream(dev, priority=-1)
    route = None
    route_steps = None
    if multi and args.route != "none":
        from starrygl.cache.cache_route import CacheRoute, CommPlan
        from starrygl.cache.NodeState import DistNodeState
        from starrygl.utils.partition_book import PartitionState
        rgen = torch.Generator().manual_seed(100 + rank)
        # per step: ROUTE_ROWS owned rows go to the other ranks (round-robin), slots on the receiver are unique
        per = ROUTE_ROWS // (world - 1)
        ranks = torch.cat([torch.full((per,), p, dtype=torch.long) for p in range(world) if p != rank])
        sizes = torch.bincount(ranks, minlength=world)
        plans = []
        for b in range(NUM_BATCHES):
            plans.append(CommPlan(send_ranks=ranks, send_sizes=sizes,
                                  send_indices=torch.randint(0, NUM_NODES, (ranks.numel(),), generator=rgen),
                                  send_remote_indices=(torch.randperm(NUM_NODES, generator=rgen)[:ranks.numel()])).to(dev))
        ps = PartitionState(loc_ids=torch.arange(NUM_NODES, device=dev), num_master_nums=NUM_NODES, node_mode='identity',
                            num_nodes=NUM_NODES)
        state = DistNodeState(ps, MEM_DIM, device=dev)
        mem = torch.randn(NUM_NODES, MEM_DIM, device=dev)
        mem_ts = torch.rand(NUM_NODES, device=dev)
        cr = CacheRoute()

        def cb(idx, rows, mode):
            state.write_packed(idx, rows)
        cb.fused_state = state
        for p in plans:     # receive counts are exchanged once per plan (set-up), steps then need no host sync
            cr._exchange_counts(p, dev)
        if args.route == "p2p":
            from starrygl.cache.p2p_route import P2PCacheRoute
            p2p = P2PCacheRoute(MEM_DIM, True, cap_rows=max(1024, ROUTE_ROWS), ring=8)

            class _P2PAdapter:      # same call shape as CacheRoute.update_with_plan for the loops below
                def update_with_plan(self, feats, plan, cb_, local_ts=None):
                    return [p2p.push(feats, plan, state, local_ts)]
            cr = _P2PAdapter()
            route_steps = [p2p.bind_step(mem, mem_ts, pl_, state, route_stream, route_recv_stream) for pl_ in plans]
        route = (cr, plans, mem, mem_ts, cb)

    batch_ptrs = [(b_roots[b].data_ptr(), b_ts[b].data_ptr()) for b in range(NUM_BATCHES)]

    issue_t = {"sample_gather": 0.0, "route_send": 0.0, "route_apply": 0.0}

    def step_device(i, ev=None, route_inline=True):
        b = i % NUM_BATCHES
        t_a = time.perf_counter()
        if ev is not None:
            pipes[i % S].run_device(b_roots[b], b_ts[b], 0, ev)
        elif use_graph:
            pipes[i % S].replay_device(b_roots[b], b_ts[b])
        elif not args.no_step_graph:
            pipes[i % S].replay_ptr(batch_ptrs[b][0])       # one call: copy the batch's roots in + one graph launch
        else:
            pipes[i % S].run_device_ptr(batch_ptrs[b][0], batch_ptrs[b][1], BATCH)
        if route is not None and route_inline:
            # the memory rows pushed to the other partitions do not depend on this batch's samples: the route runs
            # on its own stream, concurrently with sampling and gather
            cr, plans, mem, mem_ts, cb = route
            t_b = time.perf_counter()
            if route_steps is not None:
                route_steps[b]()                # one pre-bound foreign call: send + apply of this step
                t_c = time.perf_counter()
            else:
                with torch.cuda.stream(route_stream):
                    futs = cr.update_with_plan(mem, plans[b], cb, local_ts=mem_ts)
                    t_c = time.perf_counter()
                    for f in futs:
                        f.wait()
            t_d = time.perf_counter()
            issue_t["sample_gather"] += t_b - t_a
            issue_t["route_send"] += t_c - t_b
            issue_t["route_apply"] += t_d - t_c

    def barrier():
        if multi:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- value: inputs resident in HBM --------------------------------------------------------------------
    for i in range(args.warmup):
        step_device(i)
    barrier()
    for p_ in pipes:
        p_.status.check("bench warmup")
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    for k_ in issue_t:
        issue_t[k_] = 0.0
    gev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    # K steps, up to S of them in flight: the streams fork from / join into main_stream, whose two events bracket
    # the whole region on the device
    e0.record(main_stream)
    for st in streams + [route_stream, route_recv_stream]:
        st.wait_stream(main_stream)
    route_thread = None
    if route_steps is not None:
        # the route is driven from its own host thread, as a trainer would (the foreign calls release the GIL): the two
        # issue loops run side by side, the device-side ring bounds how far a rank can run ahead of its peers
        def route_loop():
            torch.cuda.set_device(dev)
            t_r = time.perf_counter()
            for i in range(args.steps):
                route_steps[(args.warmup + i) % NUM_BATCHES]()
            issue_t["route_thread_total"] = time.perf_counter() - t_r
        route_thread = threading.Thread(target=route_loop)
        route_thread.start()
    t_issue = time.perf_counter()
    for i in range(args.steps):
        step_device(args.warmup + i, None, route_inline=route_thread is None)
    t_issue = time.perf_counter() - t_issue
    if route_thread is not None:
        route_thread.join()
    # where the device time goes: end of the sampler/gather streams and end of the two route chains, each against e0
    e_pipe = torch.cuda.Event(enable_timing=True)
    e_rs, e_rr = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    join_stream = torch.cuda.Stream(dev)
    for st in streams:
        join_stream.wait_stream(st)
    e_pipe.record(join_stream)
    e_rs.record(route_stream)
    e_rr.record(route_recv_stream)
    for st in streams + [route_stream, route_recv_stream]:
        main_stream.wait_stream(st)
    e1.record(main_stream)
    barrier()
    ms = e0.elapsed_time(e1)
    for p_ in pipes:
        p_.status.check("bench")
    if os.environ.get("SGL_P2P_DBG", "0") == "2" and route_steps is not None and os.environ.get("SGL_P2P_TL_OUT"):
        import ctypes as C_
        n_tl = min(args.steps + 2 * args.warmup, 4096)
        buf = (C_.c_uint64 * (n_tl * 8))()
        _C.lib().sgl_p2p_route_timeline(p2p.ctx, buf, n_tl)
        np.save(os.environ["SGL_P2P_TL_OUT"] + f".rank{rank}.npy", np.array(buf, dtype=np.uint64).reshape(n_tl, 8))
    if os.environ.get("SGL_P2P_DBG", "0") == "2" and route_steps is not None and rank == 0:
        import ctypes as C_
        n_tl = min(args.steps + 2 * args.warmup, 4096)
        buf = (C_.c_uint64 * (n_tl * 8))()
        _C.lib().sgl_p2p_route_timeline(p2p.ctx, buf, n_tl)
        tl = np.array(buf, dtype=np.uint64).reshape(n_tl, 8).astype(np.float64)[args.warmup + 50:args.warmup + args.steps - 10] / 1e3
        sys.stderr.write("P2P timeline (us): send dur %.1f | send start->next start %.1f | apply start->first CTA done %.1f | first CTA done->end %.1f | "
                         "apply start->next start %.1f | send end -> apply first CTA done %.1f | resident before start: send %.1f apply %.1f\n" % (
                             np.median(tl[:, 1] - tl[:, 0]), np.median(np.diff(tl[:, 0])), np.median(tl[:, 3] - tl[:, 2]),
                             np.median(tl[:, 4] - tl[:, 3]), np.median(np.diff(tl[:, 2])), np.median(tl[:, 3] - tl[:, 1]),
                             np.median(tl[:, 0] - tl[:, 5]), np.median(tl[:, 2] - tl[:, 6])))
    if True:
        # the step is one foreign call (or one graph replay), so its kernels cannot be bracketed individually:
        # the dominant kernel is timed in a second pass over the same K batches, kernel by kernel on one stream
        for i in range(args.steps):
            pipe.run_device(b_roots[(args.warmup + i) % NUM_BATCHES], b_ts[(args.warmup + i) % NUM_BATCHES], 0, gev[i])
        pipe.stream.synchronize()
    gather_ms = [a.elapsed_time(b) for a, b in gev]
    # edges actually gathered per step (for the algorithmic byte count), read after the timed region
    edges = []
    for i in range(args.steps):
        pipe.run_device(b_roots[(args.warmup + i) % NUM_BATCHES], b_ts[(args.warmup + i) % NUM_BATCHES])
        pipe.stream.synchronize()
        edges.append(int(pipe.offsets[BATCH].item()))

    # ---- e2e: host buffers in, block structure out, up to S batches in flight -------------------------------
    def e2e_loop(first, count):
        tot = 0
        for i in range(count):
            p_ = pipes[i % S]
            if i >= S:                          # retire the batch that used this pipeline object before reusing it
                tot += p_.result()[0]
            b = (first + i) % NUM_BATCHES
            if args.e2e_mode == "native":
                p_.submit_host_ptr(h_ptrs[b])   # one call: roots from the pinned block + the captured step with its export
            else:
                p_.submit_host(h_roots[b], h_ts[b])
            if route_steps is not None:
                route_steps[b]()                # peer-memory route: send + apply of this step
            elif route is not None:
                cr, plans, mem, mem_ts, cb = route
                with torch.cuda.stream(route_stream):
                    for f in cr.update_with_plan(mem, plans[b], cb, local_ts=mem_ts):
                        f.wait()
        for i in range(max(0, count - S), count):
            tot += pipes[i % S].result()[0]
        return tot
    e2e_loop(0, args.warmup)
    barrier()
    t0 = time.perf_counter()
    e2e_steps = args.steps
    e2e_edges = e2e_loop(args.warmup, e2e_steps)
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    barrier()
    clk = clocks.stop() if rank == 0 else None

    t = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if multi:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()

    if rank == 0:
        peak, peak_kind = peaks()
        row_bytes = EDGE_DIM * 4
        alg = statistics.mean(edges) * (2 * row_bytes + 8)
        g_ms = statistics.mean(gather_ms)
        achieved = alg / g_ms / 1e6
        line = {"metric": "sampled+gathered events/sec", "value": world * BATCH * args.steps / (ms / 1e3),
                "unit": "events/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "host": host_info, "host_issue_ms_per_step": t_issue * 1e3 / args.steps,
                "host_issue_breakdown_ms": {k: v * 1e3 / args.steps for k, v in issue_t.items()},
                "device_ms_per_step": {"sample_gather_streams": e0.elapsed_time(e_pipe) / args.steps,
                                       "route_send_chain": e0.elapsed_time(e_rs) / args.steps,
                                       "route_apply_chain": e0.elapsed_time(e_rr) / args.steps},
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "int64", "data": "synthetic", "config": workload_config(world),
                "e2e": {"value": world * BATCH * e2e_steps / (e2e_ms / 1e3), "unit": "events/s",
                        "h2d_bytes_per_step": pipe.h2d_bytes(BATCH), "d2h_bytes_per_step": pipe.d2h_bytes(e2e_edges / max(e2e_steps, 1)),
                        "note": "pinned host roots/times in; offsets, neighbour ids, timestamps, edge ids and dt out; "
                                "gathered feature rows stay on the GPU for the model", "edges_per_step": e2e_edges / e2e_steps},
                "gpu_launches": args.steps * (pipe.kernel_launches_per_step + (2 if multi else 0)),
                "roofline": {"bound": "hbm", "kernel": "gather_bulk_kernel" if pipe.mode != 1 else "gather_lanes_kernel",
                             "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_source": peak_kind, "traffic": statistics.mean(edges) * GATHER_TRAFFIC_BYTES_PER_ROW,
                             "traffic_note": "ncu dram read+write of a 65 k-row launch scaled by rows; the output is still in L2 when "
                                             "the kernel ends, so write-back is under-counted (see profiles/)",
                             "bytes_per_launch": alg, "ms_per_launch": g_ms,
                             "edges_per_step": statistics.mean(edges)},
                "clocks": clk}
        if world == 1 and not args.no_secondary:
            del feats, pipe, pipes
            feats = pipe = pipes = None
            torch.cuda.empty_cache()
            line["secondary"] = secondary_measurements(g, dev, peak)
        if not args.no_cpu_baseline and world == 1:
            del feats, pipe, pipes, g
            torch.cuda.empty_cache()
            line["cpu_baseline"] = cpu_baseline_measure(dev, args.steps, args.warmup, 20.0)["cpu_baseline"]
        print(json.dumps(line), file=out_stream, flush=True)
    if multi:
        dist.barrier()
        from starrygl.cache.cache_route import NativeComm
        NativeComm.shutdown()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
