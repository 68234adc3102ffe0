// Sub-graph of a chunk set and a time window, as a two-level CSR: node -> distinct timestamps -> edges.
//
// Selected edges: source node in a selected chunk, t_begin <= ts < t_end, neighbour in a selected chunk.  Output:
//   out_nodes[U]        ascending ids of the nodes that keep at least one edge
//   out_node_ptr[U+1]   node u owns the timestamp groups [out_node_ptr[u], out_node_ptr[u+1])
//   out_group_ts[G]     timestamp of a group (ascending inside a node)
//   out_group_ptr[G+1]  group g owns the edges [out_group_ptr[g], out_group_ptr[g+1])
//   out_nbr/ts/eid[E]   the edges in T-CSR order
// Three kernels, nothing is sorted (the T-CSR already is) and nothing uses atomics on the data:
//   slice_count_kernel  one warp per node: window by binary search, ballot over 32 edges at a time -> edges and groups
//   slice_scan_kernel   exclusive scans of (node kept, groups, edges) over the nodes: CTA scan, last CTA scans the totals
//   slice_write_kernel  one warp per node again, writes at the scanned positions
// Algorithmic HBM bytes: per node in a selected chunk 16 (row pointer) + 8 * 2 * ceil(log2 deg) (two searches), per
// edge of the window 16 read twice (neighbour, ts; + 8 for the neighbour's chunk), per kept edge 24 written.
#include "scan.cuh"

namespace sgl {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ int64_t lower_bound_i64(const int64_t* __restrict__ a, int64_t lo, int64_t hi, int64_t v) {
  while (lo < hi) {
    const int64_t mid = lo + ((hi - lo) >> 1);
    if (__ldg(a + mid) < v) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}

struct SliceArgs {
  const int64_t *indptr, *nbr, *ts;
  const int64_t* node_chunk;   // may be null: every node is in chunk 0
  const uint8_t* chunk_mask;   // may be null: every chunk is selected
  int64_t num_nodes, num_chunks, t_begin, t_end;
};

__device__ __forceinline__ bool chunk_selected(const SliceArgs& a, int64_t node) {
  if (!a.chunk_mask) return true;
  const int64_t c = a.node_chunk ? __ldg(a.node_chunk + node) : 0;
  return c >= 0 && c < a.num_chunks && __ldg(a.chunk_mask + c) != 0;
}

// Walks the window of one node 32 edges at a time.  f(e, pos_in_node, is_head, group_in_node) is called for every kept
// edge by its lane.  Returns (edges, groups) kept, identical in all lanes.
template <typename F>
__device__ __forceinline__ void walk_node(const SliceArgs& a, int64_t node, int lane, int64_t* n_edges, int64_t* n_groups,
                                          F f) {
  int64_t ce = 0, cg = 0;
  if (chunk_selected(a, node)) {
    const int64_t rs = __ldg(a.indptr + node), re = __ldg(a.indptr + node + 1);
    if (re > rs) {
      const int64_t lo = lower_bound_i64(a.ts, rs, re, a.t_begin);
      const int64_t hi = lower_bound_i64(a.ts, lo, re, a.t_end);
      bool have_prev = false;
      int64_t prev_ts = 0;
      const uint32_t lt = (1u << lane) - 1u;
      for (int64_t base = lo; base < hi; base += 32) {
        const int64_t e = base + lane;
        int64_t t = 0;
        bool keep = false;
        if (e < hi) {
          t = __ldg(a.ts + e);
          const int64_t v = __ldg(a.nbr + e);
          keep = v >= 0 && v < a.num_nodes && chunk_selected(a, v);
        }
        const uint32_t kept = __ballot_sync(0xffffffffu, keep);
        // timestamp of the kept edge just before this lane (inside the 32, else the last one of earlier rounds)
        const uint32_t before = kept & lt;
        const int src_lane = before ? 31 - __clz(before) : 0;
        const int64_t t_before = __shfl_sync(0xffffffffu, t, src_lane);
        const bool head = keep && (before ? t_before != t : (!have_prev || prev_ts != t));
        const uint32_t heads = __ballot_sync(0xffffffffu, head);
        if (keep) f(e, ce + __popc(before), head, cg + __popc(heads & lt) - (head ? 0 : 1));
        if (kept) {
          prev_ts = __shfl_sync(0xffffffffu, t, 31 - __clz(kept));
          have_prev = true;
        }
        ce += __popc(kept);
        cg += __popc(heads);
      }
    }
  }
  *n_edges = ce;
  *n_groups = cg;
}

__global__ void __launch_bounds__(kThreads)
slice_count_kernel(SliceArgs a, uint32_t* __restrict__ cnt_edges, uint32_t* __restrict__ cnt_groups, int32_t* d_status) {
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t node = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5; node < a.num_nodes; node += n_warps) {
    int64_t ce, cg;
    walk_node(a, node, lane, &ce, &cg, [](int64_t, int64_t, bool, int64_t) {});
    if (lane == 0) {
      if (ce > 0xffffffffll) {
        dev_flag(d_status, SGL_DEV_OVERFLOW);
        ce = cg = 0;
      }
      cnt_edges[node] = (uint32_t)ce;
      cnt_groups[node] = (uint32_t)cg;
    }
  }
}

// thread per node; three exclusive scans (kept nodes, groups, edges): CTA-local offsets + scanned CTA totals
__global__ void __launch_bounds__(kThreads)
slice_scan_kernel(const uint32_t* __restrict__ cnt_edges, const uint32_t* __restrict__ cnt_groups, int64_t num_nodes,
                  uint32_t* __restrict__ loc_node, uint32_t* __restrict__ loc_group, uint32_t* __restrict__ loc_edge,
                  int64_t* __restrict__ cta_nodes, int64_t* __restrict__ cta_groups, int64_t* __restrict__ cta_edges,
                  unsigned int* done, int64_t* d_counts) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t ce = i < num_nodes ? cnt_edges[i] : 0, cg = i < num_nodes ? cnt_groups[i] : 0;
  int64_t tn, tg, te;
  const int64_t on = cta_exclusive_scan<kThreads, int64_t>(ce > 0 ? 1 : 0, &tn);
  const int64_t og = cta_exclusive_scan<kThreads, int64_t>(cg, &tg);
  const int64_t oe = cta_exclusive_scan<kThreads, int64_t>(ce, &te);
  if (i < num_nodes) {
    loc_node[i] = (uint32_t)on;
    loc_group[i] = (uint32_t)og;
    loc_edge[i] = (uint32_t)oe;
  }
  publish_and_scan_cta_totals<kThreads>(tn, cta_nodes, done + 0, d_counts + 0);
  __syncthreads();
  publish_and_scan_cta_totals<kThreads>(tg, cta_groups, done + 1, d_counts + 1);
  __syncthreads();
  publish_and_scan_cta_totals<kThreads>(te, cta_edges, done + 2, d_counts + 2);
}

__global__ void __launch_bounds__(kThreads)
slice_write_kernel(SliceArgs a, const int64_t* __restrict__ eid, const uint32_t* __restrict__ cnt_edges,
                   const uint32_t* __restrict__ loc_node, const uint32_t* __restrict__ loc_group,
                   const uint32_t* __restrict__ loc_edge, const int64_t* __restrict__ cta_nodes,
                   const int64_t* __restrict__ cta_groups, const int64_t* __restrict__ cta_edges, const int64_t* d_counts,
                   int64_t cap_edges, int64_t* __restrict__ out_nodes, int64_t* __restrict__ out_node_ptr,
                   int64_t* __restrict__ out_group_ts, int64_t* __restrict__ out_group_ptr, int64_t* __restrict__ out_nbr,
                   int64_t* __restrict__ out_ts, int64_t* __restrict__ out_eid, int32_t* d_status) {
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  const int64_t total_edges = d_counts[2];
  if (total_edges > cap_edges) {   // nothing is written beyond the caller's capacity
    if (blockIdx.x == 0 && threadIdx.x == 0) dev_flag(d_status, SGL_DEV_OVERFLOW);
    return;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    out_node_ptr[d_counts[0]] = d_counts[1];
    out_group_ptr[d_counts[1]] = total_edges;
  }
  for (int64_t node = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5; node < a.num_nodes; node += n_warps) {
    if (cnt_edges[node] == 0) continue;
    const int64_t cta = node / kThreads;
    const int64_t u = cta_nodes[cta] + loc_node[node];
    const int64_t g0 = cta_groups[cta] + loc_group[node];
    const int64_t e0 = cta_edges[cta] + loc_edge[node];
    if (lane == 0) {
      out_nodes[u] = node;
      out_node_ptr[u] = g0;
    }
    int64_t ce, cg;
    walk_node(a, node, lane, &ce, &cg, [&](int64_t e, int64_t pos, bool head, int64_t group) {
      out_nbr[e0 + pos] = __ldg(a.nbr + e);
      out_ts[e0 + pos] = __ldg(a.ts + e);
      out_eid[e0 + pos] = eid ? __ldg(eid + e) : e;
      if (head) {
        out_group_ts[g0 + group] = __ldg(a.ts + e);
        out_group_ptr[g0 + group] = e0 + pos;
      }
    });
  }
}

// Dense per-time-step groups out of the sparse ones: node u of the sparse form owns the groups
// [node_ptr[u], node_ptr[u+1]) with ascending timestamps group_ts and edge ranges group_ptr; the dense form gives every
// node ALL time steps t_begin .. t_end-1 (T = t_end - t_begin groups per node, empty where the node has no event).
// One thread per (node, time step): the first sparse group of the node with timestamp >= t by binary search.
__global__ void __launch_bounds__(kThreads)
densify_groups_kernel(const int64_t* __restrict__ node_ptr, const int64_t* __restrict__ group_ts,
                      const int64_t* __restrict__ group_ptr, int64_t u_cap, const int64_t* d_u, int64_t t_begin, int64_t T,
                      int64_t* __restrict__ out_node_ptr, int64_t* __restrict__ out_ts, int64_t* __restrict__ out_group_ptr) {
  const int64_t U = eff_count(u_cap, d_u);
  const int64_t total = U * T;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x; q <= total; q += stride) {
    if (q == total) {                       // closing entries
      out_group_ptr[total] = U ? group_ptr[node_ptr[U]] : 0;
      out_node_ptr[U] = total;
      break;
    }
    const int64_t u = q / T, t = t_begin + (q - u * T);
    int64_t lo = node_ptr[u], hi = node_ptr[u + 1];
    const int64_t end = hi;
    while (lo < hi) {
      const int64_t mid = lo + ((hi - lo) >> 1);
      if (group_ts[mid] < t) lo = mid + 1; else hi = mid;
    }
    out_ts[q] = t;
    out_group_ptr[q] = group_ptr[lo];       // lo == end: the start of the next node's edges = the end of this node's
    (void)end;
    if (q == u * T) out_node_ptr[u] = q;
  }
}

inline unsigned ctas_for(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads < 1 ? 1 : (n + kThreads - 1) / kThreads); }

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" size_t sgl_slice_window_ws_bytes(int64_t num_nodes) {
  const int64_t n = num_nodes < 1 ? 1 : num_nodes;
  return 5 * align_up((size_t)n * 4) + 3 * align_up((size_t)ctas_for(n) * 8) + align_up(16);
}

extern "C" int sgl_slice_window(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                                int64_t num_nodes, const int64_t* node_chunk, const uint8_t* chunk_mask, int64_t num_chunks,
                                int64_t t_begin, int64_t t_end, int64_t cap_edges, int64_t* out_nodes, int64_t* out_node_ptr,
                                int64_t* out_group_ts, int64_t* out_group_ptr, int64_t* out_nbr, int64_t* out_ts,
                                int64_t* out_eid, int64_t* d_counts, int32_t* d_status, void* ws, size_t ws_bytes,
                                void* stream_) {
  SGL_NVTX("sgl_slice_window");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(num_nodes >= 0 && cap_edges >= 0 && num_chunks >= 0, SGL_ERR_ARG, "slice_window: negative size");
  SGL_REQUIRE(d_counts && out_node_ptr && out_group_ptr, SGL_ERR_ARG, "slice_window: null counter / pointer array");
  SGL_REQUIRE(chunk_mask == nullptr || num_chunks > 0, SGL_ERR_ARG, "slice_window: a chunk mask needs num_chunks > 0");
  if (num_nodes == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(d_counts, 0, 3 * sizeof(int64_t), stream));
    SGL_CUDA_CHECK(cudaMemsetAsync(out_node_ptr, 0, sizeof(int64_t), stream));
    SGL_CUDA_CHECK(cudaMemsetAsync(out_group_ptr, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE(indptr && nbr && ts && out_nodes && out_group_ts && out_nbr && out_ts && out_eid, SGL_ERR_ARG,
              "slice_window: null array");
  WsCarver c(ws, ws_bytes);
  uint32_t* cnt_edges = c.take<uint32_t>(num_nodes);
  uint32_t* cnt_groups = c.take<uint32_t>(num_nodes);
  uint32_t* loc_node = c.take<uint32_t>(num_nodes);
  uint32_t* loc_group = c.take<uint32_t>(num_nodes);
  uint32_t* loc_edge = c.take<uint32_t>(num_nodes);
  int64_t* cta_nodes = c.take<int64_t>(ctas_for(num_nodes));
  int64_t* cta_groups = c.take<int64_t>(ctas_for(num_nodes));
  int64_t* cta_edges = c.take<int64_t>(ctas_for(num_nodes));
  unsigned int* done = c.take<unsigned int>(4);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "slice_window: workspace %zu < %zu bytes", ws_bytes, sgl_slice_window_ws_bytes(num_nodes));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, 16, stream));
  SliceArgs a{indptr, nbr, ts, node_chunk, chunk_mask, num_nodes, num_chunks, t_begin, t_end};
  const int grid = stream_grid(num_nodes, kThreads / 32, 16);
  slice_count_kernel<<<grid, kThreads, 0, stream>>>(a, cnt_edges, cnt_groups, d_status);
  slice_scan_kernel<<<ctas_for(num_nodes), kThreads, 0, stream>>>(cnt_edges, cnt_groups, num_nodes, loc_node, loc_group, loc_edge,
                                                                 cta_nodes, cta_groups, cta_edges, done, d_counts);
  slice_write_kernel<<<grid, kThreads, 0, stream>>>(a, eid, cnt_edges, loc_node, loc_group, loc_edge, cta_nodes, cta_groups,
                                                    cta_edges, d_counts, cap_edges, out_nodes, out_node_ptr, out_group_ts,
                                                    out_group_ptr, out_nbr, out_ts, out_eid, d_status);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_densify_time_groups(const int64_t* node_ptr, const int64_t* group_ts, const int64_t* group_ptr, int64_t n_nodes,
                                       const int64_t* d_n_nodes, int64_t t_begin, int64_t t_end, int64_t* out_node_ptr,
                                       int64_t* out_ts, int64_t* out_group_ptr, void* stream_) {
  SGL_REQUIRE(n_nodes >= 0 && t_end >= t_begin, SGL_ERR_ARG, "densify_time_groups: bad size");
  SGL_REQUIRE(out_node_ptr && out_group_ptr, SGL_ERR_ARG, "densify_time_groups: null output");
  const int64_t T = t_end - t_begin;
  SGL_REQUIRE(T == 0 || n_nodes <= (((int64_t)1 << 40) / T), SGL_ERR_UNSUPPORTED,
              "densify_time_groups: %lld nodes x %lld time steps is too large for dense groups", (long long)n_nodes, (long long)T);
  SGL_REQUIRE(n_nodes == 0 || (node_ptr && group_ptr && (T == 0 || (group_ts && out_ts))), SGL_ERR_ARG,
              "densify_time_groups: null array");
  densify_groups_kernel<<<stream_grid(n_nodes * T + 1, kThreads, 16), kThreads, 0, (cudaStream_t)stream_>>>(
      node_ptr, group_ts, group_ptr, n_nodes, d_n_nodes, t_begin, T, out_node_ptr, out_ts, out_group_ptr);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}
