// Dedup / relabel kernels of the mini-batch builder.  Everything is sort based so that local ids come out in
// the deterministic order the CPU builder produces (sorted unique), not in hash-table order:
//
//   pack -> stable radix sort (key = (id << ts_bits) | (ts - ts_base), payload = input position)
//        -> head flags + scan (CTA scan, last CTA scans the CTA totals) -> emit unique list and inverse map.
//
// Algorithmic HBM bytes: 16 read + 8 write per input pair, 16 per unique pair, plus the sort passes
// (32 B per pair and populated key byte).
#include "heads.cuh"
#include "sort.cuh"

namespace sgl {
namespace {

constexpr int kThreads = kHeadsThreads;

// ---- unique (id, ts) pairs -----------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
pairs_pack_kernel(const int64_t* __restrict__ a_id, const int64_t* __restrict__ a_ts, int64_t n_a, const int64_t* d_n_a,
                  const int64_t* __restrict__ b_id, const int64_t* __restrict__ b_ts, int64_t n_b, const int64_t* d_n_b,
                  int id_bits, int ts_bits, int64_t ts_base, uint64_t* __restrict__ keys, int64_t* d_total,
                  int32_t* d_status) {
  const int64_t na = eff_count(n_a, d_n_a), nb = eff_count(n_b, d_n_b);
  const int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (q == 0) *d_total = na + nb;
  int64_t id, t, pos;
  if (q < n_a) {
    if (q >= na) return;
    id = a_id[q]; t = a_ts[q]; pos = q;
  } else {
    int64_t qb = q - n_a;
    if (qb >= nb) return;
    id = b_id[qb]; t = b_ts[qb]; pos = na + qb;
  }
  uint64_t dt = (uint64_t)t - (uint64_t)ts_base;
  if (id < 0 || ((uint64_t)id & ~low_mask(id_bits))) { dev_flag(d_status, SGL_DEV_BAD_NODE); id = 0; }
  if (t < ts_base || (dt & ~low_mask(ts_bits))) { dev_flag(d_status, SGL_DEV_BAD_TS); dt = 0; }
  keys[pos] = ts_bits >= 64 ? dt : (((uint64_t)id << ts_bits) | dt);
}

__global__ void __launch_bounds__(kThreads)
pairs_emit_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ perm, const int64_t* d_total,
                  int64_t n_cap, const uint32_t* __restrict__ packed, const int64_t* __restrict__ cta_base, int ts_bits,
                  int64_t ts_base, int64_t n_a, const int64_t* d_n_a, int64_t* __restrict__ out_id,
                  int64_t* __restrict__ out_ts, int64_t* __restrict__ inv_a, int64_t* __restrict__ inv_b) {
  const int64_t n = eff_count(n_cap, d_total);
  const int64_t na = eff_count(n_a, d_n_a);
  const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (j >= n) return;
  uint32_t pk = packed[j];
  int64_t u = cta_base[blockIdx.x] + (pk >> 1) + (pk & 1) - 1;  // index of this key's pair in the unique list
  uint64_t k = keys[j];
  if (pk & 1) {
    out_id[u] = ts_bits >= 64 ? 0 : (int64_t)(k >> ts_bits);
    out_ts[u] = (int64_t)(k & low_mask(ts_bits)) + ts_base;
  }
  int64_t src = perm[j];
  if (src < na) {
    if (inv_a) inv_a[src] = u;
  } else if (inv_b) {
    inv_b[src - na] = u;
  }
}

// ---- CSC of one hop -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
csc_pack_kernel(const int64_t* __restrict__ dst, const int64_t* __restrict__ dst_map, const int64_t* __restrict__ ts,
                int64_t n_cap, const int64_t* d_n, int dst_bits, int ts_bits, int64_t ts_base,
                uint64_t* __restrict__ keys, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (e >= n) return;
  int64_t d = dst[e];
  if (dst_map) d = dst_map[d];
  int64_t t = ts[e];
  uint64_t dt = (uint64_t)t - (uint64_t)ts_base;
  if (d < 0 || ((uint64_t)d & ~low_mask(dst_bits))) { dev_flag(d_status, SGL_DEV_BAD_NODE); d = 0; }
  if (t < ts_base || (dt & ~low_mask(ts_bits))) { dev_flag(d_status, SGL_DEV_BAD_TS); dt = 0; }
  keys[e] = ts_bits >= 64 ? dt : (((uint64_t)d << ts_bits) | dt);
}

__global__ void __launch_bounds__(kThreads)
csc_emit_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ perm, int64_t n_cap, const int64_t* d_n,
                int64_t num_dst_cap, const int64_t* d_num_dst, int ts_bits, const int64_t* __restrict__ src_local,
                const int64_t* __restrict__ ts, const float* __restrict__ dt, const int64_t* __restrict__ eid,
                int64_t* __restrict__ indptr, int64_t* __restrict__ out_indices, int64_t* __restrict__ out_ts,
                float* __restrict__ out_dt, int64_t* __restrict__ out_eid) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t num_dst = eff_count(num_dst_cap, d_num_dst);
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  if (n == 0) {
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v <= num_dst; v += stride) indptr[v] = 0;
    return;
  }
  for (int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x; j < n; j += stride) {
    uint32_t p = perm[j];
    out_indices[j] = src_local[p];
    out_ts[j] = ts[p];
    out_dt[j] = dt[p];
    out_eid[j] = eid[p];
    int64_t d = ts_bits >= 64 ? 0 : (int64_t)(keys[j] >> ts_bits);
    int64_t prev = j == 0 ? -1 : (ts_bits >= 64 ? 0 : (int64_t)(keys[j - 1] >> ts_bits));
    for (int64_t v = prev + 1; v <= d && v <= num_dst; ++v) indptr[v] = j;
    if (j == n - 1)
      for (int64_t v = d + 1; v <= num_dst; ++v) indptr[v] = n;
  }
}

// The same for edges that already are in (dst, ts) order -- the first hop of a batch, whose targets are the layer list
// itself: target i is row i, and a target's samples come out in ascending time.  No sort: a copy plus the row pointer.
__global__ void __launch_bounds__(kThreads)
csc_emit_sorted_kernel(const int64_t* __restrict__ dst, int64_t n_cap, const int64_t* d_n, int64_t num_dst_cap,
                       const int64_t* d_num_dst, const int64_t* __restrict__ src_local, const int64_t* __restrict__ ts,
                       const float* __restrict__ dt, const int64_t* __restrict__ eid, int64_t* __restrict__ indptr,
                       int64_t* __restrict__ out_indices, int64_t* __restrict__ out_ts, float* __restrict__ out_dt,
                       int64_t* __restrict__ out_eid, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t num_dst = eff_count(num_dst_cap, d_num_dst);
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  if (n == 0) {
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v <= num_dst; v += stride) indptr[v] = 0;
    return;
  }
  for (int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x; j < n; j += stride) {
    out_indices[j] = src_local[j];
    out_ts[j] = ts[j];
    out_dt[j] = dt[j];
    out_eid[j] = eid[j];
    const int64_t d = dst[j];
    const int64_t prev = j == 0 ? -1 : dst[j - 1];
    if (d < prev || d < 0 || (d == prev && ts[j] < ts[j - 1])) dev_flag(d_status, SGL_DEV_BAD_INDEX);   // not in (dst, ts) order
    for (int64_t v = prev + 1; v <= d && v <= num_dst; ++v) indptr[v] = j;
    if (j == n - 1)
      for (int64_t v = d + 1; v <= num_dst; ++v) indptr[v] = n;
  }
}

// ---- node-level relabel ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
nodes_pack_kernel(const int64_t* __restrict__ ids, int64_t n_cap, const int64_t* d_n, int64_t num_nodes,
                  const int64_t* __restrict__ mask, int64_t epoch, int id_bits, uint64_t* __restrict__ keys,
                  int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  int64_t g = ids[i];
  uint64_t k = 1ull << id_bits;  // "already known" and invalid ids sort behind every new id
  if (g < 0 || g >= num_nodes) dev_flag(d_status, SGL_DEV_BAD_NODE);
  else if (mask[g] != epoch) k = (uint64_t)g;
  keys[i] = k;
}

__global__ void __launch_bounds__(kThreads)
nodes_assign_kernel(const uint64_t* __restrict__ keys, int64_t n_cap, const int64_t* d_n, int id_bits,
                    const uint32_t* __restrict__ packed, const int64_t* __restrict__ cta_base,
                    const int64_t* d_next_local, int64_t* __restrict__ mapper, int64_t* __restrict__ mask, int64_t epoch,
                    int64_t* __restrict__ out_new_ids) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (j >= n) return;
  uint32_t pk = packed[j];
  if (!(pk & 1)) return;
  int64_t rank = cta_base[blockIdx.x] + (pk >> 1);
  int64_t g = (int64_t)keys[j];
  mapper[g] = *d_next_local + rank;
  mask[g] = epoch;
  out_new_ids[rank] = g;
}

__global__ void __launch_bounds__(kThreads)
nodes_lookup_kernel(const int64_t* __restrict__ ids, int64_t n_cap, const int64_t* d_n, int64_t num_nodes,
                    const int64_t* __restrict__ mapper, int64_t* __restrict__ out_local, int64_t* d_next_local,
                    const int64_t* d_n_new) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < n) {
    int64_t g = ids[i];
    out_local[i] = (g >= 0 && g < num_nodes) ? mapper[g] : -1;
  }
}

__global__ void nodes_advance_kernel(int64_t* d_next_local, const int64_t* d_n_new) { *d_next_local += *d_n_new; }

// ---- roots of a time window ----------------------------------------------------------------------------------
// events of the window whose source node lies in a selected chunk get key (src << ts_bits) | (ts - base); the others
// a sentinel above every real key, so that after the sort the selected events form a prefix grouped by (src, ts)
__global__ void __launch_bounds__(kThreads)
seeds_pack_kernel(const int64_t* __restrict__ ev_src, const int64_t* __restrict__ ev_ts, int64_t n,
                  const int64_t* __restrict__ node_chunk, const uint8_t* __restrict__ chunk_mask, int64_t num_chunks,
                  int64_t num_nodes, int id_bits, int ts_bits, int64_t ts_base, uint64_t* __restrict__ keys,
                  int32_t* d_status) {
  const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (j >= n) return;
  const uint64_t sentinel = 1ull << (id_bits + ts_bits);
  int64_t s = ev_src[j], t = ev_ts[j];
  uint64_t dt = (uint64_t)t - (uint64_t)ts_base;
  uint64_t k = sentinel;
  if (s < 0 || s >= num_nodes) dev_flag(d_status, SGL_DEV_BAD_NODE);
  else if (t < ts_base || (dt & ~low_mask(ts_bits))) dev_flag(d_status, SGL_DEV_BAD_TS);
  else {
    bool take = true;
    if (chunk_mask) {
      int64_t c = node_chunk ? node_chunk[s] : 0;
      take = c >= 0 && c < num_chunks && chunk_mask[c];
    }
    if (take) k = ((uint64_t)s << ts_bits) | dt;
  }
  keys[j] = k;
}

__global__ void __launch_bounds__(kThreads)
seeds_emit_pairs_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ perm, int64_t n, int key_bits,
                        int ts_bits, int64_t ts_base, const int64_t* __restrict__ ev_eid,
                        const uint32_t* __restrict__ packed, const int64_t* __restrict__ cta_base,
                        int64_t* __restrict__ pair_node, int64_t* __restrict__ out_ts, int64_t* __restrict__ out_q_ptr,
                        int64_t* __restrict__ out_q_eid, int64_t* d_counts) {
  const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (j >= n) return;
  const uint64_t k = keys[j];
  const bool valid = (k >> key_bits) == 0;
  if (!valid) {
    if (j == 0) {  // no selected event at all
      out_q_ptr[0] = 0;
      d_counts[2] = 0;
    }
    return;
  }
  out_q_eid[j] = ev_eid[perm[j]];
  const uint32_t pk = packed[j];
  if (pk & 1) {
    int64_t p = cta_base[blockIdx.x] + (pk >> 1);
    pair_node[p] = (int64_t)(k >> ts_bits);
    out_ts[p] = (int64_t)(k & low_mask(ts_bits)) + ts_base;
    out_q_ptr[p] = j;
  }
  if (j == n - 1 || (keys[j + 1] >> key_bits) != 0) {  // last selected event closes the prefix arrays
    out_q_ptr[d_counts[1]] = j + 1;
    d_counts[2] = j + 1;
  }
}

__global__ void __launch_bounds__(kThreads)
seeds_emit_roots_kernel(const int64_t* __restrict__ pair_node, int64_t n_cap, const int64_t* d_counts,
                        const uint32_t* __restrict__ packed, const int64_t* __restrict__ cta_base,
                        int64_t* __restrict__ out_roots, int64_t* __restrict__ out_ts_ptr) {
  const int64_t n = eff_count(n_cap, d_counts + 1);
  const int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (n == 0) {
    if (p == 0) out_ts_ptr[0] = 0;
    return;
  }
  if (p >= n) return;
  const uint32_t pk = packed[p];
  if (pk & 1) {
    int64_t r = cta_base[blockIdx.x] + (pk >> 1);
    out_roots[r] = pair_node[p];
    out_ts_ptr[r] = p;
  }
  if (p == n - 1) out_ts_ptr[d_counts[0]] = n;
}

// first position with sorted[pos] >= value, one thread per value
__global__ void lower_bound_kernel(const int64_t* __restrict__ sorted, int64_t n, const int64_t* __restrict__ values,
                                   int k, int64_t* __restrict__ out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= k) return;
  int64_t v = values[i], lo = 0, hi = n;
  while (lo < hi) {
    int64_t mid = lo + ((hi - lo) >> 1);
    if (sorted[mid] < v) lo = mid + 1; else hi = mid;
  }
  out[i] = lo;
}

inline unsigned ctas_for(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads < 1 ? 1 : (n + kThreads - 1) / kThreads); }

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" size_t sgl_unique_pairs_ws_bytes(int64_t n_total) {
  if (n_total < 1) n_total = 1;
  return 2 * align_up((size_t)n_total * 8) + 3 * align_up((size_t)n_total * 4) + align_up((size_t)ctas_for(n_total) * 8) +
         2 * align_up(8) + radix_sort_ws_bytes(n_total);
}

extern "C" int sgl_unique_pairs(const int64_t* a_id, const int64_t* a_ts, int64_t n_a, const int64_t* d_n_a,
                                const int64_t* b_id, const int64_t* b_ts, int64_t n_b, const int64_t* d_n_b, int id_bits,
                                int ts_bits, int64_t ts_base, int64_t* out_id, int64_t* out_ts, int64_t* inv_a,
                                int64_t* inv_b, int64_t* d_n_unique, int32_t* d_status, void* ws, size_t ws_bytes,
                                void* stream_) {
  SGL_NVTX("sgl_unique_pairs");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n_a >= 0 && n_b >= 0, SGL_ERR_ARG, "unique_pairs: negative size");
  SGL_REQUIRE(id_bits >= 0 && ts_bits >= 0 && id_bits + ts_bits <= 64, SGL_ERR_UNSUPPORTED,
              "unique_pairs: id_bits %d + ts_bits %d exceed the 64-bit sort key", id_bits, ts_bits);
  SGL_REQUIRE(d_n_unique, SGL_ERR_ARG, "unique_pairs: d_n_unique is null");
  const int64_t n = n_a + n_b;
  if (n == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(d_n_unique, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE((n_a == 0 || (a_id && a_ts)) && (n_b == 0 || (b_id && b_ts)) && out_id && out_ts, SGL_ERR_ARG,
              "unique_pairs: null array");
  WsCarver c(ws, ws_bytes);
  uint64_t* k0 = c.take<uint64_t>(n);
  uint64_t* k1 = c.take<uint64_t>(n);
  uint32_t* v0 = c.take<uint32_t>(n);
  uint32_t* v1 = c.take<uint32_t>(n);
  uint32_t* packed = c.take<uint32_t>(n);
  int64_t* cta_sums = c.take<int64_t>(ctas_for(n));
  int64_t* d_total = c.take<int64_t>(1);
  unsigned int* done = c.take<unsigned int>(1);
  size_t sort_bytes = radix_sort_ws_bytes(n);
  char* sort_ws = c.take<char>(sort_bytes);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "unique_pairs: workspace %zu < %zu bytes", ws_bytes, sgl_unique_pairs_ws_bytes(n));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
  pairs_pack_kernel<<<ctas_for(n), kThreads, 0, stream>>>(a_id, a_ts, n_a, d_n_a, b_id, b_ts, n_b, d_n_b, id_bits, ts_bits,
                                                          ts_base, k0, d_total, d_status);
  SGL_LAUNCH_CHECK();
  int in_alt = 0;
  int rc = radix_sort_pairs(k0, v0, k1, v1, n, d_total, id_bits + ts_bits, true, &in_alt, sort_ws, sort_bytes, stream);
  if (rc) return rc;
  const uint64_t* ks = in_alt ? k1 : k0;
  const uint32_t* vs = in_alt ? v1 : v0;
  heads_scan_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, n, d_total, 64, packed, cta_sums, done, d_n_unique);
  pairs_emit_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, vs, d_total, n, packed, cta_sums, ts_bits, ts_base, n_a,
                                                          d_n_a, out_id, out_ts, inv_a, inv_b);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" size_t sgl_build_csc_ws_bytes(int64_t n_edges, int64_t num_dst) {
  (void)num_dst;
  if (n_edges < 1) n_edges = 1;
  return 2 * align_up((size_t)n_edges * 8) + 2 * align_up((size_t)n_edges * 4) + radix_sort_ws_bytes(n_edges);
}

extern "C" int sgl_build_csc(const int64_t* src_local, const int64_t* dst, const int64_t* dst_map, const int64_t* ts,
                             const float* dt, const int64_t* eid, int64_t n_edges, const int64_t* d_n_edges,
                             int64_t num_dst, const int64_t* d_num_dst, int dst_bits, int ts_bits, int64_t ts_base,
                             int64_t* out_indptr, int64_t* out_indices, int64_t* out_ts, float* out_dt, int64_t* out_eid,
                             int presorted, int32_t* d_status, void* ws, size_t ws_bytes, void* stream_) {
  SGL_NVTX("sgl_build_csc");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n_edges >= 0 && num_dst >= 0, SGL_ERR_ARG, "build_csc: negative size");
  if (presorted) {
    SGL_REQUIRE(dst_map == nullptr, SGL_ERR_ARG, "build_csc: presorted input cannot go through a dst_map");
    SGL_REQUIRE(out_indptr, SGL_ERR_ARG, "build_csc: out_indptr is null");
    SGL_REQUIRE(n_edges == 0 || (src_local && dst && ts && dt && eid && out_indices && out_ts && out_dt && out_eid), SGL_ERR_ARG,
                "build_csc: null array");
    const int64_t work_s = n_edges > num_dst + 1 ? n_edges : num_dst + 1;
    csc_emit_sorted_kernel<<<stream_grid(work_s, kThreads, 16), kThreads, 0, stream>>>(
        dst, n_edges, d_n_edges, num_dst, d_num_dst, src_local, ts, dt, eid, out_indptr, out_indices, out_ts, out_dt, out_eid,
        d_status);
    SGL_LAUNCH_CHECK();
    return SGL_OK;
  }
  SGL_REQUIRE(dst_bits >= 0 && ts_bits >= 0 && dst_bits + ts_bits <= 64, SGL_ERR_UNSUPPORTED,
              "build_csc: dst_bits %d + ts_bits %d exceed the 64-bit sort key", dst_bits, ts_bits);
  SGL_REQUIRE(out_indptr, SGL_ERR_ARG, "build_csc: out_indptr is null");
  const int64_t cap = n_edges < 1 ? 1 : n_edges;
  WsCarver c(ws, ws_bytes);
  uint64_t* k0 = c.take<uint64_t>(cap);
  uint64_t* k1 = c.take<uint64_t>(cap);
  uint32_t* v0 = c.take<uint32_t>(cap);
  uint32_t* v1 = c.take<uint32_t>(cap);
  size_t sort_bytes = radix_sort_ws_bytes(cap);
  char* sort_ws = c.take<char>(sort_bytes);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "build_csc: workspace %zu < %zu bytes", ws_bytes,
              sgl_build_csc_ws_bytes(n_edges, num_dst));
  int in_alt = 0;
  if (n_edges > 0) {
    SGL_REQUIRE(src_local && dst && ts && dt && eid && out_indices && out_ts && out_dt && out_eid, SGL_ERR_ARG,
                "build_csc: null array");
    csc_pack_kernel<<<ctas_for(n_edges), kThreads, 0, stream>>>(dst, dst_map, ts, n_edges, d_n_edges, dst_bits, ts_bits,
                                                               ts_base, k0, d_status);
    SGL_LAUNCH_CHECK();
    int rc = radix_sort_pairs(k0, v0, k1, v1, n_edges, d_n_edges, dst_bits + ts_bits, true, &in_alt, sort_ws, sort_bytes,
                              stream);
    if (rc) return rc;
  }
  int64_t work = n_edges > num_dst + 1 ? n_edges : num_dst + 1;
  csc_emit_kernel<<<stream_grid(work, kThreads, 16), kThreads, 0, stream>>>(
      in_alt ? k1 : k0, in_alt ? v1 : v0, n_edges, d_n_edges, num_dst, d_num_dst, ts_bits, src_local, ts, dt, eid,
      out_indptr, out_indices, out_ts, out_dt, out_eid);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" size_t sgl_relabel_nodes_ws_bytes(int64_t n) {
  if (n < 1) n = 1;
  return 2 * align_up((size_t)n * 8) + 3 * align_up((size_t)n * 4) + align_up((size_t)ctas_for(n) * 8) + align_up(8) +
         radix_sort_ws_bytes(n);
}

extern "C" int sgl_relabel_nodes(const int64_t* ids, int64_t n, const int64_t* d_n, int64_t num_nodes, int64_t* mapper,
                                 int64_t* mask, int64_t epoch, int64_t* d_next_local, int64_t* out_local,
                                 int64_t* out_new_ids, int64_t* d_n_new, int32_t* d_status, void* ws, size_t ws_bytes,
                                 void* stream_) {
  SGL_NVTX("sgl_relabel_nodes");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && num_nodes >= 0, SGL_ERR_ARG, "relabel_nodes: negative size");
  SGL_REQUIRE(d_next_local && d_n_new, SGL_ERR_ARG, "relabel_nodes: null counter");
  if (n == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(d_n_new, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE(ids && mapper && mask && out_local && out_new_ids, SGL_ERR_ARG, "relabel_nodes: null array");
  const int id_bits = bits_for(num_nodes > 0 ? (uint64_t)(num_nodes - 1) : 0);
  SGL_REQUIRE(id_bits < 63, SGL_ERR_UNSUPPORTED, "relabel_nodes: num_nodes too large");
  WsCarver c(ws, ws_bytes);
  uint64_t* k0 = c.take<uint64_t>(n);
  uint64_t* k1 = c.take<uint64_t>(n);
  uint32_t* v0 = c.take<uint32_t>(n);
  uint32_t* v1 = c.take<uint32_t>(n);
  uint32_t* packed = c.take<uint32_t>(n);
  int64_t* cta_sums = c.take<int64_t>(ctas_for(n));
  unsigned int* done = c.take<unsigned int>(1);
  size_t sort_bytes = radix_sort_ws_bytes(n);
  char* sort_ws = c.take<char>(sort_bytes);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "relabel_nodes: workspace %zu < %zu bytes", ws_bytes, sgl_relabel_nodes_ws_bytes(n));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
  nodes_pack_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ids, n, d_n, num_nodes, mask, epoch, id_bits, k0, d_status);
  SGL_LAUNCH_CHECK();
  int in_alt = 0;
  int rc = radix_sort_pairs(k0, v0, k1, v1, n, d_n, id_bits + 1, true, &in_alt, sort_ws, sort_bytes, stream);
  if (rc) return rc;
  const uint64_t* ks = in_alt ? k1 : k0;
  heads_scan_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, n, d_n, id_bits, packed, cta_sums, done, d_n_new);
  nodes_assign_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, n, d_n, id_bits, packed, cta_sums, d_next_local, mapper,
                                                           mask, epoch, out_new_ids);
  nodes_lookup_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ids, n, d_n, num_nodes, mapper, out_local, d_next_local, d_n_new);
  nodes_advance_kernel<<<1, 1, 0, stream>>>(d_next_local, d_n_new);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_lower_bound_i64(const int64_t* sorted, int64_t n, const int64_t* values, int k, int64_t* out,
                                   void* stream_) {
  SGL_REQUIRE(n >= 0 && k >= 0, SGL_ERR_ARG, "lower_bound: negative size");
  if (k == 0) return SGL_OK;
  SGL_REQUIRE((n == 0 || sorted) && values && out, SGL_ERR_ARG, "lower_bound: null array");
  lower_bound_kernel<<<(k + 127) / 128, 128, 0, (cudaStream_t)stream_>>>(sorted, n, values, k, out);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" size_t sgl_seeds_ws_bytes(int64_t n_events) {
  if (n_events < 1) n_events = 1;
  return 2 * align_up((size_t)n_events * 8) + 3 * align_up((size_t)n_events * 4) + align_up((size_t)n_events * 8) +
         align_up((size_t)ctas_for(n_events) * 8) + align_up(8) + radix_sort_ws_bytes(n_events);
}

extern "C" int sgl_seeds_in_window(const int64_t* ev_src, const int64_t* ev_ts, const int64_t* ev_eid, int64_t n_events,
                                   const int64_t* node_chunk, const uint8_t* chunk_mask, int64_t num_chunks,
                                   int64_t num_nodes, int id_bits, int ts_bits, int64_t ts_base, int64_t* out_roots,
                                   int64_t* out_ts_ptr, int64_t* out_ts, int64_t* out_q_ptr, int64_t* out_q_eid,
                                   int64_t* d_counts, int32_t* d_status, void* ws, size_t ws_bytes, void* stream_) {
  SGL_NVTX("sgl_seeds_in_window");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n_events >= 0 && num_nodes >= 0, SGL_ERR_ARG, "seeds_in_window: negative size");
  SGL_REQUIRE(id_bits >= 0 && ts_bits >= 0 && id_bits + ts_bits < 64, SGL_ERR_UNSUPPORTED,
              "seeds_in_window: id_bits %d + ts_bits %d leave no room for the sentinel key", id_bits, ts_bits);
  SGL_REQUIRE(d_counts && out_ts_ptr && out_q_ptr, SGL_ERR_ARG, "seeds_in_window: null output");
  if (n_events == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(d_counts, 0, 3 * sizeof(int64_t), stream));
    SGL_CUDA_CHECK(cudaMemsetAsync(out_ts_ptr, 0, sizeof(int64_t), stream));
    SGL_CUDA_CHECK(cudaMemsetAsync(out_q_ptr, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE(ev_src && ev_ts && ev_eid && out_roots && out_ts && out_q_eid, SGL_ERR_ARG, "seeds_in_window: null array");
  const int64_t n = n_events;
  WsCarver c(ws, ws_bytes);
  uint64_t* k0 = c.take<uint64_t>(n);
  uint64_t* k1 = c.take<uint64_t>(n);
  uint32_t* v0 = c.take<uint32_t>(n);
  uint32_t* v1 = c.take<uint32_t>(n);
  uint32_t* packed = c.take<uint32_t>(n);
  int64_t* pair_node = c.take<int64_t>(n);
  int64_t* cta_sums = c.take<int64_t>(ctas_for(n));
  unsigned int* done = c.take<unsigned int>(1);
  size_t sort_bytes = radix_sort_ws_bytes(n);
  char* sort_ws = c.take<char>(sort_bytes);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "seeds_in_window: workspace %zu < %zu bytes", ws_bytes, sgl_seeds_ws_bytes(n));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
  const int key_bits = id_bits + ts_bits;
  seeds_pack_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ev_src, ev_ts, n, node_chunk, chunk_mask, num_chunks, num_nodes,
                                                          id_bits, ts_bits, ts_base, k0, d_status);
  SGL_LAUNCH_CHECK();
  int in_alt = 0;
  int rc = radix_sort_pairs(k0, v0, k1, v1, n, nullptr, key_bits + 1, true, &in_alt, sort_ws, sort_bytes, stream);
  if (rc) return rc;
  const uint64_t* ks = in_alt ? k1 : k0;
  const uint32_t* vs = in_alt ? v1 : v0;
  heads_scan_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, n, nullptr, key_bits, packed, cta_sums, done, d_counts + 1);
  seeds_emit_pairs_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, vs, n, key_bits, ts_bits, ts_base, ev_eid, packed,
                                                                cta_sums, pair_node, out_ts, out_q_ptr, out_q_eid, d_counts);
  // roots = runs of equal node id among the (node, ts) pairs
  heads_scan_kernel<<<ctas_for(n), kThreads, 0, stream>>>((const uint64_t*)pair_node, n, d_counts + 1, 64, packed, cta_sums,
                                                          done, d_counts);
  seeds_emit_roots_kernel<<<ctas_for(n), kThreads, 0, stream>>>(pair_node, n, d_counts, packed, cta_sums, out_roots,
                                                                out_ts_ptr);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}
