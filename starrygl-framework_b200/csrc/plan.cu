// Route plan of one layer on the GPU: which rows of the layer's (id, ts) list this partition must push to which
// other ranks, and where they land there.
//
// Input: the layer list sorted by (id, ts) (what the batch builder produces), the owner partition of every node and
// the replica table (CSR over node id of (rank, slot)).  For every distinct node id the row with the latest timestamp
// is the last row of its run.  Rows of nodes owned here are expanded to one entry per replica on another rank, then
// ordered by rank (stable: ascending list row inside a rank).
//
//   plan_count_kernel   per row: is it the run's last row and owned here? how many foreign replicas? CTA scan,
//                       last CTA scans the CTA totals; per-rank sizes by atomic add (order independent)
//   plan_expand_kernel  writes (rank, row, slot) triplets in row order
//   radix sort on the rank (one 8-bit pass) + plan_emit_kernel gathers rows and slots in sorted order
#include "scan.cuh"
#include "sort.cuh"

namespace sgl {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
plan_count_kernel(const int64_t* __restrict__ ids, int64_t n_cap, const int64_t* d_n, const int64_t* __restrict__ node_parts,
                  int64_t num_nodes, int64_t pid, const int64_t* __restrict__ indptr, const int64_t* __restrict__ ranks,
                  int64_t num_parts, int64_t* __restrict__ local_off, int64_t* __restrict__ cta_sums,
                  unsigned int* done_counter, int64_t* d_total, unsigned long long* __restrict__ send_sizes, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  int64_t len = 0;
  if (i < n) {
    const int64_t id = ids[i];
    if (id < 0 || id >= num_nodes) {
      dev_flag(d_status, SGL_DEV_BAD_NODE);
    } else {
      if (i + 1 < n && ids[i + 1] < id) dev_flag(d_status, SGL_DEV_BAD_INDEX);   // list must be sorted by id
      const bool tail = (i == n - 1) || ids[i + 1] != id;
      if (tail && node_parts[id] == pid) {
        for (int64_t p = indptr[id]; p < indptr[id + 1]; ++p) {
          const int64_t r = ranks[p];
          if (r != pid && r >= 0 && r < num_parts) {
            ++len;
            atomicAdd(send_sizes + r, 1ull);
          }
        }
      }
    }
  }
  int64_t total;
  int64_t ex = cta_exclusive_scan<kThreads, int64_t>(len, &total);
  if (i < n) local_off[i] = ex;
  publish_and_scan_cta_totals<kThreads>(total, cta_sums, done_counter, d_total);
}

__global__ void __launch_bounds__(kThreads)
plan_expand_kernel(const int64_t* __restrict__ ids, int64_t n_cap, const int64_t* d_n, const int64_t* __restrict__ node_parts,
                   int64_t num_nodes, int64_t pid, const int64_t* __restrict__ indptr, const int64_t* __restrict__ ranks,
                   const int64_t* __restrict__ locs, int64_t num_parts, const int64_t* __restrict__ local_off,
                   const int64_t* __restrict__ cta_sums, int64_t cap, uint64_t* __restrict__ keys,
                   int64_t* __restrict__ tmp_rows, int64_t* __restrict__ tmp_locs, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  const int64_t id = ids[i];
  if (id < 0 || id >= num_nodes) return;
  const bool tail = (i == n - 1) || ids[i + 1] != id;
  if (!tail || node_parts[id] != pid) return;
  int64_t off = cta_sums[blockIdx.x] + local_off[i];
  for (int64_t p = indptr[id]; p < indptr[id + 1]; ++p) {
    const int64_t r = ranks[p];
    if (r == pid || r < 0 || r >= num_parts) continue;
    if (off >= cap) {
      dev_flag(d_status, SGL_DEV_OVERFLOW);
      return;
    }
    keys[off] = (uint64_t)r;
    tmp_rows[off] = i;
    tmp_locs[off] = locs[p];
    ++off;
  }
}

__global__ void __launch_bounds__(kThreads)
plan_emit_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ perm, int64_t cap, const int64_t* d_total,
                 const int64_t* __restrict__ tmp_rows, const int64_t* __restrict__ tmp_locs, int64_t* __restrict__ out_ranks,
                 int64_t* __restrict__ out_rows, int64_t* __restrict__ out_locs) {
  const int64_t n = eff_count(cap, d_total);
  for (int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x; j < n; j += (int64_t)gridDim.x * kThreads) {
    const uint32_t p = perm[j];
    out_ranks[j] = (int64_t)keys[j];
    out_rows[j] = tmp_rows[p];
    out_locs[j] = tmp_locs[p];
  }
}

inline int64_t ctas_for(int64_t n) { return (n + kThreads - 1) / kThreads < 1 ? 1 : (n + kThreads - 1) / kThreads; }

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" size_t sgl_plan_route_ws_bytes(int64_t n, int64_t cap) {
  if (n < 1) n = 1;
  if (cap < 1) cap = 1;
  return align_up((size_t)n * 8) + align_up((size_t)ctas_for(n) * 8) + align_up(8) + 2 * align_up((size_t)cap * 8) +
         2 * align_up((size_t)cap * 4) + 2 * align_up((size_t)cap * 8) + radix_sort_ws_bytes(cap);
}

extern "C" int sgl_plan_route(const int64_t* layer_ids, int64_t n, const int64_t* d_n, const int64_t* node_parts,
                              int64_t num_nodes, int64_t pid, const int64_t* rep_indptr, const int64_t* rep_ranks,
                              const int64_t* rep_locs, int64_t num_parts, int64_t cap, int64_t* out_ranks, int64_t* out_rows,
                              int64_t* out_locs, int64_t* d_send_sizes, int64_t* d_total, int32_t* d_status, void* ws,
                              size_t ws_bytes, void* stream_) {
  SGL_NVTX("sgl_plan_route");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && cap >= 0 && num_nodes >= 0 && num_parts >= 1 && num_parts <= 256 && pid >= 0 && pid < num_parts,
              SGL_ERR_ARG, "plan_route: bad size (1 <= num_parts <= 256, 0 <= pid < num_parts)");
  SGL_REQUIRE(d_send_sizes && d_total, SGL_ERR_ARG, "plan_route: null counter");
  SGL_CUDA_CHECK(cudaMemsetAsync(d_send_sizes, 0, (size_t)num_parts * sizeof(int64_t), stream));
  if (n == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(d_total, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE(layer_ids && node_parts && rep_indptr && rep_ranks && rep_locs && out_ranks && out_rows && out_locs, SGL_ERR_ARG,
              "plan_route: null array");
  const int64_t capc = cap < 1 ? 1 : cap;
  WsCarver c(ws, ws_bytes);
  int64_t* local_off = c.take<int64_t>(n);
  int64_t* cta_sums = c.take<int64_t>(ctas_for(n));
  unsigned int* done = c.take<unsigned int>(1);
  uint64_t* k0 = c.take<uint64_t>(capc);
  uint64_t* k1 = c.take<uint64_t>(capc);
  uint32_t* v0 = c.take<uint32_t>(capc);
  uint32_t* v1 = c.take<uint32_t>(capc);
  int64_t* tmp_rows = c.take<int64_t>(capc);
  int64_t* tmp_locs = c.take<int64_t>(capc);
  size_t sort_bytes = radix_sort_ws_bytes(capc);
  char* sort_ws = c.take<char>(sort_bytes);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "plan_route: workspace %zu < %zu bytes", ws_bytes, sgl_plan_route_ws_bytes(n, cap));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
  plan_count_kernel<<<(unsigned)ctas_for(n), kThreads, 0, stream>>>(layer_ids, n, d_n, node_parts, num_nodes, pid, rep_indptr,
                                                                    rep_ranks, num_parts, local_off, cta_sums, done, d_total,
                                                                    (unsigned long long*)d_send_sizes, d_status);
  plan_expand_kernel<<<(unsigned)ctas_for(n), kThreads, 0, stream>>>(layer_ids, n, d_n, node_parts, num_nodes, pid, rep_indptr,
                                                                     rep_ranks, rep_locs, num_parts, local_off, cta_sums, cap, k0,
                                                                     tmp_rows, tmp_locs, d_status);
  SGL_LAUNCH_CHECK();
  int in_alt = 0;
  int rc = radix_sort_pairs(k0, v0, k1, v1, capc, d_total, bits_for((uint64_t)(num_parts - 1)), true, &in_alt, sort_ws, sort_bytes,
                            stream);
  if (rc) return rc;
  plan_emit_kernel<<<stream_grid(capc, kThreads, 8), kThreads, 0, stream>>>(in_alt ? k1 : k0, in_alt ? v1 : v0, capc, d_total,
                                                                          tmp_rows, tmp_locs, out_ranks, out_rows, out_locs);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}
