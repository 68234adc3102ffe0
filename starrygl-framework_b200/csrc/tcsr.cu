// T-CSR construction: rows keyed by node id, inside a row ascending timestamp, ties in input order.
//
//   1. tcsr_scan_input_kernel   min/max timestamp + count of out-of-range keys (one pass over key, ts)
//   2. tcsr_pack_kernel         64-bit sort key = (node << ts_bits) | (ts - ts_min)
//   3. stable LSD radix sort    on the populated key bits, payload = input position
//      (when node bits + timestamp bits exceed 64: sort by timestamp first, then stably by node)
//   4. tcsr_emit_kernel         reads the sorted keys sequentially (row and timestamp of every edge), gathers only the
//                               neighbour / edge id through the permutation and writes indptr from the row
//                               boundaries of the sorted keys (no atomics, no separate prefix sum)
#include "sort.cuh"

namespace sgl {
namespace {

struct InputScan {
  long long ts_min;
  long long ts_max;
  unsigned long long bad_keys;
};

__global__ void tcsr_init_scan_kernel(InputScan* s) {
  s->ts_min = 0x7fffffffffffffffLL;
  s->ts_max = (long long)0x8000000000000000ULL;
  s->bad_keys = 0;
}

__global__ void __launch_bounds__(256)
tcsr_scan_input_kernel(const int64_t* __restrict__ key, const int64_t* __restrict__ ts, int64_t m, int64_t num_nodes,
                       InputScan* out) {
  long long lo = 0x7fffffffffffffffLL, hi = (long long)0x8000000000000000ULL;
  unsigned long long bad = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x) {
    long long t = ts[i];
    lo = t < lo ? t : lo;
    hi = t > hi ? t : hi;
    int64_t k = key[i];
    bad += (k < 0 || k >= num_nodes) ? 1 : 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    long long a = __shfl_xor_sync(0xffffffffu, lo, o);
    long long b = __shfl_xor_sync(0xffffffffu, hi, o);
    unsigned long long c = __shfl_xor_sync(0xffffffffu, bad, o);
    lo = a < lo ? a : lo;
    hi = b > hi ? b : hi;
    bad += c;
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMin(&out->ts_min, lo);
    atomicMax(&out->ts_max, hi);
    if (bad) atomicAdd(&out->bad_keys, bad);
  }
}

// mode 0: key = (node << ts_bits) | (ts - ts_min)     mode 1: key = ts - ts_min     mode 2: key = node[perm[i]]
__global__ void __launch_bounds__(256)
tcsr_pack_kernel(const int64_t* __restrict__ key, const int64_t* __restrict__ ts, const uint32_t* __restrict__ perm,
                 int64_t m, long long ts_min, int ts_bits, int mode, uint64_t* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x) {
    uint64_t v;
    if (mode == 0) {
      uint64_t dt = (uint64_t)ts[i] - (uint64_t)ts_min;
      v = ts_bits >= 64 ? dt : (((uint64_t)key[i] << ts_bits) | dt);
    } else if (mode == 1) {
      v = (uint64_t)ts[i] - (uint64_t)ts_min;
    } else {
      v = (uint64_t)key[perm[i]];
    }
    out[i] = v;
  }
}

// The sorted keys are read sequentially and already hold the row of every edge (and, when node and timestamp share one
// key, its timestamp): only the neighbour (and the edge id, when given) are gathered through the permutation.
// combined != 0: key = (node << ts_bits) | (ts - ts_min); else key = node and the timestamp is gathered too.
__global__ void __launch_bounds__(256)
tcsr_emit_kernel(const uint64_t* __restrict__ sorted_keys, const uint32_t* __restrict__ perm, int combined, int ts_bits,
                 long long ts_min, const int64_t* __restrict__ nbr, const int64_t* __restrict__ ts,
                 const int64_t* __restrict__ eid, int64_t m, int64_t num_nodes, int64_t* __restrict__ indptr,
                 int64_t* __restrict__ out_nbr, int64_t* __restrict__ out_ts, int64_t* __restrict__ out_eid,
                 int64_t* __restrict__ out_perm) {
  const bool split = combined && ts_bits < 64;
  const uint64_t ts_mask = ts_bits >= 64 ? ~0ull : ((1ull << ts_bits) - 1ull);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t p = perm[i];
    const uint64_t k = sorted_keys[i];
    out_nbr[i] = nbr[p];
    out_ts[i] = combined ? (int64_t)((k & ts_mask) + (uint64_t)ts_min) : ts[p];
    out_eid[i] = eid ? eid[p] : (int64_t)p;
    if (out_perm) out_perm[i] = (int64_t)p;
    // row boundaries: every node id in (prev_node, this_node] starts at position i
    const int64_t node = combined ? (split ? (int64_t)(k >> ts_bits) : 0) : (int64_t)k;
    int64_t prev = -1;
    if (i > 0) {
      const uint64_t kp = sorted_keys[i - 1];
      prev = combined ? (split ? (int64_t)(kp >> ts_bits) : 0) : (int64_t)kp;
    }
    for (int64_t v = prev + 1; v <= node; ++v) indptr[v] = i;
    if (i == m - 1)
      for (int64_t v = node + 1; v <= num_nodes; ++v) indptr[v] = m;
  }
}

__global__ void fill_i64_kernel(int64_t* p, int64_t n, int64_t v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" size_t sgl_tcsr_build_ws_bytes(int64_t num_nodes, int64_t m) {
  (void)num_nodes;
  if (m < 1) m = 1;
  return align_up(sizeof(InputScan)) + 2 * align_up((size_t)m * 8) + 2 * align_up((size_t)m * 4) + radix_sort_ws_bytes(m);
}

extern "C" int sgl_tcsr_build(int64_t num_nodes, int64_t m, const int64_t* key, const int64_t* nbr, const int64_t* ts,
                              const int64_t* eid, int64_t* indptr, int64_t* out_nbr, int64_t* out_ts, int64_t* out_eid,
                              int64_t* out_perm, int64_t* h_ts_range, void* ws, size_t ws_bytes, void* stream_) {
  SGL_NVTX("sgl_tcsr_build");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(num_nodes >= 0 && m >= 0, SGL_ERR_ARG, "tcsr_build: negative size");
  SGL_REQUIRE(m < ((int64_t)1 << 32), SGL_ERR_UNSUPPORTED, "tcsr_build: m=%lld needs a 64-bit permutation", (long long)m);
  SGL_REQUIRE(indptr, SGL_ERR_ARG, "tcsr_build: indptr is null");
  if (m == 0) {
    fill_i64_kernel<<<stream_grid(num_nodes + 1, 256, 4), 256, 0, stream>>>(indptr, num_nodes + 1, 0);
    SGL_LAUNCH_CHECK();
    if (h_ts_range) h_ts_range[0] = h_ts_range[1] = 0;
    return SGL_OK;
  }
  SGL_REQUIRE(key && nbr && ts && out_nbr && out_ts && out_eid, SGL_ERR_ARG, "tcsr_build: null array");
  WsCarver c(ws, ws_bytes);
  InputScan* d_scan = c.take<InputScan>(1);
  uint64_t* k0 = c.take<uint64_t>(m);
  uint64_t* k1 = c.take<uint64_t>(m);
  uint32_t* v0 = c.take<uint32_t>(m);
  uint32_t* v1 = c.take<uint32_t>(m);
  size_t sort_bytes = radix_sort_ws_bytes(m);
  char* sort_ws = c.take<char>(sort_bytes);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "tcsr_build: workspace %zu < %zu bytes", ws_bytes,
              sgl_tcsr_build_ws_bytes(num_nodes, m));

  const int grid = stream_grid(m, 256 * 4, 8);
  tcsr_init_scan_kernel<<<1, 1, 0, stream>>>(d_scan);
  tcsr_scan_input_kernel<<<grid, 256, 0, stream>>>(key, ts, m, num_nodes, d_scan);
  SGL_LAUNCH_CHECK();
  InputScan h;
  SGL_CUDA_CHECK(cudaMemcpyAsync(&h, d_scan, sizeof(h), cudaMemcpyDeviceToHost, stream));
  SGL_CUDA_CHECK(cudaStreamSynchronize(stream));
  SGL_REQUIRE(h.bad_keys == 0, SGL_ERR_RANGE, "tcsr_build: %llu edge keys outside [0, %lld)", h.bad_keys,
              (long long)num_nodes);
  if (h_ts_range) {
    h_ts_range[0] = h.ts_min;
    h_ts_range[1] = h.ts_max;
  }
  const int ts_bits = bits_for((uint64_t)h.ts_max - (uint64_t)h.ts_min);
  const int id_bits = bits_for(num_nodes > 0 ? (uint64_t)(num_nodes - 1) : 0);
  int in_alt = 0;
  const uint64_t* sorted_keys = nullptr;
  const bool combined = ts_bits + id_bits <= 64;
  if (combined) {
    tcsr_pack_kernel<<<grid, 256, 0, stream>>>(key, ts, nullptr, m, h.ts_min, ts_bits, 0, k0);
    SGL_LAUNCH_CHECK();
    int rc = radix_sort_pairs(k0, v0, k1, v1, m, nullptr, ts_bits + id_bits, true, &in_alt, sort_ws, sort_bytes, stream);
    if (rc) return rc;
    sorted_keys = in_alt ? k1 : k0;
  } else {
    // two stable rounds: by timestamp, then by node id
    tcsr_pack_kernel<<<grid, 256, 0, stream>>>(key, ts, nullptr, m, h.ts_min, ts_bits, 1, k0);
    SGL_LAUNCH_CHECK();
    int rc = radix_sort_pairs(k0, v0, k1, v1, m, nullptr, ts_bits, true, &in_alt, sort_ws, sort_bytes, stream);
    if (rc) return rc;
    uint32_t* perm1 = in_alt ? v1 : v0;
    uint64_t* kk = in_alt ? k1 : k0;       // reuse the buffer that holds the (no longer needed) sorted keys
    uint64_t* kk_alt = in_alt ? k0 : k1;
    uint32_t* vv_alt = in_alt ? v0 : v1;
    tcsr_pack_kernel<<<grid, 256, 0, stream>>>(key, ts, perm1, m, h.ts_min, ts_bits, 2, kk);
    SGL_LAUNCH_CHECK();
    int in_alt2 = 0;
    rc = radix_sort_pairs(kk, perm1, kk_alt, vv_alt, m, nullptr, id_bits, false, &in_alt2, sort_ws, sort_bytes, stream);
    if (rc) return rc;
    sorted_keys = in_alt2 ? kk_alt : kk;
    in_alt = in_alt2 ? !in_alt : in_alt;
  }
  const uint32_t* perm = in_alt ? v1 : v0;
  tcsr_emit_kernel<<<grid, 256, 0, stream>>>(sorted_keys, perm, combined ? 1 : 0, ts_bits, h.ts_min, nbr, ts, eid, m, num_nodes,
                                             indptr, out_nbr, out_ts, out_eid, out_perm);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Search index over the time-sorted rows ("fence"): for every block of 32 consecutive edges of a row the timestamp of
// the block's last edge.  Row r (edges [s, e)) owns the entries fence[(s >> 5) + r + j], j < ceil((e - s) / 32) -- a
// placement that needs no pointer array of its own: consecutive rows never overlap because
// floor((s + d) / 32) - floor(s / 32) >= ceil(d / 32) - 1.  About 1.6 % of the adjacency's size, so it stays in L2 while
// the timestamps themselves (8 bytes per edge) do not; a time-range search walks the fence and then reads ONE block of
// the row.
// ---------------------------------------------------------------------------------------------------------------
namespace sgl {
namespace {
// One thread per fence entry x: its row is the last r with (indptr[r] >> 5) + r <= x (that start position is strictly
// increasing in r), found by binary search over the row pointer -- so a hub row's tens of thousands of entries are
// written by as many threads, not by one warp.
__global__ void __launch_bounds__(256)
tcsr_fence_kernel(const int64_t* __restrict__ indptr, const int64_t* __restrict__ ts, int64_t num_nodes, int64_t len,
                  int64_t* __restrict__ fence) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t x = (int64_t)blockIdx.x * 256 + threadIdx.x; x < len; x += stride) {
    int64_t lo = 0, hi = num_nodes;          // invariant: start(lo) <= x; rows >= hi start after x
    while (hi - lo > 1) {
      const int64_t mid = lo + ((hi - lo) >> 1);
      if ((__ldg(indptr + mid) >> 5) + mid <= x) lo = mid; else hi = mid;
    }
    const int64_t s = __ldg(indptr + lo), e = __ldg(indptr + lo + 1);
    const int64_t j = x - ((s >> 5) + lo);
    if (j < ((e - s + 31) >> 5)) {
      const int64_t last = s + (j << 5) + 31;
      fence[x] = __ldg(ts + (last < e ? last : e - 1));
    }
  }
}
}  // namespace
}  // namespace sgl

extern "C" int64_t sgl_tcsr_fence_len(int64_t num_nodes, int64_t m) { return (m >> 5) + num_nodes + 1; }

extern "C" int sgl_tcsr_fence(const int64_t* indptr, const int64_t* ts, int64_t num_nodes, int64_t m, int64_t* out_fence,
                              void* stream_) {
  SGL_REQUIRE(num_nodes >= 0 && m >= 0, SGL_ERR_ARG, "tcsr_fence: negative size");
  if (num_nodes == 0 || m == 0) return SGL_OK;
  SGL_REQUIRE(indptr && ts && out_fence, SGL_ERR_ARG, "tcsr_fence: null array");
  const int64_t len = sgl_tcsr_fence_len(num_nodes, m);
  tcsr_fence_kernel<<<stream_grid(len, 256, 16), 256, 0, (cudaStream_t)stream_>>>(indptr, ts, num_nodes, len, out_fence);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}
