// Mailbox update of a mini-batch: "latest message per node" reduce, row assembly and the write into the mailbox.
//
// The reference concatenates the batch's source and destination nodes, builds one mail row per entry
// ([own memory | other end's memory | edge feature]), and keeps for every distinct node the entry with the largest
// timestamp (unique + scatter_max + index).  Here the 2B x width mail matrix is never materialised:
//
//   mail_pack_kernel     key = node id of entry j (sources first, then destinations)
//   stable radix sort    on the populated id bits, payload = entry position
//   heads_scan_kernel    run heads -> index of every entry's node in the sorted unique list, number of unique nodes
//   mail_argmax_kernel   per entry one 64-bit atomicMax on its node's slot: (orderable fp32 ts << 32) | ~position, so the
//                        winner is the largest timestamp and, among equal timestamps, the FIRST entry (order
//                        independent, hence deterministic)
//   mail_emit_kernel     one warp per unique node: winner's position and timestamp, and the mail row gathered
//                        straight from the per-event tables
//
// Timestamps are compared as fp32, like the reference, which converts them to the mailbox dtype before the reduce.
// Algorithmic HBM bytes: 8 + 4|8 read per entry + sort passes (32 B per entry and populated key byte), and per
// unique node 2 * row bytes + 20 written / read.
#include "heads.cuh"
#include "sort.cuh"

namespace sgl {
namespace {

constexpr int kThreads = kHeadsThreads;
constexpr int kMaxSeg = 4;

struct Segs {
  const float* a[kMaxSeg];   // source of the segment for entries of the first list (row = entry position)
  const float* b[kMaxSeg];   // ... of the second list (row = position - n_a)
  int64_t dim[kMaxSeg];
  int n;
};

__device__ __forceinline__ float ts_at(const void* ts, int64_t ts_len, int is_i64, int64_t pos) {
  const int64_t k = pos < ts_len ? pos : pos - ts_len;   // cat(ts, ts) when one value per event is given
  return is_i64 ? (float)((const int64_t*)ts)[k] : ((const float*)ts)[k];
}

// monotone map fp32 -> uint32 (larger float, larger integer)
__device__ __forceinline__ uint32_t orderable(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kThreads)
mail_pack_kernel(const int64_t* __restrict__ ids_a, int64_t n_a, const int64_t* __restrict__ ids_b, int64_t n_b,
                 int64_t num_nodes, uint64_t* __restrict__ keys, int32_t* d_status) {
  const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (j >= n_a + n_b) return;
  int64_t g = j < n_a ? ids_a[j] : ids_b[j - n_a];
  if (g < 0 || g >= num_nodes) {
    dev_flag(d_status, SGL_DEV_BAD_NODE);
    g = 0;
  }
  keys[j] = (uint64_t)g;
}

__global__ void __launch_bounds__(kThreads)
mail_argmax_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ perm, int64_t n,
                   const uint32_t* __restrict__ packed, const int64_t* __restrict__ cta_base, const void* ts,
                   int64_t ts_len, int ts_is_i64, unsigned long long* __restrict__ best, int64_t* __restrict__ out_index) {
  const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (j >= n) return;
  const uint32_t pk = packed[j];
  const int64_t u = cta_base[blockIdx.x] + (pk >> 1) + (pk & 1) - 1;   // this entry's node in the unique list
  if (pk & 1) out_index[u] = (int64_t)keys[j];
  const uint32_t pos = perm[j];
  const unsigned long long v = ((unsigned long long)orderable(ts_at(ts, ts_len, ts_is_i64, pos)) << 32) | (0xffffffffu - pos);
  atomicMax(best + u, v);
}

__global__ void __launch_bounds__(kThreads)
mail_emit_kernel(const unsigned long long* __restrict__ best, int64_t n_cap, const int64_t* d_num_unique, int64_t n_a,
                 const void* ts, int64_t ts_len, int ts_is_i64, Segs segs, int64_t width, int64_t* __restrict__ out_pos,
                 float* __restrict__ out_ts, float* __restrict__ out_mail) {
  const int64_t n = eff_count(n_cap, d_num_unique);
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t u = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5; u < n; u += n_warps) {
    const int64_t pos = (int64_t)(0xffffffffu - (uint32_t)best[u]);
    if (lane == 0) {
      if (out_pos) out_pos[u] = pos;
      if (out_ts) out_ts[u] = ts_at(ts, ts_len, ts_is_i64, pos);
    }
    if (!out_mail) continue;
    const bool first = pos < n_a;
    const int64_t row = first ? pos : pos - n_a;
    float* dst = out_mail + u * width;
    int64_t off = 0;
    for (int s = 0; s < segs.n; ++s) {
      const float* src = (first ? segs.a[s] : segs.b[s]) + row * segs.dim[s];
      for (int64_t e = lane; e < segs.dim[s]; e += 32) dst[off + e] = __ldg(src + e);
      off += segs.dim[s];
    }
  }
}

// mailbox[node, next_pos[node], :] = mail[u, :], the timestamp alongside, and the ring position advanced.
// One warp per row; `index` holds distinct nodes (the output of the reduce), so no two warps touch one node.
__global__ void __launch_bounds__(kThreads)
mailbox_write_kernel(const int64_t* __restrict__ index, int64_t n_cap, const int64_t* d_n, const float* __restrict__ mail,
                     const float* __restrict__ mail_ts, int64_t width, float* __restrict__ mailbox,
                     float* __restrict__ mailbox_ts, int64_t* __restrict__ next_pos, int64_t num_nodes, int64_t mailbox_size,
                     int advance, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t u = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5; u < n; u += n_warps) {
    const int64_t g = index[u];
    if (g < 0 || g >= num_nodes) {
      if (lane == 0) dev_flag(d_status, SGL_DEV_BAD_NODE);
      continue;
    }
    int64_t p = next_pos ? next_pos[g] : 0;
    if (p < 0 || p >= mailbox_size) {
      if (lane == 0) dev_flag(d_status, SGL_DEV_BAD_INDEX);
      continue;
    }
    float* dst = mailbox + (g * mailbox_size + p) * width;
    const float* src = mail + u * width;
    for (int64_t e = lane; e < width; e += 32) dst[e] = src[e];
    __syncwarp();   // every lane has read next_pos[g] before lane 0 advances it
    if (lane == 0) {
      mailbox_ts[g * mailbox_size + p] = mail_ts[u];
      if (advance && next_pos && mailbox_size > 1) next_pos[g] = (p + 1) % mailbox_size;
    }
  }
}

inline unsigned ctas_for(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads < 1 ? 1 : (n + kThreads - 1) / kThreads); }

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" size_t sgl_mail_reduce_ws_bytes(int64_t n_entries) {
  int64_t n = n_entries < 1 ? 1 : n_entries;
  return 2 * align_up((size_t)n * 8) + 3 * align_up((size_t)n * 4) + align_up((size_t)ctas_for(n) * 8) + align_up(8) +
         align_up((size_t)n * 8) + radix_sort_ws_bytes(n);
}

extern "C" int sgl_mail_reduce(const int64_t* ids_a, int64_t n_a, const int64_t* ids_b, int64_t n_b, int64_t num_nodes,
                               const void* ts, int64_t ts_len, int ts_is_i64, int n_seg, const float* const* seg_a,
                               const float* const* seg_b, const int64_t* seg_dim, int64_t* out_index, int64_t* out_pos,
                               float* out_ts, float* out_mail, int64_t* d_num_unique, int32_t* d_status, void* ws,
                               size_t ws_bytes, void* stream_) {
  SGL_NVTX("sgl_mail_reduce");
  cudaStream_t stream = (cudaStream_t)stream_;
  const int64_t n = n_a + n_b;
  SGL_REQUIRE(n_a >= 0 && n_b >= 0 && num_nodes >= 0 && n <= 0xffffffffll, SGL_ERR_ARG, "mail_reduce: bad size");
  SGL_REQUIRE(d_num_unique, SGL_ERR_ARG, "mail_reduce: null counter");
  SGL_REQUIRE(n_seg >= 0 && n_seg <= kMaxSeg, SGL_ERR_ARG, "mail_reduce: at most %d row segments", kMaxSeg);
  if (n == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(d_num_unique, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE((n_a == 0 || ids_a) && (n_b == 0 || ids_b) && ts && out_index, SGL_ERR_ARG, "mail_reduce: null array");
  SGL_REQUIRE(ts_len == n || (ts_len == n_a && n_a == n_b), SGL_ERR_ARG,
              "mail_reduce: ts must hold one value per entry, or one per event when both lists have that length");
  Segs segs;
  memset(&segs, 0, sizeof(segs));
  segs.n = out_mail ? n_seg : 0;
  int64_t width = 0;
  for (int s = 0; s < segs.n; ++s) {
    SGL_REQUIRE(seg_dim && seg_a && seg_b && seg_dim[s] >= 0, SGL_ERR_ARG, "mail_reduce: bad segment table");
    SGL_REQUIRE(seg_dim[s] == 0 || ((n_a == 0 || seg_a[s]) && (n_b == 0 || seg_b[s])), SGL_ERR_ARG,
                "mail_reduce: segment %d has a null source", s);
    segs.a[s] = seg_a[s];
    segs.b[s] = seg_b[s];
    segs.dim[s] = seg_dim[s];
    width += seg_dim[s];
  }
  const int id_bits = bits_for(num_nodes > 0 ? (uint64_t)(num_nodes - 1) : 0);
  WsCarver c(ws, ws_bytes);
  uint64_t* k0 = c.take<uint64_t>(n);
  uint64_t* k1 = c.take<uint64_t>(n);
  uint32_t* v0 = c.take<uint32_t>(n);
  uint32_t* v1 = c.take<uint32_t>(n);
  uint32_t* packed = c.take<uint32_t>(n);
  int64_t* cta_sums = c.take<int64_t>(ctas_for(n));
  unsigned int* done = c.take<unsigned int>(1);
  unsigned long long* best = c.take<unsigned long long>(n);
  size_t sort_bytes = radix_sort_ws_bytes(n);
  char* sort_ws = c.take<char>(sort_bytes);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "mail_reduce: workspace %zu < %zu bytes", ws_bytes, sgl_mail_reduce_ws_bytes(n));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
  SGL_CUDA_CHECK(cudaMemsetAsync(best, 0, (size_t)n * 8, stream));
  mail_pack_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ids_a, n_a, ids_b, n_b, num_nodes, k0, d_status);
  SGL_LAUNCH_CHECK();
  int in_alt = 0;
  int rc = radix_sort_pairs(k0, v0, k1, v1, n, nullptr, id_bits, true, &in_alt, sort_ws, sort_bytes, stream);
  if (rc) return rc;
  const uint64_t* ks = in_alt ? k1 : k0;
  const uint32_t* perm = in_alt ? v1 : v0;
  heads_scan_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, n, nullptr, 64, packed, cta_sums, done, d_num_unique);
  mail_argmax_kernel<<<ctas_for(n), kThreads, 0, stream>>>(ks, perm, n, packed, cta_sums, ts, ts_len, ts_is_i64, best, out_index);
  mail_emit_kernel<<<stream_grid(n, kThreads / 32, 8), kThreads, 0, stream>>>(best, n, d_num_unique, n_a, ts, ts_len, ts_is_i64,
                                                                             segs, width, out_pos, out_ts, out_mail);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_mailbox_write(const int64_t* index, int64_t n, const int64_t* d_n, const float* mail, const float* mail_ts,
                                 int64_t width, float* mailbox, float* mailbox_ts, int64_t* next_mail_pos, int64_t num_nodes,
                                 int64_t mailbox_size, int advance, int32_t* d_status, void* stream_) {
  SGL_NVTX("sgl_mailbox_write");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && width >= 1 && num_nodes >= 0 && mailbox_size >= 1, SGL_ERR_ARG, "mailbox_write: bad size");
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(index && mail && mail_ts && mailbox && mailbox_ts, SGL_ERR_ARG, "mailbox_write: null array");
  SGL_REQUIRE(mailbox_size == 1 || next_mail_pos, SGL_ERR_ARG, "mailbox_write: a mailbox of several slots needs next_mail_pos");
  mailbox_write_kernel<<<stream_grid(n, kThreads / 32, 8), kThreads, 0, stream>>>(index, n, d_n, mail, mail_ts, width, mailbox,
                                                                                 mailbox_ts, next_mail_pos, num_nodes,
                                                                                 mailbox_size, advance, d_status);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}
