// Row gather / scatter kernels of the feature and node-memory path.
//
//   gather_lanes_kernel<V>  flattened copy: consecutive threads move consecutive V-byte lanes (V = 16: 128-bit
//                           loads/stores; V = 4 for rows that are not 16-byte multiples), so every warp reads one
//                           contiguous piece of a source row and writes one contiguous piece of the output.
//   gather_bulk_kernel      per-warp pipeline of bulk asynchronous copies: each lane asks the copy engine for one
//                           source row (global -> shared, completion counted on an mbarrier), then one lane
//                           writes the whole stage back with a single shared -> global bulk copy.  The payload
//                           never passes through registers.  All waits are bounded.
//   cache_lookup_kernel +   hit-map lookup, deterministic miss compaction (CTA scan + last-CTA scan of CTA
//   cache_copy_kernel       totals), then one flattened copy that picks cache or backing store per row.
//   scatter_lanes_kernel    the reverse of the gather, optionally splitting a trailing timestamp column.
//
// Algorithmic HBM bytes: rows * (2 * row_bytes + 8) (+4 per id for the hit-map, +16 per miss for the miss list).
#include "common.cuh"
#include "scan.cuh"

namespace sgl {
namespace {

constexpr int kLaneThreads = 256;
constexpr int kLaneUnroll = 4;

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream(uint32_t* p, uint32_t v) {
  asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Flattened lane q -> (row i, lane l inside the row).  Rows of a power-of-two number of lanes split with a shift; other
// rows with a 32-bit division while the lane count fits 32 bits (a 64-bit division costs several times as much, and
// these kernels execute one split per 16 bytes moved).
struct LaneSplit {
  uint32_t lanes;
  int shift;        // log2(lanes) or -1
  bool small;       // every flattened index of the launch fits 32 bits
  __host__ LaneSplit(uint32_t lanes_, int64_t total) : lanes(lanes_), shift(-1), small(total <= 0xffffffffll) {
    if ((lanes & (lanes - 1)) == 0) {
      shift = 0;
      while ((1u << shift) < lanes) ++shift;
    }
  }
  __device__ __forceinline__ void operator()(int64_t q, int64_t* i, uint32_t* l) const {
    if (shift >= 0) {
      *i = q >> shift;
      *l = (uint32_t)q & (lanes - 1);
    } else if (small) {
      const uint32_t qq = (uint32_t)q, ii = qq / lanes;
      *i = ii;
      *l = qq - ii * lanes;
    } else {
      *i = q / lanes;
      *l = (uint32_t)(q - *i * lanes);
    }
  }
};

// resolve the source/destination row of item i; returns false when the row must be skipped
__device__ __forceinline__ bool resolve_row(const int64_t* __restrict__ idx, const int64_t* __restrict__ map,
                                            int64_t map_len, int64_t table_rows, int64_t i, bool wrap_negative,
                                            int32_t* d_status, int64_t* row) {
  int64_t r = __ldg(idx + i);
  if (map) {
    if (r < 0 || r >= map_len) {
      dev_flag(d_status, SGL_DEV_BAD_INDEX);
      return false;
    }
    r = __ldg(map + r);
  }
  if (r < 0) {
    if (!wrap_negative) return false;  // "not stored here": skipped silently
    r += table_rows;
  }
  if (r < 0 || r >= table_rows) {
    dev_flag(d_status, SGL_DEV_BAD_INDEX);
    return false;
  }
  *row = r;
  return true;
}

template <typename V>
__global__ void __launch_bounds__(kLaneThreads)
gather_lanes_kernel(const char* __restrict__ table, int64_t table_rows, LaneSplit split, int64_t src_pitch,
                    const int64_t* __restrict__ idx, const int64_t* __restrict__ map, int64_t map_len, int64_t n_cap,
                    const int64_t* d_n, char* __restrict__ out, int64_t dst_pitch, const float* __restrict__ ts_table,
                    float* __restrict__ out_ts, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t total = n * split.lanes;
  const int64_t stride = (int64_t)gridDim.x * kLaneThreads;
  for (int64_t q0 = (int64_t)blockIdx.x * kLaneThreads + threadIdx.x; q0 < total; q0 += stride * kLaneUnroll) {
    V v[kLaneUnroll];
    V* dst[kLaneUnroll];
#pragma unroll
    for (int u = 0; u < kLaneUnroll; ++u) {
      int64_t q = q0 + u * stride;
      dst[u] = nullptr;
      if (q < total) {
        int64_t i;
        uint32_t l;
        split(q, &i, &l);
        int64_t r;
        if (resolve_row(idx, map, map_len, table_rows, i, true, d_status, &r)) {
          v[u] = ld_stream((const V*)(table + r * src_pitch) + l);
          dst[u] = (V*)(out + i * dst_pitch) + l;
          if (l == 0 && ts_table) out_ts[i] = __ldg(ts_table + r);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kLaneUnroll; ++u)
      if (dst[u]) st_stream(dst[u], v[u]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// bulk asynchronous copy path
// ---------------------------------------------------------------------------------------------------------------
constexpr int kBulkWarps = 4;
constexpr int kBulkStages = 3;
constexpr unsigned long long kBulkWaitLimitNs = 2000000000ull;  // a wait gives up after two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait: false when the barrier did not flip within the limit
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  while (global_ns() - t0 < kBulkWaitLimitNs)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Output rows must be contiguous (dst_pitch == row_bytes); row_bytes multiple of 16; rows_per_stage <= 32.
template <int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
gather_bulk_kernel(const char* __restrict__ table, int64_t table_rows, uint32_t row_bytes, int64_t src_pitch,
                   const int64_t* __restrict__ idx, const int64_t* __restrict__ map, int64_t map_len, int64_t n_cap,
                   const int64_t* d_n, char* __restrict__ out, const float* __restrict__ ts_table,
                   float* __restrict__ out_ts, int rows_per_stage, int32_t* d_status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[WARPS][STAGES];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n = eff_count(n_cap, d_n);
  const uint32_t stage_bytes = (uint32_t)rows_per_stage * row_bytes;
  unsigned char* my_smem = smem_raw + (size_t)warp * STAGES * stage_bytes;
  const int64_t num_chunks = (n + rows_per_stage - 1) / rows_per_stage;
  const int64_t warps_total = (int64_t)gridDim.x * WARPS;
  const int64_t gwarp = (int64_t)blockIdx.x * WARPS + warp;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(smem_u32(&bars[warp][s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  __syncwarp();

  // issue the loads of this warp's k-th chunk into stage k % STAGES
  auto issue = [&](int64_t k) {
    const int64_t chunk = gwarp + k * warps_total;
    if (chunk >= num_chunks) return;
    const int s = (int)(k % STAGES);
    const int64_t row0 = chunk * rows_per_stage;
    const int rows = (int)((n - row0) < rows_per_stage ? (n - row0) : rows_per_stage);
    const uint32_t bar = smem_u32(&bars[warp][s]);
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows * row_bytes);
    __syncwarp();
    if (lane < rows) {
      int64_t r;
      if (!resolve_row(idx, map, map_len, table_rows, row0 + lane, true, d_status, &r)) r = 0;  // flagged; keep byte count
      bulk_g2s(smem_u32(my_smem + (size_t)s * stage_bytes + (size_t)lane * row_bytes), table + r * src_pitch, row_bytes,
               bar);
      if (ts_table) out_ts[row0 + lane] = __ldg(ts_table + r);
    }
  };

  for (int k = 0; k < STAGES; ++k) issue(k);
  bool failed = false;
  for (int64_t k = 0;; ++k) {
    const int64_t chunk = gwarp + k * warps_total;
    if (chunk >= num_chunks) break;
    const int s = (int)(k % STAGES);
    const uint32_t parity = (uint32_t)((k / STAGES) & 1);
    const int64_t row0 = chunk * rows_per_stage;
    const int rows = (int)((n - row0) < rows_per_stage ? (n - row0) : rows_per_stage);
    bool ok = mbar_wait_bounded(smem_u32(&bars[warp][s]), parity);
    if (!__all_sync(0xffffffffu, ok)) {
      failed = true;
      break;
    }
    if (lane == 0) {
      fence_async_smem();
      bulk_s2g(out + row0 * (int64_t)row_bytes, smem_u32(my_smem + (size_t)s * stage_bytes), (uint32_t)rows * row_bytes);
      bulk_commit();
      // the stage written back one iteration ago may be refilled once its store has finished reading shared memory
      bulk_wait_read<1>();
    }
    __syncwarp();
    if (k >= 1) issue(k - 1 + STAGES);
  }
  if (lane == 0) bulk_wait_all();
  if (failed) {
    if (lane == 0) dev_flag(d_status, SGL_DEV_TIMEOUT);
    // give copies still in flight a bounded chance to land before the CTA's shared memory is released
    for (int s = 0; s < STAGES; ++s) mbar_wait_bounded(smem_u32(&bars[warp][s]), 0);
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------------------------------------------
// cache
// ---------------------------------------------------------------------------------------------------------------
constexpr int kCacheThreads = 256;

__global__ void __launch_bounds__(kCacheThreads)
cache_lookup_kernel(const int32_t* __restrict__ hitmap, int64_t num_ids, const int64_t* __restrict__ ids, int64_t n,
                    int32_t* __restrict__ slot_ws, int32_t* __restrict__ rank_ws, int64_t* __restrict__ cta_miss,
                    unsigned int* done_counter, int64_t* d_counts, int32_t* d_status) {
  const int64_t i = (int64_t)blockIdx.x * kCacheThreads + threadIdx.x;
  int32_t slot = -1;
  int miss = 0;
  if (i < n) {
    int64_t id = __ldg(ids + i);
    if (id < 0 || id >= num_ids) {
      dev_flag(d_status, SGL_DEV_BAD_INDEX);
      slot = -2;  // neither hit nor reportable miss: row is left untouched
    } else {
      slot = __ldg(hitmap + id);
      miss = slot < 0 ? 1 : 0;
      if (slot < 0) slot = -1;
    }
  }
  int total;
  int rank = cta_exclusive_scan<kCacheThreads, int>(miss, &total);
  if (i < n) {
    slot_ws[i] = slot;
    rank_ws[i] = rank;
  }
  publish_and_scan_cta_totals<kCacheThreads>((int64_t)total, cta_miss, done_counter, d_counts + 1);
}

template <typename V>
__global__ void __launch_bounds__(kLaneThreads)
cache_copy_kernel(const char* __restrict__ cache_rows, int64_t cache_slots, const char* __restrict__ backing,
                  LaneSplit split, int64_t row_bytes, const int64_t* __restrict__ ids, int64_t n,
                  const int32_t* __restrict__ slot_ws, const int32_t* __restrict__ rank_ws,
                  const int64_t* __restrict__ cta_miss, char* __restrict__ out, int64_t* __restrict__ miss_pos,
                  int64_t* __restrict__ miss_ids, int64_t* d_counts, int32_t* d_status) {
  const int64_t total = n * split.lanes;
  const int64_t stride = (int64_t)gridDim.x * kLaneThreads;
  if (blockIdx.x == 0 && threadIdx.x == 0) d_counts[0] = n - d_counts[1];
  for (int64_t q0 = (int64_t)blockIdx.x * kLaneThreads + threadIdx.x; q0 < total; q0 += stride * kLaneUnroll) {
    V v[kLaneUnroll];
    V* dst[kLaneUnroll];
#pragma unroll
    for (int u = 0; u < kLaneUnroll; ++u) {
      int64_t q = q0 + u * stride;
      dst[u] = nullptr;
      if (q < total) {
        int64_t i;
        uint32_t l;
        split(q, &i, &l);
        int32_t slot = __ldg(slot_ws + i);
        const char* src = nullptr;
        if (slot >= 0) {
          if (slot < cache_slots) src = cache_rows + (int64_t)slot * row_bytes;
          else dev_flag(d_status, SGL_DEV_BAD_INDEX);
        } else if (slot == -1) {
          int64_t id = __ldg(ids + i);
          if (l == 0) {
            int64_t p = cta_miss[i / kCacheThreads] + rank_ws[i];
            miss_pos[p] = i;
            miss_ids[p] = id;
          }
          if (backing) src = backing + id * row_bytes;
        }
        if (src) {
          v[u] = ld_stream((const V*)src + l);
          dst[u] = (V*)(out + i * row_bytes) + l;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kLaneUnroll; ++u)
      if (dst[u]) st_stream(dst[u], v[u]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// scatter / route helpers
// ---------------------------------------------------------------------------------------------------------------
template <typename V>
__global__ void __launch_bounds__(kLaneThreads)
scatter_lanes_kernel(char* __restrict__ table, int64_t table_rows, uint32_t lanes_per_row, int64_t row_bytes,
                     int64_t dst_pitch,
                     const int64_t* __restrict__ idx, const int64_t* __restrict__ map, int64_t map_len, int64_t n_cap,
                     const int64_t* d_n, const char* __restrict__ rows, int64_t src_pitch, float* __restrict__ ts_table,
                     const float* __restrict__ ts, int split_last_col, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t total = n * lanes_per_row;
  const int64_t stride = (int64_t)gridDim.x * kLaneThreads;
  for (int64_t q = (int64_t)blockIdx.x * kLaneThreads + threadIdx.x; q < total; q += stride) {
    int64_t i = q / lanes_per_row;
    uint32_t l = (uint32_t)(q - i * lanes_per_row);
    int64_t r;
    if (!resolve_row(idx, map, map_len, table_rows, i, false, d_status, &r)) continue;
    ((V*)(table + r * dst_pitch))[l] = ((const V*)(rows + i * src_pitch))[l];
    if (l == 0 && ts_table) {
      if (split_last_col) ts_table[r] = *(const float*)(rows + i * src_pitch + row_bytes);
      else if (ts) ts_table[r] = ts[i];
    }
  }
}

// Wire rows: [dim features | ts (optional) | slot low word | slot high word | zero padding to a multiple of 4 floats]
// (the slot words and the padding exist only when remote_idx is given).  VEC = 4: 128-bit lanes, needs dim % 4 == 0.
__device__ __forceinline__ uint32_t wire_word(uint32_t e, uint32_t dim, uint32_t payload, const float* __restrict__ frow,
                                              const float* __restrict__ ts, int64_t r, uint64_t slot) {
  if (e < dim) return __float_as_uint(__ldg(frow + e));
  if (e < payload) return __float_as_uint(__ldg(ts + r));
  if (e == payload) return (uint32_t)slot;
  if (e == payload + 1) return (uint32_t)(slot >> 32);
  return 0u;
}

template <int VEC>
__global__ void __launch_bounds__(kLaneThreads)
route_pack_kernel(const float* __restrict__ feats, int64_t n_rows, uint32_t dim, const float* __restrict__ ts,
                  const int64_t* __restrict__ send_idx, const int64_t* __restrict__ remote_idx, int64_t n_send,
                  uint32_t pitch, float* __restrict__ packed, int32_t* d_status) {
  const uint32_t payload = dim + (ts ? 1u : 0u);
  const uint32_t lanes = pitch / VEC;
  const int64_t total = n_send * lanes;
  const int64_t stride = (int64_t)gridDim.x * kLaneThreads;
  for (int64_t q = (int64_t)blockIdx.x * kLaneThreads + threadIdx.x; q < total; q += stride) {
    int64_t i = q / lanes;
    uint32_t l = (uint32_t)(q - i * lanes);
    int64_t r = __ldg(send_idx + i);
    if (r < 0) r += n_rows;
    if (r < 0 || r >= n_rows) {
      dev_flag(d_status, SGL_DEV_BAD_INDEX);
      continue;
    }
    const float* frow = feats + r * dim;
    if (VEC == 4) {
      uint4 v;
      if ((l + 1) * 4 <= dim) {
        v = ld_stream((const uint4*)frow + l);
      } else {
        uint64_t slot = remote_idx ? (uint64_t)__ldg(remote_idx + i) : 0ull;
        v.x = wire_word(4 * l + 0, dim, payload, frow, ts, r, slot);
        v.y = wire_word(4 * l + 1, dim, payload, frow, ts, r, slot);
        v.z = wire_word(4 * l + 2, dim, payload, frow, ts, r, slot);
        v.w = wire_word(4 * l + 3, dim, payload, frow, ts, r, slot);
      }
      ((uint4*)packed)[q] = v;
    } else {
      uint64_t slot = (remote_idx && l >= payload) ? (uint64_t)__ldg(remote_idx + i) : 0ull;
      ((uint32_t*)packed)[q] = wire_word(l, dim, payload, frow, ts, r, slot);
    }
  }
}

template <int VEC>
__global__ void __launch_bounds__(kLaneThreads)
route_unpack_kernel(const float* __restrict__ packed, int64_t n, uint32_t width, uint32_t pitch, float* __restrict__ data,
                    int64_t data_rows, uint32_t dim, float* __restrict__ ts_table, int32_t* d_status) {
  const uint32_t lanes = (width + VEC - 1) / VEC;   // lanes that carry payload
  const int64_t total = n * lanes;
  const int64_t stride = (int64_t)gridDim.x * kLaneThreads;
  for (int64_t q = (int64_t)blockIdx.x * kLaneThreads + threadIdx.x; q < total; q += stride) {
    int64_t i = q / lanes;
    uint32_t l = (uint32_t)(q - i * lanes);
    const uint32_t* row = (const uint32_t*)packed + i * pitch;
    int64_t slot = (int64_t)((uint64_t)__ldg(row + width) | ((uint64_t)__ldg(row + width + 1) << 32));
    if (slot < 0 || slot >= data_rows) {
      dev_flag(d_status, SGL_DEV_BAD_INDEX);
      continue;
    }
    if (VEC == 4) {
      uint4 v = ld_stream((const uint4*)row + l);
      if ((l + 1) * 4 <= dim) ((uint4*)(data + slot * dim))[l] = v;
      else if (ts_table) ts_table[slot] = __uint_as_float(v.x);   // dim % 4 == 0: the lane after the features starts with ts
    } else {
      float v = __uint_as_float(__ldg(row + l));
      if (l < dim) data[slot * dim + l] = v;
      else if (ts_table) ts_table[slot] = v;
    }
  }
}

__global__ void __launch_bounds__(kLaneThreads)
route_add_kernel(float* __restrict__ x, int64_t n_rows, uint32_t dim, const int64_t* __restrict__ send_idx,
                 const float* __restrict__ outs, int64_t seg_len, int32_t* d_status) {
  const int64_t total = seg_len * dim;
  const int64_t stride = (int64_t)gridDim.x * kLaneThreads;
  for (int64_t q = (int64_t)blockIdx.x * kLaneThreads + threadIdx.x; q < total; q += stride) {
    int64_t i = q / dim;
    uint32_t l = (uint32_t)(q - i * dim);
    int64_t r = __ldg(send_idx + i);
    if (r < 0) r += n_rows;
    if (r < 0 || r >= n_rows) {
      dev_flag(d_status, SGL_DEV_BAD_INDEX);
      continue;
    }
    x[r * dim + l] += outs[q];
  }
}

// Reverse-route accumulate over ALL peer segments in one launch.  The received rows are grouped by the row of x they
// add to (row_ptr / pos: for destination row rows[u] the positions pos[row_ptr[u] .. row_ptr[u+1]) of `outs`, ascending,
// i.e. in peer order); one warp owns one destination row and adds its contributions one after the other, which is
// the summation order of a per-peer loop -- the float32 result is the same bit for bit.
__global__ void __launch_bounds__(kLaneThreads)
route_add_grouped_kernel(float* __restrict__ x, int64_t n_rows, uint32_t dim, const int64_t* __restrict__ rows,
                         const int64_t* __restrict__ row_ptr, const int64_t* __restrict__ pos, int64_t n_groups,
                         const float* __restrict__ outs, int64_t n_outs, int32_t* d_status) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kLaneThreads / 32);
  for (int64_t u = ((int64_t)blockIdx.x * kLaneThreads + threadIdx.x) >> 5; u < n_groups; u += warps) {
    int64_t r = __ldg(rows + u);
    if (r < 0) r += n_rows;
    if (r < 0 || r >= n_rows) {
      if (lane == 0) dev_flag(d_status, SGL_DEV_BAD_INDEX);
      continue;
    }
    const int64_t a = __ldg(row_ptr + u), b = __ldg(row_ptr + u + 1);
    for (uint32_t l = lane; l < dim; l += 32) {
      float acc = x[r * dim + l];
      for (int64_t j = a; j < b; ++j) {
        const int64_t p = __ldg(pos + j);
        if (p >= 0 && p < n_outs) acc += __ldg(outs + p * dim + l);
        else dev_flag(d_status, SGL_DEV_BAD_INDEX);
      }
      x[r * dim + l] = acc;
    }
  }
}

// Gather from a table whose rows live on several GPUs of one node: id = (partition << 48) | local row (the packed
// route index); the row is read straight from its owner's memory over NVLink (plain 128-bit / 32-bit loads of a peer
// mapping), so every row crosses the link once and no id or row exchange is needed.
template <typename V>
__global__ void __launch_bounds__(kLaneThreads)
shard_gather_kernel(const char* const* __restrict__ bases, const int64_t* __restrict__ shard_rows, int world,
                    uint32_t lanes_per_row, int64_t row_bytes, const int64_t* __restrict__ dist_idx, int64_t n_cap,
                    const int64_t* d_n, char* __restrict__ out, int32_t* d_status) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t total = n * lanes_per_row;
  const int64_t stride = (int64_t)gridDim.x * kLaneThreads;
  for (int64_t q0 = (int64_t)blockIdx.x * kLaneThreads + threadIdx.x; q0 < total; q0 += stride * kLaneUnroll) {
    V v[kLaneUnroll];
    V* dst[kLaneUnroll];
#pragma unroll
    for (int u = 0; u < kLaneUnroll; ++u) {
      const int64_t q = q0 + u * stride;
      dst[u] = nullptr;
      if (q < total) {
        const int64_t i = q / lanes_per_row;
        const uint32_t l = (uint32_t)(q - i * lanes_per_row);
        const int64_t id = __ldg(dist_idx + i);
        const int64_t part = (id >> 48) & 0x3FFF, loc = id & 0xFFFFFFFFFFFFll;
        if (part >= world || loc >= __ldg(shard_rows + part)) {
          dev_flag(d_status, SGL_DEV_BAD_INDEX);
        } else {
          v[u] = ld_stream((const V*)(bases[part] + loc * row_bytes) + l);
          dst[u] = (V*)(out + i * row_bytes) + l;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kLaneUnroll; ++u)
      if (dst[u]) st_stream(dst[u], v[u]);
  }
}

__global__ void dist_pack_kernel(const int64_t* __restrict__ loc, const int64_t* __restrict__ part,
                                 const uint8_t* __restrict__ shared, int64_t n, int64_t* __restrict__ dist) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    uint64_t d = ((uint64_t)loc[i] & 0xFFFFFFFFFFFFull) | (((uint64_t)part[i] & 0x3FFFull) << 48);
    if (shared && shared[i]) d |= (1ull << 62);
    dist[i] = (int64_t)d;
  }
}

__global__ void dist_unpack_kernel(const int64_t* __restrict__ dist, int64_t n, int64_t* __restrict__ loc,
                                   int64_t* __restrict__ part, uint8_t* __restrict__ shared) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t d = dist[i];
    if (loc) loc[i] = d & 0xFFFFFFFFFFFFll;
    if (part) part[i] = (d >> 48) & 0x3FFF;
    if (shared) shared[i] = (d >> 62) != 0;  // arithmetic shift, then "non-zero", as the reference's bool cast
  }
}

constexpr int kReplicaThreads = 256;

__global__ void __launch_bounds__(kReplicaThreads)
replica_count_kernel(const int64_t* __restrict__ indptr, int64_t num_nodes, const int64_t* __restrict__ ids, int64_t n,
                     int64_t* __restrict__ local_off, int64_t* __restrict__ cta_sums, unsigned int* done_counter,
                     int64_t* out_total, int32_t* d_status) {
  const int64_t i = (int64_t)blockIdx.x * kReplicaThreads + threadIdx.x;
  int64_t len = 0;
  if (i < n) {
    int64_t id = ids[i];
    if (id < 0 || id >= num_nodes) dev_flag(d_status, SGL_DEV_BAD_NODE);
    else len = indptr[id + 1] - indptr[id];
  }
  int64_t total;
  int64_t ex = cta_exclusive_scan<kReplicaThreads, int64_t>(len, &total);
  if (i < n) local_off[i] = ex;
  publish_and_scan_cta_totals<kReplicaThreads>(total, cta_sums, done_counter, out_total);
}

__global__ void __launch_bounds__(kReplicaThreads)
replica_expand_kernel(const int64_t* __restrict__ indptr, const int64_t* __restrict__ ranks,
                      const int64_t* __restrict__ locs, int64_t num_nodes, const int64_t* __restrict__ ids, int64_t n,
                      int64_t cap, const int64_t* __restrict__ local_off, const int64_t* __restrict__ cta_sums,
                      int64_t* __restrict__ out_src, int64_t* __restrict__ out_rank, int64_t* __restrict__ out_loc,
                      int64_t* __restrict__ out_offsets, int32_t* d_status) {
  const int64_t i = (int64_t)blockIdx.x * kReplicaThreads + threadIdx.x;
  if (i >= n) return;
  int64_t off = cta_sums[blockIdx.x] + local_off[i];
  out_offsets[i] = off;
  int64_t id = ids[i];
  if (id < 0 || id >= num_nodes) return;
  int64_t s = indptr[id], e = indptr[id + 1];
  for (int64_t p = s; p < e; ++p, ++off) {
    if (off >= cap) {
      dev_flag(d_status, SGL_DEV_OVERFLOW);
      return;
    }
    out_src[off] = i;
    out_rank[off] = ranks[p];
    out_loc[off] = locs[p];
  }
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }


// ---- device-counted prefix copy ------------------------------------------------------------------------------
// Copies the first *d_count elements of up to 8 arrays in one launch (an array with a negative element size is
// copied whole: that many bytes).  The destination may be pinned host memory: a batch's result then crosses PCIe with
// exactly the bytes it has, although its size is only known on the device.
struct PrefixCopy {
  const char* src[8];
  char* dst[8];
  int64_t elem_bytes[8];
  int n;
};

__global__ void __launch_bounds__(256)
copy_prefix_kernel(PrefixCopy pc, const int64_t* __restrict__ d_count, int64_t cap) {
  int64_t cnt = *d_count;
  cnt = cnt < 0 ? 0 : (cnt > cap ? cap : cnt);
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int a = 0; a < pc.n; ++a) {
    const int64_t bytes = pc.elem_bytes[a] < 0 ? -pc.elem_bytes[a] : cnt * pc.elem_bytes[a];
    const int64_t vec = bytes >> 4;
    const uint4* s = (const uint4*)pc.src[a];
    uint4* d = (uint4*)pc.dst[a];
    for (int64_t u = tid; u < vec; u += stride) d[u] = s[u];
    for (int64_t b = (vec << 4) + tid; b < bytes; b += stride) pc.dst[a][b] = pc.src[a][b];
  }
}

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" int sgl_gather_rows(const void* table, int64_t table_rows, int64_t row_bytes, int64_t src_pitch,
                               const int64_t* idx, const int64_t* map, int64_t map_len, int64_t n, const int64_t* d_n,
                               void* out, int64_t dst_pitch, const float* ts_table, float* out_ts, int mode,
                               int32_t* d_status, void* stream_) {
  SGL_NVTX("sgl_gather_rows");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && table_rows >= 0 && row_bytes > 0, SGL_ERR_ARG, "gather_rows: bad size");
  SGL_REQUIRE(src_pitch >= row_bytes && dst_pitch >= row_bytes, SGL_ERR_ARG, "gather_rows: pitch smaller than row");
  SGL_REQUIRE(row_bytes % 4 == 0 && src_pitch % 4 == 0 && dst_pitch % 4 == 0, SGL_ERR_UNSUPPORTED,
              "gather_rows: rows must be multiples of 4 bytes");
  SGL_REQUIRE((ts_table == nullptr) == (out_ts == nullptr), SGL_ERR_ARG, "gather_rows: ts_table/out_ts must come together");
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(table && idx && out, SGL_ERR_ARG, "gather_rows: null array");
  SGL_REQUIRE(map == nullptr || map_len > 0, SGL_ERR_ARG, "gather_rows: empty map");
  const bool vec_ok = row_bytes % 16 == 0 && src_pitch % 16 == 0 && dst_pitch % 16 == 0 && aligned16(table) && aligned16(out);
  // bulk configuration: 4 warps x 3 stages per CTA, two CTAs per SM, about 5.5 KB per stage (8 rows of 688 bytes)
  constexpr int64_t kBulkBudget = 200 * 1024 / 2;
  int rows_per_stage = (int)(kBulkBudget / ((int64_t)kBulkWarps * kBulkStages * row_bytes));
  {
    const int want_rows = (int)((5632 + row_bytes - 1) / row_bytes);
    if (rows_per_stage > want_rows) rows_per_stage = want_rows;
    if (rows_per_stage > 32) rows_per_stage = 32;
  }
  if (mode == SGL_GATHER_AUTO) {
    // measured on B200: the bulk-copy pipeline beats 128-bit lanes from 512-byte rows up; below that they tie.  Rows
    // of which fewer than two fit a stage (above about 4 KB) go through the lanes kernel.
    const bool bulk_ok = vec_ok && dst_pitch == row_bytes && row_bytes >= 512 && rows_per_stage >= 2 && n >= 1024;
    mode = bulk_ok ? SGL_GATHER_BULK : (vec_ok ? SGL_GATHER_VEC : 0);
  }
  if (mode == SGL_GATHER_BULK) {
    SGL_REQUIRE(vec_ok && dst_pitch == row_bytes, SGL_ERR_UNSUPPORTED,
                "gather_rows: bulk mode needs 16-byte rows and a dense output");
    SGL_REQUIRE(rows_per_stage >= 2, SGL_ERR_UNSUPPORTED, "gather_rows: row of %lld bytes too large for bulk mode",
                (long long)row_bytes);
    const size_t smem = (size_t)kBulkWarps * kBulkStages * rows_per_stage * row_bytes;
    const int64_t chunks = (n + rows_per_stage - 1) / rows_per_stage;
    int64_t ctas = (chunks + kBulkWarps - 1) / kBulkWarps;
    if (ctas > (int64_t)kNumSM * 2) ctas = (int64_t)kNumSM * 2;  // persistent CTAs
    SGL_CUDA_CHECK(cudaFuncSetAttribute(gather_bulk_kernel<kBulkWarps, kBulkStages>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    gather_bulk_kernel<kBulkWarps, kBulkStages><<<(unsigned)ctas, kBulkWarps * 32, smem, stream>>>(
        (const char*)table, table_rows, (uint32_t)row_bytes, src_pitch, idx, map, map_len, n, d_n, (char*)out, ts_table,
        out_ts, rows_per_stage, d_status);
    SGL_LAUNCH_CHECK();
    return SGL_OK;
  }
  if (mode == SGL_GATHER_VEC) {
    SGL_REQUIRE(vec_ok, SGL_ERR_UNSUPPORTED, "gather_rows: 128-bit mode needs 16-byte aligned rows");
    const uint32_t lanes = (uint32_t)(row_bytes / 16);
    const int grid = stream_grid(n * lanes, kLaneThreads * kLaneUnroll, 8);
    gather_lanes_kernel<uint4><<<grid, kLaneThreads, 0, stream>>>((const char*)table, table_rows, LaneSplit(lanes, n * lanes), src_pitch, idx,
                                                                 map, map_len, n, d_n, (char*)out, dst_pitch, ts_table,
                                                                 out_ts, d_status);
  } else {
    const uint32_t lanes = (uint32_t)(row_bytes / 4);
    const int grid = stream_grid(n * lanes, kLaneThreads * kLaneUnroll, 8);
    gather_lanes_kernel<uint32_t><<<grid, kLaneThreads, 0, stream>>>((const char*)table, table_rows, LaneSplit(lanes, n * lanes), src_pitch,
                                                                    idx, map, map_len, n, d_n, (char*)out, dst_pitch,
                                                                    ts_table, out_ts, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_copy_prefix(int n_arrays, const void* const* src, void* const* dst, const int64_t* elem_bytes,
                               const int64_t* d_count, int64_t cap, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n_arrays >= 0 && n_arrays <= 8 && cap >= 0 && d_count, SGL_ERR_ARG, "copy_prefix: at most 8 arrays, non-null count");
  if (n_arrays == 0) return SGL_OK;
  PrefixCopy pc;
  memset(&pc, 0, sizeof(pc));
  pc.n = n_arrays;
  int64_t most = 0;
  for (int a = 0; a < n_arrays; ++a) {
    SGL_REQUIRE(src && dst && elem_bytes && src[a] && dst[a] && elem_bytes[a] != 0, SGL_ERR_ARG, "copy_prefix: bad array %d", a);
    SGL_REQUIRE((((uintptr_t)src[a] | (uintptr_t)dst[a]) & 15) == 0, SGL_ERR_ARG, "copy_prefix: array %d is not 16-byte aligned", a);
    pc.src[a] = (const char*)src[a];
    pc.dst[a] = (char*)dst[a];
    pc.elem_bytes[a] = elem_bytes[a];
    const int64_t b = elem_bytes[a] < 0 ? -elem_bytes[a] : cap * elem_bytes[a];
    most = most > b ? most : b;
  }
  copy_prefix_kernel<<<stream_grid(most / 16 + 1, 256 * 4, 2), 256, 0, stream>>>(pc, d_count, cap);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" size_t sgl_cache_gather_ws_bytes(int64_t n) {
  if (n < 1) n = 1;
  int64_t ctas = (n + kCacheThreads - 1) / kCacheThreads;
  return 2 * align_up((size_t)n * 4) + align_up((size_t)ctas * 8) + align_up(sizeof(unsigned int));
}

extern "C" int sgl_cache_gather(const void* cache_rows, int64_t cache_slots, const int32_t* hitmap, int64_t num_ids,
                                const void* backing, int64_t row_bytes, const int64_t* ids, int64_t n, void* out,
                                int64_t* miss_pos, int64_t* miss_ids, int64_t* d_counts, int32_t* d_status, void* ws,
                                size_t ws_bytes, void* stream_) {
  SGL_NVTX("sgl_cache_gather");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && row_bytes > 0 && row_bytes % 4 == 0, SGL_ERR_ARG, "cache_gather: bad size");
  SGL_REQUIRE(d_counts, SGL_ERR_ARG, "cache_gather: d_counts is null");
  if (n == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(d_counts, 0, 2 * sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE(cache_rows && hitmap && ids && out && miss_pos && miss_ids, SGL_ERR_ARG, "cache_gather: null array");
  WsCarver c(ws, ws_bytes);
  int32_t* slot_ws = c.take<int32_t>(n);
  int32_t* rank_ws = c.take<int32_t>(n);
  const int64_t ctas = (n + kCacheThreads - 1) / kCacheThreads;
  int64_t* cta_miss = c.take<int64_t>(ctas);
  unsigned int* done = c.take<unsigned int>(1);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "cache_gather: workspace %zu < %zu bytes", ws_bytes, sgl_cache_gather_ws_bytes(n));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
  cache_lookup_kernel<<<(unsigned)ctas, kCacheThreads, 0, stream>>>(hitmap, num_ids, ids, n, slot_ws, rank_ws, cta_miss,
                                                                   done, d_counts, d_status);
  const bool vec_ok = row_bytes % 16 == 0 && aligned16(cache_rows) && aligned16(out) && (backing == nullptr || aligned16(backing));
  if (vec_ok) {
    const uint32_t lanes = (uint32_t)(row_bytes / 16);
    const int grid = stream_grid(n * lanes, kLaneThreads * kLaneUnroll, 8);
    cache_copy_kernel<uint4><<<grid, kLaneThreads, 0, stream>>>((const char*)cache_rows, cache_slots, (const char*)backing,
                                                               LaneSplit(lanes, n * lanes), row_bytes, ids, n, slot_ws, rank_ws, cta_miss,
                                                               (char*)out, miss_pos, miss_ids, d_counts, d_status);
  } else {
    const uint32_t lanes = (uint32_t)(row_bytes / 4);
    const int grid = stream_grid(n * lanes, kLaneThreads * kLaneUnroll, 8);
    cache_copy_kernel<uint32_t><<<grid, kLaneThreads, 0, stream>>>((const char*)cache_rows, cache_slots,
                                                                  (const char*)backing, LaneSplit(lanes, n * lanes), row_bytes, ids, n, slot_ws,
                                                                  rank_ws, cta_miss, (char*)out, miss_pos, miss_ids,
                                                                  d_counts, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_scatter_rows(void* table, int64_t table_rows, int64_t row_bytes, int64_t dst_pitch, const int64_t* idx,
                                const int64_t* map, int64_t map_len, int64_t n, const int64_t* d_n, const void* rows,
                                int64_t src_pitch, float* ts_table, const float* ts, int split_last_col,
                                int32_t* d_status, void* stream_) {
  SGL_NVTX("sgl_scatter_rows");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && table_rows >= 0 && row_bytes > 0 && row_bytes % 4 == 0, SGL_ERR_ARG, "scatter_rows: bad size");
  SGL_REQUIRE(dst_pitch >= row_bytes && src_pitch >= row_bytes + (split_last_col ? 4 : 0), SGL_ERR_ARG,
              "scatter_rows: pitch smaller than row");
  SGL_REQUIRE(!split_last_col || ts_table, SGL_ERR_ARG, "scatter_rows: split_last_col needs ts_table");
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(table && idx && rows, SGL_ERR_ARG, "scatter_rows: null array");
  const bool vec_ok = row_bytes % 16 == 0 && src_pitch % 16 == 0 && dst_pitch % 16 == 0 && aligned16(table) && aligned16(rows);
  if (vec_ok) {
    const uint32_t lanes = (uint32_t)(row_bytes / 16);
    const int grid = stream_grid(n * lanes, kLaneThreads, 16);
    scatter_lanes_kernel<uint4><<<grid, kLaneThreads, 0, stream>>>((char*)table, table_rows, lanes, row_bytes, dst_pitch, idx,
                                                                  map, map_len, n, d_n, (const char*)rows, src_pitch,
                                                                  ts_table, ts, split_last_col, d_status);
  } else {
    const uint32_t lanes = (uint32_t)(row_bytes / 4);
    const int grid = stream_grid(n * lanes, kLaneThreads, 16);
    scatter_lanes_kernel<uint32_t><<<grid, kLaneThreads, 0, stream>>>((char*)table, table_rows, lanes, row_bytes, dst_pitch,
                                                                     idx, map, map_len, n, d_n, (const char*)rows,
                                                                     src_pitch, ts_table, ts, split_last_col, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int64_t sgl_wire_pitch(int64_t dim, int has_ts, int has_slot) {
  int64_t w = dim + (has_ts ? 1 : 0);
  return has_slot ? (w + 2 + 3) / 4 * 4 : w;
}

extern "C" int sgl_route_pack(const float* feats, int64_t n_rows, int64_t dim, const float* ts, const int64_t* send_idx,
                              const int64_t* remote_idx, int64_t n_send, float* packed, int32_t* d_status,
                              void* stream_) {
  SGL_NVTX("sgl_route_pack");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n_send >= 0 && n_rows >= 0 && dim > 0, SGL_ERR_ARG, "route_pack: bad size");
  if (n_send == 0) return SGL_OK;
  SGL_REQUIRE(feats && send_idx && packed, SGL_ERR_ARG, "route_pack: null array");
  const int64_t pitch = sgl_wire_pitch(dim, ts != nullptr, remote_idx != nullptr);
  const bool vec = dim % 4 == 0 && pitch % 4 == 0 && aligned16(feats) && aligned16(packed);
  if (vec) {
    const int grid = stream_grid(n_send * (pitch / 4), kLaneThreads, 16);
    route_pack_kernel<4><<<grid, kLaneThreads, 0, stream>>>(feats, n_rows, (uint32_t)dim, ts, send_idx, remote_idx, n_send,
                                                           (uint32_t)pitch, packed, d_status);
  } else {
    const int grid = stream_grid(n_send * pitch, kLaneThreads, 16);
    route_pack_kernel<1><<<grid, kLaneThreads, 0, stream>>>(feats, n_rows, (uint32_t)dim, ts, send_idx, remote_idx, n_send,
                                                           (uint32_t)pitch, packed, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_route_unpack(const float* packed, int64_t n, int64_t width, float* data, int64_t data_rows,
                                int64_t dim, float* ts_table, int32_t* d_status, void* stream_) {
  SGL_NVTX("sgl_route_unpack");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && data_rows >= 0 && dim > 0, SGL_ERR_ARG, "route_unpack: bad size");
  SGL_REQUIRE(width == dim || width == dim + 1, SGL_ERR_ARG, "route_unpack: width %lld must be dim or dim+1 (dim=%lld)",
              (long long)width, (long long)dim);
  SGL_REQUIRE(width == dim || ts_table, SGL_ERR_ARG, "route_unpack: rows carry a timestamp but ts_table is null");
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(packed && data, SGL_ERR_ARG, "route_unpack: null array");
  const int64_t pitch = sgl_wire_pitch(dim, width > dim, 1);
  const bool vec = dim % 4 == 0 && aligned16(packed) && aligned16(data);
  if (vec) {
    const int grid = stream_grid(n * ((width + 3) / 4), kLaneThreads, 16);
    route_unpack_kernel<4><<<grid, kLaneThreads, 0, stream>>>(packed, n, (uint32_t)width, (uint32_t)pitch, data, data_rows,
                                                             (uint32_t)dim, ts_table, d_status);
  } else {
    const int grid = stream_grid(n * width, kLaneThreads, 16);
    route_unpack_kernel<1><<<grid, kLaneThreads, 0, stream>>>(packed, n, (uint32_t)width, (uint32_t)pitch, data, data_rows,
                                                             (uint32_t)dim, ts_table, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_route_add_rows(float* x, int64_t n_rows, int64_t dim, const int64_t* send_idx, const float* outs,
                                  int64_t seg_len, int32_t* d_status, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(seg_len >= 0 && n_rows >= 0 && dim > 0, SGL_ERR_ARG, "route_add_rows: bad size");
  if (seg_len == 0) return SGL_OK;
  SGL_REQUIRE(x && send_idx && outs, SGL_ERR_ARG, "route_add_rows: null array");
  const int grid = stream_grid(seg_len * dim, kLaneThreads, 16);
  route_add_kernel<<<grid, kLaneThreads, 0, stream>>>(x, n_rows, (uint32_t)dim, send_idx, outs, seg_len, d_status);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_route_add_grouped(float* x, int64_t n_rows, int64_t dim, const int64_t* rows, const int64_t* row_ptr,
                                     const int64_t* pos, int64_t n_groups, const float* outs, int64_t n_outs,
                                     int32_t* d_status, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n_groups >= 0 && n_rows >= 0 && n_outs >= 0 && dim > 0, SGL_ERR_ARG, "route_add_grouped: bad size");
  if (n_groups == 0) return SGL_OK;
  SGL_REQUIRE(x && rows && row_ptr && pos && outs, SGL_ERR_ARG, "route_add_grouped: null array");
  const int grid = stream_grid(n_groups, kLaneThreads / 32, 16);
  route_add_grouped_kernel<<<grid, kLaneThreads, 0, stream>>>(x, n_rows, (uint32_t)dim, rows, row_ptr, pos, n_groups, outs,
                                                             n_outs, d_status);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_shard_gather(const void* const* d_bases, const int64_t* d_shard_rows, int world, int64_t row_bytes,
                                const int64_t* dist_idx, int64_t n, const int64_t* d_n, void* out, int32_t* d_status,
                                void* stream_) {
  SGL_NVTX("sgl_shard_gather");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && world >= 1 && world <= 0x3FFF && row_bytes > 0 && row_bytes % 4 == 0, SGL_ERR_ARG,
              "shard_gather: bad size (rows must be multiples of 4 bytes)");
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(d_bases && d_shard_rows && dist_idx && out, SGL_ERR_ARG, "shard_gather: null array");
  // the shard base pointers are device values: their 16-byte alignment is the caller's contract (cudaMalloc gives 256)
  if (row_bytes % 16 == 0 && aligned16(out)) {
    const uint32_t lanes = (uint32_t)(row_bytes / 16);
    shard_gather_kernel<uint4><<<stream_grid(n * lanes, kLaneThreads * kLaneUnroll, 8), kLaneThreads, 0, stream>>>(
        (const char* const*)d_bases, d_shard_rows, world, lanes, row_bytes, dist_idx, n, d_n, (char*)out, d_status);
  } else {
    const uint32_t lanes = (uint32_t)(row_bytes / 4);
    shard_gather_kernel<uint32_t><<<stream_grid(n * lanes, kLaneThreads * kLaneUnroll, 8), kLaneThreads, 0, stream>>>(
        (const char* const*)d_bases, d_shard_rows, world, lanes, row_bytes, dist_idx, n, d_n, (char*)out, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_dist_pack(const int64_t* loc, const int64_t* part, const uint8_t* shared, int64_t n, int64_t* dist,
                             void* stream_) {
  SGL_REQUIRE(n >= 0, SGL_ERR_ARG, "dist_pack: negative size");
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(loc && part && dist, SGL_ERR_ARG, "dist_pack: null array");
  dist_pack_kernel<<<stream_grid(n, 256, 8), 256, 0, (cudaStream_t)stream_>>>(loc, part, shared, n, dist);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_dist_unpack(const int64_t* dist, int64_t n, int64_t* loc, int64_t* part, uint8_t* shared,
                               void* stream_) {
  SGL_REQUIRE(n >= 0, SGL_ERR_ARG, "dist_unpack: negative size");
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(dist, SGL_ERR_ARG, "dist_unpack: null array");
  dist_unpack_kernel<<<stream_grid(n, 256, 8), 256, 0, (cudaStream_t)stream_>>>(dist, n, loc, part, shared);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" size_t sgl_replica_lookup_ws_bytes(int64_t n) {
  if (n < 1) n = 1;
  int64_t ctas = (n + kReplicaThreads - 1) / kReplicaThreads;
  return align_up((size_t)n * 8) + align_up((size_t)ctas * 8) + align_up(sizeof(unsigned int));
}

extern "C" int sgl_replica_lookup(const int64_t* indptr, const int64_t* ranks, const int64_t* locs, int64_t num_nodes,
                                  const int64_t* ids, int64_t n, int64_t cap, int64_t* out_src, int64_t* out_rank,
                                  int64_t* out_loc, int64_t* out_offsets, int32_t* d_status, void* ws, size_t ws_bytes,
                                  void* stream_) {
  SGL_NVTX("sgl_replica_lookup");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n >= 0 && cap >= 0 && num_nodes >= 0, SGL_ERR_ARG, "replica_lookup: negative size");
  SGL_REQUIRE(out_offsets, SGL_ERR_ARG, "replica_lookup: out_offsets is null");
  if (n == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(out_offsets, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE(indptr && ranks && locs && ids && out_src && out_rank && out_loc, SGL_ERR_ARG, "replica_lookup: null array");
  WsCarver c(ws, ws_bytes);
  int64_t* local_off = c.take<int64_t>(n);
  const int64_t ctas = (n + kReplicaThreads - 1) / kReplicaThreads;
  int64_t* cta_sums = c.take<int64_t>(ctas);
  unsigned int* done = c.take<unsigned int>(1);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "replica_lookup: workspace %zu < %zu bytes", ws_bytes,
              sgl_replica_lookup_ws_bytes(n));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
  replica_count_kernel<<<(unsigned)ctas, kReplicaThreads, 0, stream>>>(indptr, num_nodes, ids, n, local_off, cta_sums, done,
                                                                      out_offsets + n, d_status);
  replica_expand_kernel<<<(unsigned)ctas, kReplicaThreads, 0, stream>>>(indptr, ranks, locs, num_nodes, ids, n, cap,
                                                                       local_off, cta_sums, out_src, out_rank, out_loc,
                                                                       out_offsets, d_status);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}
