// Stable LSD radix sort, 8 bits per pass, three kernels per pass:
//   1. sort_hist_kernel    per-CTA digit histogram of its tile (4096 keys)          -> block_hist[digit][cta]
//   2. sort_scan_kernel    one CTA per digit: exclusive scan over CTAs + digit total
//   3. sort_scatter_kernel re-reads the tile, ranks keys stably (warp match + per-warp running counters), lays the
//                          tile out in digit order in shared memory and writes every digit's run with consecutive
//                          threads (coalesced runs instead of scattered 8- and 4-byte stores)
// HBM traffic per pass and key: 8 B (histogram read) + 12 B read + 12 B write.
#include "sort.cuh"

namespace sgl {

namespace {

__device__ __forceinline__ uint32_t digit_of(uint64_t key, int shift) {
  return (uint32_t)(key >> shift) & (kSortRadix - 1);
}

__global__ void __launch_bounds__(kSortThreads)
sort_hist_kernel(const uint64_t* __restrict__ keys, int64_t n_cap, const int64_t* d_n, int shift,
                 uint32_t* __restrict__ block_hist, int num_blocks) {
  __shared__ uint32_t hist[kSortRadix];
  const int64_t n = eff_count(n_cap, d_n);
  hist[threadIdx.x] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t base = (int64_t)blockIdx.x * kSortTile + (int64_t)warp * (kSortItems * 32) + lane;
#pragma unroll
  for (int c = 0; c < kSortItems; ++c) {
    int64_t i = base + c * 32;
    if (i < n) atomicAdd(&hist[digit_of(keys[i], shift)], 1u);
  }
  __syncthreads();
  block_hist[(size_t)threadIdx.x * num_blocks + blockIdx.x] = hist[threadIdx.x];
}

// one CTA per digit: exclusive scan of block_hist[digit][0..num_blocks) in place, total -> digit_total[digit]
__global__ void __launch_bounds__(256)
sort_scan_kernel(uint32_t* __restrict__ block_hist, int num_blocks, uint32_t* __restrict__ digit_total) {
  __shared__ uint32_t warp_sums[8];
  __shared__ uint32_t carry_s;
  uint32_t* row = block_hist + (size_t)blockIdx.x * num_blocks;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < num_blocks; base += 256) {
    int i = base + threadIdx.x;
    uint32_t v = i < num_blocks ? row[i] : 0;
    uint32_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    uint32_t woff = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < warp) woff += warp_sums[w];
    uint32_t carry = carry_s;
    if (i < num_blocks) row[i] = carry + woff + x - v;
    __syncthreads();
    if (threadIdx.x == 255) carry_s = carry + woff + x;
    __syncthreads();
  }
  if (threadIdx.x == 0) digit_total[blockIdx.x] = carry_s;
}

// Shared memory of the scatter kernel: the tile's keys and payloads in digit order, the per-warp digit counters and
// two per-digit tables.
constexpr size_t kScatterSmem = (size_t)kSortTile * 12 + (size_t)(kSortThreads / 32) * kSortRadix * 4 + 2 * kSortRadix * 4;

__global__ void __launch_bounds__(kSortThreads, 3)   // three tiles per SM: their load / rank / write phases overlap
sort_scatter_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n_cap,
                    const int64_t* d_n, int shift, const uint32_t* __restrict__ block_hist, int num_blocks,
                    const uint32_t* __restrict__ digit_total, uint64_t* __restrict__ out_keys,
                    uint32_t* __restrict__ out_vals) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint64_t* s_keys = (uint64_t*)smem;                                             // [kSortTile]
  uint32_t* s_vals = (uint32_t*)(s_keys + kSortTile);                             // [kSortTile]
  uint32_t(*warp_cnt)[kSortRadix] = (uint32_t(*)[kSortRadix])(s_vals + kSortTile);  // [warps][radix]
  uint32_t* glob_base = (uint32_t*)(warp_cnt + kSortThreads / 32);                // [radix] where this tile's run of a digit starts
  uint32_t* tile_start = glob_base + kSortRadix;                                  // [radix] start of the digit inside the tile
  __shared__ uint32_t scan_tmp[8];
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t tile_base = (int64_t)blockIdx.x * kSortTile;
  if (tile_base >= n) return;                                   // nothing in this tile (device-side count below capacity)
  const int tile_n = (int)(n - tile_base < kSortTile ? n - tile_base : kSortTile);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // global start of every digit (exclusive scan of the 256 totals) + this tile's offset inside the digit
  {
    uint32_t v = digit_total[threadIdx.x];
    uint32_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) scan_tmp[warp] = x;
    __syncthreads();
    uint32_t woff = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < warp) woff += scan_tmp[w];
    glob_base[threadIdx.x] = woff + x - v + block_hist[(size_t)threadIdx.x * num_blocks + blockIdx.x];
  }
#pragma unroll
  for (int w = 0; w < kSortThreads / 32; ++w) warp_cnt[w][threadIdx.x] = 0;
  __syncthreads();

  // warp w owns items [w * 512, (w + 1) * 512) of the tile, 32 at a time: (warp, round, lane) order = key order
  const int64_t base = tile_base + (int64_t)warp * (kSortItems * 32) + lane;
  uint64_t k[kSortItems];
  uint32_t v[kSortItems];
#pragma unroll
  for (int c = 0; c < kSortItems; ++c) {
    const int64_t i = base + c * 32;
    k[c] = i < n ? keys[i] : 0;
    v[c] = i < n ? (vals ? vals[i] : (uint32_t)i) : 0u;
    if (i < n) atomicAdd(&warp_cnt[warp][digit_of(k[c], shift)], 1u);
  }
  __syncthreads();
  // per digit: counts of the warps -> start of every warp's keys inside the tile (digit-major, then warp order)
  {
    uint32_t run = 0;
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) {
      const uint32_t c = warp_cnt[w][threadIdx.x];
      warp_cnt[w][threadIdx.x] = run;
      run += c;
    }
    uint32_t x = run;   // keys of this digit in the tile
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    __syncthreads();    // scan_tmp is free again
    if (lane == 31) scan_tmp[warp] = x;
    __syncthreads();
    uint32_t woff = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < warp) woff += scan_tmp[w];
    const uint32_t start = woff + x - run;
    tile_start[threadIdx.x] = start;
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) warp_cnt[w][threadIdx.x] += start;
  }
  __syncthreads();
  // stable rank of every key inside the tile; the tile is laid out in digit order in shared memory
  const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int c = 0; c < kSortItems; ++c) {
    const int64_t i = base + c * 32;
    const bool valid = i < n;
    const uint32_t d = valid ? digit_of(k[c], shift) : (uint32_t)kSortRadix;
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    const uint32_t rank = __popc(peers & lt_mask);
    uint32_t pos = 0;
    if (valid) pos = warp_cnt[warp][d] + rank;
    __syncwarp();
    if (valid && rank == 0) warp_cnt[warp][d] += __popc(peers);
    __syncwarp();
    if (valid) {
      s_keys[pos] = k[c];
      s_vals[pos] = v[c];
    }
  }
  __syncthreads();
  // write-out: consecutive threads take consecutive tile positions, i.e. runs of one digit -> consecutive addresses
  for (int j = threadIdx.x; j < tile_n; j += kSortThreads) {
    const uint64_t key = s_keys[j];
    const uint32_t d = digit_of(key, shift);
    const uint32_t g = glob_base[d] + ((uint32_t)j - tile_start[d]);
    out_keys[g] = key;
    out_vals[g] = s_vals[j];
  }
}

}  // namespace

size_t radix_sort_ws_bytes(int64_t n) {
  int64_t nb = (n + kSortTile - 1) / kSortTile;
  if (nb < 1) nb = 1;
  return align_up((size_t)nb * kSortRadix * sizeof(uint32_t)) + align_up(kSortRadix * sizeof(uint32_t));
}

int radix_sort_pairs(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n,
                     const int64_t* d_n, int num_bits, bool iota_vals, int* result_in_alt, void* ws, size_t ws_bytes,
                     cudaStream_t stream) {
  SGL_REQUIRE(n >= 0 && n < ((int64_t)1 << 32), SGL_ERR_ARG, "radix sort: n=%lld outside [0, 2^32)", (long long)n);
  SGL_REQUIRE(num_bits >= 0 && num_bits <= 64, SGL_ERR_ARG, "radix sort: num_bits=%d", num_bits);
  *result_in_alt = 0;
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(keys && vals && keys_alt && vals_alt, SGL_ERR_ARG, "radix sort: null buffer");
  const int num_blocks = (int)((n + kSortTile - 1) / kSortTile);
  WsCarver c(ws, ws_bytes);
  uint32_t* block_hist = c.take<uint32_t>((size_t)num_blocks * kSortRadix);
  uint32_t* digit_total = c.take<uint32_t>(kSortRadix);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "radix sort: workspace %zu < %zu bytes", ws_bytes, radix_sort_ws_bytes(n));
  int passes = (num_bits + kSortRadixBits - 1) / kSortRadixBits;
  if (passes == 0 && iota_vals) passes = 1;  // still has to materialise the payload
  uint64_t *kin = keys, *kout = keys_alt;
  uint32_t *vin = vals, *vout = vals_alt;
  static bool smem_set = false;   // the attribute is per device function and context: set it once per process and device
  static int smem_dev = -1;
  int dev = 0;
  SGL_CUDA_CHECK(cudaGetDevice(&dev));
  if (!smem_set || smem_dev != dev) {
    SGL_CUDA_CHECK(cudaFuncSetAttribute(sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScatterSmem));
    smem_set = true;
    smem_dev = dev;
  }
  for (int p = 0; p < passes; ++p) {
    int shift = p * kSortRadixBits;
    sort_hist_kernel<<<num_blocks, kSortThreads, 0, stream>>>(kin, n, d_n, shift, block_hist, num_blocks);
    sort_scan_kernel<<<kSortRadix, 256, 0, stream>>>(block_hist, num_blocks, digit_total);
    sort_scatter_kernel<<<num_blocks, kSortThreads, kScatterSmem, stream>>>(kin, (p == 0 && iota_vals) ? nullptr : vin, n, d_n,
                                                                 shift, block_hist, num_blocks, digit_total, kout, vout);
    SGL_LAUNCH_CHECK();
    uint64_t* tk = kin; kin = kout; kout = tk;
    uint32_t* tv = vin; vin = vout; vout = tv;
  }
  *result_in_alt = (passes & 1);
  return SGL_OK;
}

}  // namespace sgl

extern "C" size_t sgl_radix_sort_ws_bytes(int64_t n) { return sgl::radix_sort_ws_bytes(n); }

extern "C" int sgl_radix_sort_u64_u32(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n,
                                      int num_bits, int* h_result_in_alt, void* ws, size_t ws_bytes, void* stream) {
  int dummy = 0;
  return sgl::radix_sort_pairs(keys, vals, keys_alt, vals_alt, n, nullptr, num_bits, false,
                               h_result_in_alt ? h_result_in_alt : &dummy, ws, ws_bytes, (cudaStream_t)stream);
}
