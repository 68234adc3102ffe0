// Stable LSD radix sort, 8 or 9 bits per pass (whichever needs fewer passes for the key width), three kernels per pass:
//   1. sort_hist_kernel    per-CTA digit histogram of its tile (4096 keys)          -> block_hist[digit][cta]
//   2. sort_scan_kernel    one CTA per digit: exclusive scan over CTAs + digit total
//   3. sort_scatter_kernel re-reads the tile, ranks keys stably (warp match + per-warp running counters), lays the
//                          tile out in digit order in shared memory and writes every digit's run with consecutive
//                          threads (coalesced runs instead of scattered 8- and 4-byte stores)
// HBM traffic per pass and key: 8 B (histogram read) + 12 B read + 12 B write.
#include "sort.cuh"

namespace sgl {

namespace {

constexpr int kMaxRadixBits = 9;
constexpr int kMaxRadix = 1 << kMaxRadixBits;
constexpr int kWarps = kSortThreads / 32;

template <int BITS>
__device__ __forceinline__ uint32_t digit_of(uint64_t key, int shift) {
  return (uint32_t)(key >> shift) & ((1u << BITS) - 1u);
}

// exclusive scan of one value per thread across the CTA (256 threads); tmp = 8 words of shared memory
__device__ __forceinline__ uint32_t cta_scan_u32(uint32_t v, uint32_t* tmp) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();   // tmp may still be read from an earlier call
  if (lane == 31) tmp[warp] = x;
  __syncthreads();
  uint32_t woff = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w)
    if (w < warp) woff += tmp[w];
  return woff + x - v;
}

// Thread t owns the digits [t * DPT, (t + 1) * DPT), DPT = radix / 256.
template <int BITS>
__global__ void __launch_bounds__(kSortThreads)
sort_hist_kernel(const uint64_t* __restrict__ keys, int64_t n_cap, const int64_t* d_n, int shift,
                 uint32_t* __restrict__ block_hist, int num_blocks) {
  constexpr int RADIX = 1 << BITS, DPT = RADIX / kSortThreads;
  __shared__ uint32_t hist[RADIX];
  const int64_t n = eff_count(n_cap, d_n);
#pragma unroll
  for (int q = 0; q < DPT; ++q) hist[threadIdx.x * DPT + q] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t base = (int64_t)blockIdx.x * kSortTile + (int64_t)warp * (kSortItems * 32) + lane;
#pragma unroll
  for (int c = 0; c < kSortItems; ++c) {
    int64_t i = base + c * 32;
    if (i < n) atomicAdd(&hist[digit_of<BITS>(keys[i], shift)], 1u);
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < DPT; ++q) {
    const int d = threadIdx.x * DPT + q;
    block_hist[(size_t)d * num_blocks + blockIdx.x] = hist[d];
  }
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
constexpr size_t scatter_smem(int bits) { return (size_t)kSortTile * 12 + (size_t)(kWarps + 2) * ((size_t)1 << bits) * 4; }

template <int BITS>
__global__ void __launch_bounds__(kSortThreads, 3)   // three tiles per SM: their load / rank / write phases overlap
sort_scatter_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n_cap,
                    const int64_t* d_n, int shift, const uint32_t* __restrict__ block_hist, int num_blocks,
                    const uint32_t* __restrict__ digit_total, uint64_t* __restrict__ out_keys,
                    uint32_t* __restrict__ out_vals) {
  constexpr int RADIX = 1 << BITS, DPT = RADIX / kSortThreads;
  extern __shared__ __align__(16) unsigned char smem[];
  uint64_t* s_keys = (uint64_t*)smem;                                 // [kSortTile]
  uint32_t* s_vals = (uint32_t*)(s_keys + kSortTile);                 // [kSortTile]
  uint32_t(*warp_cnt)[RADIX] = (uint32_t(*)[RADIX])(s_vals + kSortTile);  // [warps][radix]
  uint32_t* glob_base = (uint32_t*)(warp_cnt + kWarps);               // [radix] where this tile's run of a digit starts
  uint32_t* tile_start = glob_base + RADIX;                           // [radix] start of the digit inside the tile
  __shared__ uint32_t scan_tmp[kWarps];
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t tile_base = (int64_t)blockIdx.x * kSortTile;
  if (tile_base >= n) return;                                   // nothing in this tile (device-side count below capacity)
  const int tile_n = (int)(n - tile_base < kSortTile ? n - tile_base : kSortTile);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d0 = threadIdx.x * DPT;

  // global start of every digit (exclusive scan of the totals) + this tile's offset inside the digit
  {
    uint32_t t[DPT], sum = 0;
#pragma unroll
    for (int q = 0; q < DPT; ++q) {
      t[q] = digit_total[d0 + q];
      sum += t[q];
    }
    uint32_t start = cta_scan_u32(sum, scan_tmp);
#pragma unroll
    for (int q = 0; q < DPT; ++q) {
      glob_base[d0 + q] = start + block_hist[(size_t)(d0 + q) * num_blocks + blockIdx.x];
      start += t[q];
    }
  }
#pragma unroll
  for (int w = 0; w < kWarps; ++w)
#pragma unroll
    for (int q = 0; q < DPT; ++q) warp_cnt[w][d0 + q] = 0;
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
    if (i < n) atomicAdd(&warp_cnt[warp][digit_of<BITS>(k[c], shift)], 1u);
  }
  __syncthreads();
  // per digit: counts of the warps -> start of every warp's keys inside the tile (digit-major, then warp order)
  {
    uint32_t cnt[DPT], sum = 0;
#pragma unroll
    for (int q = 0; q < DPT; ++q) {
      uint32_t run = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const uint32_t c = warp_cnt[w][d0 + q];
        warp_cnt[w][d0 + q] = run;
        run += c;
      }
      cnt[q] = run;   // keys of this digit in the tile
      sum += run;
    }
    uint32_t start = cta_scan_u32(sum, scan_tmp);
#pragma unroll
    for (int q = 0; q < DPT; ++q) {
      tile_start[d0 + q] = start;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) warp_cnt[w][d0 + q] += start;
      start += cnt[q];
    }
  }
  __syncthreads();
  // stable rank of every key inside the tile; the tile is laid out in digit order in shared memory
  const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int c = 0; c < kSortItems; ++c) {
    const int64_t i = base + c * 32;
    const bool valid = i < n;
    const uint32_t d = valid ? digit_of<BITS>(k[c], shift) : (uint32_t)RADIX;
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
    const uint32_t d = digit_of<BITS>(key, shift);
    const uint32_t g = glob_base[d] + ((uint32_t)j - tile_start[d]);
    out_keys[g] = key;
    out_vals[g] = s_vals[j];
  }
}

template <int BITS>
int run_passes(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n, const int64_t* d_n,
               int passes, bool iota_vals, uint32_t* block_hist, uint32_t* digit_total, int num_blocks, cudaStream_t stream) {
  static int smem_dev = -1;   // the attribute is per device function and context: set it once per process and device
  int dev = 0;
  SGL_CUDA_CHECK(cudaGetDevice(&dev));
  if (smem_dev != dev) {
    SGL_CUDA_CHECK(cudaFuncSetAttribute(sort_scatter_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)scatter_smem(BITS)));
    smem_dev = dev;
  }
  uint64_t *kin = keys, *kout = keys_alt;
  uint32_t *vin = vals, *vout = vals_alt;
  for (int p = 0; p < passes; ++p) {
    const int shift = p * BITS;
    sort_hist_kernel<BITS><<<num_blocks, kSortThreads, 0, stream>>>(kin, n, d_n, shift, block_hist, num_blocks);
    sort_scan_kernel<<<1 << BITS, 256, 0, stream>>>(block_hist, num_blocks, digit_total);
    sort_scatter_kernel<BITS><<<num_blocks, kSortThreads, scatter_smem(BITS), stream>>>(
        kin, (p == 0 && iota_vals) ? nullptr : vin, n, d_n, shift, block_hist, num_blocks, digit_total, kout, vout);
    SGL_LAUNCH_CHECK();
    uint64_t* tk = kin; kin = kout; kout = tk;
    uint32_t* tv = vin; vin = vout; vout = tv;
  }
  return SGL_OK;
}

}  // namespace

size_t radix_sort_ws_bytes(int64_t n) {
  int64_t nb = (n + kSortTile - 1) / kSortTile;
  if (nb < 1) nb = 1;
  return align_up((size_t)nb * kMaxRadix * sizeof(uint32_t)) + align_up(kMaxRadix * sizeof(uint32_t));
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
  uint32_t* block_hist = c.take<uint32_t>((size_t)num_blocks * kMaxRadix);
  uint32_t* digit_total = c.take<uint32_t>(kMaxRadix);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "radix sort: workspace %zu < %zu bytes", ws_bytes, radix_sort_ws_bytes(n));
  // 9-bit digits when they save a pass (e.g. 44 key bits: 5 passes instead of 6); their runs per tile are half as long
  int passes8 = (num_bits + 7) / 8, passes9 = (num_bits + 8) / 9;
  if (passes8 == 0 && iota_vals) passes8 = passes9 = 1;  // still has to materialise the payload
  const bool wide = passes9 < passes8;
  const int passes = wide ? passes9 : passes8;
  int rc = wide ? run_passes<9>(keys, vals, keys_alt, vals_alt, n, d_n, passes, iota_vals, block_hist, digit_total, num_blocks, stream)
                : run_passes<8>(keys, vals, keys_alt, vals_alt, n, d_n, passes, iota_vals, block_hist, digit_total, num_blocks, stream);
  if (rc) return rc;
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
