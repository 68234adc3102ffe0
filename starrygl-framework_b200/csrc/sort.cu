// Stable LSD radix sort, 8 bits per pass, three kernels per pass:
//   1. sort_hist_kernel    per-CTA digit histogram of its tile (4096 keys)          -> block_hist[digit][cta]
//   2. sort_scan_kernel    one CTA per digit: exclusive scan over CTAs + digit total
//   3. sort_scatter_kernel re-reads the tile, ranks keys stably (warp match + per-warp running counters)
//                          and writes key/payload to their final place for this digit
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

__global__ void __launch_bounds__(kSortThreads)
sort_scatter_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n_cap,
                    const int64_t* d_n, int shift, const uint32_t* __restrict__ block_hist, int num_blocks,
                    const uint32_t* __restrict__ digit_total, uint64_t* __restrict__ out_keys,
                    uint32_t* __restrict__ out_vals) {
  __shared__ uint32_t digit_base[kSortRadix];
  __shared__ uint32_t warp_cnt[kSortThreads / 32][kSortRadix];
  __shared__ uint32_t scan_tmp[8];
  const int64_t n = eff_count(n_cap, d_n);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // exclusive scan of the 256 digit totals (global start of every digit) + this CTA's offset inside the digit
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
    digit_base[threadIdx.x] = woff + x - v + block_hist[(size_t)threadIdx.x * num_blocks + blockIdx.x];
  }
#pragma unroll
  for (int w = 0; w < kSortThreads / 32; ++w) warp_cnt[w][threadIdx.x] = 0;
  __syncthreads();

  const int64_t base = (int64_t)blockIdx.x * kSortTile + (int64_t)warp * (kSortItems * 32) + lane;
  uint64_t k[kSortItems];
#pragma unroll
  for (int c = 0; c < kSortItems; ++c) {
    int64_t i = base + c * 32;
    k[c] = i < n ? keys[i] : 0;
    if (i < n) atomicAdd(&warp_cnt[warp][digit_of(k[c], shift)], 1u);
  }
  __syncthreads();
  // per digit: turn the per-warp counts into per-warp start positions (warp order = key order)
  {
    uint32_t run = digit_base[threadIdx.x];
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) {
      uint32_t c = warp_cnt[w][threadIdx.x];
      warp_cnt[w][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
  const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int c = 0; c < kSortItems; ++c) {
    int64_t i = base + c * 32;
    bool valid = i < n;
    uint32_t d = valid ? digit_of(k[c], shift) : (uint32_t)kSortRadix;
    uint32_t peers = __match_any_sync(0xffffffffu, d);
    uint32_t rank = __popc(peers & lt_mask);
    uint32_t pos = 0;
    if (valid) pos = warp_cnt[warp][d] + rank;
    __syncwarp();
    if (valid && rank == 0) warp_cnt[warp][d] += __popc(peers);
    __syncwarp();
    if (valid) {
      out_keys[pos] = k[c];
      out_vals[pos] = vals ? vals[i] : (uint32_t)i;
    }
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
  for (int p = 0; p < passes; ++p) {
    int shift = p * kSortRadixBits;
    sort_hist_kernel<<<num_blocks, kSortThreads, 0, stream>>>(kin, n, d_n, shift, block_hist, num_blocks);
    sort_scan_kernel<<<kSortRadix, 256, 0, stream>>>(block_hist, num_blocks, digit_total);
    sort_scatter_kernel<<<num_blocks, kSortThreads, 0, stream>>>(kin, (p == 0 && iota_vals) ? nullptr : vin, n, d_n,
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
