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

// ---------------------------------------------------------------------------------------------------------------
// Mini-batch sizes (up to kSmallMaxKeys keys): ONE kernel per pass, up to 11 bits per pass.
//
// The relabel sorts of a mini-batch are a few hundred thousand keys of 40-odd bits.  At that size the three-kernel pass
// above is bound by its launches, so the pass is restructured around what is cheap for few tiles:
//
//   small_hist_kernel   one read of the keys: the digit totals of EVERY pass (shared-memory histograms flushed with
//                       global atomics) and the per-tile histogram of the first pass.
//   small_pass_kernel   tile t finds where its keys of digit d start by itself: digit starts from an in-kernel scan of
//                       the pass's totals, plus the counts of the tiles before it read straight from the per-tile
//                       histogram (tile-major, so a thread adds up its four digits with one 128-bit load per earlier
//                       tile, all loads independent; with <= 64 tiles that is cheaper than a scan kernel and its launch).  While it
//                       writes its keys to their sorted places it adds them to the NEXT pass's per-tile histogram
//                       (the tile a key lands in is known from its destination), so no pass needs a histogram kernel.
//   small_single_kernel up to one tile (8,192 keys): all passes inside one CTA, the tile never leaves shared memory.
//
// Tiles are 8,192 keys (512 threads x 16); ranks inside a tile are stable: a warp owns 512 consecutive keys, counts them
// per digit in its own 16-bit counters, and a key's rank = keys of its digit in earlier warps + in its warp's earlier
// rounds + in lower lanes of its round.
// Nothing waits on another CTA: the dependencies between passes are kernel boundaries.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kSmallThreads = 512;
constexpr int kSmallWarps = kSmallThreads / 32;
constexpr int kSmallItems = 16;
constexpr int kSmallTile = kSmallThreads * kSmallItems;   // 8,192 keys
constexpr int kSmallMaxBits = 11;
constexpr int kSmallRadix = 1 << kSmallMaxBits;           // 2,048 digits at most
constexpr int kSmallDpt = kSmallRadix / kSmallThreads;    // digits per thread in the per-digit phases
constexpr int kSmallMaxTiles = 64;
constexpr int64_t kSmallMaxKeys = (int64_t)kSmallTile * kSmallMaxTiles;
constexpr int kSmallMaxPasses = 6;

struct SmallSmem {
  uint64_t keys[kSmallTile];                       // the tile in digit order
  uint32_t vals[kSmallTile];
  unsigned short warp_cnt[kSmallWarps][kSmallRadix];   // per-warp digit counts, then start of the warp's keys of a digit
  uint32_t glob_base[kSmallRadix];                 // global position of the tile's first key of a digit
  unsigned short tile_start[kSmallRadix];          // position of the digit's run inside the tile
  uint32_t scan_tmp[kSmallWarps];
};

__device__ __forceinline__ uint32_t small_cta_scan(uint32_t v, uint32_t* tmp, uint32_t* total) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();
  if (lane == 31) tmp[warp] = x;
  __syncthreads();
  uint32_t woff = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kSmallWarps; ++w) {
    const uint32_t t = tmp[w];
    if (w < warp) woff += t;
    tot += t;
  }
  if (total) *total = tot;
  return woff + x - v;
}

// Ranks the tile's keys (held in registers, item c of a thread = tile position warp*512 + c*32 + lane; invalid items
// have valid bit clear) on `digit` and lays keys and payloads out in digit order in shared memory.  On return
// sm.tile_start[d] is the start of digit d's run; the per-digit counts of the tile are returned through cnt_out
// (kSmallDpt digits per thread, digit = threadIdx.x * kSmallDpt + q).
//
// Counting: every lane adds 1 to its digit's 16-bit counter of the warp with one shared-memory atomic on the 32-bit word
// that holds two counters; the value it gets back is its rank among the warp's earlier keys of that digit -- unless
// another lane of the same round hit the same digit, in which case the hardware's order among them is arbitrary.  With
// up to 2,048 digits that is rare; it is detected (a counter that moved by more than one past a lane's own value) and
// only then are the round's ranks recomputed in lane order with a warp match.
__device__ __forceinline__ void small_rank_tile(SmallSmem& sm, const uint64_t (&k)[kSmallItems], const uint32_t (&v)[kSmallItems],
                                                uint32_t valid_mask, int shift, int bits, uint32_t (&cnt_out)[kSmallDpt]) {
  static_assert(kSmallDpt == 4, "four 16-bit counters = one 64-bit word per thread and warp row");
  const uint32_t mask = (1u << bits) - 1u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d0 = threadIdx.x * kSmallDpt;
#pragma unroll
  for (int w = 0; w < kSmallWarps; ++w) *(uint2*)&sm.warp_cnt[w][d0] = make_uint2(0u, 0u);
  __syncthreads();
  const uint32_t lt_mask = (1u << lane) - 1u;
  uint32_t* my_words = (uint32_t*)sm.warp_cnt[warp];
  unsigned short rk[kSmallItems];
#pragma unroll
  for (int c = 0; c < kSmallItems; ++c) {
    const bool valid = (valid_mask >> c) & 1u;
    const uint32_t d = valid ? ((uint32_t)(k[c] >> shift) & mask) : 0u;
    const uint32_t sh = (d & 1u) * 16u;
    uint32_t mine = 0;
    if (valid) mine = (atomicAdd(&my_words[d >> 1], 1u << sh) >> sh) & 0xffffu;
    __syncwarp();
    uint32_t now = 0;
    if (valid) now = sm.warp_cnt[warp][d];
    if (__any_sync(0xffffffffu, valid && now - mine > 1u)) {
      // two lanes of this round share a digit: ranks in lane order.  now = count before the round + size of the group
      const uint32_t peers = __match_any_sync(0xffffffffu, valid ? d : 0xffffffffu);
      mine = now - __popc(peers) + __popc(peers & lt_mask);
    }
    __syncwarp();
    rk[c] = (unsigned short)mine;
  }
  __syncthreads();
  // per digit: counts of the warps -> start of every warp's keys of the digit (digit-major, then warp order); a thread's
  // four digits are one 64-bit word of a warp's counter row
  uint32_t run[kSmallDpt] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int w = 0; w < kSmallWarps; ++w) {
    const uint2 c = *(const uint2*)&sm.warp_cnt[w][d0];
    run[0] += c.x & 0xffffu;
    run[1] += c.x >> 16;
    run[2] += c.y & 0xffffu;
    run[3] += c.y >> 16;
  }
  uint32_t start = small_cta_scan(run[0] + run[1] + run[2] + run[3], sm.scan_tmp, nullptr);
  uint32_t off[kSmallDpt];
#pragma unroll
  for (int q = 0; q < kSmallDpt; ++q) {
    cnt_out[q] = run[q];
    sm.tile_start[d0 + q] = (unsigned short)start;
    off[q] = start;
    start += run[q];
  }
#pragma unroll
  for (int w = 0; w < kSmallWarps; ++w) {
    const uint2 c = *(const uint2*)&sm.warp_cnt[w][d0];
    *(uint2*)&sm.warp_cnt[w][d0] = make_uint2((off[0] & 0xffffu) | (off[1] << 16), (off[2] & 0xffffu) | (off[3] << 16));
    off[0] += c.x & 0xffffu;
    off[1] += c.x >> 16;
    off[2] += c.y & 0xffffu;
    off[3] += c.y >> 16;
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < kSmallItems; ++c) {
    if ((valid_mask >> c) & 1u) {
      const uint32_t d = (uint32_t)(k[c] >> shift) & mask;
      const uint32_t pos = (uint32_t)sm.warp_cnt[warp][d] + rk[c];
      sm.keys[pos] = k[c];
      sm.vals[pos] = v[c];
    }
  }
  __syncthreads();
}

// ghist[pass][digit] += digit totals of this tile for every pass; hist0[tile][digit] = first-pass histogram of the tile
__global__ void __launch_bounds__(kSmallThreads)
small_hist_kernel(const uint64_t* __restrict__ keys, int64_t n_cap, const int64_t* d_n, int passes, int bits,
                  uint32_t* __restrict__ ghist, uint32_t* __restrict__ hist0, int num_tiles) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* h = (uint32_t*)smem_raw;   // [passes][kSmallRadix]
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t tile_base = (int64_t)blockIdx.x * kSmallTile;
  if (tile_base >= n) return;
  const uint32_t mask = (1u << bits) - 1u;
  const int radix = 1 << bits;
  for (int j = threadIdx.x; j < passes * kSmallRadix; j += kSmallThreads) h[j] = 0;
  __syncthreads();
#pragma unroll 4
  for (int c = 0; c < kSmallItems; ++c) {
    const int64_t i = tile_base + (int64_t)c * kSmallThreads + threadIdx.x;
    if (i < n) {
      const uint64_t key = keys[i];
      for (int p = 0; p < passes; ++p) atomicAdd(&h[p * kSmallRadix + ((uint32_t)(key >> (p * bits)) & mask)], 1u);
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < passes * kSmallRadix; j += kSmallThreads) {
    const int p = j / kSmallRadix, d = j - p * kSmallRadix;
    if (d >= radix) continue;
    const uint32_t c = h[j];
    if (c) atomicAdd(&ghist[p * kSmallRadix + d], c);
    if (p == 0) hist0[(size_t)blockIdx.x * kSmallRadix + d] = c;
  }
}

__global__ void __launch_bounds__(kSmallThreads, 1)
small_pass_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n_cap, const int64_t* d_n,
                  int shift, int bits, const uint32_t* __restrict__ ghist_p, const uint32_t* __restrict__ hist_p,
                  uint32_t* __restrict__ hist_next, int next_shift, int num_tiles, uint64_t* __restrict__ out_keys,
                  uint32_t* __restrict__ out_vals) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SmallSmem& sm = *(SmallSmem*)smem_raw;
  const int64_t n = eff_count(n_cap, d_n);
  const int tile = blockIdx.x;
  const int64_t tile_base = (int64_t)tile * kSmallTile;
  if (tile_base >= n) return;
  const int tile_n = (int)(n - tile_base < kSmallTile ? n - tile_base : kSmallTile);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t mask = (1u << bits) - 1u;
  const int radix = 1 << bits;
  const int d0 = threadIdx.x * kSmallDpt;

  // the tile's keys: issued first so that the loads are in flight while the digit bases are computed
  uint64_t k[kSmallItems];
  uint32_t v[kSmallItems];
  uint32_t valid_mask = 0;
  const int64_t base = tile_base + (int64_t)warp * (kSmallItems * 32) + lane;
#pragma unroll
  for (int c = 0; c < kSmallItems; ++c) {
    const int64_t i = base + c * 32;
    const bool ok = i < n;
    k[c] = ok ? keys[i] : 0;
    v[c] = ok ? (vals ? vals[i] : (uint32_t)i) : 0u;
    valid_mask |= (ok ? 1u : 0u) << c;
  }
  // global start of every digit: exclusive scan of the pass's totals
  {
    uint32_t t[kSmallDpt], sum = 0;
#pragma unroll
    for (int q = 0; q < kSmallDpt; ++q) {
      t[q] = (d0 + q < radix) ? ghist_p[d0 + q] : 0u;
      sum += t[q];
    }
    uint32_t start = small_cta_scan(sum, sm.scan_tmp, nullptr);
#pragma unroll
    for (int q = 0; q < kSmallDpt; ++q) {
      sm.glob_base[d0 + q] = start;
      start += t[q];
    }
  }
  __syncthreads();
  // + the keys of the digit in the tiles before this one: the thread's four digits are one 128-bit word of a tile's
  // histogram; the loads of the earlier tiles are independent of each other
  {
    static_assert(kSmallDpt == 4, "one uint4 per thread and tile");
    const uint4* col = (const uint4*)hist_p + threadIdx.x;
    uint4 acc = make_uint4(0, 0, 0, 0);
    int t = 0;
    for (; t + 4 <= tile; t += 4) {
      const uint4 a = __ldg(col + (size_t)(t + 0) * (kSmallRadix / 4)), b = __ldg(col + (size_t)(t + 1) * (kSmallRadix / 4));
      const uint4 c2 = __ldg(col + (size_t)(t + 2) * (kSmallRadix / 4)), d2 = __ldg(col + (size_t)(t + 3) * (kSmallRadix / 4));
      acc.x += a.x + b.x + c2.x + d2.x;
      acc.y += a.y + b.y + c2.y + d2.y;
      acc.z += a.z + b.z + c2.z + d2.z;
      acc.w += a.w + b.w + c2.w + d2.w;
    }
    for (; t < tile; ++t) {
      const uint4 a = __ldg(col + (size_t)t * (kSmallRadix / 4));
      acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    }
    sm.glob_base[d0 + 0] += acc.x;
    sm.glob_base[d0 + 1] += acc.y;
    sm.glob_base[d0 + 2] += acc.z;
    sm.glob_base[d0 + 3] += acc.w;
  }
  uint32_t cnt[kSmallDpt];
  small_rank_tile(sm, k, v, valid_mask, shift, bits, cnt);   // (starts with a barrier: glob_base is complete after it)
  // write-out: consecutive threads take consecutive tile positions, i.e. runs of one digit -> consecutive addresses
  const uint32_t next_mask = mask;
  for (int j = threadIdx.x; j < tile_n; j += kSmallThreads) {
    const uint64_t key = sm.keys[j];
    const uint32_t d = (uint32_t)(key >> shift) & mask;
    const uint32_t g = sm.glob_base[d] + ((uint32_t)j - sm.tile_start[d]);
    out_keys[g] = key;
    out_vals[g] = sm.vals[j];
    if (hist_next) atomicAdd(&hist_next[(size_t)(g / kSmallTile) * kSmallRadix + ((uint32_t)(key >> next_shift) & next_mask)], 1u);
  }
}

// n <= one tile: every pass inside the CTA; (keys, vals) are read once and written once
__global__ void __launch_bounds__(kSmallThreads, 1)
small_single_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n_cap, const int64_t* d_n,
                    int passes, int bits, uint64_t* __restrict__ out_keys, uint32_t* __restrict__ out_vals) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SmallSmem& sm = *(SmallSmem*)smem_raw;
  int64_t n = eff_count(n_cap, d_n);
  if (n > kSmallTile) n = kSmallTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t mask = (1u << bits) - 1u;
  uint64_t k[kSmallItems];
  uint32_t v[kSmallItems];
  uint32_t valid_mask = 0;
  const int pos0 = warp * (kSmallItems * 32) + lane;
#pragma unroll
  for (int c = 0; c < kSmallItems; ++c) {
    const int i = pos0 + c * 32;
    const bool ok = i < n;
    k[c] = ok ? keys[i] : 0;
    v[c] = ok ? (vals ? vals[i] : (uint32_t)i) : 0u;
    valid_mask |= (ok ? 1u : 0u) << c;
  }
  uint32_t cnt[kSmallDpt];
  for (int p = 0; p < passes; ++p) {
    small_rank_tile(sm, k, v, valid_mask, p * bits, bits, cnt);
    if (p + 1 < passes) {
#pragma unroll
      for (int c = 0; c < kSmallItems; ++c) {
        const int i = pos0 + c * 32;
        if (i < n) {
          k[c] = sm.keys[i];
          v[c] = sm.vals[i];
        }
      }
      __syncthreads();
    }
  }
  for (int j = threadIdx.x; j < n; j += kSmallThreads) {
    out_keys[j] = sm.keys[j];
    out_vals[j] = sm.vals[j];
  }
}

inline size_t small_ws_bytes() {
  return align_up((size_t)kSmallMaxPasses * kSmallRadix * 4) + align_up((size_t)kSmallMaxPasses * kSmallRadix * kSmallMaxTiles * 4);
}

// passes and bits per pass for a key width (balanced: 44 bits -> 4 x 11, 40 bits -> 4 x 10)
inline void small_plan(int num_bits, bool iota_vals, int* passes, int* bits) {
  int p = (num_bits + kSmallMaxBits - 1) / kSmallMaxBits;
  if (p == 0 && iota_vals) p = 1;   // still has to materialise the payload
  *passes = p;
  *bits = p ? (num_bits + p - 1) / p : 0;
  if (*bits < 1) *bits = 1;
}

int run_small(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n, const int64_t* d_n,
              int num_bits, bool iota_vals, int* result_in_alt, void* ws, size_t ws_bytes, cudaStream_t stream) {
  int passes, bits;
  small_plan(num_bits, iota_vals, &passes, &bits);
  *result_in_alt = 0;
  if (passes == 0) return SGL_OK;
  static int attr_dev = -1;   // the attribute is per device function and context: set it once per process and device
  int dev = 0;
  SGL_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    SGL_CUDA_CHECK(cudaFuncSetAttribute(small_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmallSmem)));
    SGL_CUDA_CHECK(cudaFuncSetAttribute(small_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmallSmem)));
    SGL_CUDA_CHECK(cudaFuncSetAttribute(small_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kSmallMaxPasses * kSmallRadix * 4));
    attr_dev = dev;
  }
  if (n <= kSmallTile) {
    small_single_kernel<<<1, kSmallThreads, sizeof(SmallSmem), stream>>>(keys, iota_vals ? nullptr : vals, n, d_n, passes, bits,
                                                                         keys_alt, vals_alt);
    SGL_LAUNCH_CHECK();
    *result_in_alt = 1;
    return SGL_OK;
  }
  const int num_tiles = (int)((n + kSmallTile - 1) / kSmallTile);
  WsCarver c(ws, ws_bytes);
  uint32_t* ghist = c.take<uint32_t>((size_t)kSmallMaxPasses * kSmallRadix);
  uint32_t* hist = c.take<uint32_t>((size_t)kSmallMaxPasses * kSmallRadix * kSmallMaxTiles);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "radix sort: workspace %zu < %zu bytes", ws_bytes, small_ws_bytes());
  // per-pass histogram p ([tile][digit]) lives at hist + p * kSmallRadix * num_tiles (packed for the actual tile count)
  const size_t per_pass = (size_t)kSmallRadix * num_tiles;
  SGL_CUDA_CHECK(cudaMemsetAsync(ghist, 0, (size_t)passes * kSmallRadix * 4, stream));
  SGL_CUDA_CHECK(cudaMemsetAsync(hist, 0, (size_t)passes * per_pass * 4, stream));
  small_hist_kernel<<<num_tiles, kSmallThreads, (size_t)passes * kSmallRadix * 4, stream>>>(keys, n, d_n, passes, bits, ghist, hist,
                                                                                          num_tiles);
  uint64_t *kin = keys, *kout = keys_alt;
  uint32_t *vin = vals, *vout = vals_alt;
  for (int p = 0; p < passes; ++p) {
    uint32_t* next = p + 1 < passes ? hist + (size_t)(p + 1) * per_pass : nullptr;
    small_pass_kernel<<<num_tiles, kSmallThreads, sizeof(SmallSmem), stream>>>(
        kin, (p == 0 && iota_vals) ? nullptr : vin, n, d_n, p * bits, bits, ghist + (size_t)p * kSmallRadix,
        hist + (size_t)p * per_pass, next, (p + 1) * bits, num_tiles, kout, vout);
    uint64_t* tk = kin; kin = kout; kout = tk;
    uint32_t* tv = vin; vin = vout; vout = tv;
  }
  SGL_LAUNCH_CHECK();
  *result_in_alt = passes & 1;
  return SGL_OK;
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
  const size_t big = align_up((size_t)nb * kMaxRadix * sizeof(uint32_t)) + align_up(kMaxRadix * sizeof(uint32_t));
  const size_t small = n <= kSmallMaxKeys ? small_ws_bytes() : 0;
  return big > small ? big : small;
}

int radix_sort_pairs(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n,
                     const int64_t* d_n, int num_bits, bool iota_vals, int* result_in_alt, void* ws, size_t ws_bytes,
                     cudaStream_t stream) {
  SGL_REQUIRE(n >= 0 && n < ((int64_t)1 << 32), SGL_ERR_ARG, "radix sort: n=%lld outside [0, 2^32)", (long long)n);
  SGL_REQUIRE(num_bits >= 0 && num_bits <= 64, SGL_ERR_ARG, "radix sort: num_bits=%d", num_bits);
  *result_in_alt = 0;
  if (n == 0) return SGL_OK;
  SGL_REQUIRE(keys && vals && keys_alt && vals_alt, SGL_ERR_ARG, "radix sort: null buffer");
  if (n <= kSmallMaxKeys) return run_small(keys, vals, keys_alt, vals_alt, n, d_n, num_bits, iota_vals, result_in_alt, ws, ws_bytes, stream);
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

// number of kernels one sort of n keys of num_bits bits launches (for launch accounting; memsets are not kernels)
extern "C" int sgl_radix_sort_launches(int64_t n, int num_bits) {
  if (n <= 0) return 0;
  if (n <= sgl::kSmallMaxKeys) {
    int passes, bits;
    sgl::small_plan(num_bits, true, &passes, &bits);
    return n <= sgl::kSmallTile ? (passes ? 1 : 0) : 1 + passes;
  }
  const int p8 = (num_bits + 7) / 8, p9 = (num_bits + 8) / 9;
  return 3 * (p9 < p8 ? p9 : p8);
}

extern "C" int sgl_radix_sort_u64_u32(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n,
                                      int num_bits, int* h_result_in_alt, void* ws, size_t ws_bytes, void* stream) {
  int dummy = 0;
  return sgl::radix_sort_pairs(keys, vals, keys_alt, vals_alt, n, nullptr, num_bits, false,
                               h_result_in_alt ? h_result_in_alt : &dummy, ws, ws_bytes, (cudaStream_t)stream);
}
