// Head flags of a sorted key list + scan: shared by the dedup / relabel kernels and the mailbox reduce.
#pragma once
#include "scan.cuh"

namespace sgl {
namespace {

constexpr int kHeadsThreads = 256;

__device__ __forceinline__ uint64_t low_mask(int bits) { return bits >= 64 ? ~0ull : ((1ull << bits) - 1ull); }

// head flag of every sorted key (first of its run) and its CTA-local exclusive rank, packed as rank*2 + head.
// Keys >= limit (when limit_bits < 64) are ignored: used by the node relabel to park already-known ids at the end.
__global__ void __launch_bounds__(kHeadsThreads)
heads_scan_kernel(const uint64_t* __restrict__ keys, int64_t n_cap, const int64_t* d_n, int limit_bits,
                  uint32_t* __restrict__ packed, int64_t* __restrict__ cta_sums, unsigned int* done_counter,
                  int64_t* grand_total) {
  const int64_t n = eff_count(n_cap, d_n);
  const int64_t j = (int64_t)blockIdx.x * kHeadsThreads + threadIdx.x;
  int head = 0;
  if (j < n) {
    uint64_t k = keys[j];
    bool counted = limit_bits >= 64 || (k >> limit_bits) == 0;
    head = counted && (j == 0 || keys[j - 1] != k) ? 1 : 0;
  }
  int total;
  int ex = cta_exclusive_scan<kHeadsThreads, int>(head, &total);
  if (j < n) packed[j] = ((uint32_t)ex << 1) | (uint32_t)head;
  publish_and_scan_cta_totals<kHeadsThreads>((int64_t)total, cta_sums, done_counter, grand_total);
}

}  // namespace
}  // namespace sgl
