// CTA-level scan helpers and the "last CTA scans the per-CTA totals" pattern (no spinning anywhere:
// a fence plus an atomic counter decides which CTA is the last one to finish).
#pragma once
#include "common.cuh"

namespace sgl {

// inclusive warp scan
template <typename T>
__device__ __forceinline__ T warp_inclusive_scan(T x, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    T y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  return x;
}

// Exclusive scan of one value per thread across the CTA (THREADS multiple of 32, <= 1024).
// Returns the exclusive prefix; *total (optional) receives the CTA sum in every thread.
template <int THREADS, typename T>
__device__ __forceinline__ T cta_exclusive_scan(T v, T* total) {
  __shared__ T s_w[THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T x = warp_inclusive_scan(v, lane);
  if (lane == 31) s_w[warp] = x;
  __syncthreads();
  T woff = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) {
    T s = s_w[w];
    if (w < warp) woff += s;
    tot += s;
  }
  __syncthreads();
  if (total) *total = tot;
  return woff + x - v;
}

// Every CTA calls this once with its total (same value in all threads).  cta_sums[blockIdx.x] is published;
// the last CTA to arrive replaces cta_sums[0..gridDim.x) by its exclusive scan, writes the grand total to
// *grand_total and re-arms *done_counter (0) for the next launch.  Kernels that consume the scanned values
// must be launched after this kernel on the same stream.
template <int THREADS>
__device__ __forceinline__ void publish_and_scan_cta_totals(int64_t my_total, int64_t* cta_sums,
                                                           unsigned int* done_counter, int64_t* grand_total) {
  __shared__ bool s_last;
  __shared__ int64_t s_carry;
  if (threadIdx.x == 0) {
    cta_sums[blockIdx.x] = my_total;
    __threadfence();
    unsigned prev = atomicAdd(done_counter, 1u);
    s_last = (prev == gridDim.x - 1);
    s_carry = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int64_t base = 0; base < gridDim.x; base += THREADS) {
    int64_t idx = base + threadIdx.x;
    int64_t v = idx < gridDim.x ? ((volatile int64_t*)cta_sums)[idx] : 0;
    int64_t tot;
    int64_t ex = cta_exclusive_scan<THREADS, int64_t>(v, &tot);
    int64_t carry = s_carry;
    if (idx < gridDim.x) cta_sums[idx] = carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) s_carry = carry + tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (grand_total) *grand_total = s_carry;
    *done_counter = 0;
  }
}

}  // namespace sgl
