// Stable LSD radix sort of (uint64 key, uint32 payload) pairs -- host-side launcher interface.
#pragma once
#include "common.cuh"

namespace sgl {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 16;
constexpr int kSortTile = kSortThreads * kSortItems;  // keys per CTA

size_t radix_sort_ws_bytes(int64_t n);

// Sorts on key bits [0, num_bits).  vals may be nullptr on input: the payload is then the input position.
// The data ping-pong between (keys, vals) and (keys_alt, vals_alt); *result_in_alt says where they end.
// `d_n` (optional) is a device count <= n: only the first *d_n items are sorted.
int radix_sort_pairs(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n,
                     const int64_t* d_n, int num_bits, bool iota_vals, int* result_in_alt, void* ws, size_t ws_bytes,
                     cudaStream_t stream);

inline int bits_for(uint64_t max_value) {
  int b = 0;
  while (b < 64 && (max_value >> b) != 0) ++b;
  return b;
}

}  // namespace sgl
