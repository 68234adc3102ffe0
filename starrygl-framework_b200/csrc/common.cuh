// Shared helpers of libsgl_b200: error reporting, launch checks, warp primitives.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <nvtx3/nvToolsExt.h>

#include "../../include/sgl_b200.h"

#define SGL_STR2(x) #x
#define SGL_STR(x) SGL_STR2(x)

namespace sgl {

// number of SMs on a B200; grids of the streaming kernels are sized in multiples of it
constexpr int kNumSM = 148;

void set_error(const char* fmt, ...);

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// carve `bytes` out of a caller workspace; returns nullptr when it does not fit
struct WsCarver {
  char* base;
  size_t cap;
  size_t off = 0;
  WsCarver(void* ws, size_t bytes) : base((char*)ws), cap(bytes) {}
  template <typename T>
  T* take(size_t count) {
    size_t b = align_up(count * sizeof(T));
    if (base == nullptr || off + b > cap) {
      off = cap + 1;
      return nullptr;
    }
    T* p = (T*)(base + off);
    off += b;
    return p;
  }
  bool ok() const { return off <= cap; }
};

#define SGL_CUDA_CHECK(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      sgl::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return SGL_ERR_CUDA;                                                                \
    }                                                                                     \
  } while (0)

#define SGL_LAUNCH_CHECK() SGL_CUDA_CHECK(cudaGetLastError())

#define SGL_REQUIRE(cond, code, ...)  \
  do {                                \
    if (!(cond)) {                    \
      sgl::set_error(__VA_ARGS__);    \
      return (code);                  \
    }                                 \
  } while (0)

// Named range on the profiler's timeline for the duration of an entry point (one per stage of the data path: T-CSR
// build, sampling, relabel, gather, plan, route ...).  Header-only NVTX: without an attached tool this is a null check.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};
#define SGL_NVTX(name) sgl::NvtxRange sgl_nvtx_range_(name)

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ void dev_flag(int32_t* status, int bit) {
  if (status) atomicOr(status, bit);
}

// effective count: device override when present, clamped to the launch capacity
__device__ __forceinline__ int64_t eff_count(int64_t n_cap, const int64_t* d_n) {
  if (d_n == nullptr) return n_cap;
  int64_t v = *d_n;
  return v < 0 ? 0 : (v > n_cap ? n_cap : v);
}

// grid size for a grid-stride streaming kernel: enough CTAs for the work, capped at a multiple of the SM count
inline int stream_grid(int64_t work_items, int per_block, int ctas_per_sm) {
  int64_t need = (work_items + per_block - 1) / per_block;
  int64_t cap = (int64_t)kNumSM * ctas_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

}  // namespace sgl
