// Cache route over NVLink peer memory: pack + transfer in ONE kernel, no collective library call per step.
//
// Every rank owns a buffer that all ranks of the node map (CUDA IPC):
//     flags[world][ring]   flags[q][slot] = step + 1 once sender q's rows of that step have landed here
//     acks [world]         acks[p] = number of this rank's steps that receiver p has applied (written by p)
//     stage[world][ring][cap_rows][pitch]   wire rows from sender q, ring slot = step % ring
//
// send kernel (rank r, step s):  waits until every receiver has applied step s - ring (so the slot is free), builds
//     the wire rows [features | ts | slot | pad] exactly like route_pack_kernel and stores them with 128-bit stores
//     straight into the receivers' stage[r][s % ring] over NVLink; the last CTA to finish (fence + counter) publishes
//     flags[r][s % ring] = s + 1 on every receiver.
// recv kernel (rank p, step s):  waits for the flags of all senders, scatters the rows from its own stage into the
//     node-state table (same work as route_unpack_kernel), then the last CTA acknowledges to every sender.
//
// The two kernels of a step run on DIFFERENT GPUs (one process per GPU), never as two launches on one GPU.  Every
// wait is bounded by a wall-clock limit; on expiry the kernel raises SGL_DEV_TIMEOUT in the status word, publishes
// nothing and returns, so the context stays usable.  Every rank must run send and recv for every step (zero rows are
// fine): the handshake is per step, not per row.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace sgl {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kThreads = 64;    // small CTAs: they fit into the register/thread gaps a busy GPU has left, so they start promptly
constexpr int kUnroll = 4;   // lanes in flight per thread in the route kernels
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

struct P2PCfg {
  int dbg;
  unsigned long long* tl;   // optional timeline buffer [steps][8] (diagnostics)
  int rank, world, ring;
  int64_t cap_rows;
  uint32_t pitch;
  unsigned long long* flags;
  unsigned long long* acks;
  float* stage;
  unsigned long long* peer_flags[kMaxWorld];
  unsigned long long* peer_acks[kMaxWorld];
  float* peer_stage[kMaxWorld];
};

struct Splits {
  int64_t off[kMaxWorld + 1];
};

struct Ctx {
  P2PCfg cfg;
  unsigned int* counters;   // [2] device: arrival counters of the send / recv kernels
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// spin until *p >= want; false when the limit expires
__device__ __forceinline__ bool wait_at_least(const unsigned long long* p, unsigned long long want) {
  const volatile unsigned long long* vp = p;
  if (*vp >= want) return true;
  const unsigned long long t0 = now_ns();
  while (now_ns() - t0 < kWaitLimitNs) {
    if (*vp >= want) return true;
    __nanosleep(200);
  }
  return false;
}

__device__ __forceinline__ uint32_t wire_word2(uint32_t e, uint32_t dim, uint32_t payload, const float* __restrict__ frow,
                                               const float* __restrict__ ts, int64_t r, uint64_t slot) {
  if (e < dim) return __float_as_uint(__ldg(frow + e));
  if (e < payload) return __float_as_uint(__ldg(ts + r));
  if (e == payload) return (uint32_t)slot;
  if (e == payload + 1) return (uint32_t)(slot >> 32);
  return 0u;
}

__device__ __forceinline__ int segment_of(const Splits& s, int world, int64_t i) {
  int p = 0;
  while (p + 1 < world && i >= s.off[p + 1]) ++p;
  return p;
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
p2p_send_kernel(P2PCfg c, const float* __restrict__ feats, int64_t n_rows, uint32_t dim, const float* __restrict__ ts,
                const int64_t* __restrict__ send_idx, const int64_t* __restrict__ remote_idx, Splits seg,
                unsigned long long step, unsigned int* done_counter, int32_t* d_status) {
  __shared__ int s_ok;
  __shared__ bool s_last;
  if (threadIdx.x == 0) s_ok = 1;
  if (c.tl && blockIdx.x == 0 && threadIdx.x == 0 && step < 4096) c.tl[step * 8 + 0] = now_ns();
  __syncthreads();
  // flow control: the ring slot may be overwritten once every receiver has applied the step that used it last
  if (threadIdx.x < c.world && step >= (unsigned long long)c.ring) {
    if (!wait_at_least(c.acks + threadIdx.x, step - c.ring + 1)) s_ok = 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  if (ok) {
    const int slot = (int)(step % c.ring);
    const uint32_t payload = dim + (ts ? 1u : 0u);
    const uint32_t lanes = c.pitch / VEC;
    const int64_t n_send = seg.off[c.world];
    const int64_t total = n_send * lanes;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    // kUnroll lanes per thread and iteration, in three phases (indices, rows, stores), so that the two dependent
    // loads of every lane overlap with those of the other lanes: a small grid then moves a small message in about
    // two memory latencies, and few CTAs have to find a free slot on a busy GPU
    for (int64_t q0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; q0 < total; q0 += stride * kUnroll) {
      int64_t row_i[kUnroll], src_r[kUnroll];
      uint64_t slotv[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t q = q0 + u * stride;
        row_i[u] = -1;
        if (q < total) {
          row_i[u] = q / lanes;
          src_r[u] = __ldg(send_idx + row_i[u]);
          slotv[u] = (uint64_t)__ldg(remote_idx + row_i[u]);
        }
      }
      uint4 v[kUnroll];
      void* dst[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        dst[u] = nullptr;
        if (row_i[u] < 0) continue;
        const int64_t i = row_i[u];
        const uint32_t l = (uint32_t)(q0 + u * stride - i * lanes);
        int64_t r = src_r[u];
        if (r < 0) r += n_rows;
        if (r < 0 || r >= n_rows) {
          dev_flag(d_status, SGL_DEV_BAD_INDEX);
          continue;
        }
        const int p = segment_of(seg, c.world, i);
        float* dst_row = c.peer_stage[p] + (((int64_t)c.rank * c.ring + slot) * c.cap_rows + (i - seg.off[p])) * c.pitch;
        const float* frow = feats + r * dim;
        if (VEC == 4) {
          if ((l + 1) * 4 <= dim) {
            v[u] = __ldg((const uint4*)frow + l);
          } else {
            v[u].x = wire_word2(4 * l + 0, dim, payload, frow, ts, r, slotv[u]);
            v[u].y = wire_word2(4 * l + 1, dim, payload, frow, ts, r, slotv[u]);
            v[u].z = wire_word2(4 * l + 2, dim, payload, frow, ts, r, slotv[u]);
            v[u].w = wire_word2(4 * l + 3, dim, payload, frow, ts, r, slotv[u]);
          }
          dst[u] = (uint4*)dst_row + l;
        } else {
          v[u].x = wire_word2(l, dim, payload, frow, ts, r, slotv[u]);
          dst[u] = (uint32_t*)dst_row + l;
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (!dst[u]) continue;
        if (VEC == 4) *(uint4*)dst[u] = v[u];
        else *(uint32_t*)dst[u] = v[u].x;
      }
    }
  } else if (threadIdx.x == 0) {
    dev_flag(d_status, SGL_DEV_TIMEOUT);
  }
  // publish.  One system-scope fence per CTA instead of one per thread: the CTA barrier makes every thread's stores
  // happen-before thread 0's fence, and fences are cumulative, so thread 0's fence + counter increment orders the whole
  // CTA's rows before anything the last CTA does after it has seen all increments.  (A system fence is expensive
  // while the GPU streams other data; 20,000 of them per launch dominated this kernel's latency.)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned prev = atomicAdd(done_counter, 1u);
    s_last = prev == gridDim.x - 1;
    if (s_last) __threadfence_system();
  }
  __syncthreads();
  if (!s_last) return;
  const bool failed = d_status && (*(volatile int32_t*)d_status & SGL_DEV_TIMEOUT);
  if (threadIdx.x < c.world && !failed) {
    volatile unsigned long long* f = c.peer_flags[threadIdx.x] + (int64_t)c.rank * c.ring + (step % c.ring);
    *f = step + 1;
  }
  if (c.tl && threadIdx.x == 0 && step < 4096) c.tl[step * 8 + 1] = now_ns();
  if (threadIdx.x == 0) *done_counter = 0;
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
p2p_recv_kernel(P2PCfg c, Splits seg, uint32_t width, float* __restrict__ data, int64_t data_rows, uint32_t dim,
                float* __restrict__ ts_table, unsigned long long step, unsigned int* done_counter, int32_t* d_status) {
  __shared__ int s_ok;
  __shared__ bool s_last;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const int slot = (int)(step % c.ring);
  if (c.tl && blockIdx.x == 0 && threadIdx.x == 0 && step < 4096) c.tl[step * 8 + 2] = now_ns();
  if (threadIdx.x < c.world) {
    if (!wait_at_least(c.flags + (int64_t)threadIdx.x * c.ring + slot, step + 1)) s_ok = 0;
    __threadfence_system();   // acquire side: the rows written before the flag are visible after this fence ...
  }
  __syncthreads();            // ... and, through the barrier, to every thread of the CTA
  if (c.tl && blockIdx.x == 0 && threadIdx.x == 0 && step < 4096) c.tl[step * 8 + 3] = now_ns();
  const bool ok = s_ok != 0;
  if (ok) {
    const uint32_t lanes = (width + VEC - 1) / VEC;
    const int64_t n_recv = seg.off[c.world];
    const int64_t total = n_recv * lanes;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t q0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; q0 < total; q0 += stride * kUnroll) {
      // plain loads throughout: the stage was written by another GPU, the read-only cache must not be used for it
      uint4 v[kUnroll];
      int64_t dslot[kUnroll];
      uint32_t lane_l[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t q = q0 + u * stride;
        dslot[u] = -1;
        if (q >= total) continue;
        const int64_t i = q / lanes;
        const uint32_t l = (uint32_t)(q - i * lanes);
        const int sdr = segment_of(seg, c.world, i);
        const uint32_t* row = (const uint32_t*)(c.stage + (((int64_t)sdr * c.ring + slot) * c.cap_rows + (i - seg.off[sdr])) * c.pitch);
        dslot[u] = (int64_t)((uint64_t)row[width] | ((uint64_t)row[width + 1] << 32));
        lane_l[u] = l;
        if (VEC == 4) v[u] = ((const uint4*)row)[l];
        else v[u].x = row[l];
        if (dslot[u] < 0 || dslot[u] >= data_rows) {
          dev_flag(d_status, SGL_DEV_BAD_INDEX);
          dslot[u] = -1;
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (dslot[u] < 0) continue;
        const uint32_t l = lane_l[u];
        if (VEC == 4) {
          if ((l + 1) * 4 <= dim) ((uint4*)(data + dslot[u] * dim))[l] = v[u];
          else if (ts_table) ts_table[dslot[u]] = __uint_as_float(v[u].x);
        } else {
          if (l < dim) data[dslot[u] * dim + l] = __uint_as_float(v[u].x);
          else if (ts_table) ts_table[dslot[u]] = __uint_as_float(v[u].x);
        }
      }
    }
  } else if (threadIdx.x == 0) {
    dev_flag(d_status, SGL_DEV_TIMEOUT);
  }
  // all reads of the staging slot are done before the senders are told they may overwrite it (same one-fence-per-CTA
  // pattern as in the send kernel)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned prev = atomicAdd(done_counter, 1u);
    s_last = prev == gridDim.x - 1;
    if (s_last) __threadfence_system();
  }
  __syncthreads();
  if (!s_last) return;
  const bool failed = d_status && (*(volatile int32_t*)d_status & SGL_DEV_TIMEOUT);
  if (threadIdx.x < c.world && !failed) {
    volatile unsigned long long* a = c.peer_acks[threadIdx.x] + c.rank;   // "rank has applied your step"
    *a = step + 1;
  }
  if (c.tl && threadIdx.x == 0 && step < 4096) c.tl[step * 8 + 4] = now_ns();
  if (threadIdx.x == 0) *done_counter = 0;
}

inline size_t header_bytes(int world, int ring) { return align_up((size_t)world * ring * 8 + (size_t)world * 8, 256); }

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" size_t sgl_p2p_buffer_bytes(int world, int ring, int64_t cap_rows, int64_t pitch_floats) {
  if (world < 1 || ring < 1 || cap_rows < 0 || pitch_floats < 1) return 0;
  return header_bytes(world, ring) + (size_t)world * ring * (size_t)cap_rows * (size_t)pitch_floats * 4;
}

extern "C" int sgl_p2p_alloc(size_t bytes, void** out_ptr, char* out_handle, size_t handle_bytes) {
  SGL_REQUIRE(out_ptr && out_handle && handle_bytes >= sizeof(cudaIpcMemHandle_t), SGL_ERR_ARG,
              "p2p_alloc: handle buffer must hold %zu bytes", sizeof(cudaIpcMemHandle_t));
  void* p = nullptr;
  SGL_CUDA_CHECK(cudaMalloc(&p, bytes < 256 ? 256 : bytes));
  SGL_CUDA_CHECK(cudaMemset(p, 0, bytes < 256 ? 256 : bytes));
  cudaIpcMemHandle_t h;
  SGL_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
  memcpy(out_handle, &h, sizeof(h));
  *out_ptr = p;
  return SGL_OK;
}

extern "C" int sgl_p2p_open(const char* handle, void** out_ptr) {
  SGL_REQUIRE(handle && out_ptr, SGL_ERR_ARG, "p2p_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  SGL_CUDA_CHECK(cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return SGL_OK;
}

extern "C" int sgl_p2p_close(void* peer_ptr) {
  if (peer_ptr) SGL_CUDA_CHECK(cudaIpcCloseMemHandle(peer_ptr));
  return SGL_OK;
}

extern "C" int sgl_p2p_free(void* ptr) {
  if (ptr) SGL_CUDA_CHECK(cudaFree(ptr));
  return SGL_OK;
}

extern "C" int sgl_p2p_route_create(int rank, int world, int ring, int64_t cap_rows, int64_t pitch_floats,
                                    void* const* h_bases, void** out_ctx) {
  SGL_REQUIRE(out_ctx && h_bases && world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world && ring >= 2 &&
                  cap_rows >= 1 && pitch_floats >= 1,
              SGL_ERR_ARG, "p2p_route_create: bad argument (world <= %d, ring >= 2)", kMaxWorld);
  Ctx* x = new Ctx();
  P2PCfg& c = x->cfg;
  c.dbg = getenv("SGL_P2P_DBG") ? atoi(getenv("SGL_P2P_DBG")) : 0;   // 2 = record a per-step kernel timeline (diagnostics)
  c.rank = rank; c.world = world; c.ring = ring; c.cap_rows = cap_rows; c.pitch = (uint32_t)pitch_floats;
  const size_t hb = header_bytes(world, ring);
  for (int p = 0; p < world; ++p) {
    SGL_REQUIRE(h_bases[p], SGL_ERR_ARG, "p2p_route_create: base pointer of rank %d is null", p);
    char* b = (char*)h_bases[p];
    c.peer_flags[p] = (unsigned long long*)b;
    c.peer_acks[p] = (unsigned long long*)b + (size_t)world * ring;
    c.peer_stage[p] = (float*)(b + hb);
  }
  c.flags = c.peer_flags[rank];
  c.acks = c.peer_acks[rank];
  c.stage = c.peer_stage[rank];
  SGL_CUDA_CHECK(cudaMalloc(&x->counters, 256));
  SGL_CUDA_CHECK(cudaMemset(x->counters, 0, 256));
  c.tl = nullptr;
  if (c.dbg & 2) {
    SGL_CUDA_CHECK(cudaMalloc(&c.tl, 4096 * 8 * 8));
    SGL_CUDA_CHECK(cudaMemset(c.tl, 0, 4096 * 8 * 8));
  }
  *out_ctx = x;
  return SGL_OK;
}

extern "C" int sgl_p2p_route_destroy(void* ctx) {
  if (!ctx) return SGL_OK;
  Ctx* x = (Ctx*)ctx;
  cudaFree(x->counters);
  delete x;
  return SGL_OK;
}

// number of CTAs of a route kernel: enough for the rows, capped (SGL_P2P_MAX_CTAS, tuning aid) -- small messages are
// latency-bound and every extra CTA adds fence traffic and a longer wait for the last one
static int p2p_grid(int64_t lanes_total) {
  static int cap = -1;
  if (cap < 0) {
    const char* e = getenv("SGL_P2P_MAX_CTAS");
    cap = e ? atoi(e) : kNumSM * 8;
    if (cap < 1) cap = 1;
  }
  int g = stream_grid(lanes_total, kThreads * kUnroll, 8);
  return g < cap ? g : cap;
}

static int make_splits(const Ctx* x, const int64_t* h_rows, Splits* s, const char* what) {
  s->off[0] = 0;
  for (int p = 0; p < x->cfg.world; ++p) {
    SGL_REQUIRE(h_rows[p] >= 0 && h_rows[p] <= x->cfg.cap_rows, SGL_ERR_ARG, "%s: %lld rows for rank %d exceed the staging capacity %lld",
                what, (long long)h_rows[p], p, (long long)x->cfg.cap_rows);
    s->off[p + 1] = s->off[p] + h_rows[p];
  }
  for (int p = x->cfg.world; p < kMaxWorld; ++p) s->off[p + 1] = s->off[x->cfg.world];
  return SGL_OK;
}

extern "C" int sgl_p2p_route_send(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                                  const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows,
                                  uint64_t step, int32_t* d_status, void* stream_) {
  SGL_REQUIRE(ctx && h_send_rows && dim > 0, SGL_ERR_ARG, "p2p_route_send: bad argument");
  Ctx* x = (Ctx*)ctx;
  Splits seg;
  int rc = make_splits(x, h_send_rows, &seg, "p2p_route_send");
  if (rc) return rc;
  const int64_t n_send = seg.off[x->cfg.world];
  const int64_t pitch = sgl_wire_pitch(dim, ts != nullptr, 1);
  SGL_REQUIRE(pitch == x->cfg.pitch, SGL_ERR_ARG, "p2p_route_send: wire pitch %lld differs from the context's %u",
              (long long)pitch, x->cfg.pitch);
  SGL_REQUIRE(n_send == 0 || (feats && send_idx && remote_idx), SGL_ERR_ARG, "p2p_route_send: null array");
  cudaStream_t stream = (cudaStream_t)stream_;
  const bool vec = dim % 4 == 0 && ((uintptr_t)feats & 15) == 0;
  if (vec) {
    const int grid = p2p_grid(n_send * (pitch / 4));
    p2p_send_kernel<4><<<grid, kThreads, 0, stream>>>(x->cfg, feats, n_rows, (uint32_t)dim, ts, send_idx, remote_idx, seg, step,
                                                     x->counters, d_status);
  } else {
    const int grid = p2p_grid(n_send * pitch);
    p2p_send_kernel<1><<<grid, kThreads, 0, stream>>>(x->cfg, feats, n_rows, (uint32_t)dim, ts, send_idx, remote_idx, seg, step,
                                                     x->counters, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_p2p_route_recv(void* ctx, const int64_t* h_recv_rows, float* data, int64_t data_rows, int64_t dim,
                                  int has_ts, float* ts_table, uint64_t step, int32_t* d_status, void* stream_) {
  SGL_REQUIRE(ctx && h_recv_rows && dim > 0, SGL_ERR_ARG, "p2p_route_recv: bad argument");
  SGL_REQUIRE(!has_ts || ts_table, SGL_ERR_ARG, "p2p_route_recv: rows carry a timestamp but ts_table is null");
  Ctx* x = (Ctx*)ctx;
  Splits seg;
  int rc = make_splits(x, h_recv_rows, &seg, "p2p_route_recv");
  if (rc) return rc;
  const int64_t n_recv = seg.off[x->cfg.world];
  const int64_t width = dim + (has_ts ? 1 : 0);
  SGL_REQUIRE(sgl_wire_pitch(dim, has_ts, 1) == x->cfg.pitch, SGL_ERR_ARG, "p2p_route_recv: wire pitch differs from the context's");
  SGL_REQUIRE(n_recv == 0 || data, SGL_ERR_ARG, "p2p_route_recv: null table");
  cudaStream_t stream = (cudaStream_t)stream_;
  const bool vec = dim % 4 == 0 && ((uintptr_t)data & 15) == 0;
  if (vec) {
    const int grid = p2p_grid(n_recv * ((width + 3) / 4));
    p2p_recv_kernel<4><<<grid, kThreads, 0, stream>>>(x->cfg, seg, (uint32_t)width, data, data_rows, (uint32_t)dim, ts_table,
                                                     step, x->counters + 32, d_status);
  } else {
    const int grid = p2p_grid(n_recv * width);
    p2p_recv_kernel<1><<<grid, kThreads, 0, stream>>>(x->cfg, seg, (uint32_t)width, data, data_rows, (uint32_t)dim, ts_table,
                                                     step, x->counters + 32, d_status);
  }
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_p2p_route_step(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                                  const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows,
                                  const int64_t* h_recv_rows, float* data, int64_t data_rows, float* ts_table,
                                  uint64_t step, int32_t* d_status, void* stream) {
  int rc = sgl_p2p_route_send(ctx, feats, n_rows, dim, ts, send_idx, remote_idx, h_send_rows, step, d_status, stream);
  if (rc) return rc;
  return sgl_p2p_route_recv(ctx, h_recv_rows, data, data_rows, dim, ts != nullptr, ts_table, step, d_status, stream);
}

// diagnostics: copies the per-step kernel timeline (ns; send start/end, apply start/flags seen/end) to the host
extern "C" int sgl_p2p_route_timeline(void* ctx, unsigned long long* h_out, int64_t steps) {
  Ctx* x = (Ctx*)ctx;
  SGL_REQUIRE(x && x->cfg.tl && h_out && steps <= 4096, SGL_ERR_ARG, "p2p_route_timeline: not enabled (SGL_P2P_DBG=2)");
  SGL_CUDA_CHECK(cudaMemcpy(h_out, x->cfg.tl, (size_t)steps * 8 * 8, cudaMemcpyDeviceToHost));
  return SGL_OK;
}
