// Cache route over NVLink peer memory: pack + transfer in ONE kernel, no collective library call per step.
//
// Every rank owns a buffer that all ranks of the node map (CUDA IPC):
//     acks [world]         acks[p] = number of this rank's steps that receiver p has applied (written by p)
//     meta [world][ring]   meta[q][slot] = (plain << 63) | (rows << 32) | tag: how many rows sender q pushed here in the
//                          step that uses the slot, and in which of the two wire forms (below).  The receiver learns its row counts from these words, so a plan that was built on
//                          the device (its sizes never visit the host) needs no count exchange and no host sync.
//     stage[world][ring][cap_rows][pitch / 2]   16-byte lines from sender q, ring slot = step % ring
//
// The wire row of a node is [features | ts | slot lo | slot hi | pad] (pitch 32-bit words, a multiple of 4), the same
// row route_pack_kernel builds.  On the staging buffer every 16-byte line carries two data words and two copies of
// the step's tag:  { w0, tag, w1, tag },  tag = (uint32)(step + 1).  The receiver polls the lines themselves until
// both tags match, so the data needs no separate "rows have landed" flag: no fence, no arrival counter and no last
// CTA on the sender, and the receiver starts on the first lines while the rest are still in flight.  (A line is
// written with one 16-byte store; only 8-byte halves are assumed to arrive atomically, hence one tag per half.)  A
// ring slot is reused every `ring` steps, and a line left from an earlier use carries that step's tag, never the
// current one.
//
// send kernel (rank r, step s):  waits until every receiver has applied step s - ring (so the slot is free), builds
//     the wire rows and stores the tagged lines straight into the receivers' stage[r][s % ring] over NVLink.
// gate kernel (rank p, step s):  one warp waits for every sender's meta word of the step.
// recv kernel (rank p, step s):  behind the gate in the stream; polls the lines of all senders (tagged form), scatters
//     the rows into the node-state table (same work as route_unpack_kernel); the last CTA to finish acknowledges the
//     step to every sender.
//
// Large messages: tagging doubles the bytes on the wire, which is the wrong trade once a message is bandwidth-bound.
// A pair whose message of a step has at least `bulk_rows` rows, and every pair of a step in which the sender pushes at
// least `bulk_total_rows` rows in total (the link out of a GPU is shared by its pairs), uses
// plain wire rows instead -- 128-bit stores into the first half of the same staging region -- followed by one
// system-scope fence per CTA and an arrival counter; the last CTA of the send kernel then writes the pair's meta word,
// which for such a pair doubles as the "rows have landed" flag (for a small pair the meta word is written up front and
// the lines validate themselves).  Small and large pairs can be mixed inside one step.
// (A region that held plain rows and is reused for tagged lines contains arbitrary words, not old tags: a stale line
// passes for a fresh one only if two of its words both equal the new 32-bit tag, a 2^-64 event per line.)
//
// The two kernels of a step run on DIFFERENT GPUs (one process per GPU), never as two launches on one GPU.  Every
// wait is bounded by a wall-clock limit; on expiry the kernel raises SGL_DEV_TIMEOUT in the status word, publishes
// nothing and returns, so the context stays usable.  Every rank must run send and recv for every step (zero rows are
// fine): the handshake is per step, not per row.
#include <string.h>

#include "common.cuh"

namespace sgl {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kThreads = 128;   // 4 warps per CTA, one or two rows per warp at a time
constexpr int kSendThreads = kThreads;
constexpr int kFlatUnroll = 4;   // quads in flight per thread in the plain-rows form of the send kernel
constexpr int kRowsInFlight = 1;   // rows per warp and iteration; more in flight measured slower (299 vs 371 GB/s at 40 MB)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // default bound of every device-side wait (sgl_p2p_route_configure changes it)

struct P2PCfg {
  unsigned long long wait_ns;   // bound of every device-side wait
  int rank, world, ring;
  int64_t cap_rows;
  uint32_t pitch;           // 32-bit words per wire row; a row occupies pitch / 2 lines
  int64_t bulk_rows;        // a pair's message with at least this many rows travels as plain rows + completion word
  int64_t bulk_total_rows;  // ... and so does every pair of a step in which this rank sends at least this many rows
  unsigned long long* acks;
  unsigned long long* meta;
  uint4* stage;
  unsigned long long* peer_acks[kMaxWorld];
  unsigned long long* peer_meta[kMaxWorld];
  uint4* peer_stage[kMaxWorld];
};

struct Splits {
  int64_t off[kMaxWorld + 1];
};

struct Ctx {
  P2PCfg cfg;
  unsigned int* counters;   // device: arrival counters of the send ([0]) and recv ([32]) kernels, credit words [16..24), then the gate words
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// No kernel of this file may hold an SM's registers and thread slots while it waits for another GPU: the work it waits
// for (the peer's send or apply kernel) may in turn be waiting for a kernel of THIS GPU that then finds no room to become
// resident -- with several steps queued on two streams that is a cycle, which only the wait limits would break.  So
// every wait for a peer is done by a one-warp kernel in front of the wide kernel it guards (the "credit" kernel before a
// send, the "gate" kernel before an apply), and the kernels are launched plainly, in stream order (no programmatic
// dependent launch: a dependent that becomes resident early would hold resources while its predecessor waits).

// spin until *p >= want; false when the limit expires
__device__ __forceinline__ bool wait_at_least(const unsigned long long* p, unsigned long long want, unsigned long long limit_ns) {
  const volatile unsigned long long* vp = p;
  if (*vp >= want) return true;
  const unsigned long long t0 = now_ns();
  while (now_ns() - t0 < limit_ns) {
    if (*vp >= want) return true;
    __nanosleep(200);
  }
  return false;
}

__device__ __forceinline__ void store_line(uint4* p, uint32_t w0, uint32_t w1, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(w0), "r"(tag), "r"(w1), "r"(tag) : "memory");
}

__device__ __forceinline__ uint4 load_line(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// a quad of a plain wire row in this GPU's staging buffer: written by a peer, so never through L1 (cached at L2 only);
// unlike load_line the compiler may keep several of these in flight
__device__ __forceinline__ uint4 load_quad_l2(const uint4* p) {
  uint4 v;
  asm("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// re-reads a line until both halves carry the tag; false when the limit expires
__device__ __noinline__ bool poll_line(const uint4* p, uint32_t tag, uint4* v, unsigned long long limit_ns) {
  const unsigned long long t0 = now_ns();
  do {
    *v = load_line(p);
    if (v->y == tag && v->w == tag) return true;
    __nanosleep(100);
  } while (now_ns() - t0 < limit_ns);
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

// quad l (wire words 4l .. 4l+3) of the row built from table row r; r == -2 marks a row that could not be read
__device__ __forceinline__ uint4 wire_quad(uint32_t l, uint32_t dim, uint32_t payload, int vec_ok, const float* __restrict__ feats,
                                           const float* __restrict__ ts, int64_t r, uint64_t slot) {
  uint4 v;
  if (r < 0) {
    const uint32_t e = 4 * l;
    v.x = (e + 0 == payload || e + 0 == payload + 1) ? 0xffffffffu : 0u;
    v.y = (e + 1 == payload || e + 1 == payload + 1) ? 0xffffffffu : 0u;
    v.z = (e + 2 == payload || e + 2 == payload + 1) ? 0xffffffffu : 0u;
    v.w = (e + 3 == payload || e + 3 == payload + 1) ? 0xffffffffu : 0u;
    return v;
  }
  const float* frow = feats + r * dim;
  if (vec_ok && (l + 1) * 4 <= dim) return __ldg((const uint4*)frow + l);
  v.x = wire_word2(4 * l + 0, dim, payload, frow, ts, r, slot);
  v.y = wire_word2(4 * l + 1, dim, payload, frow, ts, r, slot);
  v.z = wire_word2(4 * l + 2, dim, payload, frow, ts, r, slot);
  v.w = wire_word2(4 * l + 3, dim, payload, frow, ts, r, slot);
  return v;
}

__device__ __forceinline__ int segment_of(const int64_t* off, int world, int64_t i) {
  int p = 0;
  while (p + 1 < world && i >= off[p + 1]) ++p;
  return p;
}

__device__ __forceinline__ unsigned long long meta_word(int64_t rows, unsigned long long step, bool plain) {
  return ((unsigned long long)plain << 63) | ((unsigned long long)rows << 32) | (unsigned long long)(uint32_t)(step + 1);
}

// Flow control of a step's send, one warp: the ring slot may be overwritten once every receiver has applied the step
// that used it last.  *credit = 1 when all acknowledgements are there, 0 (and SGL_DEV_TIMEOUT) when the wait ran out.
__global__ void __launch_bounds__(32)
p2p_credit_kernel(P2PCfg c, unsigned long long step, unsigned int* __restrict__ credit, int32_t* d_status) {
  bool ok = true;
  if ((int)threadIdx.x < c.world && step >= (unsigned long long)c.ring)
    ok = wait_at_least(c.acks + threadIdx.x, step - c.ring + 1, c.wait_ns);
  const bool all_ok = __all_sync(0xffffffffu, ok);
  if (threadIdx.x == 0) {
    if (!all_ok) dev_flag(d_status, SGL_DEV_TIMEOUT);
    *credit = all_ok ? 1u : 0u;
  }
}

// A route kernel competes for issue slots with whatever else runs on its SM (warps are scheduled round robin, stream
// priority only decides which CTA is placed first), so on a busy GPU its duration is set by its instruction count per
// warp, not by memory latency.  Hence one WARP per row: the row's index, destination and segment are computed once
// per row with no division, a lane handles a quad (4 consecutive wire words = 2 lines), and many small warps rather
// than few long-running ones share the work.
//
// Row counts per destination come from the host (seg, d_sizes == nullptr) or from device memory (d_sizes[world], the
// send sizes a device-built plan left there); counts above the staging capacity are cut and flagged.
__global__ void __launch_bounds__(kSendThreads)
p2p_send_kernel(P2PCfg c, const float* __restrict__ feats, int64_t n_rows, uint32_t dim, const float* __restrict__ ts,
                const int64_t* __restrict__ send_idx, const int64_t* __restrict__ remote_idx, Splits seg,
                const int64_t* __restrict__ d_sizes, unsigned long long step, int vec_ok, unsigned int* done_counter,
                const unsigned int* __restrict__ credit, int32_t* d_status) {
  __shared__ int s_ok;
  __shared__ bool s_last;
  __shared__ int64_t s_off[kMaxWorld + 1];   // exclusive prefix of the row counts per destination (what is SENT)
  __shared__ int64_t s_src[kMaxWorld + 1];   // the same prefix over the plan's own counts (where the rows sit in send_idx)
  if (threadIdx.x == 0) {
    s_ok = *credit != 0;                      // 0: the credit kernel's wait for the receivers ran out -- send nothing

    s_off[0] = s_src[0] = 0;
    for (int p = 0; p < c.world; ++p) {
      int64_t have = d_sizes ? d_sizes[p] : seg.off[p + 1] - seg.off[p];
      if (have < 0) have = 0;
      int64_t cnt = have;
      if (cnt > c.cap_rows) {
        dev_flag(d_status, SGL_DEV_OVERFLOW);
        cnt = c.cap_rows;
      }
      s_off[p + 1] = s_off[p] + cnt;
      s_src[p + 1] = s_src[p] + have;
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const uint32_t tag = (uint32_t)(step + 1);
  const uint32_t payload = dim + (ts ? 1u : 0u);
  const uint32_t quads = c.pitch / 4;
  const uint32_t lane = threadIdx.x & 31u;
  const int64_t ring_slot = (int64_t)(step % c.ring);
  const bool all_plain = s_off[c.world] >= c.bulk_total_rows;
  bool any_bulk = false;
  for (int p = 0; p < c.world; ++p) {
    const int64_t cnt = s_off[p + 1] - s_off[p];
    any_bulk |= cnt > 0 && (all_plain || cnt >= c.bulk_rows);
  }
  // small pairs: the count goes out first, the tagged lines validate themselves
  if (ok && blockIdx.x == 0 && threadIdx.x < c.world) {
    const int64_t cnt = s_off[threadIdx.x + 1] - s_off[threadIdx.x];
    if (!(cnt > 0 && (all_plain || cnt >= c.bulk_rows))) {
      volatile unsigned long long* m = c.peer_meta[threadIdx.x] + (int64_t)c.rank * c.ring + ring_slot;
      *m = meta_word(cnt, step, false);
    }
  }
  const int64_t n_send = ok ? s_off[c.world] : 0;
  const int64_t n_warps = (int64_t)gridDim.x * (kSendThreads / 32);
  const int64_t slot_base = ((int64_t)c.rank * c.ring + ring_slot) * c.cap_rows;
  // A step whose pairs all travel as plain rows is bandwidth work: one 16-byte quad per thread over the flattened
  // (row, quad) index, kFlatUnroll quads in flight per thread, every load independent of every other -- the layout of the
  // row-gather kernel, whose stores fill a peer's memory at 0.8 of the copy engine's rate (measured), where one warp per
  // row reached 0.5-0.6.
  bool flat = n_send > 0;
  for (int p = 0; p < c.world; ++p) {
    const int64_t cnt = s_off[p + 1] - s_off[p];
    flat = flat && (cnt == 0 || all_plain || cnt >= c.bulk_rows);
  }
  if (flat) {
    const int64_t total = n_send * quads;
    const int64_t stride = (int64_t)gridDim.x * kSendThreads;
    const bool small = total <= 0xffffffffll;
    for (int64_t q0 = (int64_t)blockIdx.x * kSendThreads + threadIdx.x; q0 < total; q0 += stride * kFlatUnroll) {
      uint4 v[kFlatUnroll];
      uint4* d[kFlatUnroll];
#pragma unroll
      for (int u = 0; u < kFlatUnroll; ++u) {
        const int64_t q = q0 + u * stride;
        d[u] = nullptr;
        if (q >= total) continue;
        int64_t i;
        uint32_t l;
        if (small) {
          const uint32_t qq = (uint32_t)q, ii = qq / quads;
          i = ii;
          l = qq - ii * quads;
        } else {
          i = q / quads;
          l = (uint32_t)(q - i * quads);
        }
        const int p = segment_of(s_off, c.world, i);
        const int64_t in_seg = i - s_off[p];
        const int64_t src = s_src[p] + in_seg;
        int64_t r = __ldg(send_idx + src);
        const uint64_t slotv = (uint64_t)__ldg(remote_idx + src);
        if (r < 0) r += n_rows;
        if (r < 0 || r >= n_rows) {
          if (l == 0) dev_flag(d_status, SGL_DEV_BAD_INDEX);
          r = -2;                                           // sent as zeros with slot -1, which the receiver skips
        }
        v[u] = wire_quad(l, dim, payload, vec_ok, feats, ts, r, slotv);
        d[u] = c.peer_stage[p] + slot_base * (c.pitch / 2) + in_seg * (c.pitch / 4) + l;
      }
#pragma unroll
      for (int u = 0; u < kFlatUnroll; ++u)
        if (d[u]) *d[u] = v[u];
    }
  }
  // Two rows per warp and round: the index loads of both are in flight together, and per quad both rows' table loads are
  // issued before either store (a warp is alone with the latency of its dependent loads: few CTAs, many rows per warp).
  for (int64_t i0 = ((int64_t)blockIdx.x * kSendThreads + threadIdx.x) >> 5; i0 < n_send && !flat; i0 += 2 * n_warps) {
    int64_t r[2];
    uint64_t slotv[2];
    uint4* dst[2];
    bool bulk[2], have[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t i = i0 + k * n_warps;
      have[k] = i < n_send;
      r[k] = -2; slotv[k] = 0; dst[k] = nullptr; bulk[k] = false;
      if (!have[k]) continue;
      const int p = segment_of(s_off, c.world, i);
      const int64_t in_seg = i - s_off[p];
      const int64_t src = s_src[p] + in_seg;                // position in the plan's index arrays
      r[k] = __ldg(send_idx + src);                         // one address per warp: a single broadcast load
      slotv[k] = (uint64_t)__ldg(remote_idx + src);
      bulk[k] = all_plain || s_off[p + 1] - s_off[p] >= c.bulk_rows;
      // the pair's region starts at the same place in both layouts; a plain row takes pitch / 4 lines, a tagged one pitch / 2
      uint4* region = c.peer_stage[p] + slot_base * (c.pitch / 2);
      dst[k] = region + in_seg * (bulk[k] ? c.pitch / 4 : c.pitch / 2);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (!have[k]) continue;
      if (r[k] < 0) r[k] += n_rows;
      if (r[k] < 0 || r[k] >= n_rows) {
        if (lane == 0) dev_flag(d_status, SGL_DEV_BAD_INDEX);
        r[k] = -2;                                          // sent as zeros with slot -1, which the receiver skips
      }
    }
    for (uint32_t l = lane; l < quads; l += 32) {
      uint4 q[2];
#pragma unroll
      for (int k = 0; k < 2; ++k)
        if (have[k]) q[k] = wire_quad(l, dim, payload, vec_ok, feats, ts, r[k], slotv[k]);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (!have[k]) continue;
        if (bulk[k]) {
          dst[k][l] = q[k];
        } else {
          store_line(dst[k] + 2 * l, q[k].x, q[k].y, tag);
          store_line(dst[k] + 2 * l + 1, q[k].z, q[k].w, tag);
        }
      }
    }
  }
  if (!any_bulk) return;
  // plain rows are published by the pair's meta word.  One system-scope fence per CTA: the CTA barrier makes every
  // thread's stores happen-before thread 0's fence, and fences are cumulative, so thread 0's fence + counter increment
  // orders the whole CTA's rows before anything the last CTA does after it has seen all increments.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(done_counter, 1u);
    s_last = prev == gridDim.x - 1;
    if (s_last) __threadfence_system();
  }
  __syncthreads();
  if (!s_last) return;
  const bool failed = !ok || (d_status && (*(volatile int32_t*)d_status & SGL_DEV_TIMEOUT));
  if (threadIdx.x < c.world && !failed) {
    const int64_t cnt = s_off[threadIdx.x + 1] - s_off[threadIdx.x];
    if (cnt > 0 && (all_plain || cnt >= c.bulk_rows)) {
      volatile unsigned long long* m = c.peer_meta[threadIdx.x] + (int64_t)c.rank * c.ring + ring_slot;
      *m = meta_word(cnt, step, true);
    }
  }
  if (threadIdx.x == 0) *done_counter = 0;
}

// The wait for the senders is NOT done by the wide apply kernel: CTAs that spin on a word another GPU has yet to write
// hold their SM's registers and thread slots, and enough of them keep this GPU's own send kernel -- which the peers'
// apply kernels are waiting for in the same way -- from ever becoming resident.  One warp waits instead (bounded), leaves
// the senders' words in gate[world], and the wide kernel behind it in the stream starts when every sender has at least
// begun (tagged lines) or finished (plain rows) this step.
__global__ void __launch_bounds__(32)
p2p_gate_kernel(P2PCfg c, unsigned long long step, unsigned long long* __restrict__ gate, int32_t* d_status) {
  const uint32_t tag = (uint32_t)(step + 1);
  if ((int)threadIdx.x >= c.world) return;
  const volatile unsigned long long* m = c.meta + (int64_t)threadIdx.x * c.ring + (int64_t)(step % c.ring);
  unsigned long long w = *m;
  if ((uint32_t)w != tag) {
    const unsigned long long t0 = now_ns();
    bool got = false;
    while (now_ns() - t0 < c.wait_ns) {
      w = *m;
      if ((uint32_t)w == tag) { got = true; break; }
      __nanosleep(100);
    }
    if (!got) {
      w = 0;
      dev_flag(d_status, SGL_DEV_TIMEOUT);
    }
  }
  __threadfence_system();   // acquire side: plain rows written before the meta word are visible to what follows
  gate[threadIdx.x] = w;
}

// One warp per incoming row: every lane reads the line(s) holding the row's slot (one broadcast load per line) and
// the 2 lines of its own quad, and re-polls (bounded) only what has not landed yet.  The number of rows per sender is
// what the sender's meta word says; when the host also named a count (expect.off, check != 0) a difference is flagged.
__global__ void __launch_bounds__(kThreads)
p2p_recv_kernel(P2PCfg c, Splits expect, int check, uint32_t width, float* __restrict__ data, int64_t data_rows, uint32_t dim,
                float* __restrict__ ts_table, unsigned long long step, int vec_ok, unsigned int* done_counter,
                const unsigned long long* __restrict__ gate, int32_t* d_status) {
  __shared__ int s_ok;
  __shared__ bool s_last;
  __shared__ int64_t s_cnt[kMaxWorld];
  __shared__ int64_t s_off[kMaxWorld + 1];
  __shared__ bool s_plain[kMaxWorld];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const uint32_t tag = (uint32_t)(step + 1);
  const uint32_t quads = (width + 3) / 4;                // quads that hold features / ts
  const uint32_t la = width / 2, lb = (width + 1) / 2;   // lines of the slot's low and high word
  const uint32_t lane = threadIdx.x & 31u;
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  const int64_t ring_slot = (int64_t)(step % c.ring);
  // every sender's meta word of this step, as the gate kernel saw it: its row count; for a large pair also the sign that
  // its plain rows landed (a word without the step's tag: the gate's wait ran out)
  if (threadIdx.x < c.world) {
    const unsigned long long w = gate[threadIdx.x];
    if ((uint32_t)w != tag) s_ok = 0;
    int64_t cnt = (uint32_t)w == tag ? (int64_t)((w >> 32) & 0x7fffffffull) : 0;
    s_plain[threadIdx.x] = (w >> 63) != 0;
    if (cnt > c.cap_rows) cnt = c.cap_rows;
    if (check && s_ok && cnt != expect.off[threadIdx.x + 1] - expect.off[threadIdx.x]) dev_flag(d_status, SGL_DEV_MISMATCH);
    s_cnt[threadIdx.x] = cnt;
  }
  // No fence here: the gate kernel saw the senders' words, fenced, and COMPLETED before this kernel started; the rows sit
  // in this GPU's own memory and are read with volatile loads (L2, the point of coherence for peer writes), never from L1.
  __syncthreads();
  if (threadIdx.x == 0) {
    s_off[0] = 0;
    for (int p = 0; p < c.world; ++p) s_off[p + 1] = s_off[p] + s_cnt[p];
  }
  __syncthreads();
  bool ok = s_ok != 0;
  const int64_t n_recv = ok ? s_off[c.world] : 0;
  // Every sender's rows arrived as plain rows: bandwidth work, one quad per thread over the flattened (row, quad) index,
  // kFlatUnroll quads in flight per thread (the row's slot words are one or two more loads that hit L2).
  bool flat = n_recv > 0;
  for (int p = 0; p < c.world; ++p) flat = flat && (s_cnt[p] == 0 || s_plain[p]);
  if (flat) {
    const int64_t total = n_recv * quads;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const bool small = total <= 0xffffffffll;
    for (int64_t q0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; q0 < total; q0 += stride * kFlatUnroll) {
      uint4 v[kFlatUnroll];
      int64_t ds[kFlatUnroll];
      uint32_t ll[kFlatUnroll];
#pragma unroll
      for (int u = 0; u < kFlatUnroll; ++u) {
        const int64_t q = q0 + u * stride;
        ds[u] = -1;
        ll[u] = 0;
        if (q >= total) continue;
        int64_t i;
        uint32_t l;
        if (small) {
          const uint32_t qq = (uint32_t)q, ii = qq / quads;
          i = ii;
          l = qq - ii * quads;
        } else {
          i = q / quads;
          l = (uint32_t)(q - i * quads);
        }
        const int sdr = segment_of(s_off, c.world, i);
        const uint4* prow = c.stage + ((int64_t)sdr * c.ring + ring_slot) * c.cap_rows * (c.pitch / 2) + (i - s_off[sdr]) * (c.pitch / 4);
        const uint4 qa = load_quad_l2(prow + width / 4);
        const uint4 qb = (width + 1) / 4 == width / 4 ? qa : load_quad_l2(prow + (width + 1) / 4);
        v[u] = load_quad_l2(prow + l);
        const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
        const int64_t dslot = (int64_t)((uint64_t)wa[width & 3] | ((uint64_t)wb[(width + 1) & 3] << 32));
        if (dslot < 0 || dslot >= data_rows) {
          if (l == 0) dev_flag(d_status, SGL_DEV_BAD_INDEX);
        } else {
          ds[u] = dslot;
          ll[u] = l;
        }
      }
#pragma unroll
      for (int u = 0; u < kFlatUnroll; ++u) {
        if (ds[u] < 0) continue;
        if (vec_ok && (ll[u] + 1) * 4 <= dim) {
          ((uint4*)(data + ds[u] * dim))[ll[u]] = v[u];
        } else {
          const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t e = 4 * ll[u] + k;
            if (e < dim) data[ds[u] * dim + e] = __uint_as_float(w[k]);
            else if (e < width && ts_table) ts_table[ds[u]] = __uint_as_float(w[k]);
          }
        }
      }
    }
  }
  for (int64_t i = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5; i < n_recv && ok && !flat; i += n_warps) {
    const int sdr = segment_of(s_off, c.world, i);
    const uint4* region = c.stage + ((int64_t)sdr * c.ring + ring_slot) * c.cap_rows * (c.pitch / 2);
    if (s_plain[sdr]) {
      // plain wire row (pitch / 4 quads); volatile loads: the row was written by another GPU
      const uint4* prow = region + (i - s_off[sdr]) * (c.pitch / 4);
      const uint4 qa = load_line(prow + width / 4), qb = load_line(prow + (width + 1) / 4);
      const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
      const int64_t dslot = (int64_t)((uint64_t)wa[width & 3] | ((uint64_t)wb[(width + 1) & 3] << 32));
      const bool bad = dslot < 0 || dslot >= data_rows;
      if (bad && lane == 0) dev_flag(d_status, SGL_DEV_BAD_INDEX);
      for (uint32_t l = lane; l < quads && !bad; l += 32) {
        const uint4 q = load_line(prow + l);
        if (vec_ok && (l + 1) * 4 <= dim) {
          ((uint4*)(data + dslot * dim))[l] = q;
        } else {
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t e = 4 * l + k;
            if (e < dim) data[dslot * dim + e] = __uint_as_float(w[k]);
            else if (e < width && ts_table) ts_table[dslot] = __uint_as_float(w[k]);
          }
        }
      }
      continue;
    }
    const uint4* row = region + (i - s_off[sdr]) * (c.pitch / 2);
    // all loads in flight first; the rows have normally landed long ago
    uint4 sa = load_line(row + la);
    uint4 sb = la == lb ? sa : load_line(row + lb);
    uint4 a = make_uint4(0, tag, 0, tag), b = a;
    if (lane < quads) {
      a = load_line(row + 2 * lane);
      b = load_line(row + 2 * lane + 1);
    }
    if (sa.y != tag || sa.w != tag) ok = ok && poll_line(row + la, tag, &sa, c.wait_ns);
    if (la == lb) sb = sa;
    else if (sb.y != tag || sb.w != tag) ok = ok && poll_line(row + lb, tag, &sb, c.wait_ns);
    if (!ok) break;
    const uint32_t lo = (width & 1) ? sa.z : sa.x;
    const uint32_t hi = ((width + 1) & 1) ? sb.z : sb.x;
    const int64_t dslot = (int64_t)((uint64_t)lo | ((uint64_t)hi << 32));
    const bool bad = dslot < 0 || dslot >= data_rows;
    if (bad && lane == 0) dev_flag(d_status, SGL_DEV_BAD_INDEX);
    for (uint32_t l = lane; l < quads; l += 32) {
      if (l != lane) {
        a = load_line(row + 2 * l);
        b = load_line(row + 2 * l + 1);
      }
      if (a.y != tag || a.w != tag) ok = ok && poll_line(row + 2 * l, tag, &a, c.wait_ns);
      if (b.y != tag || b.w != tag) ok = ok && poll_line(row + 2 * l + 1, tag, &b, c.wait_ns);
      if (!ok || bad) break;
      if (vec_ok && (l + 1) * 4 <= dim) {
        ((uint4*)(data + dslot * dim))[l] = make_uint4(a.x, a.z, b.x, b.z);
      } else {
        const uint32_t w[4] = {a.x, a.z, b.x, b.z};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t e = 4 * l + k;
          if (e < dim) data[dslot * dim + e] = __uint_as_float(w[k]);
          else if (e < width && ts_table) ts_table[dslot] = __uint_as_float(w[k]);
        }
      }
    }
  }
  if (!ok) {
    s_ok = 0;
    dev_flag(d_status, SGL_DEV_TIMEOUT);
  }
  // Acknowledge once every CTA has read its lines.  A thread reaches the barrier only after the values of its polls
  // have been examined, so its loads of the slot are complete by then; the counter is incremented after the CTA's
  // barrier and the acknowledgement is stored after the last increment, so no load of this step can still be in
  // flight when a sender sees the acknowledgement.  No fence is needed for that: nothing this kernel WRITES has to
  // be visible to the senders (the table it writes is read by later kernels of this stream only).
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned prev = atomicAdd(done_counter, 1u);
    s_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  const bool failed = s_ok == 0 || (d_status && (*(volatile int32_t*)d_status & SGL_DEV_TIMEOUT));
  if (threadIdx.x < c.world && !failed) {
    volatile unsigned long long* ak = c.peer_acks[threadIdx.x] + c.rank;   // "rank has applied your step"
    *ak = step + 1;
  }
  if (threadIdx.x == 0) *done_counter = 0;
}

inline size_t header_bytes(int world, int ring) { return align_up((size_t)world * 8 + (size_t)world * ring * 8, 256); }

}  // namespace
}  // namespace sgl

using namespace sgl;

extern "C" size_t sgl_p2p_buffer_bytes(int world, int ring, int64_t cap_rows, int64_t pitch_floats) {
  if (world < 1 || ring < 1 || cap_rows < 0 || pitch_floats < 1) return 0;
  if (pitch_floats % 4) return 0;
  // every 16-byte line holds two wire words and two tags: twice the bytes of the plain wire rows
  return header_bytes(world, ring) + (size_t)world * ring * (size_t)cap_rows * (size_t)pitch_floats * 8;
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
                  cap_rows >= 1 && cap_rows < ((int64_t)1 << 31) && pitch_floats >= 4 && pitch_floats % 4 == 0,
              SGL_ERR_ARG, "p2p_route_create: bad argument (world <= %d, ring >= 2, pitch a multiple of 4)", kMaxWorld);
  for (int p = 0; p < world; ++p)
    SGL_REQUIRE(h_bases[p], SGL_ERR_ARG, "p2p_route_create: base pointer of rank %d is null", p);
  unsigned int* counters = nullptr;   // 256 bytes of arrival counters, then the gate words [ring][kMaxWorld]
  const size_t aux_bytes = 256 + (size_t)ring * kMaxWorld * sizeof(unsigned long long);
  SGL_CUDA_CHECK(cudaMalloc(&counters, aux_bytes));
  if (cudaMemset(counters, 0, aux_bytes) != cudaSuccess) {
    cudaFree(counters);
    set_error("p2p_route_create: cudaMemset of the arrival counters failed");
    return SGL_ERR_CUDA;
  }
  Ctx* x = new Ctx();
  x->counters = counters;
  P2PCfg& c = x->cfg;
  c.wait_ns = kWaitLimitNs;
  c.rank = rank; c.world = world; c.ring = ring; c.cap_rows = cap_rows; c.pitch = (uint32_t)pitch_floats;
  const size_t hb = header_bytes(world, ring);
  for (int p = 0; p < world; ++p) {
    char* b = (char*)h_bases[p];
    c.peer_acks[p] = (unsigned long long*)b;
    c.peer_meta[p] = (unsigned long long*)b + world;
    c.peer_stage[p] = (uint4*)(b + hb);
  }
  c.acks = c.peer_acks[rank];
  c.meta = c.peer_meta[rank];
  c.stage = c.peer_stage[rank];
  // a pair's message of 256 KiB and more, and every pair of a step in which this rank sends four times that in total,
  // travels as plain rows (sgl_p2p_route_configure changes the limit)
  c.bulk_rows = ((256 << 10) + pitch_floats * 4 - 1) / (pitch_floats * 4);
  c.bulk_total_rows = 4 * c.bulk_rows;
  *out_ctx = x;
  return SGL_OK;
}

extern "C" int sgl_p2p_route_configure(void* ctx, int64_t wait_ms, int64_t bulk_bytes) {
  SGL_REQUIRE(ctx, SGL_ERR_ARG, "p2p_route_configure: null context");
  P2PCfg& c = ((Ctx*)ctx)->cfg;
  if (wait_ms >= 0) {
    SGL_REQUIRE(wait_ms >= 1 && wait_ms <= 60000, SGL_ERR_ARG, "p2p_route_configure: wait_ms %lld outside [1, 60000]",
                (long long)wait_ms);
    c.wait_ns = (unsigned long long)wait_ms * 1000000ull;
  }
  if (bulk_bytes >= 0) {
    c.bulk_rows = bulk_bytes == 0 ? 1 : (bulk_bytes + c.pitch * 4 - 1) / ((int64_t)c.pitch * 4);
    c.bulk_total_rows = 4 * c.bulk_rows;
  }
  return SGL_OK;
}

extern "C" int sgl_p2p_route_destroy(void* ctx) {
  if (!ctx) return SGL_OK;
  Ctx* x = (Ctx*)ctx;
  cudaFree(x->counters);
  delete x;
  return SGL_OK;
}

// number of CTAs of a route kernel: enough for the rows, at most four per SM -- small messages are latency-bound and
// every extra CTA adds fence traffic and a longer wait for the last one
static int p2p_grid(int64_t rows) { return stream_grid(rows, kThreads / 32, 4); }
// Send kernel: two rows per warp and round in the tagged form; the flattened plain-rows form strides over whatever grid it
// gets.  Four CTAs per SM for both kernels is the measured optimum on two B200s (40-96 MB per step, send and apply
// running side by side): with eight the two kernels and the incoming writes slow each other, with two or fewer too few
// stores are in flight for the link (send/apply CTAs per SM -> GB/s per direction at 40 MB: 8/8 356, 4/4 437, 2/8 287,
// 1/8 167).
static int send_grid(int64_t rows) { return stream_grid((rows + 1) / 2, kSendThreads / 32, 4); }

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

static int send_impl(Ctx* x, const float* feats, int64_t n_rows, int64_t dim, const float* ts, const int64_t* send_idx,
                     const int64_t* remote_idx, const Splits& seg, const int64_t* d_sizes, int64_t grid_rows, uint64_t step,
                     int32_t* d_status, void* stream_) {
  const int64_t pitch = sgl_wire_pitch(dim, ts != nullptr, 1);
  SGL_REQUIRE(pitch == x->cfg.pitch, SGL_ERR_ARG, "p2p_route_send: wire pitch %lld differs from the context's %u",
              (long long)pitch, x->cfg.pitch);
  SGL_REQUIRE(grid_rows == 0 || (feats && send_idx && remote_idx), SGL_ERR_ARG, "p2p_route_send: null array");
  const int vec_ok = dim % 4 == 0 && ((uintptr_t)feats & 15) == 0;
  unsigned int* credit = x->counters + 16 + (unsigned)(step % 8);   // one word per step in flight (8 >= streams' depth)
  p2p_credit_kernel<<<1, 32, 0, (cudaStream_t)stream_>>>(x->cfg, (unsigned long long)step, credit, d_status);
  p2p_send_kernel<<<send_grid(grid_rows), kSendThreads, 0, (cudaStream_t)stream_>>>(
      x->cfg, feats, n_rows, (uint32_t)dim, ts, send_idx, remote_idx, seg, d_sizes, (unsigned long long)step, vec_ok, x->counters,
      credit, d_status);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_p2p_route_send(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                                  const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows,
                                  uint64_t step, int32_t* d_status, void* stream) {
  SGL_NVTX("sgl_p2p_route_send");
  SGL_REQUIRE(ctx && h_send_rows && dim > 0, SGL_ERR_ARG, "p2p_route_send: bad argument");
  Ctx* x = (Ctx*)ctx;
  Splits seg;
  int rc = make_splits(x, h_send_rows, &seg, "p2p_route_send");
  if (rc) return rc;
  return send_impl(x, feats, n_rows, dim, ts, send_idx, remote_idx, seg, nullptr, seg.off[x->cfg.world], step, d_status, stream);
}

extern "C" int sgl_p2p_route_send_dev(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                                      const int64_t* send_idx, const int64_t* remote_idx, const int64_t* d_send_rows,
                                      int64_t rows_hint, uint64_t step, int32_t* d_status, void* stream) {
  SGL_NVTX("sgl_p2p_route_send_dev");
  SGL_REQUIRE(ctx && d_send_rows && dim > 0 && rows_hint >= 0, SGL_ERR_ARG, "p2p_route_send_dev: bad argument");
  Splits seg;
  memset(&seg, 0, sizeof(seg));
  return send_impl((Ctx*)ctx, feats, n_rows, dim, ts, send_idx, remote_idx, seg, d_send_rows, rows_hint < 1 ? 1 : rows_hint, step,
                   d_status, stream);
}

static int recv_impl(Ctx* x, const Splits& expect, int check, int64_t grid_rows, float* data, int64_t data_rows, int64_t dim,
                     int has_ts, float* ts_table, uint64_t step, int32_t* d_status, void* stream_) {
  SGL_REQUIRE(!has_ts || ts_table, SGL_ERR_ARG, "p2p_route_recv: rows carry a timestamp but ts_table is null");
  const int64_t width = dim + (has_ts ? 1 : 0);
  SGL_REQUIRE(sgl_wire_pitch(dim, has_ts, 1) == x->cfg.pitch, SGL_ERR_ARG, "p2p_route_recv: wire pitch differs from the context's");
  SGL_REQUIRE(grid_rows == 0 || data, SGL_ERR_ARG, "p2p_route_recv: null table");
  const int vec_ok = dim % 4 == 0 && ((uintptr_t)data & 15) == 0;
  unsigned long long* gate = (unsigned long long*)((char*)x->counters + 256) + (size_t)(step % x->cfg.ring) * kMaxWorld;
  p2p_gate_kernel<<<1, 32, 0, (cudaStream_t)stream_>>>(x->cfg, (unsigned long long)step, gate, d_status);
  p2p_recv_kernel<<<p2p_grid(grid_rows), kThreads, 0, (cudaStream_t)stream_>>>(
      x->cfg, expect, check, (uint32_t)width, data, data_rows, (uint32_t)dim, has_ts ? ts_table : (float*)nullptr,
      (unsigned long long)step, vec_ok, x->counters + 32, (const unsigned long long*)gate, d_status);
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_p2p_route_recv(void* ctx, const int64_t* h_recv_rows, float* data, int64_t data_rows, int64_t dim,
                                  int has_ts, float* ts_table, uint64_t step, int32_t* d_status, void* stream) {
  SGL_NVTX("sgl_p2p_route_recv");
  SGL_REQUIRE(ctx && h_recv_rows && dim > 0, SGL_ERR_ARG, "p2p_route_recv: bad argument");
  Ctx* x = (Ctx*)ctx;
  Splits seg;
  int rc = make_splits(x, h_recv_rows, &seg, "p2p_route_recv");
  if (rc) return rc;
  return recv_impl(x, seg, 1, seg.off[x->cfg.world], data, data_rows, dim, has_ts, ts_table, step, d_status, stream);
}

extern "C" int sgl_p2p_route_recv_dev(void* ctx, int64_t rows_hint, float* data, int64_t data_rows, int64_t dim, int has_ts,
                                      float* ts_table, uint64_t step, int32_t* d_status, void* stream) {
  SGL_NVTX("sgl_p2p_route_recv_dev");
  SGL_REQUIRE(ctx && dim > 0 && rows_hint >= 0 && data, SGL_ERR_ARG, "p2p_route_recv_dev: bad argument");
  Splits seg;
  memset(&seg, 0, sizeof(seg));
  return recv_impl((Ctx*)ctx, seg, 0, rows_hint < 1 ? 1 : rows_hint, data, data_rows, dim, has_ts, ts_table, step, d_status, stream);
}

extern "C" int sgl_p2p_route_step(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                                  const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows,
                                  const int64_t* h_recv_rows, float* data, int64_t data_rows, float* ts_table,
                                  uint64_t step, int32_t* d_status, void* stream) {
  int rc = sgl_p2p_route_send(ctx, feats, n_rows, dim, ts, send_idx, remote_idx, h_send_rows, step, d_status, stream);
  if (rc) return rc;
  return sgl_p2p_route_recv(ctx, h_recv_rows, data, data_rows, dim, ts != nullptr, ts_table, step, d_status, stream);
}
