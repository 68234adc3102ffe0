// Temporal neighbour sampling, one warp per target, two kernels per hop:
//
//   sample_count_kernel  warp-cooperative 32-ary search of the row's time-sorted timestamps for the
//                        candidate window [lo, cut); stores the window and min(fanout, cut-lo); the last
//                        CTA to finish turns the per-CTA totals into CTA base offsets (no spinning: a
//                        fence + counter decides who is last).
//   sample_fill_kernel   CTA-local exclusive scan of the counts (+ CTA base) gives every target its
//                        output offset.  Windows that are copied as they are (recent: the tail of the
//                        window; uniform with no more candidates than the fan-out) are written one
//                        OUTPUT ELEMENT per thread -- every lane busy, stores coalesced, all loads of a
//                        thread independent of each other; a target that draws (uniform: Floyd's
//                        k-subset with Philox4x32-10, ranked ascending) is handled by one warp.
//
// Algorithmic HBM bytes per target: 16 (indptr pair) + 16 (target id, time) + 8*ceil(log2 deg) (search
// probes) + k_eff*24 (nbr, ts, eid reads) + k_eff*36 (five output arrays) + 8 (offset).
#include "common.cuh"
#include "scan.cuh"

namespace sgl {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kCtaThreads = kWarpsPerCta * 32;
// Targets per warp (TPW) of the count kernel is chosen per launch: 1 for small batches (every target gets its own
// warp: enough warps to hide the latency of the few dependent loads), 32 for larger ones, where the searches run one
// target per LANE (8-ary steps: seven independent probes per round, so a 32-edge block takes two rounds) and the
// number of CTAs -- hence the length of the last-CTA scan -- stays small.
constexpr int kFillTargets = 32;   // targets per CTA of the fill kernel when the count kernel ran 256 per CTA

// first position p in [lo, hi) with ts[p] >= bound (hi when none); all 32 lanes cooperate and agree
__device__ __forceinline__ int64_t warp_lower_bound(const int64_t* __restrict__ ts, int64_t lo, int64_t hi,
                                                    int64_t bound, int lane) {
  while (hi - lo > 32) {
    int64_t stride = (hi - lo + 31) >> 5;
    int64_t p = lo + (int64_t)(lane + 1) * stride - 1;
    if (p > hi - 1) p = hi - 1;
    bool less = __ldg(ts + p) < bound;
    unsigned b = __ballot_sync(0xffffffffu, less);
    int c = __popc(b);  // probes are monotone, so the true ones are lanes [0, c)
    if (c == 32) return hi;
    int64_t p_first_false = lo + (int64_t)(c + 1) * stride - 1;
    if (p_first_false > hi - 1) p_first_false = hi - 1;
    if (c > 0) {
      int64_t p_last_true = lo + (int64_t)c * stride - 1;
      if (p_last_true > hi - 1) p_last_true = hi - 1;
      lo = p_last_true + 1;
    }
    hi = p_first_false;
  }
  bool less = (lo + lane < hi) && (__ldg(ts + lo + lane) < bound);
  return lo + __popc(__ballot_sync(0xffffffffu, less));
}

struct Philox {
  uint32_t c[4];
  __device__ __forceinline__ Philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    c[0] = c0; c[1] = c1; c[2] = c2; c[3] = c3;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
      uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
      uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
      c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
  }
};

// first position p in [lo, hi) with ts[p] >= bound, one lane on its own: k-ary steps with independent probes (every
// probe of a lane is its own 32-byte sector, so far-apart probes cost load/store-unit slots: 3 per round while the
// range is wide, 7 once it is narrow and the probes share a few lines), then the last <= 8 candidates at once
__device__ __forceinline__ int64_t lane_lower_bound(const int64_t* __restrict__ ts, int64_t lo, int64_t hi, int64_t bound) {
  while (hi - lo > 256) {
    const int64_t q = (hi - lo) >> 2;
    int c = 0;                          // the probes are monotone: the first c of them are "less"
#pragma unroll
    for (int j = 1; j < 4; ++j) c += (__ldg(ts + lo + j * q) < bound) ? 1 : 0;
    const int64_t nlo = c ? lo + c * q + 1 : lo;
    if (c < 3) hi = lo + (c + 1) * q;
    lo = nlo;
  }
  while (hi - lo > 8) {
    const int64_t q = (hi - lo) >> 3;   // >= 1, and lo + 7 q < hi
    int c = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j) c += (__ldg(ts + lo + j * q) < bound) ? 1 : 0;
    const int64_t nlo = c ? lo + c * q + 1 : lo;
    if (c < 7) hi = lo + (c + 1) * q;
    lo = nlo;
  }
  int c = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) c += (lo + j < hi && __ldg(ts + lo + j) < bound) ? 1 : 0;
  return lo + c;
}

// The same bound through the fence of the row (timestamp of the last edge of every 32-edge block, see sgl_tcsr_fence):
// the block that holds the answer is found in the fence -- a small array that lives in L2 -- and only that block of the
// row is read: one or two 128-byte lines of the timestamps per search instead of 32 scattered sectors per round.
__device__ __forceinline__ int64_t warp_fenced_lower_bound(const int64_t* __restrict__ ts, const int64_t* __restrict__ fence_row,
                                                           int64_t s, int64_t e, int64_t bound, int lane) {
  int64_t p0 = s;
  if (e - s > 32) {
    const int64_t nb = (e - s + 31) >> 5;
    const int64_t j = warp_lower_bound(fence_row, 0, nb, bound, lane);
    if (j >= nb) return e;
    p0 = s + (j << 5);
  }
  const bool less = (p0 + lane < e) && (__ldg(ts + p0 + lane) < bound);
  return p0 + __popc(__ballot_sync(0xffffffffu, less));
}

__device__ __forceinline__ int64_t lane_fenced_lower_bound(const int64_t* __restrict__ ts, const int64_t* __restrict__ fence_row,
                                                           int64_t s, int64_t e, int64_t bound) {
  if (e - s <= 32) return lane_lower_bound(ts, s, e, bound);
  const int64_t nb = (e - s + 31) >> 5;
  const int64_t j = lane_lower_bound(fence_row, 0, nb, bound);
  if (j >= nb) return e;
  const int64_t p0 = s + (j << 5), p1 = p0 + 32 < e ? p0 + 32 : e;
  return lane_lower_bound(ts, p0, p1, bound);
}

template <int TPW>
__global__ void __launch_bounds__(kCtaThreads)
sample_count_kernel(const int64_t* __restrict__ indptr, const int64_t* __restrict__ ts, const int64_t* __restrict__ fence,
                    int64_t num_nodes,
                    const int64_t* __restrict__ targets, const int64_t* __restrict__ target_ts, int64_t n_cap,
                    const int64_t* d_n, int fanout, int equal_root_time, int64_t allowed_offset,
                    int64_t* __restrict__ win_lo, int64_t* __restrict__ win_cut, int32_t* __restrict__ cnt,
                    int64_t* __restrict__ cta_sums, unsigned int* done_counter, int64_t* __restrict__ out_offsets,
                    int32_t* d_status) {
  constexpr int TPC = kWarpsPerCta * TPW;
  const int64_t n = eff_count(n_cap, d_n);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t my_cnt = 0;   // count of target (blockIdx.x * TPC + threadIdx.x), held by thread threadIdx.x < TPC
  if (TPW == 32) {
    const int64_t i = (int64_t)blockIdx.x * TPC + threadIdx.x;
    if (i < n) {
      int64_t node = targets[i], t = target_ts[i], lo = 0, cut = 0;
      if (node < 0 || node >= num_nodes) {
        dev_flag(d_status, SGL_DEV_BAD_NODE);
      } else {
        int64_t s = __ldg(indptr + node), e = __ldg(indptr + node + 1);
        if (fence) {
          const int64_t* frow = fence + (s >> 5) + node;
          cut = lane_fenced_lower_bound(ts, frow, s, e, t + (equal_root_time ? 1 : 0));
          lo = s;
          if (allowed_offset >= 0) {
            lo = lane_fenced_lower_bound(ts, frow, s, e, t - allowed_offset);
            if (lo > cut) lo = cut;
          }
        } else {
          cut = lane_lower_bound(ts, s, e, t + (equal_root_time ? 1 : 0));
          lo = allowed_offset >= 0 ? lane_lower_bound(ts, s, cut, t - allowed_offset) : s;
        }
      }
      int64_t cand = cut - lo;
      my_cnt = (int32_t)(cand < fanout ? cand : fanout);
      win_lo[i] = lo;
      win_cut[i] = cut;
      cnt[i] = my_cnt;
    }
  } else {
    __shared__ int32_t s_cnt[TPC];
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
      const int slot = warp * TPW + j;
      const int64_t i = (int64_t)blockIdx.x * TPC + slot;
      int32_t c = 0;
      if (i < n) {
        int64_t node = targets[i];
        int64_t t = target_ts[i];
        int64_t lo = 0, cut = 0;
        if (node < 0 || node >= num_nodes) {
          if (lane == 0) dev_flag(d_status, SGL_DEV_BAD_NODE);
        } else {
          int64_t s = __ldg(indptr + node), e = __ldg(indptr + node + 1);
          lo = s;
          cut = s;
          if (e > s && fence) {
            const int64_t* frow = fence + (s >> 5) + node;
            cut = warp_fenced_lower_bound(ts, frow, s, e, t + (equal_root_time ? 1 : 0), lane);
            if (allowed_offset >= 0 && cut > s) {
              lo = warp_fenced_lower_bound(ts, frow, s, e, t - allowed_offset, lane);
              if (lo > cut) lo = cut;
            }
          } else if (e > s) {
            cut = warp_lower_bound(ts, s, e, t + (equal_root_time ? 1 : 0), lane);
            if (allowed_offset >= 0 && cut > s) lo = warp_lower_bound(ts, s, cut, t - allowed_offset, lane);
          }
        }
        int64_t cand = cut - lo;
        c = (int32_t)(cand < fanout ? cand : fanout);
        if (lane == 0) {
          win_lo[i] = lo;
          win_cut[i] = cut;
          cnt[i] = c;
        }
      }
      if (lane == 0) s_cnt[slot] = c;
    }
    __syncthreads();
    if (threadIdx.x < TPC) my_cnt = s_cnt[threadIdx.x];
  }
  int cta_total;
  cta_exclusive_scan<kCtaThreads, int>(my_cnt, &cta_total);
  // grand total -> out_offsets[n_cap]; the slots of the targets themselves are written by the fill kernel
  publish_and_scan_cta_totals<kCtaThreads>((int64_t)cta_total, cta_sums, done_counter, out_offsets + n_cap);
}

// CT = targets per CTA of the count kernel (whose scanned totals are the CTA bases), FT = targets of this CTA
// (FT divides CT): the CTA rebuilds the prefix inside its count CTA from the counts, which are a coalesced read of at
// most 1 KB that hits L2.
template <int CT, int FT>
__global__ void __launch_bounds__(kCtaThreads)
sample_fill_kernel(const int64_t* __restrict__ nbr, const int64_t* __restrict__ ts, const int64_t* __restrict__ eid,
                   const int64_t* __restrict__ target_ts, int64_t n_cap, const int64_t* d_n, int fanout, int policy,
                   int keep_root_time, uint64_t seed, uint32_t rng_stream, const int64_t* __restrict__ win_lo,
                   const int64_t* __restrict__ win_cut, const int32_t* __restrict__ cnt,
                   const int64_t* __restrict__ cta_base, int64_t* __restrict__ out_nbr, int64_t* __restrict__ out_dst,
                   int64_t* __restrict__ out_ts, float* __restrict__ out_dt, int64_t* __restrict__ out_dt_i64,
                   int64_t* __restrict__ out_eid, int64_t* __restrict__ out_offsets) {
  static_assert(CT % FT == 0 && CT <= kCtaThreads && FT % kWarpsPerCta == 0, "fill CTAs tile the count CTAs");
  __shared__ int32_t s_ex[FT + 1];   // offset of the target's first element inside the count CTA's output; [FT] = end
  __shared__ int32_t s_cnt[FT];
  __shared__ int64_t s_lo[FT], s_cut[FT], s_t[FT];
  const int64_t n = eff_count(n_cap, d_n);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t first = (int64_t)blockIdx.x * FT;          // this CTA's first target
  const int64_t count_cta = first / CT;
  const int sub = (int)(first - count_cta * CT);           // where this CTA's targets start inside the count CTA
  const int64_t base = cta_base[count_cta];
  {
    const int64_t i = count_cta * CT + threadIdx.x;
    const bool in_ct = threadIdx.x < CT;
    const int slot = (int)threadIdx.x - sub;
    const bool mine = in_ct && slot >= 0 && slot < FT;
    const int c = (in_ct && i < n) ? cnt[i] : 0;
    int64_t lo = 0, cut = 0, t = 0;
    if (mine && i < n) {
      lo = win_lo[i];
      cut = win_cut[i];
      t = target_ts[i];
    }
    const int ex = cta_exclusive_scan<kCtaThreads, int>(c, nullptr);
    if (mine) {
      s_ex[slot] = ex;
      s_cnt[slot] = c;
      s_lo[slot] = lo;
      s_cut[slot] = cut;
      s_t[slot] = t;
      if (slot == FT - 1) s_ex[FT] = ex + c;
      // offsets past the valid targets all equal the total, so out_offsets[n..n_cap] stays a valid prefix array
      if (i < n_cap) out_offsets[i] = base + ex;
    }
  }
  __syncthreads();
  const bool draws = policy == SGL_POLICY_UNIFORM;
  // windows copied as they are: one output element per thread
  for (int o = s_ex[0] + (int)threadIdx.x; o < s_ex[FT]; o += kCtaThreads) {
    int a = 0, b = FT;               // last slot with s_ex[slot] <= o (its next offset is > o, so it is not empty)
    while (b - a > 1) {
      const int m = (a + b) >> 1;
      if (s_ex[m] <= o) a = m; else b = m;
    }
    const int c = s_cnt[a];
    const int64_t cut = s_cut[a];
    if (draws && cut - s_lo[a] > fanout) continue;
    const int64_t p = cut - c + (o - s_ex[a]);   // recent: tail of the window; uniform with cand <= k: the whole window
    const int64_t t = s_t[a];
    const int64_t ets = __ldg(ts + p);
    const int64_t g = base + o;
    out_nbr[g] = __ldg(nbr + p);
    out_eid[g] = __ldg(eid + p);
    out_ts[g] = keep_root_time ? t : ets;
    out_dt[g] = (float)(t - ets);
    if (out_dt_i64) out_dt_i64[g] = ets - t;
    out_dst[g] = first + a;
  }
  if (!draws) return;
  // targets that draw: one warp per target
#pragma unroll 1
  for (int slot = warp; slot < FT; slot += kWarpsPerCta) {
    const int64_t i = first + slot;
    if (i >= n) break;
    const int64_t lo = s_lo[slot], cut = s_cut[slot];
    const int64_t cand = cut - lo;
    if (cand <= fanout) continue;
    const int64_t t = s_t[slot];
    const int64_t off = base + s_ex[slot];
    if (fanout > 32) {
      // more draws than lanes: the same selection, with the picks of the target kept in this warp's shared memory
      extern __shared__ uint64_t s_picks_all[];
      uint64_t* picks = s_picks_all + (size_t)warp * fanout;
      for (int d = lane; d < fanout; d += 32) {
        Philox ph((uint32_t)i, (uint32_t)((uint64_t)i >> 32), (uint32_t)d, rng_stream, (uint32_t)seed, (uint32_t)(seed >> 32));
        const uint64_t u = (uint64_t)ph.c[0] | ((uint64_t)ph.c[1] << 32);
        picks[d] = u % (uint64_t)(cand - fanout + d + 1);
      }
      __syncwarp();
      for (int d = 1; d < fanout; ++d) {          // draw d against the (final) draws before it
        const uint64_t mine = picks[d];
        bool clash = false;
        for (int q = lane; q < d; q += 32) clash |= picks[q] == mine;
        clash = __any_sync(0xffffffffu, clash);
        __syncwarp();
        if (clash && lane == 0) picks[d] = (uint64_t)(cand - fanout + d);
        __syncwarp();
      }
      for (int d = lane; d < fanout; d += 32) {   // rank ascending, then copy
        const uint64_t pick = picks[d];
        int rank = 0;
        for (int q = 0; q < fanout; ++q) rank += picks[q] < pick ? 1 : 0;
        const int64_t p = lo + (int64_t)pick;
        const int64_t o = off + rank;
        const int64_t ets = __ldg(ts + p);
        out_nbr[o] = __ldg(nbr + p);
        out_eid[o] = __ldg(eid + p);
        out_ts[o] = keep_root_time ? t : ets;
        out_dt[o] = (float)(t - ets);
        if (out_dt_i64) out_dt_i64[o] = ets - t;
        out_dst[o] = i;
      }
      __syncwarp();
    } else {
      // Floyd's subset selection: draw j picks t_j uniform in [0, cand-k+j]; a repeat is replaced by cand-k+j
      uint64_t pick = 0;
      if (lane < fanout) {
        Philox ph((uint32_t)i, (uint32_t)((uint64_t)i >> 32), (uint32_t)lane, rng_stream, (uint32_t)seed,
                  (uint32_t)(seed >> 32));
        uint64_t u = (uint64_t)ph.c[0] | ((uint64_t)ph.c[1] << 32);
        uint64_t bound = (uint64_t)(cand - fanout + lane + 1);
        pick = u % bound;
      }
      for (int d = 1; d < fanout; ++d) {
        uint64_t mine = __shfl_sync(0xffffffffu, pick, d);
        bool clash = lane < d && pick == mine;
        if (__any_sync(0xffffffffu, clash) && lane == d) pick = (uint64_t)(cand - fanout + d);
      }
      // rank ascending
      int rank = 0;
      for (int d = 0; d < fanout; ++d) {
        uint64_t other = __shfl_sync(0xffffffffu, pick, d);
        rank += (other < pick) ? 1 : 0;
      }
      if (lane < fanout) {
        int64_t p = lo + (int64_t)pick;
        int64_t o = off + rank;
        int64_t ets = __ldg(ts + p);
        out_nbr[o] = __ldg(nbr + p);
        out_eid[o] = __ldg(eid + p);
        out_ts[o] = keep_root_time ? t : ets;
        out_dt[o] = (float)(t - ets);
        if (out_dt_i64) out_dt_i64[o] = ets - t;
        out_dst[o] = i;
      }
    }
  }
}

}  // namespace
}  // namespace sgl

using namespace sgl;

static inline int sample_tpw(int64_t n) { return n <= 16384 ? 1 : 32; }

static inline int64_t sample_num_ctas(int64_t n, int tpw) {
  int64_t tpc = (int64_t)kWarpsPerCta * tpw;
  int64_t b = (n + tpc - 1) / tpc;
  return b < 1 ? 1 : b;
}

extern "C" size_t sgl_sample_ws_bytes(int64_t n_targets) {
  if (n_targets < 1) n_targets = 1;
  return 2 * align_up((size_t)n_targets * 8) + align_up((size_t)n_targets * 4) +
         align_up((size_t)sample_num_ctas(n_targets, 1) * 8) + align_up(sizeof(unsigned int));
}

template <int TPW>
static void launch_sample(int64_t ctas, cudaStream_t stream, const int64_t* indptr, const int64_t* nbr, const int64_t* ts,
                          const int64_t* eid, const int64_t* fence, int64_t num_nodes, const int64_t* targets, const int64_t* target_ts,
                          int64_t n_targets, const int64_t* d_n, int fanout, int policy, int equal_root_time,
                          int64_t allowed_offset, int keep_root_time, uint64_t seed, uint32_t rng_stream, int64_t* win_lo,
                          int64_t* win_cut, int32_t* cnt, int64_t* cta_sums, unsigned int* done, int64_t* out_nbr,
                          int64_t* out_dst, int64_t* out_ts, float* out_dt, int64_t* out_dt_i64, int64_t* out_eid,
                          int64_t* out_offsets, int32_t* d_status) {
  sample_count_kernel<TPW><<<(unsigned)ctas, kCtaThreads, 0, stream>>>(indptr, ts, fence, num_nodes, targets, target_ts,
                                                                       n_targets, d_n, fanout, equal_root_time,
                                                                       allowed_offset, win_lo, win_cut, cnt, cta_sums, done,
                                                                       out_offsets, d_status);
  const size_t pick_smem = (policy == SGL_POLICY_UNIFORM && fanout > 32) ? (size_t)kWarpsPerCta * fanout * sizeof(uint64_t) : 0;
  constexpr int CT = kWarpsPerCta * TPW, FT = CT < kFillTargets ? CT : kFillTargets;
  const unsigned fill_ctas = (unsigned)((n_targets + FT - 1) / FT);
  sample_fill_kernel<CT, FT><<<fill_ctas, kCtaThreads, pick_smem, stream>>>(nbr, ts, eid, target_ts, n_targets, d_n, fanout, policy,
                                                                           keep_root_time, seed, rng_stream, win_lo, win_cut, cnt,
                                                                           cta_sums, out_nbr, out_dst, out_ts, out_dt, out_dt_i64,
                                                                           out_eid, out_offsets);
}

static int sample_layer_impl(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                             const int64_t* fence, int64_t num_nodes, const int64_t* targets, const int64_t* target_ts,
                             int64_t n_targets, const int64_t* d_n, int fanout, int policy, int equal_root_time,
                             int64_t allowed_offset, int keep_root_time, uint64_t seed, uint32_t rng_stream, int64_t* out_nbr,
                             int64_t* out_dst, int64_t* out_ts, float* out_dt, int64_t* out_dt_i64, int64_t* out_eid,
                             int64_t* out_offsets, int32_t* d_status, void* ws, size_t ws_bytes, void* stream_) {
  SGL_NVTX("sgl_sample_layer");
  cudaStream_t stream = (cudaStream_t)stream_;
  SGL_REQUIRE(n_targets >= 0 && num_nodes >= 0, SGL_ERR_ARG, "sample_layer: negative size");
  SGL_REQUIRE(fanout >= 1, SGL_ERR_ARG, "sample_layer: fanout=%d must be >= 1", fanout);
  SGL_REQUIRE(policy == SGL_POLICY_RECENT || policy == SGL_POLICY_UNIFORM, SGL_ERR_ARG,
              "sample_layer: unknown policy %d", policy);
  SGL_REQUIRE(policy != SGL_POLICY_UNIFORM || fanout <= SGL_MAX_UNIFORM_FANOUT, SGL_ERR_UNSUPPORTED,
              "sample_layer: uniform fanout %d > %d", fanout, SGL_MAX_UNIFORM_FANOUT);
  SGL_REQUIRE(out_offsets, SGL_ERR_ARG, "sample_layer: out_offsets is null");
  SGL_REQUIRE(n_targets < ((int64_t)1 << 34), SGL_ERR_UNSUPPORTED, "sample_layer: too many targets");
  if (n_targets == 0) {
    SGL_CUDA_CHECK(cudaMemsetAsync(out_offsets, 0, sizeof(int64_t), stream));
    return SGL_OK;
  }
  SGL_REQUIRE(indptr && nbr && ts && eid && targets && target_ts && out_nbr && out_dst && out_ts && out_dt && out_eid,
              SGL_ERR_ARG, "sample_layer: null array");
  WsCarver c(ws, ws_bytes);
  int64_t* win_lo = c.take<int64_t>(n_targets);
  int64_t* win_cut = c.take<int64_t>(n_targets);
  int32_t* cnt = c.take<int32_t>(n_targets);
  const int tpw = sample_tpw(n_targets);
  const int64_t ctas = sample_num_ctas(n_targets, tpw);
  int64_t* cta_sums = c.take<int64_t>(sample_num_ctas(n_targets, 1));
  unsigned int* done = c.take<unsigned int>(1);
  SGL_REQUIRE(c.ok(), SGL_ERR_WORKSPACE, "sample_layer: workspace %zu < %zu bytes", ws_bytes,
              sgl_sample_ws_bytes(n_targets));
  SGL_CUDA_CHECK(cudaMemsetAsync(done, 0, sizeof(unsigned int), stream));
#define SGL_SAMPLE_ARGS                                                                                               \
  ctas, stream, indptr, nbr, ts, eid, fence, num_nodes, targets, target_ts, n_targets, d_n, fanout, policy, equal_root_time, \
      allowed_offset, keep_root_time, seed, rng_stream, win_lo, win_cut, cnt, cta_sums, done, out_nbr, out_dst,       \
      out_ts, out_dt, out_dt_i64, out_eid, out_offsets, d_status
  if (tpw == 1) launch_sample<1>(SGL_SAMPLE_ARGS);
  else launch_sample<32>(SGL_SAMPLE_ARGS);
#undef SGL_SAMPLE_ARGS
  SGL_LAUNCH_CHECK();
  return SGL_OK;
}

extern "C" int sgl_sample_layer(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                                int64_t num_nodes, const int64_t* targets, const int64_t* target_ts, int64_t n_targets,
                                const int64_t* d_n, int fanout, int policy, int equal_root_time, int64_t allowed_offset,
                                int keep_root_time, uint64_t seed, uint32_t rng_stream, int64_t* out_nbr,
                                int64_t* out_dst, int64_t* out_ts, float* out_dt, int64_t* out_dt_i64,
                                int64_t* out_eid, int64_t* out_offsets, int32_t* d_status, void* ws, size_t ws_bytes,
                                void* stream) {
  return sample_layer_impl(indptr, nbr, ts, eid, nullptr, num_nodes, targets, target_ts, n_targets, d_n, fanout, policy,
                           equal_root_time, allowed_offset, keep_root_time, seed, rng_stream, out_nbr, out_dst, out_ts, out_dt,
                           out_dt_i64, out_eid, out_offsets, d_status, ws, ws_bytes, stream);
}

extern "C" int sgl_sample_layer_fenced(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                                       const int64_t* fence, int64_t num_nodes, const int64_t* targets, const int64_t* target_ts,
                                       int64_t n_targets, const int64_t* d_n, int fanout, int policy, int equal_root_time,
                                       int64_t allowed_offset, int keep_root_time, uint64_t seed, uint32_t rng_stream,
                                       int64_t* out_nbr, int64_t* out_dst, int64_t* out_ts, float* out_dt, int64_t* out_dt_i64,
                                       int64_t* out_eid, int64_t* out_offsets, int32_t* d_status, void* ws, size_t ws_bytes,
                                       void* stream) {
  return sample_layer_impl(indptr, nbr, ts, eid, fence, num_nodes, targets, target_ts, n_targets, d_n, fanout, policy,
                           equal_root_time, allowed_offset, keep_root_time, seed, rng_stream, out_nbr, out_dst, out_ts, out_dt,
                           out_dt_i64, out_eid, out_offsets, d_status, ws, ws_bytes, stream);
}

extern "C" int sgl_sample_gather_fenced(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                                        const int64_t* fence, int64_t num_nodes, const int64_t* targets, const int64_t* target_ts,
                                        int64_t n_targets, int fanout, int policy, int equal_root_time, int64_t allowed_offset,
                                        int keep_root_time, uint64_t seed, uint32_t rng_stream, int64_t* out_nbr, int64_t* out_dst,
                                        int64_t* out_ts, float* out_dt, int64_t* out_eid, int64_t* out_offsets,
                                        const void* feat_table, int64_t feat_rows, int64_t row_bytes, int64_t src_pitch,
                                        void* out_feats, int gather_mode, int32_t* d_status, void* ws, size_t ws_bytes, void* stream) {
  int rc = sample_layer_impl(indptr, nbr, ts, eid, fence, num_nodes, targets, target_ts, n_targets, nullptr, fanout, policy,
                             equal_root_time, allowed_offset, keep_root_time, seed, rng_stream, out_nbr, out_dst, out_ts, out_dt,
                             nullptr, out_eid, out_offsets, d_status, ws, ws_bytes, stream);
  if (rc != SGL_OK || n_targets == 0) return rc;
  return sgl_gather_rows(feat_table, feat_rows, row_bytes, src_pitch, out_eid, nullptr, 0, n_targets * fanout,
                         out_offsets + n_targets, out_feats, row_bytes, nullptr, nullptr, gather_mode, d_status, stream);
}

extern "C" int sgl_sample_gather(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                                 int64_t num_nodes, const int64_t* targets, const int64_t* target_ts, int64_t n_targets,
                                 int fanout, int policy, int equal_root_time, int64_t allowed_offset, int keep_root_time,
                                 uint64_t seed, uint32_t rng_stream, int64_t* out_nbr, int64_t* out_dst, int64_t* out_ts,
                                 float* out_dt, int64_t* out_eid, int64_t* out_offsets, const void* feat_table,
                                 int64_t feat_rows, int64_t row_bytes, int64_t src_pitch, void* out_feats, int gather_mode,
                                 int32_t* d_status, void* ws, size_t ws_bytes, void* stream) {
  SGL_NVTX("sgl_sample_gather");
  int rc = sgl_sample_layer(indptr, nbr, ts, eid, num_nodes, targets, target_ts, n_targets, nullptr, fanout, policy,
                            equal_root_time, allowed_offset, keep_root_time, seed, rng_stream, out_nbr, out_dst, out_ts,
                            out_dt, nullptr, out_eid, out_offsets, d_status, ws, ws_bytes, stream);
  if (rc != SGL_OK || n_targets == 0) return rc;
  return sgl_gather_rows(feat_table, feat_rows, row_bytes, src_pitch, out_eid, nullptr, 0, n_targets * fanout,
                         out_offsets + n_targets, out_feats, row_bytes, nullptr, nullptr, gather_mode, d_status, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// Sampling without caller-provided scratch.
//
// Some hosts of this library cannot hand it device memory on demand: a sampler thread that runs next to a training
// loop must not call cudaMalloc (it stalls every stream of the device while it runs), and a process whose HBM has
// been handed in full to another framework's pool has no allocator of its own to ask.  For them the scratch of one
// hop lives in a fixed array inside the library image instead.  Every GPU that loads the library carries the array
// (about 1.3 MB) until the process exits.
// ---------------------------------------------------------------------------------------------------------------
namespace {
constexpr int64_t kStaticMaxTargets = SGL_STATIC_SAMPLE_MAX_TARGETS;
// same layout as the caller-provided workspace of sgl_sample_layer for kStaticMaxTargets targets
constexpr size_t kStaticScratchBytes = 2 * ((kStaticMaxTargets * 8 + 255) / 256 * 256) + ((kStaticMaxTargets * 4 + 255) / 256 * 256) +
                                       ((kStaticMaxTargets / kWarpsPerCta * 8 + 255) / 256 * 256) + 256;
static __device__ __align__(256) unsigned char g_static_sample_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices];   // device address of the array, per device, filled on first use
}  // namespace

extern "C" int sgl_sample_layer_static(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                                       int64_t num_nodes, const int64_t* targets, const int64_t* target_ts,
                                       int64_t n_targets, int fanout, int policy, int equal_root_time,
                                       int64_t allowed_offset, int keep_root_time, uint64_t seed, uint32_t rng_stream,
                                       int64_t* out_nbr, int64_t* out_dst, int64_t* out_ts, float* out_dt, int64_t* out_eid,
                                       int64_t* out_offsets, int32_t* d_status, void* stream) {
  SGL_REQUIRE(n_targets >= 0 && n_targets <= kStaticMaxTargets, SGL_ERR_ARG,
              "sample_layer_static: %lld targets exceed the built-in scratch (at most %lld per call); use sgl_sample_layer "
              "with your own workspace for larger batches", (long long)n_targets, (long long)kStaticMaxTargets);
  int dev = -1;
  SGL_CUDA_CHECK(cudaGetDevice(&dev));
  SGL_REQUIRE(dev >= 0 && dev < kMaxDevices, SGL_ERR_UNSUPPORTED, "sample_layer_static: device index %d not supported", dev);
  if (g_static_scratch_addr[dev] == nullptr) {
    // In host code the array's name is only a handle; the address kernels can use has to be asked for, once per
    // device, with that device current.
    void* p = nullptr;
    SGL_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_sample_scratch));
    SGL_REQUIRE(p != nullptr, SGL_ERR_CUDA, "sample_layer_static: no device address for the built-in scratch");
    g_static_scratch_addr[dev] = p;
  }
  // sgl_sample_layer clears the one word of the scratch that has to start at zero (the CTA arrival counter) on the
  // stream before its kernels; everything else in the array is written before it is read.
  return sgl_sample_layer(indptr, nbr, ts, eid, num_nodes, targets, target_ts, n_targets, nullptr, fanout, policy,
                          equal_root_time, allowed_offset, keep_root_time, seed, rng_stream, out_nbr, out_dst, out_ts,
                          out_dt, nullptr, out_eid, out_offsets, d_status, g_static_scratch_addr[dev], kStaticScratchBytes,
                          stream);
}
