/*
 * CPU oracle in C (OpenMP) -- TEST INFRASTRUCTURE ONLY: the checker and the timed CPU baseline.
 * Nothing in the shipped package links or calls this file.
 *
 * Restates the reference's CPU path (paths inside the reference project):
 *   orc_tcsr_build    MaterializedMultiLayerBuilder.__init__        prepare_sample.py:179-203
 *   orc_sample_layer  _jit_sample_kernel (continuous graph branch)  prepare_sample.py:32-172
 *                     two passes over the targets -- count, prefix sum, fill -- parallel over targets,
 *                     exactly the structure of the numba kernel (prange over tasks)
 *   orc_gather_rows   DistNodeState.__getitem__ / index_select      starrygl/cache/NodeState.py:36-44
 *   orc_cache_gather  CachedNodeState.get hit/miss split (design)   starrygl/cache/NodeState.py:152-194
 * The uniform policy draws its k distinct positions with Philox4x32-10 + Floyd's algorithm, the same
 * counter layout as oracle_np.uniform_positions, so GPU results can be compared bit for bit.
 * Parity pin: tests/test_oracle_golden.py checks these functions against vectors produced by the reference.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <omp.h>

typedef int64_t i64;

int orc_num_threads(void) { return omp_get_max_threads(); }
void orc_set_threads(int n) { omp_set_num_threads(n); }

/* ---- T-CSR: counting sort by key, then a stable sort by ts inside each row --------------------- */
typedef struct { i64 ts; i64 pos; } tp_t;
static int cmp_tp(const void* a, const void* b) {
  const tp_t *x = a, *y = b;
  if (x->ts != y->ts) return x->ts < y->ts ? -1 : 1;
  return x->pos < y->pos ? -1 : (x->pos > y->pos);
}

int orc_tcsr_build(i64 n, i64 m, const i64* key, const i64* nbr, const i64* ts, const i64* eid, i64* indptr,
                   i64* o_nbr, i64* o_ts, i64* o_eid, i64* o_perm) {
  memset(indptr, 0, (size_t)(n + 1) * sizeof(i64));
  for (i64 i = 0; i < m; ++i) {
    if (key[i] < 0 || key[i] >= n) return -1;
    indptr[key[i] + 1]++;
  }
  for (i64 v = 0; v < n; ++v) indptr[v + 1] += indptr[v];
  i64* fill = malloc((size_t)(n + 1) * sizeof(i64));
  tp_t* tmp = malloc((size_t)(m ? m : 1) * sizeof(tp_t));
  memcpy(fill, indptr, (size_t)(n + 1) * sizeof(i64));
  for (i64 i = 0; i < m; ++i) {
    i64 p = fill[key[i]]++;
    tmp[p].ts = ts[i];
    tmp[p].pos = i;
  }
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 v = 0; v < n; ++v) qsort(tmp + indptr[v], (size_t)(indptr[v + 1] - indptr[v]), sizeof(tp_t), cmp_tp);
#pragma omp parallel for
  for (i64 p = 0; p < m; ++p) {
    i64 i = tmp[p].pos;
    o_nbr[p] = nbr[i];
    o_ts[p] = ts[i];
    o_eid[p] = eid ? eid[i] : i;
    if (o_perm) o_perm[p] = i;
  }
  free(fill);
  free(tmp);
  return 0;
}

/* ---- Philox4x32-10 ---------------------------------------------------------------------------------- */
static void philox(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    c[1] = (uint32_t)p1; c[3] = (uint32_t)p0; c[0] = n0; c[2] = n2;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
}

static void uniform_positions(i64 cand, int k, uint64_t seed, uint32_t stream, i64 slot, i64* out) {
  for (int j = 0; j < k; ++j) {
    uint32_t c[4] = {(uint32_t)slot, (uint32_t)((uint64_t)slot >> 32), (uint32_t)j, stream};
    philox(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    uint64_t u = (uint64_t)c[0] | ((uint64_t)c[1] << 32);
    i64 bound = cand - k + j + 1;
    i64 t = (i64)(u % (uint64_t)bound);
    for (int q = 0; q < j; ++q)
      if (out[q] == t) { t = bound - 1; break; }
    out[j] = t;
  }
  for (int a = 1; a < k; ++a) {   /* insertion sort, k is small */
    i64 v = out[a];
    int b = a - 1;
    while (b >= 0 && out[b] > v) { out[b + 1] = out[b]; --b; }
    out[b + 1] = v;
  }
}

static i64 lower_bound(const i64* a, i64 n, i64 v) {
  i64 lo = 0, hi = n;
  while (lo < hi) {
    i64 mid = lo + ((hi - lo) >> 1);
    if (a[mid] < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

/* offsets[n_targets+1] out; data arrays need capacity n_targets*fanout; returns the total. policy 0 recent, 1 uniform */
i64 orc_sample_layer(const i64* indptr, const i64* nbr, const i64* ts, const i64* eid, const i64* targets,
                     const i64* target_ts, i64 n_targets, int fanout, int policy, int equal_root_time,
                     i64 allowed_offset, int keep_root_time, uint64_t seed, uint32_t stream, i64* o_nbr, i64* o_dst,
                     i64* o_ts, float* o_dt, i64* o_eid, i64* offsets) {
  i64* lo_a = malloc((size_t)(n_targets ? n_targets : 1) * sizeof(i64));
  i64* cut_a = malloc((size_t)(n_targets ? n_targets : 1) * sizeof(i64));
  /* pass 1: count */
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < n_targets; ++i) {
    i64 s = indptr[targets[i]], e = indptr[targets[i] + 1], t = target_ts[i];
    i64 cut = lower_bound(ts + s, e - s, t + (equal_root_time ? 1 : 0));
    i64 lo = allowed_offset >= 0 ? lower_bound(ts + s, cut, t - allowed_offset) : 0;
    i64 cand = cut - lo;
    lo_a[i] = s + lo;
    cut_a[i] = s + cut;
    offsets[i + 1] = cand < fanout ? cand : fanout;
  }
  offsets[0] = 0;
  for (i64 i = 0; i < n_targets; ++i) offsets[i + 1] += offsets[i];
  /* pass 2: fill */
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < n_targets; ++i) {
    i64 c = offsets[i + 1] - offsets[i];
    if (c == 0) continue;
    i64 w = offsets[i], t = target_ts[i], lo = lo_a[i], cut = cut_a[i];
    i64 pos[64];
    if (policy == 1 && cut - lo > fanout) {
      uniform_positions(cut - lo, fanout, seed, stream, i, pos);
      for (int j = 0; j < c; ++j) pos[j] += lo;
    }
    for (i64 j = 0; j < c; ++j) {
      i64 p = (policy == 1 && cut - lo > fanout) ? pos[j] : cut - c + j;
      o_nbr[w + j] = nbr[p];
      o_dst[w + j] = i;
      o_ts[w + j] = keep_root_time ? t : ts[p];
      o_dt[w + j] = (float)(t - ts[p]);
      o_eid[w + j] = eid[p];
    }
  }
  free(lo_a);
  free(cut_a);
  return offsets[n_targets];
}

/* ---- gather ----------------------------------------------------------------------------------------- */
void orc_gather_rows(const char* table, i64 rows, i64 row_bytes, const i64* idx, i64 n, char* out) {
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < n; ++i) {
    i64 r = idx[i] < 0 ? idx[i] + rows : idx[i];
    memcpy(out + i * row_bytes, table + r * row_bytes, (size_t)row_bytes);
  }
}

/* returns the number of misses; miss_pos/miss_ids in ascending position */
i64 orc_cache_gather(const char* cache, const int32_t* hitmap, const char* backing, i64 row_bytes, const i64* ids, i64 n,
                     char* out, i64* miss_pos, i64* miss_ids) {
  i64 nm = 0;
  for (i64 i = 0; i < n; ++i)
    if (hitmap[ids[i]] < 0) { miss_pos[nm] = i; miss_ids[nm] = ids[i]; ++nm; }
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < n; ++i) {
    int32_t s = hitmap[ids[i]];
    memcpy(out + i * row_bytes, s >= 0 ? cache + (i64)s * row_bytes : backing + ids[i] * row_bytes, (size_t)row_bytes);
  }
  return nm;
}
