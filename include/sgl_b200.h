/*
 * sgl_b200.h -- C ABI of libsgl_b200.so: the per-mini-batch data path of a temporal-GNN trainer
 * (T-CSR build, temporal neighbour sampling, relabel, feature/memory gather through a cache, route
 * pack/unpack) as hand-written sm_100a CUDA kernels.
 *
 * Conventions
 *   - Every function returns 0 on success or a negative SGL_ERR_* code; sgl_last_error() gives the
 *     message of the last failure on the calling thread.  Nothing throws across this boundary.
 *   - Pointers are DEVICE pointers unless the parameter name starts with h_.  `stream` is a
 *     cudaStream_t passed as void*; work is only ever enqueued on that stream (never on the default
 *     stream unless the caller passes it) and, unless stated, the call returns without synchronising.
 *   - The library allocates no device memory on these paths: scratch comes from the caller as
 *     (ws, ws_bytes); the *_ws_bytes() functions give the required size.  ws must be 256-byte aligned.
 *   - `d_status` is an optional device int32 the kernels OR error bits into (SGL_DEV_*); the caller
 *     zeroes it and reads it back at its own synchronisation points.
 *   - Counts that are only known on the device (the number of edges a hop produced) can be chained to
 *     the next call through `d_n` parameters: a device int64 that overrides the host count, which then
 *     only acts as the capacity the launch is sized for.
 *   - Callable from any host thread (no Python, no global locks); the device of the pointers must be
 *     current on the calling thread.
 *
 * Each entry point names the reference interface it replaces (path inside the reference project).
 */
#ifndef SGL_B200_H
#define SGL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SGL_OK 0
#define SGL_ERR_ARG (-1)         /* bad argument (null pointer, negative size, misaligned buffer) */
#define SGL_ERR_WORKSPACE (-2)   /* workspace too small */
#define SGL_ERR_CUDA (-3)        /* a CUDA runtime call failed */
#define SGL_ERR_RANGE (-4)       /* an id or timestamp outside the declared range was found */
#define SGL_ERR_UNSUPPORTED (-5) /* valid request the kernels do not cover (see message) */

/* bits OR-ed into *d_status by kernels */
#define SGL_DEV_BAD_NODE 1   /* node id outside [0, num_nodes) */
#define SGL_DEV_BAD_TS 2     /* timestamp outside the declared [ts_base, ts_base + 2^ts_bits) window */
#define SGL_DEV_BAD_INDEX 4  /* row index outside the table */
#define SGL_DEV_OVERFLOW 8   /* an output capacity was exceeded */
#define SGL_DEV_TIMEOUT 16   /* a bounded device-side wait gave up (copy engine or peer did not signal in time) */
#define SGL_DEV_MISMATCH 32  /* a peer's message size differs from the size the receiver was told to expect */

#define SGL_POLICY_RECENT 0
#define SGL_POLICY_UNIFORM 1
#define SGL_MAX_UNIFORM_FANOUT 512   /* picks of a target are kept in shared memory: 8 warps x 512 x 8 bytes per CTA */

const char* sgl_last_error(void);
/* Library version and the SM architecture the kernels were compiled for ("sm_100a"). */
const char* sgl_build_info(void);

/* ------------------------------------------------------------------------------------------------
 * Stable LSD radix sort of 64-bit keys carrying a 32-bit payload (used by the T-CSR build and the
 * relabel; exported so it can be tested on its own).  Sorts on key bits [0, num_bits).  On return
 * *h_result_in_alt tells whether the sorted data are in (keys, vals) [0] or in (keys_alt, vals_alt) [1].
 * Replaces: thrust::sort calls in csrc/include/starrygl/sample.cu.hpp:1078, :1197, :1795.
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_radix_sort_ws_bytes(int64_t n);
/* kernels launched by one sort of n keys of num_bits key bits (launch accounting of callers that replay captured graphs) */
int sgl_radix_sort_launches(int64_t n, int num_bits);
int sgl_radix_sort_u64_u32(uint64_t* keys, uint32_t* vals, uint64_t* keys_alt, uint32_t* vals_alt, int64_t n,
                           int num_bits, int* h_result_in_alt, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * T-CSR construction.  Rows are keyed by `key` (node id in [0, num_nodes)); inside a row edges are in
 * ascending `ts`, ties in input order.  eid may be NULL (edge id = input position).
 * Outputs: indptr[num_nodes+1], nbr/ts/eid[m] in row order, perm[m] (optional) = input position of
 * every sorted edge.  h_ts_range[2] (optional, host) receives min and max timestamp.
 * Synchronises the stream once (the number of sort passes depends on the timestamp range).
 * Replaces: Graph::Graph + build_graph_kernel (csrc/include/starrygl/sample.cu.hpp:985-1185, :83-114)
 * reached through from_edge_index (csrc/srcs/starrygl/export.cu:229-250); CPU twin
 * MaterializedMultiLayerBuilder.__init__ (prepare_sample.py:179-203).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_tcsr_build_ws_bytes(int64_t num_nodes, int64_t m);
int sgl_tcsr_build(int64_t num_nodes, int64_t m, const int64_t* key, const int64_t* nbr, const int64_t* ts,
                   const int64_t* eid, int64_t* indptr, int64_t* out_nbr, int64_t* out_ts, int64_t* out_eid,
                   int64_t* out_perm, int64_t* h_ts_range, void* ws, size_t ws_bytes, void* stream);

/* Search index over the T-CSR rows ("fence"): the timestamp of the last edge of every block of 32 consecutive edges of a
 * row; row r with edges [s, e) owns out_fence[(s >> 5) + r + j], j < ceil((e - s) / 32).  sgl_tcsr_fence_len() entries
 * (about 1.6 % of the adjacency, small enough to stay in L2).  The *_fenced sampling entry points search it first and
 * then read one block of the row instead of probing the row itself round after round; results are identical.
 * Replaces: the dependent probes of binary_lower_bound / binary_upper_bound over the whole row
 * (csrc/include/starrygl/sample.cu.hpp:218-295). */
int64_t sgl_tcsr_fence_len(int64_t num_nodes, int64_t m);
int sgl_tcsr_fence(const int64_t* indptr, const int64_t* ts, int64_t num_nodes, int64_t m, int64_t* out_fence, void* stream);

/* ------------------------------------------------------------------------------------------------
 * One hop of temporal neighbour sampling, one warp per target.
 * Target i = (targets[i], target_ts[i]).  Candidates: row edges with ts < t (ts <= t when
 * equal_root_time; additionally ts >= t - allowed_offset when allowed_offset >= 0).
 *   RECENT : the last min(fanout, candidates), ascending time.
 *   UNIFORM: all candidates if there are <= fanout, else fanout distinct positions chosen with
 *            Philox4x32-10 keyed by (seed; target index i, rng_stream), ascending position.
 * Outputs are compact, in target order: out_nbr/out_dst/out_ts/out_eid int64, out_dt float32 = t - ts,
 * out_dst = i; out_offsets[n_targets+1] (exclusive prefix of per-target counts; last = total).
 * out_dt_i64 (optional) additionally receives ts - t as int64, the sign and type of the reference's
 * CUDA result type (TemporalNeighbor.neighbors_dt, csrc/include/starrygl/sample.cu.hpp:751, :811).
 * Output arrays need capacity n_targets * fanout.  keep_root_time writes t instead of the edge time.
 * d_n (optional): device count of valid targets (<= n_targets).
 * Replaces: sample_src_in_chunks_khop + static_recent_neighbor_num / recent_sample_single_hop_kernel /
 * static_neighbor_num / uniform_sample_single_hop_kernel (csrc/include/starrygl/sample.cu.hpp:1532-1716,
 * :706-827); CPU twin _jit_sample_kernel (prepare_sample.py:32-172).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_sample_ws_bytes(int64_t n_targets);
int sgl_sample_layer(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                     int64_t num_nodes, const int64_t* targets, const int64_t* target_ts, int64_t n_targets,
                     const int64_t* d_n, int fanout, int policy, int equal_root_time, int64_t allowed_offset,
                     int keep_root_time, uint64_t seed, uint32_t rng_stream, int64_t* out_nbr, int64_t* out_dst,
                     int64_t* out_ts, float* out_dt, int64_t* out_dt_i64, int64_t* out_eid, int64_t* out_offsets,
                     int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* sgl_sample_layer / sgl_sample_gather with the rows' fence (sgl_tcsr_fence; NULL = search the rows directly). */
int sgl_sample_layer_fenced(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                            const int64_t* fence, int64_t num_nodes, const int64_t* targets, const int64_t* target_ts,
                            int64_t n_targets, const int64_t* d_n, int fanout, int policy, int equal_root_time,
                            int64_t allowed_offset, int keep_root_time, uint64_t seed, uint32_t rng_stream, int64_t* out_nbr,
                            int64_t* out_dst, int64_t* out_ts, float* out_dt, int64_t* out_dt_i64, int64_t* out_eid,
                            int64_t* out_offsets, int32_t* d_status, void* ws, size_t ws_bytes, void* stream);
int sgl_sample_gather_fenced(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                             const int64_t* fence, int64_t num_nodes, const int64_t* targets, const int64_t* target_ts,
                             int64_t n_targets, int fanout, int policy, int equal_root_time, int64_t allowed_offset,
                             int keep_root_time, uint64_t seed, uint32_t rng_stream, int64_t* out_nbr, int64_t* out_dst,
                             int64_t* out_ts, float* out_dt, int64_t* out_eid, int64_t* out_offsets, const void* feat_table,
                             int64_t feat_rows, int64_t row_bytes, int64_t src_pitch, void* out_feats, int gather_mode,
                             int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * sgl_sample_layer for callers that cannot provide scratch memory.  (No counterpart in the reference: its
 * sampler allocates thrust vectors inside every call.)
 *
 * Who needs it: a sampler thread running beside a training loop, where a cudaMalloc would stall every stream
 * of the GPU for its duration, and hosts whose device memory belongs entirely to another framework's pool, so
 * that there is nothing left to allocate from.  Here the scratch of the hop is a fixed array inside the
 * library itself (about 1.3 MB, resident on every GPU that loads the library until the process exits); the
 * call performs no cudaMalloc / cudaFree and uses no allocating library routine.  Inputs and outputs are the
 * caller's, exactly as for sgl_sample_layer (no device-side target count, no int64 dt output).
 *
 * Limits and rules:
 *   - at most SGL_STATIC_SAMPLE_MAX_TARGETS targets per call; more is refused with SGL_ERR_ARG and a message;
 *   - the first call on each device looks up the array's device address (that device must be current); make
 *     that first call before starting any stream capture;
 *   - all calls on a device share the one array, which still holds whatever the previous call left there;
 *     the word that must start at zero is cleared on the stream by the call itself.  Two calls that can run
 *     at the same time on the GPU (different streams, different host threads) race on it: serialise them.
 * ---------------------------------------------------------------------------------------------- */
#define SGL_STATIC_SAMPLE_MAX_TARGETS 65536
int sgl_sample_layer_static(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                            int64_t num_nodes, const int64_t* targets, const int64_t* target_ts, int64_t n_targets,
                            int fanout, int policy, int equal_root_time, int64_t allowed_offset, int keep_root_time,
                            uint64_t seed, uint32_t rng_stream, int64_t* out_nbr, int64_t* out_dst, int64_t* out_ts,
                            float* out_dt, int64_t* out_eid, int64_t* out_offsets, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * One hop of sampling followed by the gather of the sampled edges' feature rows, in one call:
 * sgl_sample_layer(...) and then out_feats[j, :] = feat_table[out_eid[j], :] for the edges the hop produced
 * (their number never reaches the host: the gather reads it from out_offsets[n_targets]).  out_feats needs
 * capacity n_targets * fanout rows of row_bytes.  gather_mode is an SGL_GATHER_* value.
 * Replaces: the sampler call plus the edge-feature read a mini-batch triggers
 * (starrygl/graph/graph.py:139-151 and starrygl/nn/model/tgn.py:161-162).
 * ---------------------------------------------------------------------------------------------- */
int sgl_sample_gather(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid,
                      int64_t num_nodes, const int64_t* targets, const int64_t* target_ts, int64_t n_targets,
                      int fanout, int policy, int equal_root_time, int64_t allowed_offset, int keep_root_time,
                      uint64_t seed, uint32_t rng_stream, int64_t* out_nbr, int64_t* out_dst, int64_t* out_ts,
                      float* out_dt, int64_t* out_eid, int64_t* out_offsets, const void* feat_table,
                      int64_t feat_rows, int64_t row_bytes, int64_t src_pitch, void* out_feats, int gather_mode,
                      int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * (node, ts)-pair relabel.  Input = two concatenated segments A (n_a items) then B (n_b items);
 * output = the sorted (id, then ts) unique union, its size (*d_n_unique, device), and for every input
 * item the rank of its pair in the union (inv_a, inv_b; either may be NULL).  Timestamps must lie in
 * [ts_base, ts_base + 2^ts_bits) and ids in [0, 2^id_bits); id_bits + ts_bits <= 64.
 * d_n_a / d_n_b (optional) are device counts overriding n_a / n_b (which remain the capacities).
 * Replaces: _get_unique_pairs (A only) and _merge_and_map_nodes (A = current list, B = new pairs)
 * (prepare_sample.py:205-213, :231-246).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_unique_pairs_ws_bytes(int64_t n_total);
int sgl_unique_pairs(const int64_t* a_id, const int64_t* a_ts, int64_t n_a, const int64_t* d_n_a,
                     const int64_t* b_id, const int64_t* b_ts, int64_t n_b, const int64_t* d_n_b, int id_bits,
                     int ts_bits, int64_t ts_base, int64_t* out_id, int64_t* out_ts, int64_t* inv_a, int64_t* inv_b,
                     int64_t* d_n_unique, int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * CSC of one sampled hop: stable order by (dst_local, ts); indptr over the num_dst rows of the
 * previous node list.  dst_map (optional): dst_local = dst_map[dst[e]] (the previous hop's inverse map),
 * else dst_local = dst[e].  num_dst may be overridden by the device count d_num_dst (indptr is then
 * written for d_num_dst+1 entries; capacity num_dst+1).  presorted != 0 (dst_map must be NULL): the edges already are
 * in (dst, ts) order -- the first hop of a batch, whose target i is row i of the list -- and the sort is skipped
 * (the order is checked: a violation raises SGL_DEV_BAD_INDEX).
 * Replaces: _build_csc_from_pairs (prepare_sample.py:215-229).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_build_csc_ws_bytes(int64_t n_edges, int64_t num_dst);
int sgl_build_csc(const int64_t* src_local, const int64_t* dst, const int64_t* dst_map, const int64_t* ts,
                  const float* dt, const int64_t* eid, int64_t n_edges, const int64_t* d_n_edges, int64_t num_dst,
                  const int64_t* d_num_dst, int dst_bits, int ts_bits, int64_t ts_base, int64_t* out_indptr,
                  int64_t* out_indices, int64_t* out_ts, float* out_dt, int64_t* out_eid, int presorted,
                  int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Node-level relabel of one id list against an epoch table.  mapper[num_nodes] and mask[num_nodes]
 * persist across calls; ids whose mask != epoch are new: they get consecutive local ids starting at
 * *d_next_local in ascending global id, are appended to out_new_ids, and the tables are updated.
 * out_local[i] = local id of ids[i].  *d_next_local is advanced; *d_n_new receives the number appended.
 * Replaces: Remapper::remapper + mark_new_ids_kernel / update_new_ids_kernel
 * (csrc/include/starrygl/sample.cu.hpp:1719-1824).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_relabel_nodes_ws_bytes(int64_t n);
int sgl_relabel_nodes(const int64_t* ids, int64_t n, const int64_t* d_n, int64_t num_nodes, int64_t* mapper,
                      int64_t* mask, int64_t epoch, int64_t* d_next_local, int64_t* out_local, int64_t* out_new_ids,
                      int64_t* d_n_new, int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Row gather: out[i, :] = table[row(i), :], row(i) = map ? map[idx[i]] : idx[i]; a negative row counts
 * from the end (the indexing rule of the reference's tensor indexing).  row_bytes is the payload per
 * row, src_pitch / dst_pitch the distance between rows in bytes.  ts_table (optional, float32): also
 * out_ts[i] = ts_table[row(i)].  Rows that are 16-byte multiples on 16-byte aligned bases move as
 * 128-bit lanes or as bulk asynchronous copies staged through shared memory; others as 4-byte lanes.
 * Replaces: DistNodeState.__getitem__ / IDMapper.to_local (starrygl/cache/NodeState.py:36-44,
 * starrygl/utils/partition_book.py:106-133), edge-feature and mailbox row reads
 * (starrygl/nn/model/tgn.py:161-162, starrygl/nn/memory/mailbox.py:92-93), tensor_gather
 * (csrc/include/starrygl/feature.cu.hpp:42-88).
 * ---------------------------------------------------------------------------------------------- */
#define SGL_GATHER_AUTO 0
#define SGL_GATHER_VEC 1   /* 128-bit lanes */
#define SGL_GATHER_BULK 2  /* cp.async.bulk through shared memory */
int sgl_gather_rows(const void* table, int64_t table_rows, int64_t row_bytes, int64_t src_pitch, const int64_t* idx,
                    const int64_t* map, int64_t map_len, int64_t n, const int64_t* d_n, void* out, int64_t dst_pitch,
                    const float* ts_table, float* out_ts, int mode, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Gather through a device-resident cache.  slot = hitmap[ids[i]] (int32; < 0 = miss).  Hits are copied
 * from cache_rows[slot]; misses from backing[ids[i]] when backing != NULL (any device-accessible
 * memory, e.g. mapped pinned host memory), else left untouched.  The misses are compacted in
 * ascending i into miss_pos (position i) and miss_ids (ids[i]); counts[0] = hits, counts[1] = misses.
 * Replaces: the hit/miss split designed in CachedNodeState.get (starrygl/cache/NodeState.py:152-194).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_cache_gather_ws_bytes(int64_t n);
int sgl_cache_gather(const void* cache_rows, int64_t cache_slots, const int32_t* hitmap, int64_t num_ids,
                     const void* backing, int64_t row_bytes, const int64_t* ids, int64_t n, void* out,
                     int64_t* miss_pos, int64_t* miss_ids, int64_t* d_counts, int32_t* d_status, void* ws,
                     size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Device-counted prefix copy: dst[a][0 .. *d_count * elem_bytes[a]) = src[a][...] for up to 8 arrays in one
 * launch (*d_count clamped to [0, cap]); an array with elem_bytes[a] < 0 is copied whole (-elem_bytes[a] bytes,
 * for fixed-size companions such as the offsets).  src / dst / elem_bytes are HOST arrays; the pointers in them are device
 * pointers or pinned host pointers, 16-byte aligned.  With dst in pinned host memory a result whose length only
 * the device knows (the sampled edges of a batch) crosses PCIe with exactly its bytes and without a host round trip.
 * No reference counterpart (the reference's CUDA sampler sizes its result arrays on the host,
 * csrc/include/starrygl/sample.cu.hpp:898-903).
 * ---------------------------------------------------------------------------------------------- */
int sgl_copy_prefix(int n_arrays, const void* const* src, void* const* dst, const int64_t* elem_bytes,
                    const int64_t* d_count, int64_t cap, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Row scatter: table[row(i), :] = rows[i, :] for rows with row(i) >= 0 (row(i) = map ? map[idx[i]] :
 * idx[i]); optional ts_table[row(i)] = ts[i].  With split_last_col the source rows carry one extra
 * trailing float32 column that goes to ts_table instead of `ts` (the embedding||ts wire rows).
 * Duplicate destination rows inside one call are a data race (as in the reference).
 * Replaces: DistNodeState.update (starrygl/cache/NodeState.py:46-61), remote_write_callback
 * (starrygl/cache/NodeState.py:269-274).
 * ---------------------------------------------------------------------------------------------- */
int sgl_scatter_rows(void* table, int64_t table_rows, int64_t row_bytes, int64_t dst_pitch, const int64_t* idx,
                     const int64_t* map, int64_t map_len, int64_t n, const int64_t* d_n, const void* rows,
                     int64_t src_pitch, float* ts_table, const float* ts, int split_last_col, int32_t* d_status,
                     void* stream);

/* ------------------------------------------------------------------------------------------------
 * Route pack: the send buffer of the all-to-all, already grouped by destination rank because send_idx is.
 *   packed[i, 0:D] = feats[send_idx[i], 0:D]
 *   packed[i, D]   = ts[send_idx[i]]                 when ts != NULL
 *   packed[i, W:W+2] = remote_idx[i] (int64 as two 32-bit words, W = D or D+1)   when remote_idx != NULL
 * float32 rows; the row pitch is sgl_wire_pitch(D, ts != NULL, remote_idx != NULL) floats: W without slots, else
 * W + 2 rounded up to a multiple of 4 (zero padded) so that rows move as 128-bit lanes when D % 4 == 0.  Replaces: torch.cat([emb, ts]) + local_features[plan.send_indices] and the
 * separate index message (starrygl/cache/NodeState.py:267, starrygl/cache/cache_route.py:243-258), and
 * x[send_index] (starrygl/route/route.py:428).
 * ---------------------------------------------------------------------------------------------- */
int64_t sgl_wire_pitch(int64_t dim, int has_ts, int has_slot);
int sgl_route_pack(const float* feats, int64_t n_rows, int64_t dim, const float* ts, const int64_t* send_idx,
                   const int64_t* remote_idx, int64_t n_send, float* packed, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Route unpack (receiver side of the wire format above, row pitch sgl_wire_pitch(dim, width > dim, 1)): slot =
 * the int64 after the payload; data[slot, 0:dim] = row[0:dim]; ts_table[slot] = row[dim] when ts_table != NULL (width = dim + 1).
 * Replaces: remote_write_callback (starrygl/cache/NodeState.py:269-274).
 * ---------------------------------------------------------------------------------------------- */
int sgl_route_unpack(const float* packed, int64_t n, int64_t width, float* data, int64_t data_rows, int64_t dim,
                     float* ts_table, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Native communicator (one per process / GPU) for the variable-size all-to-all of the route layer: grouped
 * ncclSend/ncclRecv on the caller's stream.  Rank 0 creates the id (SGL_COMM_ID_BYTES bytes) and hands it to
 * the other ranks out of band (e.g. through the launcher's key-value store); every rank then calls sgl_comm_init
 * with its device current.  Replaces: create_nccl_id / DistContext (csrc/include/starrygl/commContext.cu.hpp:11-51).
 * ---------------------------------------------------------------------------------------------- */
#define SGL_COMM_ID_BYTES 128
int sgl_comm_unique_id(char* out_id, size_t id_bytes);
int sgl_comm_init(void** out_comm, int rank, int world, const char* id_bytes);
int sgl_comm_destroy(void* comm);
/* rank / size of a communicator (DistContext::get_rank / get_size, csrc/include/starrygl/commContext.cu.hpp:54-60). */
int sgl_comm_info(void* comm, int* out_rank, int* out_world);
/* Enable peer access from the current device to the listed devices that this process can see; *out_accessible =
 * how many of them (the current one included) are now reachable.  Replaces: init_p2p
 * (csrc/include/starrygl/feature.cu.hpp:30-40 as exported at :715). */
int sgl_init_p2p(const int* devices, int n, int* out_accessible);

/* Rows of row_floats float32: segment p of `send` (h_send_rows[p] rows, host array of world entries) goes to rank
 * p; segment p of `recv` (h_recv_rows[p] rows) arrives from rank p.  Enqueued on `stream`, no synchronisation.
 * Replaces: DistContext::send_data_to_all / send_indices_to_all (csrc/include/starrygl/commContext.cu.hpp:85-174)
 * and dist.all_to_all_single with split sizes (starrygl/cache/cache_route.py:243-258, starrygl/route/route.py:430). */
int sgl_route_exchange(void* comm, const float* send, const int64_t* h_send_rows, float* recv,
                       const int64_t* h_recv_rows, int64_t row_floats, void* stream);

/* One cache-route step in one call: pack (sgl_route_pack into send_buf), exchange, and -- when apply != 0 --
 * unpack (sgl_route_unpack from recv_buf into data / ts_table).  send_buf / recv_buf hold sum(h_send_rows) /
 * sum(h_recv_rows) rows of sgl_wire_pitch(dim, ts != NULL, 1) floats.  With apply == 0 the caller applies the received rows
 * later with sgl_route_unpack (the reference applies them when the returned future is waited on).
 * Replaces: CacheRoute.update_with_plan + remote_write_callback (starrygl/cache/cache_route.py:211-277,
 * starrygl/cache/NodeState.py:245-282). */
int sgl_cache_route_step(void* comm, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                         const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows,
                         const int64_t* h_recv_rows, float* send_buf, float* recv_buf, float* data, int64_t data_rows,
                         float* ts_table, int apply, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Cache route over NVLink peer memory (one node): the pack and the transfer are ONE kernel that stores the wire
 * rows straight into the receivers' staging buffers, as 16-byte lines that carry the step's tag next to the data
 * (the receiver polls the lines themselves; there is no separate flag and no fence); a second kernel on the
 * receiver applies them and acknowledges the step.  A pair's message of 256 KiB and more, and every message of a step
 * in which the sender pushes four times that in total (sgl_p2p_route_configure changes the limit), is bandwidth-bound
 * and travels as plain rows followed by a fence and a per-pair word instead.
 * Every sender also tells every receiver how many rows it pushed (one 8-byte word per pair and step), so the
 * receiver needs no count exchange: a plan whose sizes exist only in device memory (sgl_plan_route's d_send_sizes)
 * is routed without a host synchronisation (sgl_p2p_route_send_dev / sgl_p2p_route_recv_dev).
 * No collective-library call per step.  Consecutive route
 * kernels of a stream are launched with programmatic stream serialization: they may become resident early but
 * touch nothing before the previous kernel of the stream has completed.  Set-up (not on the batch path, allocates): every rank allocates one buffer
 * of sgl_p2p_buffer_bytes() with sgl_p2p_alloc (zeroed, returns a 64-byte inter-process handle), the handles
 * are exchanged out of band, every rank maps the others with sgl_p2p_open and builds a context from the
 * world-sized array of base pointers (its own entry = its own buffer).
 * Per step, on every rank, with the same `step` number (0, 1, 2, ...): sgl_p2p_route_send (rows for rank p =
 * h_send_rows[p], grouped by destination like the plan's send_indices), later sgl_p2p_route_recv
 * (h_recv_rows[q] rows expected from rank q; a different count on the wire raises SGL_DEV_MISMATCH) which writes
 * data[slot] / ts_table[slot].  Both are asynchronous on the
 * stream.  A rank may run ahead of a peer by at most `ring` steps; device-side waits are bounded (2 s unless
 * configured) and end in SGL_DEV_TIMEOUT in *d_status instead of hanging.  At most cap_rows rows per (sender,
 * receiver, step); a device-side count above that is cut and raises SGL_DEV_OVERFLOW.
 * The *_dev forms size their launch for rows_hint rows (any value works; it only sets the number of CTAs).
 * Replaces: the same reference code as sgl_cache_route_step; ShardTensor's peer-memory design
 * (csrc/include/starrygl/feature.cu.hpp:142-422) is the closest reference counterpart.
 * ---------------------------------------------------------------------------------------------- */
#define SGL_P2P_HANDLE_BYTES 64
size_t sgl_p2p_buffer_bytes(int world, int ring, int64_t cap_rows, int64_t pitch_floats);
int sgl_p2p_alloc(size_t bytes, void** out_ptr, char* out_handle, size_t handle_bytes);
int sgl_p2p_open(const char* handle, void** out_ptr);
int sgl_p2p_close(void* peer_ptr);
int sgl_p2p_free(void* ptr);
int sgl_p2p_route_create(int rank, int world, int ring, int64_t cap_rows, int64_t pitch_floats, void* const* h_bases,
                         void** out_ctx);
/* wait_ms: bound of every device-side wait (1..60000); bulk_bytes: message size from which a pair uses plain rows
 * (0 = always; a sender whose step totals four times that uses them for all its pairs).  A negative value leaves the
 * setting as it is.  The sender tells the receiver which form it used, so ranks may differ in this setting. */
int sgl_p2p_route_configure(void* ctx, int64_t wait_ms, int64_t bulk_bytes);
int sgl_p2p_route_destroy(void* ctx);
int sgl_p2p_route_send(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                       const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows, uint64_t step,
                       int32_t* d_status, void* stream);
int sgl_p2p_route_send_dev(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                           const int64_t* send_idx, const int64_t* remote_idx, const int64_t* d_send_rows,
                           int64_t rows_hint, uint64_t step, int32_t* d_status, void* stream);
int sgl_p2p_route_recv(void* ctx, const int64_t* h_recv_rows, float* data, int64_t data_rows, int64_t dim, int has_ts,
                       float* ts_table, uint64_t step, int32_t* d_status, void* stream);
int sgl_p2p_route_recv_dev(void* ctx, int64_t rows_hint, float* data, int64_t data_rows, int64_t dim, int has_ts,
                           float* ts_table, uint64_t step, int32_t* d_status, void* stream);
/* send + recv of one step in one call (for callers that apply the received rows right away) */
int sgl_p2p_route_step(void* ctx, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                       const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows,
                       const int64_t* h_recv_rows, float* data, int64_t data_rows, float* ts_table, uint64_t step,
                       int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Reverse route accumulate: x[send_idx[s + j], :] += outs[s + j, :] for the peer segment [s, s + len);
 * one call per peer segment, in peer order, keeps the reference's summation order.
 * Replaces: the per-peer loop of RouteContext._recv_post (starrygl/route/route.py:461-464).
 * ---------------------------------------------------------------------------------------------- */
int sgl_route_add_rows(float* x, int64_t n_rows, int64_t dim, const int64_t* send_idx, const float* outs,
                       int64_t seg_len, int32_t* d_status, void* stream);

/* All peer segments of the reverse route in one launch.  The received rows `outs` are grouped by destination:
 * group u adds outs[pos[j], :] for j in [row_ptr[u], row_ptr[u+1]) -- positions ascending, i.e. in peer order -- to
 * x[rows[u], :], one contribution after the other, which gives the float32 result of the per-peer loop bit for bit.
 * The grouping (a stable sort of the route's send_index) is built once per route.
 * Replaces: the whole loop of RouteContext._recv_post (starrygl/route/route.py:456-466). */
int sgl_route_add_grouped(float* x, int64_t n_rows, int64_t dim, const int64_t* rows, const int64_t* row_ptr,
                          const int64_t* pos, int64_t n_groups, const float* outs, int64_t n_outs, int32_t* d_status,
                          void* stream);

/* ------------------------------------------------------------------------------------------------
 * Gather from a row table sharded over the GPUs of one node: out[i, :] = shard[part(i)][loc(i), :] with
 * dist_idx[i] = (part << 48) | loc (sgl_dist_pack).  d_bases[world] (DEVICE array) holds every shard's base address as
 * seen from this GPU -- its own memory or a peer mapping (sgl_p2p_open) -- d_shard_rows[world] the shards' row counts.
 * Rows are read from their owner directly over NVLink: no id exchange, no row exchange, no reorder pass.
 * Replaces: ShardTensor::operator[] (csrc/include/starrygl/feature.cu.hpp:298-422: split ids by owner, exchange ids,
 * owner-side tensor_gather :42-88, exchange rows, scatter to the original order).
 * ---------------------------------------------------------------------------------------------- */
int sgl_shard_gather(const void* const* d_bases, const int64_t* d_shard_rows, int world, int64_t row_bytes,
                     const int64_t* dist_idx, int64_t n, const int64_t* d_n, void* out, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * DistRouteIndex packing: dist = (loc & (2^48-1)) | ((part & 0x3FFF) << 48) | (shared << 62).
 * Replaces: DistRouteIndex (starrygl/utils/partition_book.py:7-52); device twins get_partition /
 * get_loc / is_shared (csrc/include/starrygl/feature.cu.hpp:16-28).
 * ---------------------------------------------------------------------------------------------- */
int sgl_dist_pack(const int64_t* loc, const int64_t* part, const uint8_t* shared, int64_t n, int64_t* dist,
                  void* stream);
int sgl_dist_unpack(const int64_t* dist, int64_t n, int64_t* loc, int64_t* part, uint8_t* shared, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Replica lookup: for ids[i] the CSR row [indptr[id], indptr[id+1]) of (rank, loc) replicas is expanded:
 * out_src = i repeated, out_rank, out_loc; out_offsets[n+1] = exclusive prefix of row lengths.
 * Output capacity `cap`; overflow sets SGL_DEV_OVERFLOW.
 * Replaces: CSRReplicaTable.lookup (starrygl/cache/replica_table.py:16-82).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_replica_lookup_ws_bytes(int64_t n);
int sgl_replica_lookup(const int64_t* indptr, const int64_t* ranks, const int64_t* locs, int64_t num_nodes,
                       const int64_t* ids, int64_t n, int64_t cap, int64_t* out_src, int64_t* out_rank,
                       int64_t* out_loc, int64_t* out_offsets, int32_t* d_status, void* ws, size_t ws_bytes,
                       void* stream);

/* ------------------------------------------------------------------------------------------------
 * Sub-graph of a chunk set and a time window as a two-level CSR (node -> distinct timestamps -> edges).
 * Kept edges: source node in a selected chunk (chunk_mask[node_chunk[src]] != 0; null mask = all), t_begin <= ts <
 * t_end, neighbour in a selected chunk too.  Outputs: out_nodes[U] (ascending ids of nodes that keep an edge),
 * out_node_ptr[U+1] into the groups, out_group_ts[G], out_group_ptr[G+1] into the edges, out_nbr / out_ts /
 * out_eid[E] in T-CSR order; d_counts = {U, G, E}.  Capacities: out_nodes and out_node_ptr num_nodes (+1), the group
 * and edge arrays cap_edges (+1); more kept edges than cap_edges raise SGL_DEV_OVERFLOW and nothing is written.
 * Replaces: Graph::slice_by_chunk_ts + count_edges_kernel / write_edges_kernel
 * (csrc/include/starrygl/sample.cu.hpp:1189-1291, :300-520).  The reference's version indexes its chunk table by
 * block number instead of chunk id and drops the first timestamp group of every node; the contract here is the
 * one stated above (window half open like the root extraction).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_slice_window_ws_bytes(int64_t num_nodes);
int sgl_slice_window(const int64_t* indptr, const int64_t* nbr, const int64_t* ts, const int64_t* eid, int64_t num_nodes,
                     const int64_t* node_chunk, const uint8_t* chunk_mask, int64_t num_chunks, int64_t t_begin,
                     int64_t t_end, int64_t cap_edges, int64_t* out_nodes, int64_t* out_node_ptr, int64_t* out_group_ts,
                     int64_t* out_group_ptr, int64_t* out_nbr, int64_t* out_ts, int64_t* out_eid, int64_t* d_counts,
                     int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* Dense per-time-step groups (the reference's use_full_timestamps form, for graphs whose timestamps are snapshot
 * numbers): every one of the n_nodes nodes of a two-level CSR (node_ptr / group_ts / group_ptr as written by
 * sgl_slice_window, or roots / ts_ptr / ts / q_ptr as written by sgl_seeds_in_window) gets ALL time steps
 * t_begin .. t_end-1: out_node_ptr[u] = u * T, out_ts[u * T + j] = t_begin + j, out_group_ptr[u * T + j] = first edge of
 * the node with timestamp >= t_begin + j (empty groups where the node has no event at that step); capacities
 * n_nodes + 1, n_nodes * T and n_nodes * T + 1.  d_n_nodes (optional) = device count of nodes.
 * Replaces: the use_full_timestamps branches of count_edges_kernel / write_edges_kernel and filter_seeds_kernel /
 * collect_seeds_kernel (csrc/include/starrygl/sample.cu.hpp:353-357, :454-483, :578-581, :667-683). */
int sgl_densify_time_groups(const int64_t* node_ptr, const int64_t* group_ts, const int64_t* group_ptr, int64_t n_nodes,
                            const int64_t* d_n_nodes, int64_t t_begin, int64_t t_end, int64_t* out_node_ptr, int64_t* out_ts,
                            int64_t* out_group_ptr, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Mailbox update of a mini-batch: latest message per node + row assembly, and the write into the mailbox.
 *
 * sgl_mail_reduce: entries = ids_a[n_a] followed by ids_b[n_b] (the batch's source nodes, then its destination
 * nodes); entry j has timestamp ts[j] (ts_len == n_a + n_b) or ts[j mod ts_len] (ts_len == n_a == n_b: one value
 * per event, used for both ends); ts is int64 (ts_is_i64) or fp32 and is compared as fp32.  For every distinct
 * node id (ascending in out_index) the entry with the largest timestamp wins, the first such entry on ties.
 * Outputs (capacity n_a + n_b, valid length *d_num_unique): out_index, out_pos (winning entry, optional), out_ts
 * (optional), out_mail (optional): row u = concatenation of n_seg segments (at most 4), segment s read from
 * seg_a[s][pos * seg_dim[s] ...] when the winner pos is an entry of the first list, else from
 * seg_b[s][(pos - n_a) * seg_dim[s] ...]; the seg_* arrays are HOST arrays of device pointers / sizes.
 * The per-entry mail matrix of the reference is never built.
 * Replaces: mailbox.get_update_mail (starrygl/nn/memory/mailbox.py:56-84: cat, unique, torch_scatter.scatter_max,
 * index) and the 'max' reduce at the head of mailbox.set_mailbox_local (:41-47).
 *
 * sgl_mailbox_write: mailbox[index[u], next_mail_pos[index[u]], :] = mail[u, :], mailbox_ts likewise, and (advance
 * != 0, mailbox_size > 1) next_mail_pos[index[u]] = (pos + 1) mod mailbox_size.  index must hold distinct nodes
 * (the output of the reduce).  mailbox is [num_nodes, mailbox_size, width] fp32, mailbox_ts [num_nodes,
 * mailbox_size] fp32, next_mail_pos [num_nodes] int64 (may be null when mailbox_size == 1).
 * Replaces: the writes of mailbox.set_mailbox_local (starrygl/nn/memory/mailbox.py:49-54).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_mail_reduce_ws_bytes(int64_t n_entries);
int sgl_mail_reduce(const int64_t* ids_a, int64_t n_a, const int64_t* ids_b, int64_t n_b, int64_t num_nodes, const void* ts,
                    int64_t ts_len, int ts_is_i64, int n_seg, const float* const* seg_a, const float* const* seg_b,
                    const int64_t* seg_dim, int64_t* out_index, int64_t* out_pos, float* out_ts, float* out_mail,
                    int64_t* d_num_unique, int32_t* d_status, void* ws, size_t ws_bytes, void* stream);
int sgl_mailbox_write(const int64_t* index, int64_t n, const int64_t* d_n, const float* mail, const float* mail_ts,
                      int64_t width, float* mailbox, float* mailbox_ts, int64_t* next_mail_pos, int64_t num_nodes,
                      int64_t mailbox_size, int advance, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Route plan of one layer: which rows of the layer's node list this partition pushes to which other ranks.
 * layer_ids[n] = node ids of the layer list, sorted (rows of one node adjacent, latest timestamp last -- the
 * (id, ts) order of sgl_unique_pairs).  For every node owned here (node_parts[id] == pid) the LAST row of its run
 * is sent to every replica on another rank (replica table: CSR rep_indptr / rep_ranks / rep_locs over node id).
 * Outputs, grouped by destination rank, ascending row inside a rank: out_ranks, out_rows (row of the layer list
 * to read), out_locs (slot on the receiver); d_send_sizes[num_parts]; *d_total entries (capacity cap, overflow
 * raises SGL_DEV_OVERFLOW).  These are the four arrays of a CommPlan.
 * Replaces: MaterializedMultiLayerBuilder._compute_layer_route (prepare_sample.py:266-310).
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_plan_route_ws_bytes(int64_t n, int64_t cap);
int sgl_plan_route(const int64_t* layer_ids, int64_t n, const int64_t* d_n, const int64_t* node_parts, int64_t num_nodes,
                   int64_t pid, const int64_t* rep_indptr, const int64_t* rep_ranks, const int64_t* rep_locs,
                   int64_t num_parts, int64_t cap, int64_t* out_ranks, int64_t* out_rows, int64_t* out_locs,
                   int64_t* d_send_sizes, int64_t* d_total, int32_t* d_status, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Roots of a batch = the events of one time window.  Input: the window's slice of the time-ordered event
 * arrays (source node, timestamp, edge id; n_events items).  Events whose source node lies in a selected
 * chunk (chunk_mask[node_chunk[src]] != 0; both NULL = every node) are grouped by (src, ts):
 *   out_roots[r]                     distinct source nodes, ascending
 *   out_ts[out_ts_ptr[r] .. out_ts_ptr[r+1])   the root's distinct event timestamps, ascending
 *   out_q_eid[out_q_ptr[q] .. out_q_ptr[q+1])  edge ids of the events behind (root, timestamp) pair q, input order
 * d_counts[3] = {#roots, #pairs, #selected events}.  All outputs need capacity n_events (+1 for the ptr arrays).
 * Replaces: get_seeds_in_chunks + filter_seeds_kernel / collect_seeds_kernel
 * (csrc/include/starrygl/sample.cu.hpp:1303-1449, :517-705) for using_full_timestamp = false.
 * ---------------------------------------------------------------------------------------------- */
size_t sgl_seeds_ws_bytes(int64_t n_events);
int sgl_seeds_in_window(const int64_t* ev_src, const int64_t* ev_ts, const int64_t* ev_eid, int64_t n_events,
                        const int64_t* node_chunk, const uint8_t* chunk_mask, int64_t num_chunks, int64_t num_nodes,
                        int id_bits, int ts_bits, int64_t ts_base, int64_t* out_roots, int64_t* out_ts_ptr,
                        int64_t* out_ts, int64_t* out_q_ptr, int64_t* out_q_eid, int64_t* d_counts, int32_t* d_status,
                        void* ws, size_t ws_bytes, void* stream);

/* out[i] = first position p with sorted[p] >= values[i] (n when none); k values.  Used to find the slice of the
 * time-ordered event arrays that a window [t_begin, t_end) covers. */
int sgl_lower_bound_i64(const int64_t* sorted, int64_t n, const int64_t* values, int k, int64_t* out, void* stream);

/* ------------------------------------------------------------------------------------------------
 * CUDA-graph helpers for launch-bound steps.  Between sgl_graph_capture_begin(stream) and
 * sgl_graph_capture_end(stream, &exec) every asynchronous call of this library on `stream` is recorded instead
 * of executed (thread-local capture mode; sgl_tcsr_build synchronises and cannot be captured).  sgl_graph_launch
 * optionally copies copy_bytes from copy_src to copy_dst on the stream first (the step's varying input, e.g. the
 * batch's roots, into the buffer the captured kernels read) and then replays the recorded sequence with one
 * launch.  (No counterpart in the reference, which issues every kernel from the host.)
 * ---------------------------------------------------------------------------------------------- */
int sgl_graph_capture_begin(void* stream);
int sgl_graph_capture_end(void* stream, void** out_exec);
int sgl_graph_launch(void* exec, const void* copy_src, void* copy_dst, size_t copy_bytes, void* stream);
int sgl_graph_destroy(void* exec);

#ifdef __cplusplus
}
#endif
#endif /* SGL_B200_H */
