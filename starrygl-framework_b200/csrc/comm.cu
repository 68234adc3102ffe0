// Native communicator of the route layer: variable-size all-to-all as grouped ncclSend/ncclRecv on the caller's
// stream, with the pack (gather into the send buffer) and unpack (scatter from the receive buffer) kernels enqueued
// by the same foreign call, so that one route step costs one host call and no host synchronisation.
//
// NCCL is bound at run time (dlopen / dlsym): a process that already carries an NCCL (PyTorch ships its own) keeps
// using exactly that copy, and the library loads on machines without NCCL as long as no communicator is created.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include "common.cuh"

namespace sgl {
struct Comm {
  ncclComm_t nccl;
  int rank, world;
};

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*GroupStart)();
  ncclResult_t (*GroupEnd)();
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  const char* (*GetErrorString)(ncclResult_t);
};

static bool load_nccl(NcclApi* api) {
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // the copy the process already uses, if any
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return false;
#define SGL_SYM(field, name) *(void**)(&api->field) = dlsym(h, name); if (!api->field) return false
  SGL_SYM(GetUniqueId, "ncclGetUniqueId");
  SGL_SYM(CommInitRank, "ncclCommInitRank");
  SGL_SYM(CommDestroy, "ncclCommDestroy");
  SGL_SYM(GroupStart, "ncclGroupStart");
  SGL_SYM(GroupEnd, "ncclGroupEnd");
  SGL_SYM(Send, "ncclSend");
  SGL_SYM(Recv, "ncclRecv");
  SGL_SYM(GetErrorString, "ncclGetErrorString");
#undef SGL_SYM
  return true;
}

// Resolved once per process; a function-local static is initialised under the language's own lock, so host threads
// that race here all wait for the one dlopen / dlsym sequence and see its result.
static NcclApi* nccl_api() {
  static NcclApi api;
  static const bool ok = load_nccl(&api);
  return ok ? &api : nullptr;
}
}  // namespace sgl

using namespace sgl;

#define SGL_NEED_NCCL()                                                              \
  NcclApi* N = nccl_api();                                                           \
  SGL_REQUIRE(N, SGL_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded")
#define ncclGetUniqueId N->GetUniqueId
#define ncclCommInitRank N->CommInitRank
#define ncclCommDestroy N->CommDestroy
#define ncclGroupStart N->GroupStart
#define ncclGroupEnd N->GroupEnd
#define ncclSend N->Send
#define ncclRecv N->Recv
#define ncclGetErrorString N->GetErrorString

#define SGL_NCCL_CHECK(expr)                                                                     \
  do {                                                                                           \
    ncclResult_t _r = (expr);                                                                    \
    if (_r != ncclSuccess) {                                                                     \
      sgl::set_error("%s failed: %s (%s:%d)", #expr, ncclGetErrorString(_r), __FILE__, __LINE__); \
      return SGL_ERR_CUDA;                                                                       \
    }                                                                                            \
  } while (0)

extern "C" int sgl_comm_unique_id(char* out_id, size_t id_bytes) {
  SGL_REQUIRE(out_id && id_bytes >= sizeof(ncclUniqueId), SGL_ERR_ARG, "comm_unique_id: buffer must hold %zu bytes",
              sizeof(ncclUniqueId));
  SGL_NEED_NCCL();
  ncclUniqueId id;
  SGL_NCCL_CHECK(ncclGetUniqueId(&id));
  memcpy(out_id, &id, sizeof(id));
  return SGL_OK;
}

extern "C" int sgl_comm_init(void** out_comm, int rank, int world, const char* id_bytes) {
  SGL_REQUIRE(out_comm && id_bytes && world >= 1 && rank >= 0 && rank < world, SGL_ERR_ARG, "comm_init: bad argument");
  SGL_NEED_NCCL();
  ncclUniqueId id;
  memcpy(&id, id_bytes, sizeof(id));
  Comm* c = new Comm{nullptr, rank, world};
  ncclResult_t r = ncclCommInitRank(&c->nccl, world, id, rank);
  if (r != ncclSuccess) {
    set_error("ncclCommInitRank failed: %s", ncclGetErrorString(r));
    delete c;
    return SGL_ERR_CUDA;
  }
  *out_comm = c;
  return SGL_OK;
}

extern "C" int sgl_comm_destroy(void* comm) {
  if (!comm) return SGL_OK;
  SGL_NEED_NCCL();
  Comm* c = (Comm*)comm;
  ncclCommDestroy(c->nccl);
  delete c;
  return SGL_OK;
}

// rows of row_floats float32 each; segment p of `send` (h_send_rows[p] rows) goes to rank p, segment p of `recv`
// comes from rank p
static int exchange(Comm* c, const float* send, const int64_t* h_send_rows, float* recv, const int64_t* h_recv_rows,
                    int64_t row_floats, cudaStream_t stream) {
  SGL_NEED_NCCL();
  SGL_NCCL_CHECK(ncclGroupStart());
  // a failing send / recv must not leave the group open for the next call of this thread: remember the first error,
  // close the group, then report
  ncclResult_t first = ncclSuccess;
  int64_t so = 0, ro = 0;
  for (int p = 0; p < c->world && first == ncclSuccess; ++p) {
    if (h_send_rows[p] > 0)
      first = ncclSend(send + so * row_floats, (size_t)(h_send_rows[p] * row_floats), ncclFloat, p, c->nccl, stream);
    if (first == ncclSuccess && h_recv_rows[p] > 0)
      first = ncclRecv(recv + ro * row_floats, (size_t)(h_recv_rows[p] * row_floats), ncclFloat, p, c->nccl, stream);
    so += h_send_rows[p];
    ro += h_recv_rows[p];
  }
  const ncclResult_t end = ncclGroupEnd();
  if (first == ncclSuccess) first = end;
  if (first != ncclSuccess) {
    sgl::set_error("route exchange failed: %s", ncclGetErrorString(first));
    return SGL_ERR_CUDA;
  }
  return SGL_OK;
}

extern "C" int sgl_route_exchange(void* comm, const float* send, const int64_t* h_send_rows, float* recv,
                                  const int64_t* h_recv_rows, int64_t row_floats, void* stream) {
  SGL_NVTX("sgl_route_exchange");
  SGL_REQUIRE(comm && h_send_rows && h_recv_rows && row_floats > 0, SGL_ERR_ARG, "route_exchange: bad argument");
  return exchange((Comm*)comm, send, h_send_rows, recv, h_recv_rows, row_floats, (cudaStream_t)stream);
}

extern "C" int sgl_cache_route_step(void* comm, const float* feats, int64_t n_rows, int64_t dim, const float* ts,
                                    const int64_t* send_idx, const int64_t* remote_idx, const int64_t* h_send_rows,
                                    const int64_t* h_recv_rows, float* send_buf, float* recv_buf, float* data,
                                    int64_t data_rows, float* ts_table, int apply, int32_t* d_status, void* stream) {
  SGL_NVTX("sgl_cache_route_step");
  SGL_REQUIRE(comm && h_send_rows && h_recv_rows, SGL_ERR_ARG, "cache_route_step: bad argument");
  Comm* c = (Comm*)comm;
  int64_t n_send = 0, n_recv = 0;
  for (int p = 0; p < c->world; ++p) {
    SGL_REQUIRE(h_send_rows[p] >= 0 && h_recv_rows[p] >= 0, SGL_ERR_ARG, "cache_route_step: negative split size");
    n_send += h_send_rows[p];
    n_recv += h_recv_rows[p];
  }
  const int64_t width = dim + (ts ? 1 : 0);
  // a rank with nothing to send still takes part in the exchange (its peers may send to it)
  SGL_REQUIRE(n_send == 0 || remote_idx, SGL_ERR_ARG, "cache_route_step: remote_idx is null");
  int rc = n_send ? sgl_route_pack(feats, n_rows, dim, ts, send_idx, remote_idx, n_send, send_buf, d_status, stream) : SGL_OK;
  if (rc) return rc;
  rc = exchange(c, send_buf, h_send_rows, recv_buf, h_recv_rows, sgl_wire_pitch(dim, ts != nullptr, 1), (cudaStream_t)stream);
  if (rc) return rc;
  if (apply) rc = sgl_route_unpack(recv_buf, n_recv, width, data, data_rows, dim, ts_table, d_status, stream);
  return rc;
}

extern "C" int sgl_comm_info(void* comm, int* out_rank, int* out_world) {
  SGL_REQUIRE(comm, SGL_ERR_ARG, "comm_info: null communicator");
  Comm* c = (Comm*)comm;
  if (out_rank) *out_rank = c->rank;
  if (out_world) *out_world = c->world;
  return SGL_OK;
}

// Peer access from the current device to the listed devices of this process (needed only when one process drives
// several GPUs; mappings of other processes' memory enable it themselves when they are opened).
extern "C" int sgl_init_p2p(const int* devices, int n, int* out_accessible) {
  SGL_REQUIRE(n >= 0 && (n == 0 || devices), SGL_ERR_ARG, "init_p2p: bad device list");
  int cur = 0, count = 0, ok = 0;
  SGL_CUDA_CHECK(cudaGetDevice(&cur));
  SGL_CUDA_CHECK(cudaGetDeviceCount(&count));
  for (int i = 0; i < n; ++i) {
    const int d = devices[i];
    if (d == cur) { ++ok; continue; }
    if (d < 0 || d >= count) continue;     // a device of another process: nothing to enable from here
    int can = 0;
    SGL_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, cur, d));
    if (!can) continue;
    cudaError_t e = cudaDeviceEnablePeerAccess(d, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
    SGL_CUDA_CHECK(e);
    ++ok;
  }
  if (out_accessible) *out_accessible = ok;
  return SGL_OK;
}
