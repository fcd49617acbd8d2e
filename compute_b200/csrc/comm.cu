// Collectives of the C ABI: one communicator rank per process and GPU, NCCL underneath.
//
// The reference's CollectiveOps holds AllReduce only and no implementation
// (collectiveops.go:10-39 of gomlx/compute); the all-gather at a column-shard boundary is the
// extension its interface sketches (collectiveops.go:31-32).  NCCL is resolved at run time
// (dlopen of libnccl.so.2, or of the library CUDABACKEND_NCCL_LIB names), so the library has no
// link-time dependency on it: without NCCL these entry points return CB_ERR_NOT_IMPLEMENTED and
// everything else works.
//
// Failure handling (the reference has none: it is one process on one device).  A communicator made
// with a time limit (cb_comm_init_rank_timeout, limit > 0) is non-blocking, so no NCCL call can park
// the host thread for ever: initialisation and every enqueue are followed by polling
// ncclCommGetAsyncError under the limit; when it passes or NCCL reports an asynchronous error the
// communicator is aborted (ncclCommAbort, which also ends its kernels on the device), the call
// returns CB_ERR_TIMEOUT / CB_ERR_CUDA, and every later call on the handle fails at once.  A
// non-blocking enqueue is handed to a helper thread inside NCCL, which costs tens of microseconds
// per call, so cb_comm_init_rank (no limit) keeps the blocking kind for the per-step path.  For
// both kinds cb_comm_sync is the host-side watchdog for work already enqueued: it waits for the
// stream under a limit and aborts the communicator when a peer has left.
#include "common.cuh"

#include <chrono>
#include <climits>
#include <dlfcn.h>
#include <mutex>
#include <string.h>
#include <thread>

struct cb_comm {
  void* nccl = nullptr;     // ncclComm_t
  int dev = 0, nranks = 0, rank = 0;
  double timeout_s = 0.0;   // limit of every wait on this communicator
  bool nonblocking = false;
  bool aborted = false;
};

namespace cb {
namespace {

struct NcclId { char internal[128]; };
typedef int (*get_unique_id_fn)(NcclId*);
typedef int (*comm_init_rank_fn)(void**, int, NcclId, int);
typedef int (*comm_destroy_fn)(void*);
typedef int (*all_gather_fn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*all_reduce_fn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef const char* (*error_string_fn)(int);
// The configuration record as NCCL 2.18 defined it; later libraries accept it by its size and version fields
// and take their defaults for what was added since.
struct NcclConfig {
  size_t size; unsigned magic, version;
  int blocking, cga_cluster_size, min_ctas, max_ctas;
  const char* net_name;
  int split_share;
};
typedef int (*comm_init_rank_config_fn)(void**, int, NcclId, int, NcclConfig*);
typedef int (*get_async_error_fn)(void*, int*);
typedef int (*comm_abort_fn)(void*);
constexpr int NCCL_IN_PROGRESS = 7;       // ncclInProgress

struct Nccl {
  void* lib = nullptr;
  get_unique_id_fn get_unique_id = nullptr;
  comm_init_rank_fn comm_init_rank = nullptr;
  comm_destroy_fn comm_destroy = nullptr;
  all_gather_fn all_gather = nullptr;
  all_reduce_fn all_reduce = nullptr;
  error_string_fn error_string = nullptr;
  comm_init_rank_config_fn comm_init_rank_config = nullptr;
  get_async_error_fn get_async_error = nullptr;
  comm_abort_fn comm_abort = nullptr;
  bool ok = false;
  bool can_abort = false;     // the three entry points non-blocking operation needs are present
};

Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* named = getenv("CUDABACKEND_NCCL_LIB");
    if (named && named[0]) n.lib = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) return;
    n.get_unique_id = (get_unique_id_fn)dlsym(n.lib, "ncclGetUniqueId");
    n.comm_init_rank = (comm_init_rank_fn)dlsym(n.lib, "ncclCommInitRank");
    n.comm_destroy = (comm_destroy_fn)dlsym(n.lib, "ncclCommDestroy");
    n.all_gather = (all_gather_fn)dlsym(n.lib, "ncclAllGather");
    n.all_reduce = (all_reduce_fn)dlsym(n.lib, "ncclAllReduce");
    n.error_string = (error_string_fn)dlsym(n.lib, "ncclGetErrorString");
    n.comm_init_rank_config = (comm_init_rank_config_fn)dlsym(n.lib, "ncclCommInitRankConfig");
    n.get_async_error = (get_async_error_fn)dlsym(n.lib, "ncclCommGetAsyncError");
    n.comm_abort = (comm_abort_fn)dlsym(n.lib, "ncclCommAbort");
    n.ok = n.get_unique_id && n.comm_init_rank && n.comm_destroy && n.all_gather && n.all_reduce;
    n.can_abort = n.comm_init_rank_config && n.get_async_error && n.comm_abort;
  });
  return n;
}

int need_nccl() {
  if (!nccl().ok) return fail(CB_ERR_NOT_IMPLEMENTED, "collectives need NCCL: libnccl.so.2 could not be loaded");
  return CB_OK;
}

int nccl_check(int r, const char* what) {
  if (r == 0) return CB_OK;
  const char* msg = nccl().error_string ? nccl().error_string(r) : "?";
  return fail(CB_ERR_CUDA, "%s failed: NCCL error %d (%s)", what, r, msg);
}

double default_timeout_s() {
  if (const char* t = getenv("CUDABACKEND_COMM_TIMEOUT_S")) { const double v = atof(t); if (v > 0.0) return v; }
  return 600.0;
}

// Ends the communicator after a failure: its kernels stop, its resources go, the handle stays (marked) so that
// later calls fail cleanly and cb_comm_destroy still frees it.
void abort_comm(cb_comm* c) {
  if (c->aborted) return;
  c->aborted = true;
  if (c->nccl && nccl().comm_abort) nccl().comm_abort(c->nccl);
  c->nccl = nullptr;
}

int check_alive(const cb_comm* c, const char* what) {
  if (c->aborted) return fail(CB_ERR_INVALID_ARG, "%s: the communicator (rank %d of %d) was aborted after an earlier failure", what, c->rank, c->nranks);
  return CB_OK;
}

// After a call on a non-blocking communicator: polls the asynchronous state until it leaves "in progress".
// r is what the call itself returned.
int settle(cb_comm* c, int r, const char* what) {
  if (!c->nonblocking) return nccl_check(r, what);
  if (r != 0 && r != NCCL_IN_PROGRESS) { const int st = nccl_check(r, what); abort_comm(c); return st; }
  const auto t0 = std::chrono::steady_clock::now();
  for (long long spin = 0;; spin++) {
    int state = 0;
    const int q = nccl().get_async_error(c->nccl, &state);
    if (q != 0) { const int st = nccl_check(q, "ncclCommGetAsyncError"); abort_comm(c); return st; }
    if (state == 0) return CB_OK;
    if (state != NCCL_IN_PROGRESS) { const int st = nccl_check(state, what); abort_comm(c); return st; }
    const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (waited > c->timeout_s) {
      abort_comm(c);
      return fail(CB_ERR_TIMEOUT, "%s: rank %d of %d still in progress after %.1f s (a peer that never joined or has left?); communicator aborted",
                  what, c->rank, c->nranks, waited);
    }
    if (waited > 2e-3) std::this_thread::sleep_for(std::chrono::microseconds(100));     // spin for the first two milliseconds
    else std::this_thread::yield();
  }
}

// ncclDataType_t of a dtype code, or -1
int nccl_dtype(int dtype) {
  switch (dtype) {
    case CB_I8: return 0;
    case CB_U8: return 1;
    case CB_I32: return 2;
    case CB_U32: return 3;
    case CB_I64: return 4;
    case CB_U64: return 5;
    case CB_F16: return 6;
    case CB_F32: return 7;
    case CB_F64: return 8;
    case CB_BF16: return 9;
    default: return -1;
  }
}

}  // namespace
}  // namespace cb

using namespace cb;

extern "C" {

int cb_comm_unique_id(unsigned char* id) {
  clear_error();
  if (!id) return fail(CB_ERR_INVALID_ARG, "cb_comm_unique_id: null id");
  CB_TRY(need_nccl());
  NcclId nid;
  CB_TRY(nccl_check(nccl().get_unique_id(&nid), "ncclGetUniqueId"));
  memcpy(id, nid.internal, CB_COMM_ID_BYTES);
  return CB_OK;
}

int cb_comm_init_rank_timeout(int dev, int nranks, int rank, const unsigned char* id, double timeout_s, cb_comm** comm) {
  clear_error();
  if (!id || !comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_init_rank: null argument");
  *comm = nullptr;
  if (nranks < 1 || rank < 0 || rank >= nranks) return fail(CB_ERR_INVALID_ARG, "cb_comm_init_rank: rank %d of %d", rank, nranks);
  CB_TRY(need_nccl());
  if (dev >= 0) CB_TRY(set_device(dev));          // dev < 0: the calling thread's current device
  NcclId nid;
  memcpy(nid.internal, id, CB_COMM_ID_BYTES);
  cb_comm* c = new cb_comm();
  c->dev = dev; c->nranks = nranks; c->rank = rank;
  c->timeout_s = timeout_s > 0.0 ? timeout_s : default_timeout_s();
  int st;
  if (nccl().can_abort && timeout_s > 0.0) {
    NcclConfig cfg;
    cfg.size = sizeof(cfg); cfg.magic = 0xcafebeefu; cfg.version = 21800;
    cfg.blocking = 0;
    cfg.cga_cluster_size = cfg.min_ctas = cfg.max_ctas = cfg.split_share = INT_MIN;     // "undefined": the library's defaults
    cfg.net_name = nullptr;
    c->nonblocking = true;
    const int r = nccl().comm_init_rank_config(&c->nccl, nranks, nid, rank, &cfg);
    if (r == 4 || r == 5) {      // ncclInvalidArgument / ncclInvalidUsage: a library that does not take this record
      c->nonblocking = false;
      c->nccl = nullptr;
      st = nccl_check(nccl().comm_init_rank(&c->nccl, nranks, nid, rank), "ncclCommInitRank");
    } else {
      st = settle(c, r, "ncclCommInitRankConfig");
    }
  } else {
    st = nccl_check(nccl().comm_init_rank(&c->nccl, nranks, nid, rank), "ncclCommInitRank");
  }
  if (st != CB_OK) { delete c; return st; }
  *comm = c;
  return CB_OK;
}

int cb_comm_init_rank(int dev, int nranks, int rank, const unsigned char* id, cb_comm** comm) {
  return cb_comm_init_rank_timeout(dev, nranks, rank, id, 0.0, comm);
}

int cb_comm_check(cb_comm* comm) {
  clear_error();
  if (!comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_check: null communicator");
  CB_TRY(check_alive(comm, "cb_comm_check"));
  if (!nccl().get_async_error) return CB_OK;
  int state = 0;
  const int q = nccl().get_async_error(comm->nccl, &state);
  if (q != 0) { const int st = nccl_check(q, "ncclCommGetAsyncError"); abort_comm(comm); return st; }
  if (state == 0 || state == NCCL_IN_PROGRESS) return CB_OK;
  const int st = nccl_check(state, "asynchronous NCCL operation");
  abort_comm(comm);
  return st;
}

int cb_comm_sync(cb_comm* comm, cb_stream stream, double timeout_s) {
  clear_error();
  if (!comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_sync: null communicator");
  CB_TRY(check_alive(comm, "cb_comm_sync"));
  if (comm->dev >= 0) CB_TRY(set_device(comm->dev));
  const double limit = timeout_s > 0.0 ? timeout_s : comm->timeout_s;
  const auto t0 = std::chrono::steady_clock::now();
  for (long long spin = 0;; spin++) {
    const cudaError_t q = cudaStreamQuery((cudaStream_t)stream);
    if (q == cudaSuccess) return cb_comm_check(comm);
    if (q != cudaErrorNotReady) { abort_comm(comm); return fail(CB_ERR_CUDA, "cb_comm_sync: %s", cudaGetErrorString(q)); }
    CB_TRY(cb_comm_check(comm));
    const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (waited > limit) {
      abort_comm(comm);        // ends the collective's kernel on the device; the stream then drains
      return fail(CB_ERR_TIMEOUT, "cb_comm_sync: rank %d of %d: the stream did not finish in %.1f s (a peer has left?); communicator aborted",
                  comm->rank, comm->nranks, waited);
    }
    if (spin > 100) std::this_thread::sleep_for(std::chrono::microseconds(200));
    else std::this_thread::yield();
  }
}

int cb_comm_size(const cb_comm* comm, int* nranks, int* rank) {
  clear_error();
  if (!comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_size: null communicator");
  if (nranks) *nranks = comm->nranks;
  if (rank) *rank = comm->rank;
  return CB_OK;
}

int cb_comm_allgather(cb_comm* comm, const void* send, void* recv, size_t bytes_per_rank, cb_stream stream) {
  clear_error();
  if (!comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_allgather: null communicator");
  CB_TRY(check_alive(comm, "cb_comm_allgather"));
  if (bytes_per_rank == 0) return CB_OK;
  if (!send || !recv) return fail(CB_ERR_INVALID_ARG, "cb_comm_allgather: null buffer");
  if (comm->dev >= 0) CB_TRY(set_device(comm->dev));
  return settle(comm, nccl().all_gather(send, recv, bytes_per_rank, /*ncclInt8*/ 0, comm->nccl, (cudaStream_t)stream), "ncclAllGather");
}

int cb_comm_allreduce(cb_comm* comm, const void* send, void* recv, size_t count, int32_t dtype, int32_t op, cb_stream stream) {
  clear_error();
  if (!comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_allreduce: null communicator");
  CB_TRY(check_alive(comm, "cb_comm_allreduce"));
  if (count == 0) return CB_OK;
  if (!send || !recv) return fail(CB_ERR_INVALID_ARG, "cb_comm_allreduce: null buffer");
  const int dt = nccl_dtype(dtype);
  if (dt < 0) return fail(CB_ERR_NOT_IMPLEMENTED, "AllReduce: dtype %s", dtype_name(dtype));
  if (op < CB_REDUCE_SUM || op > CB_REDUCE_MIN) return fail(CB_ERR_INVALID_ARG, "AllReduce: unknown reduction %d", op);
  if (comm->dev >= 0) CB_TRY(set_device(comm->dev));
  return settle(comm, nccl().all_reduce(send, recv, count, dt, op, comm->nccl, (cudaStream_t)stream), "ncclAllReduce");
}

int cb_comm_destroy(cb_comm* comm) {
  clear_error();
  if (!comm) return CB_OK;
  int st = CB_OK;
  if (comm->nccl && !comm->aborted && nccl().ok) {
    const int r = nccl().comm_destroy(comm->nccl);
    st = (comm->nonblocking && r == NCCL_IN_PROGRESS) ? CB_OK : nccl_check(r, "ncclCommDestroy");
  }
  delete comm;
  return st;
}

}  // extern "C"
