// Collectives of the C ABI: one communicator rank per process and GPU, NCCL underneath.
//
// The reference's CollectiveOps holds AllReduce only and no implementation
// (collectiveops.go:10-39 of gomlx/compute); the all-gather at a column-shard boundary is the
// extension its interface sketches (collectiveops.go:31-32).  NCCL is resolved at run time
// (dlopen of libnccl.so.2), so the library has no link-time dependency on it: without NCCL
// these entry points return CB_ERR_NOT_IMPLEMENTED and everything else works.
#include "common.cuh"

#include <dlfcn.h>
#include <mutex>
#include <string.h>

struct cb_comm {
  void* nccl = nullptr;     // ncclComm_t
  int dev = 0, nranks = 0, rank = 0;
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

struct Nccl {
  void* lib = nullptr;
  get_unique_id_fn get_unique_id = nullptr;
  comm_init_rank_fn comm_init_rank = nullptr;
  comm_destroy_fn comm_destroy = nullptr;
  all_gather_fn all_gather = nullptr;
  all_reduce_fn all_reduce = nullptr;
  error_string_fn error_string = nullptr;
  bool ok = false;
};

Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) return;
    n.get_unique_id = (get_unique_id_fn)dlsym(n.lib, "ncclGetUniqueId");
    n.comm_init_rank = (comm_init_rank_fn)dlsym(n.lib, "ncclCommInitRank");
    n.comm_destroy = (comm_destroy_fn)dlsym(n.lib, "ncclCommDestroy");
    n.all_gather = (all_gather_fn)dlsym(n.lib, "ncclAllGather");
    n.all_reduce = (all_reduce_fn)dlsym(n.lib, "ncclAllReduce");
    n.error_string = (error_string_fn)dlsym(n.lib, "ncclGetErrorString");
    n.ok = n.get_unique_id && n.comm_init_rank && n.comm_destroy && n.all_gather && n.all_reduce;
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

int cb_comm_init_rank(int dev, int nranks, int rank, const unsigned char* id, cb_comm** comm) {
  clear_error();
  if (!id || !comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_init_rank: null argument");
  if (nranks < 1 || rank < 0 || rank >= nranks) return fail(CB_ERR_INVALID_ARG, "cb_comm_init_rank: rank %d of %d", rank, nranks);
  CB_TRY(need_nccl());
  CB_TRY(set_device(dev));
  NcclId nid;
  memcpy(nid.internal, id, CB_COMM_ID_BYTES);
  cb_comm* c = new cb_comm();
  c->dev = dev; c->nranks = nranks; c->rank = rank;
  const int st = nccl_check(nccl().comm_init_rank(&c->nccl, nranks, nid, rank), "ncclCommInitRank");
  if (st != CB_OK) { delete c; return st; }
  *comm = c;
  return CB_OK;
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
  if (bytes_per_rank == 0) return CB_OK;
  if (!send || !recv) return fail(CB_ERR_INVALID_ARG, "cb_comm_allgather: null buffer");
  CB_TRY(set_device(comm->dev));
  return nccl_check(nccl().all_gather(send, recv, bytes_per_rank, /*ncclInt8*/ 0, comm->nccl, (cudaStream_t)stream), "ncclAllGather");
}

int cb_comm_allreduce(cb_comm* comm, const void* send, void* recv, size_t count, int32_t dtype, int32_t op, cb_stream stream) {
  clear_error();
  if (!comm) return fail(CB_ERR_INVALID_ARG, "cb_comm_allreduce: null communicator");
  if (count == 0) return CB_OK;
  if (!send || !recv) return fail(CB_ERR_INVALID_ARG, "cb_comm_allreduce: null buffer");
  const int dt = nccl_dtype(dtype);
  if (dt < 0) return fail(CB_ERR_NOT_IMPLEMENTED, "AllReduce: dtype %s", dtype_name(dtype));
  if (op < CB_REDUCE_SUM || op > CB_REDUCE_MIN) return fail(CB_ERR_INVALID_ARG, "AllReduce: unknown reduction %d", op);
  CB_TRY(set_device(comm->dev));
  return nccl_check(nccl().all_reduce(send, recv, count, dt, op, comm->nccl, (cudaStream_t)stream), "ncclAllReduce");
}

int cb_comm_destroy(cb_comm* comm) {
  clear_error();
  if (!comm) return CB_OK;
  int st = CB_OK;
  if (comm->nccl && nccl().ok) st = nccl_check(nccl().comm_destroy(comm->nccl), "ncclCommDestroy");
  delete comm;
  return st;
}

}  // extern "C"
