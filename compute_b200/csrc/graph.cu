// Host-side graph layer: Backend / Builder / Function / Executable / Buffer of the
// gomlx/compute interface for the accelerated path, over this library's own C ABI.
// A Function records a short list of nodes; Compile turns it into a launch plan
// (one cb_plan per node, chosen by shape and dtype); Execute is a sequence of
// stream launches over pooled device buffers.
//
// Reference behaviour mirrored here:
//   builder / executable protocol   builder.go:29-82, executable.go:10-37, function.go:23-134
//   DotGeneral lowering             internal/gobackend/dot/dot.go:165-285, shapeinference/dotgeneral.go:16-152
//   FusedQuantizedDense validation  internal/gobackend/fusedops/quantizeddense.go:58-142
//   SDPA validation                 internal/gobackend/fusedops/sdpa.go:98-210
//   input validation at Execute     internal/gobackend/exec.go:176-233
#include "common.cuh"
#include "../../include/cudabackend_graph.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <vector>
#include <string.h>

using cb::fail;

namespace {

struct Shape {
  int32_t dtype = 0;
  std::vector<int64_t> dims;
  int64_t size() const { int64_t n = 1; for (auto d : dims) n *= d; return n; }
  // Int4 / Uint4 are packed two per byte over the flat element order (dtypes/dtype_enum.go:91-116)
  size_t bytes() const { return (dtype == CB_I4 || dtype == CB_U4) ? ((size_t)size() + 1) / 2 : (size_t)size() * cb::dtype_size(dtype); }
  bool operator==(const Shape& o) const { return dtype == o.dtype && dims == o.dims; }
  std::string str() const {
    std::ostringstream s;
    s << "(" << cb::dtype_name(dtype) << ")[";
    for (size_t i = 0; i < dims.size(); i++) s << (i ? " " : "") << dims[i];
    s << "]";
    return s.str();
  }
};

enum NodeKind { N_PARAM, N_CONST, N_DOT, N_QDENSE, N_SDPA, N_RESHAPE, N_SLICE, N_IOTA, N_CONVERT, N_TRANSPOSE,
                N_GELU, N_SOFTMAX, N_LAYERNORM, N_COLS_BIAS, N_BINARY, N_UNARY, N_REDUCE, N_BROADCAST, N_RMSNORM,
                N_ALLREDUCE, N_ALLGATHER, N_EMBEDDING };

bool is_float(int d) { return d == CB_F16 || d == CB_F32 || d == CB_F64 || d == CB_BF16 || d == CB_F8E4M3FN || d == CB_F8E5M2; }
bool is_half(int d) { return d == CB_F16 || d == CB_BF16; }
// dtypes a buffer, parameter or constant may have: the plain ones, and packed 4-bit weights
bool storable(int d) { return (cb::dtype_size(d) != 0 && d <= CB_BF16) || d == CB_I4 || d == CB_U4; }

// Size-bucketed pool of device allocations (the role of Backend.GetBuffer / PutBuffer,
// internal/gobackend/buffers.go:117-180): cudaMalloc / cudaFree stay off the Execute path.
struct DevicePool {
  std::mutex mu;
  std::map<size_t, std::vector<void*>> free_lists;
  static size_t bucket(size_t n) {
    if (n < 256) return 256;
    size_t top = (size_t)1 << (63 - __builtin_clzll((unsigned long long)n));
    size_t step = top >> 2;                       // two more bits of resolution
    return (n + step - 1) / step * step;
  }
  int get(int dev, size_t bytes, void** p) {
    const size_t b = bucket(bytes);
    {
      std::lock_guard<std::mutex> l(mu);
      auto it = free_lists.find(b);
      if (it != free_lists.end() && !it->second.empty()) {
        *p = it->second.back();
        it->second.pop_back();
        return CB_OK;
      }
    }
    return cb_alloc(dev, b, p);
  }
  void put(size_t bytes, void* p) {
    if (!p) return;
    std::lock_guard<std::mutex> l(mu);
    free_lists[bucket(bytes)].push_back(p);
  }
  void release_all(int dev) {
    std::lock_guard<std::mutex> l(mu);
    for (auto& kv : free_lists)
      for (void* p : kv.second) cb_free(dev, p);
    free_lists.clear();
  }
};

}  // namespace

// Page-locked staging buffers for BufferFromFlatData / ToFlatData: the copy to or from the caller's
// (pageable) slice is a plain memcpy, the transfer itself runs on a stream of this library and never
// touches the default stream.
struct PinnedPool {
  std::mutex mu;
  std::map<size_t, std::vector<void*>> free_lists;
  int get(size_t bytes, void** p, size_t* cap) {
    size_t b = 4096;
    while (b < bytes) b <<= 1;
    *cap = b;
    {
      std::lock_guard<std::mutex> l(mu);
      auto it = free_lists.find(b);
      if (it != free_lists.end() && !it->second.empty()) { *p = it->second.back(); it->second.pop_back(); return CB_OK; }
    }
    return cb_host_alloc(b, p);
  }
  void put(size_t cap, void* p) { std::lock_guard<std::mutex> l(mu); free_lists[cap].push_back(p); }
  void release_all() {
    std::lock_guard<std::mutex> l(mu);
    for (auto& kv : free_lists) for (void* p : kv.second) cb_host_free(p);
    free_lists.clear();
  }
};
constexpr size_t PINNED_STAGING_MAX = (size_t)16 << 20;     // larger transfers go directly (one-off uploads of weights)

struct cbg_backend {
  int n_devices = 0;
  PinnedPool pinned;
  bool fallback_only = false;
  bool trace = false;                 // option "trace" or CUDABACKEND_TRACE=1: per-launch device times of every Execute
  bool no_graphs = false;             // option "no_graphs": never replay an Execute as a CUDA graph
  std::atomic<bool> finalized{false};
  std::string name = "cuda", description;
  std::vector<std::unique_ptr<DevicePool>> pools;
  std::mutex stream_mu;
  std::vector<std::vector<cb_stream>> streams;   // idle streams per device
  int get_stream(int dev, cb_stream* s) {
    {
      std::lock_guard<std::mutex> l(stream_mu);
      if (!streams[dev].empty()) { *s = streams[dev].back(); streams[dev].pop_back(); return CB_OK; }
    }
    return cb_stream_create(dev, s);
  }
  void put_stream(int dev, cb_stream s) {
    std::lock_guard<std::mutex> l(stream_mu);
    streams[dev].push_back(s);
  }
};

struct cbg_buffer {
  cbg_backend* be = nullptr;
  int dev = 0;
  Shape shape;
  void* ptr = nullptr;
  bool valid = true;
};

struct cbg_value {
  NodeKind kind;
  Shape shape;
  std::vector<cbg_value*> inputs;
  cbg_function* fn = nullptr;
  int index = 0;
  std::string name;                 // parameters
  int param_index = -1;
  std::vector<uint8_t> const_data;  // constants
  cb_dot_desc dot{};
  cb_qdense_desc qd{};
  cb_sdpa_desc sdpa{};
  std::vector<int64_t> starts, limits, strides;
  std::vector<int32_t> perm;
  int axis = 0;
  int64_t small_dims[4] = {0, 0, 0, 0};   // softmax [outer, axis, inner]; layer norm [rows, norm size, 1]; column slice [rows, total, first, width]
  double epsilon = 0.0;               // layer norm, rms norm
  int flags = 0;                      // gelu: exact; layer norm: 1 gamma, 2 beta; rms norm: 1 gamma
  int op = 0;                         // binary / unary / reduce op; AllReduce: cb_reduce_op; AllGather: the gather axis
  std::vector<int32_t> axis_flags;    // reduce: 1 for every reduced axis; BroadcastInDim: the broadcast axes
  std::vector<std::vector<int>> replica_groups;   // collectives: indices into the device assignment
  std::string sharding;               // Parameter: the ShardingSpec it was declared with (text form), or empty
};

struct cbg_function {
  cbg_builder* builder = nullptr;
  std::vector<std::unique_ptr<cbg_value>> nodes;
  std::vector<cbg_value*> params, outputs;
  bool returned = false;
};

struct cbg_builder {
  cbg_backend* be = nullptr;
  std::string name;
  std::unique_ptr<cbg_function> main;
  bool compiled = false;
  int spmd = 0;
  std::vector<int> assignment;
};

struct DevPlans {                             // the launch plan of one device
  std::vector<cb_plan*> plans;                // per node (NULL for parameters, constants, reshapes, skipped nodes)
  std::vector<size_t> ws_bytes;
};

struct cbg_exec {
  cbg_backend* be = nullptr;
  std::string name;
  std::unique_ptr<cbg_function> fn;          // owns the nodes
  std::vector<char> live;                    // per node: its value is needed (outputs and their operands)
  std::vector<int> group_of;                 // per node: -1, or the index of the grouped launch it belongs to
  std::vector<std::vector<int>> groups;      // grouped FusedQuantizedDense launches: member nodes; the first member launches
  int replicas = 1;
  std::vector<int> assignment;
  std::mutex mu;
  std::map<int, DevPlans> dev_plans;                                 // device -> plans (built at Compile for the assigned devices)
  std::map<int, std::vector<void*>> const_dev;                       // device -> per-node constant copy
  std::map<int, std::vector<std::vector<void*>>> idle_ws;            // device -> sets of prepared workspaces
  std::string last_trace;                                            // the trace of the latest traced Execute (under mu)
  // Replay as CUDA graphs (one device, no collectives): an Execute whose input buffers are the ones of an earlier call is
  // launched as one instantiated graph instead of node by node.  An instance owns the memory of every intermediate value
  // and its workspaces, so its kernel parameters never change; results are copied out into fresh buffers.
  struct GraphInstance {
    int dev = 0;
    std::vector<void*> key;                    // the input pointers it was captured with
    int seen = 0;                              // calls with this key so far; captured at the second
    cudaGraphExec_t exec = nullptr;
    std::vector<void*> mem, ws;                // per node: the memory the graph reads and writes, and its workspaces
    std::vector<void*> owned_mem;              // the allocations behind mem (parameters and constants are not the instance's)
    bool busy = false;                         // one replay at a time (the instance's memory is shared state)
    int launches = 0;
  };
  std::vector<std::unique_ptr<GraphInstance>> graphs;                // under mu
  bool graphs_off = false;                                           // set when a capture failed: stay on the plain path
  int graph_replays = 0;
  bool finalized = false;
};

namespace {

cbg_value* add_node(cbg_function* f, NodeKind kind, const Shape& shape, std::vector<cbg_value*> inputs) {
  auto v = std::make_unique<cbg_value>();
  v->kind = kind;
  v->shape = shape;
  v->inputs = std::move(inputs);
  v->fn = f;
  v->index = (int)f->nodes.size();
  f->nodes.push_back(std::move(v));
  return f->nodes.back().get();
}

int check_fn(const cbg_function* f, const char* op) {
  cb::clear_error();
  if (!f) return fail(CB_ERR_INVALID_ARG, "%s: function is NULL", op);
  if (f->builder->be->finalized.load()) return fail(CB_ERR_INVALID_ARG, "%s: backend has been finalized", op);
  if (f->builder->compiled) return fail(CB_ERR_INVALID_ARG, "%s: builder %s was already compiled", op, f->builder->name.c_str());
  if (f->returned) return fail(CB_ERR_INVALID_ARG, "%s: function already has its Return", op);
  return CB_OK;
}

// VerifyAndCastValues: every operand must be a live value of this function.
int check_values(const cbg_function* f, const char* op, std::initializer_list<const cbg_value*> vs) {
  for (const cbg_value* v : vs) {
    if (!v) return fail(CB_ERR_INVALID_ARG, "%s: nil value among the operands", op);
    if (v->fn != f) return fail(CB_ERR_INVALID_ARG, "%s: operand was created by a different function/builder", op);
  }
  return CB_OK;
}

int make_dims(const char* op, int rank, const int64_t* dims, std::vector<int64_t>* out) {
  if (rank < 0 || rank > 8) return fail(CB_ERR_INVALID_ARG, "%s: rank %d is not supported (max 8)", op, rank);
  out->clear();
  for (int i = 0; i < rank; i++) {
    if (dims[i] < 0) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dynamic or negative dimension %lld is not supported", op, (long long)dims[i]);
    out->push_back(dims[i]);
  }
  return CB_OK;
}

int out_shape(const cbg_value* v, int32_t* dtype, int* rank, int64_t* dims) {
  if (dtype) *dtype = v->shape.dtype;
  if (rank) *rank = (int)v->shape.dims.size();
  if (dims) for (size_t i = 0; i < v->shape.dims.size(); i++) dims[i] = v->shape.dims[i];
  return CB_OK;
}

int convert_node(cbg_function* f, cbg_value* x, int32_t dtype, cbg_value** v) {
  if (x->shape.dtype == dtype) { *v = x; return CB_OK; }
  if (cb::dtype_size(dtype) == 0 || dtype > CB_BF16 || x->shape.dtype > CB_BF16)
    return fail(CB_ERR_NOT_IMPLEMENTED, "ConvertDType: %s -> %s is not implemented", cb::dtype_name(x->shape.dtype), cb::dtype_name(dtype));
  Shape s = x->shape;
  s.dtype = dtype;
  *v = add_node(f, N_CONVERT, s, {x});
  return CB_OK;
}

cbg_value* transpose_node(cbg_function* f, cbg_value* x, const std::vector<int>& perm) {
  bool identity = true;
  for (size_t i = 0; i < perm.size(); i++) identity &= (perm[i] == (int)i);
  if (identity) return x;
  Shape s = x->shape;
  for (size_t i = 0; i < perm.size(); i++) s.dims[i] = x->shape.dims[perm[i]];
  cbg_value* v = add_node(f, N_TRANSPOSE, s, {x});
  v->perm.assign(perm.begin(), perm.end());
  return v;
}

cbg_value* reshape_node(cbg_function* f, cbg_value* x, const std::vector<int64_t>& dims) {
  if (x->shape.dims == dims) return x;
  Shape s;
  s.dtype = x->shape.dtype;
  s.dims = dims;
  return add_node(f, N_RESHAPE, s, {x});
}

// host <-> device through a pinned staging buffer and a pooled stream (to_device: host -> device)
int staged_copy(cbg_backend* be, int dev, void* dptr, void* host, size_t bytes, bool to_device) {
  if (bytes == 0) return CB_OK;
  // The caller's memory is itself page-locked (from cb_host_alloc, or registered): no staging copy is needed.
  cudaPointerAttributes attr;
  if (cb::host_range_is_page_locked(host, bytes) || (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost)) {
    cb_stream s = nullptr;
    CB_TRY(be->get_stream(dev, &s));
    int st = to_device ? cb_h2d(dev, dptr, host, bytes, s) : cb_d2h(dev, host, dptr, bytes, s);
    if (st == CB_OK) st = cb_stream_sync(dev, s);
    be->put_stream(dev, s);
    return st;
  }
  (void)cudaGetLastError();
  if (bytes > PINNED_STAGING_MAX) return to_device ? cb_h2d(dev, dptr, host, bytes, nullptr) : cb_d2h(dev, host, dptr, bytes, nullptr);
  void* pin = nullptr;
  size_t cap = 0;
  CB_TRY(be->pinned.get(bytes, &pin, &cap));
  cb_stream s = nullptr;
  int st = be->get_stream(dev, &s);
  if (st == CB_OK) {
    if (to_device) {
      memcpy(pin, host, bytes);
      st = cb_h2d(dev, dptr, pin, bytes, s);
      if (st == CB_OK) st = cb_stream_sync(dev, s);
    } else {
      st = cb_d2h(dev, pin, dptr, bytes, s);
      if (st == CB_OK) st = cb_stream_sync(dev, s);
      if (st == CB_OK) memcpy(host, pin, bytes);
    }
    be->put_stream(dev, s);
  }
  be->pinned.put(cap, pin);
  return st;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- Backend
int cbg_backend_new(const char* config, cbg_backend** backend) {
  cb::clear_error();
  if (!backend) return fail(CB_ERR_INVALID_ARG, "backend output pointer is NULL");
  *backend = nullptr;
  auto b = std::make_unique<cbg_backend>();
  std::string cfg = config ? config : "";
  std::stringstream ss(cfg);
  std::string item;
  while (std::getline(ss, item, ',')) {
    if (item.empty()) continue;
    if (item == "fallback_only") b->fallback_only = true;
    else if (item == "trace") b->trace = true;
    else if (item == "no_graphs") b->no_graphs = true;
    else if (item.rfind("devices=", 0) == 0) { /* accepted; device visibility is the process's */ }
    else return fail(CB_ERR_INVALID_ARG, "unknown configuration option \"%s\" for the cuda backend", item.c_str());
  }
  if (const char* t = getenv("CUDABACKEND_TRACE")) b->trace = b->trace || (t[0] && strcmp(t, "0") != 0);   // read once, here
  int n = 0;
  CB_TRY(cb_init(&n));
  b->n_devices = n;
  for (int i = 0; i < n; i++) b->pools.push_back(std::make_unique<DevicePool>());
  b->streams.resize(n);
  char desc[256];
  CB_TRY(cb_device_desc(0, desc, sizeof(desc)));
  b->description = std::string("cudabackend (sm_100a kernels for FusedQuantizedDense, DotGeneral, FusedScaledDotProductAttention) on ") + desc;
  *backend = b.release();
  return CB_OK;
}

const char* cbg_backend_name(const cbg_backend* b) { return b ? b->name.c_str() : ""; }
const char* cbg_backend_description(const cbg_backend* b) { return b ? b->description.c_str() : ""; }
int cbg_backend_num_devices(const cbg_backend* b) { return b ? b->n_devices : 0; }
int cbg_backend_device_description(const cbg_backend* b, int dev, char* buf, size_t n) { return cb_device_desc(dev, buf, n); }

int cbg_backend_capabilities(const cbg_backend* b, int32_t* ops, int* n_ops, int32_t* dtypes, int* n_dtypes) {
  // OpType codes of optype.go: Parameter 1, Constant 2, DotGeneral 32, AllReduce 112, AllGather 114, FusedSoftmax 116,
  // FusedLayerNorm 117, FusedGelu 118, FusedDense 119, FusedScaledDotProductAttention 120,
  // FusedAttentionQKVProjection 122, FusedQuantizedDense 123, QuantizedEmbeddingLookup 124.  The helper ops (Reshape, Slice, Iota, ConvertDType,
  // Transpose) exist to serve DotGeneral, and the element-wise / reduce ops to serve a decoder block, for the float
  // dtypes only: they are deliberately not advertised, so that the compliance suite's per-op sweeps over every dtype
  // skip them.
  static const int32_t k_ops[] = {1, 2, 32, 112, 114, 116, 117, 118, 119, 120, 122, 123, 124};
  static const int32_t k_dtypes[] = {CB_BOOL, CB_I8, CB_I32, CB_I64, CB_U8, CB_F16, CB_F32, CB_F64, CB_BF16};
  const int no = (int)(sizeof(k_ops) / sizeof(k_ops[0])), nd = (int)(sizeof(k_dtypes) / sizeof(k_dtypes[0]));
  if (ops && n_ops) for (int i = 0; i < std::min(*n_ops, no); i++) ops[i] = k_ops[i];
  if (dtypes && n_dtypes) for (int i = 0; i < std::min(*n_dtypes, nd); i++) dtypes[i] = k_dtypes[i];
  if (n_ops) *n_ops = no;
  if (n_dtypes) *n_dtypes = nd;
  return CB_OK;
}

int cbg_backend_finalize(cbg_backend* b) {
  cb::clear_error();
  if (!b) return CB_OK;
  if (b->finalized.exchange(true)) return CB_OK;
  for (int d = 0; d < b->n_devices; d++) {
    b->pools[d]->release_all(d);
    std::lock_guard<std::mutex> l(b->stream_mu);
    for (cb_stream s : b->streams[d]) cb_stream_destroy(d, s);
    b->streams[d].clear();
  }
  b->pinned.release_all();
  return CB_OK;
}

int cbg_backend_is_finalized(const cbg_backend* b) { return (!b || b->finalized.load()) ? 1 : 0; }

int cbg_backend_free(cbg_backend* b) {
  if (b) { cbg_backend_finalize(b); delete b; }
  return CB_OK;
}

// ---------------------------------------------------------------- Buffer
int cbg_buffer_from_flat(cbg_backend* b, int dev, const void* host_flat, int32_t dtype, int rank,
                         const int64_t* dims, cbg_buffer** buffer) {
  cb::clear_error();
  if (!b || !buffer) return fail(CB_ERR_INVALID_ARG, "BufferFromFlatData: NULL argument");
  *buffer = nullptr;
  if (b->finalized.load()) return fail(CB_ERR_INVALID_ARG, "BufferFromFlatData: backend has been finalized");
  if (dev < 0 || dev >= b->n_devices) return fail(CB_ERR_INVALID_ARG, "BufferFromFlatData: device %d out of range [0,%d)", dev, b->n_devices);
  if (!storable(dtype)) return fail(CB_ERR_NOT_IMPLEMENTED, "BufferFromFlatData: dtype %s is not supported", cb::dtype_name(dtype));
  auto buf = std::make_unique<cbg_buffer>();
  buf->be = b;
  buf->dev = dev;
  buf->shape.dtype = dtype;
  CB_TRY(make_dims("BufferFromFlatData", rank, dims, &buf->shape.dims));
  if (buf->shape.bytes() > 0 && !host_flat) return fail(CB_ERR_INVALID_ARG, "BufferFromFlatData: flat data is NULL");
  CB_TRY(b->pools[dev]->get(dev, buf->shape.bytes(), &buf->ptr));
  int st = staged_copy(b, dev, buf->ptr, const_cast<void*>(host_flat), buf->shape.bytes(), true);
  if (st != CB_OK) { b->pools[dev]->put(buf->shape.bytes(), buf->ptr); return st; }
  *buffer = buf.release();
  return CB_OK;
}

static int check_buffer(const cbg_buffer* buf, const char* op) {
  cb::clear_error();
  if (!buf) return fail(CB_ERR_INVALID_ARG, "%s: buffer is NULL", op);
  if (!buf->valid) return fail(CB_ERR_INVALID_ARG, "%s: buffer was finalized or donated", op);
  if (buf->be->finalized.load()) return fail(CB_ERR_INVALID_ARG, "%s: backend has been finalized", op);
  return CB_OK;
}

int cbg_buffer_shape(const cbg_buffer* buf, int32_t* dtype, int* rank, int64_t* dims) {
  CB_TRY(check_buffer(buf, "Buffer.Shape"));
  if (dtype) *dtype = buf->shape.dtype;
  if (rank) *rank = (int)buf->shape.dims.size();
  if (dims) for (size_t i = 0; i < buf->shape.dims.size(); i++) dims[i] = buf->shape.dims[i];
  return CB_OK;
}

int cbg_buffer_device_num(const cbg_buffer* buf, int* dev) {
  CB_TRY(check_buffer(buf, "Buffer.DeviceNum"));
  *dev = buf->dev;
  return CB_OK;
}

int cbg_buffer_to_flat(const cbg_buffer* buf, void* host_flat, size_t n_bytes) {
  CB_TRY(check_buffer(buf, "Buffer.ToFlatData"));
  if (n_bytes != buf->shape.bytes())
    return fail(CB_ERR_INVALID_ARG, "Buffer.ToFlatData: flat has %zu bytes, buffer %s needs %zu", n_bytes, buf->shape.str().c_str(), buf->shape.bytes());
  return staged_copy(buf->be, buf->dev, buf->ptr, host_flat, n_bytes, false);
}

int cbg_buffer_copy_to_device(const cbg_buffer* buf, int dev, cbg_buffer** out) {
  CB_TRY(check_buffer(buf, "Buffer.CopyToDevice"));
  if (dev < 0 || dev >= buf->be->n_devices) return fail(CB_ERR_INVALID_ARG, "Buffer.CopyToDevice: device %d out of range", dev);
  auto nb = std::make_unique<cbg_buffer>();
  nb->be = buf->be;
  nb->dev = dev;
  nb->shape = buf->shape;
  CB_TRY(buf->be->pools[dev]->get(dev, nb->shape.bytes(), &nb->ptr));
  int st = cb_d2d(dev, nb->ptr, buf->dev, buf->ptr, nb->shape.bytes(), nullptr);
  if (st != CB_OK) { buf->be->pools[dev]->put(nb->shape.bytes(), nb->ptr); return st; }
  *out = nb.release();
  return CB_OK;
}

int cbg_buffer_device_ptr(const cbg_buffer* buf, void** dptr) {
  CB_TRY(check_buffer(buf, "Buffer.DevicePtr"));
  *dptr = buf->ptr;
  return CB_OK;
}

int cbg_buffer_finalize(cbg_buffer* buf) {
  cb::clear_error();
  if (!buf) return CB_OK;
  if (buf->valid && buf->ptr) {
    if (buf->be->finalized.load()) cb_free(buf->dev, buf->ptr);
    else buf->be->pools[buf->dev]->put(buf->shape.bytes(), buf->ptr);
  }
  delete buf;
  return CB_OK;
}

// ---------------------------------------------------------------- Builder
int cbg_builder_new(cbg_backend* b, const char* name, cbg_builder** builder) {
  cb::clear_error();
  if (!b || !builder) return fail(CB_ERR_INVALID_ARG, "Builder: NULL argument");
  if (b->finalized.load()) return fail(CB_ERR_INVALID_ARG, "Builder: backend has been finalized");
  auto bld = std::make_unique<cbg_builder>();
  bld->be = b;
  bld->name = name ? name : "";
  bld->main = std::make_unique<cbg_function>();
  bld->main->builder = bld.get();
  *builder = bld.release();
  return CB_OK;
}

int cbg_builder_main(cbg_builder* bld, cbg_function** fn) {
  cb::clear_error();
  if (!bld || !fn) return fail(CB_ERR_INVALID_ARG, "Builder.Main: NULL argument");
  if (!bld->main) return fail(CB_ERR_INVALID_ARG, "Builder.Main: builder %s was already compiled", bld->name.c_str());
  *fn = bld->main.get();
  return CB_OK;
}

int cbg_builder_distributed_spmd(cbg_builder* bld, int num_devices) {
  cb::clear_error();
  if (!bld) return fail(CB_ERR_INVALID_ARG, "Builder.DistributedSPMD: builder is NULL");
  if (num_devices < 1 || num_devices > bld->be->n_devices)
    return fail(CB_ERR_INVALID_ARG, "Builder.DistributedSPMD: %d devices requested, %d available", num_devices, bld->be->n_devices);
  bld->spmd = num_devices;
  return CB_OK;
}

int cbg_builder_device_assignment(cbg_builder* bld, const int* devices, int n) {
  cb::clear_error();
  if (!bld) return fail(CB_ERR_INVALID_ARG, "Builder.DeviceAssignment: builder is NULL");
  for (int i = 0; i < n; i++)
    if (devices[i] < 0 || devices[i] >= bld->be->n_devices)
      return fail(CB_ERR_INVALID_ARG, "Builder.DeviceAssignment: device %d out of range [0,%d)", devices[i], bld->be->n_devices);
  bld->assignment.assign(devices, devices + n);
  return CB_OK;
}

int cbg_builder_free(cbg_builder* bld) { delete bld; return CB_OK; }

// ---------------------------------------------------------------- Function
int cbg_fn_parameter(cbg_function* f, const char* name, int32_t dtype, int rank, const int64_t* dims, cbg_value** v) {
  CB_TRY(check_fn(f, "Parameter"));
  if (!storable(dtype)) return fail(CB_ERR_NOT_IMPLEMENTED, "Parameter: dtype %s is not supported", cb::dtype_name(dtype));
  Shape s;
  s.dtype = dtype;
  CB_TRY(make_dims("Parameter", rank, dims, &s.dims));
  cbg_value* n = add_node(f, N_PARAM, s, {});
  n->name = name ? name : "";
  n->param_index = (int)f->params.size();
  f->params.push_back(n);
  *v = n;
  return CB_OK;
}

int cbg_fn_constant(cbg_function* f, const void* host_flat, int32_t dtype, int rank, const int64_t* dims, cbg_value** v) {
  CB_TRY(check_fn(f, "Constant"));
  if (!storable(dtype)) return fail(CB_ERR_NOT_IMPLEMENTED, "Constant: dtype %s is not supported", cb::dtype_name(dtype));
  Shape s;
  s.dtype = dtype;
  CB_TRY(make_dims("Constant", rank, dims, &s.dims));
  if (s.bytes() > 0 && !host_flat) return fail(CB_ERR_INVALID_ARG, "Constant: flat data is NULL");
  cbg_value* n = add_node(f, N_CONST, s, {});
  n->const_data.assign((const uint8_t*)host_flat, (const uint8_t*)host_flat + s.bytes());   // the graph owns a copy
  *v = n;
  return CB_OK;
}

int cbg_fn_shape(const cbg_value* v, int32_t* dtype, int* rank, int64_t* dims) {
  cb::clear_error();
  if (!v) return fail(CB_ERR_INVALID_ARG, "Shape: value is NULL");
  return out_shape(v, dtype, rank, dims);
}

int cbg_fn_return(cbg_function* f, cbg_value* const* outputs, int n) {
  CB_TRY(check_fn(f, "Return"));
  if (n <= 0) return fail(CB_ERR_INVALID_ARG, "Return: a function must return at least one value");
  for (int i = 0; i < n; i++) CB_TRY(check_values(f, "Return", {outputs[i]}));
  f->outputs.assign(outputs, outputs + n);
  f->returned = true;
  return CB_OK;
}

int cbg_fn_reshape(cbg_function* f, cbg_value* x, int rank, const int64_t* dims, cbg_value** v) {
  CB_TRY(check_fn(f, "Reshape"));
  CB_TRY(check_values(f, "Reshape", {x}));
  std::vector<int64_t> d;
  CB_TRY(make_dims("Reshape", rank, dims, &d));
  int64_t n = 1;
  for (auto e : d) n *= e;
  if (n != x->shape.size())
    return fail(CB_ERR_INVALID_ARG, "Reshape: cannot reshape %s (size %lld) into a shape of size %lld", x->shape.str().c_str(), (long long)x->shape.size(), (long long)n);
  *v = reshape_node(f, x, d);
  return CB_OK;
}

int cbg_fn_slice(cbg_function* f, cbg_value* x, const int64_t* starts, const int64_t* limits, const int64_t* strides, cbg_value** v) {
  CB_TRY(check_fn(f, "Slice"));
  CB_TRY(check_values(f, "Slice", {x}));
  const int r = (int)x->shape.dims.size();
  Shape s = x->shape;
  std::vector<int64_t> st(r), li(r), sr(r);
  for (int i = 0; i < r; i++) {
    st[i] = starts[i]; li[i] = limits[i]; sr[i] = strides ? strides[i] : 1;
    if (sr[i] < 1 || st[i] < 0 || li[i] > x->shape.dims[i] || st[i] > li[i])
      return fail(CB_ERR_INVALID_ARG, "Slice: axis %d start=%lld limit=%lld stride=%lld invalid for operand %s", i,
                  (long long)st[i], (long long)li[i], (long long)sr[i], x->shape.str().c_str());
    s.dims[i] = (li[i] - st[i] + sr[i] - 1) / sr[i];
  }
  cbg_value* n = add_node(f, N_SLICE, s, {x});
  n->starts = st; n->limits = li; n->strides = sr;
  *v = n;
  return CB_OK;
}

int cbg_fn_iota(cbg_function* f, int32_t dtype, int rank, const int64_t* dims, int axis, cbg_value** v) {
  CB_TRY(check_fn(f, "Iota"));
  Shape s;
  s.dtype = dtype;
  CB_TRY(make_dims("Iota", rank, dims, &s.dims));
  if (rank < 1) return fail(CB_ERR_INVALID_ARG, "Iota: shape must have rank >= 1");
  if (axis < 0 || axis >= rank) return fail(CB_ERR_INVALID_ARG, "Iota: axis %d out of range for rank %d", axis, rank);
  if (cb::dtype_size(dtype) == 0 || dtype > CB_BF16 || dtype == CB_BOOL)
    return fail(CB_ERR_NOT_IMPLEMENTED, "Iota: dtype %s is not supported", cb::dtype_name(dtype));
  cbg_value* n = add_node(f, N_IOTA, s, {});
  n->axis = axis;
  *v = n;
  return CB_OK;
}

int cbg_fn_convert_dtype(cbg_function* f, cbg_value* x, int32_t dtype, cbg_value** v) {
  CB_TRY(check_fn(f, "ConvertDType"));
  CB_TRY(check_values(f, "ConvertDType", {x}));
  return convert_node(f, x, dtype, v);
}

int cbg_fn_transpose(cbg_function* f, cbg_value* x, const int* permutation, cbg_value** v) {
  CB_TRY(check_fn(f, "Transpose"));
  CB_TRY(check_values(f, "Transpose", {x}));
  const int r = (int)x->shape.dims.size();
  std::vector<int> perm(permutation, permutation + r);
  std::vector<bool> seen(r, false);
  for (int a : perm) {
    if (a < 0 || a >= r || seen[a]) return fail(CB_ERR_INVALID_ARG, "Transpose: invalid permutation for rank %d", r);
    seen[a] = true;
  }
  *v = transpose_node(f, x, perm);
  return CB_OK;
}

int cbg_fn_dot_general(cbg_function* f, cbg_value* lhs, const int* lhs_contract, int n_contract,
                       const int* lhs_batch, int n_batch, cbg_value* rhs, const int* rhs_contract,
                       const int* rhs_batch, int32_t acc_dtype, int32_t out_dtype, cbg_value** v) {
  CB_TRY(check_fn(f, "DotGeneral"));
  CB_TRY(check_values(f, "DotGeneral", {lhs, rhs}));
  const Shape &ls = lhs->shape, &rs = rhs->shape;
  const int lr = (int)ls.dims.size(), rr = (int)rs.dims.size();
  // ---- shape inference (shapeinference/dotgeneral.go:16-152)
  if (ls.dtype != rs.dtype)
    return fail(CB_ERR_INVALID_ARG, "DotGeneral requires inputs with the same DType, got lhs=%s and rhs=%s", cb::dtype_name(ls.dtype), cb::dtype_name(rs.dtype));
  if (n_contract < 0 || n_batch < 0) return fail(CB_ERR_INVALID_ARG, "DotGeneral: negative axis count");
  std::vector<bool> lu(lr, false), ru(rr, false);
  auto use = [&](const char* side, const char* what, int axis, int rank, std::vector<bool>& used) -> int {
    if (axis < 0 || axis >= rank) return fail(CB_ERR_INVALID_ARG, "DotGeneral %s %s axis %d out of bounds for rank %d", side, what, axis, rank);
    if (used[axis]) return fail(CB_ERR_INVALID_ARG, "DotGeneral %s axis %d used more than once in contracting/batch", side, axis);
    used[axis] = true;
    return CB_OK;
  };
  for (int i = 0; i < n_contract; i++) {
    CB_TRY(use("lhs", "contracting", lhs_contract[i], lr, lu));
    CB_TRY(use("rhs", "contracting", rhs_contract[i], rr, ru));
    if (ls.dims[lhs_contract[i]] != rs.dims[rhs_contract[i]])
      return fail(CB_ERR_INVALID_ARG, "DotGeneral contracting dimensions do not match: lhs[%d]=%lld, rhs[%d]=%lld", lhs_contract[i],
                  (long long)ls.dims[lhs_contract[i]], rhs_contract[i], (long long)rs.dims[rhs_contract[i]]);
  }
  for (int i = 0; i < n_batch; i++) {
    CB_TRY(use("lhs", "batch", lhs_batch[i], lr, lu));
    CB_TRY(use("rhs", "batch", rhs_batch[i], rr, ru));
    if (ls.dims[lhs_batch[i]] != rs.dims[rhs_batch[i]])
      return fail(CB_ERR_INVALID_ARG, "DotGeneral batch dimensions do not match: lhs[%d]=%lld, rhs[%d]=%lld", lhs_batch[i],
                  (long long)ls.dims[lhs_batch[i]], rhs_batch[i], (long long)rs.dims[rhs_batch[i]]);
  }
  const int32_t in_dtype = ls.dtype;
  const int32_t final_dtype = out_dtype ? out_dtype : in_dtype;
  Shape api;   // batch..., lhs cross..., rhs cross...
  api.dtype = final_dtype;
  std::vector<int> lcross, rcross;
  for (int i = 0; i < n_batch; i++) api.dims.push_back(ls.dims[lhs_batch[i]]);
  for (int a = 0; a < lr; a++) if (!lu[a]) { lcross.push_back(a); api.dims.push_back(ls.dims[a]); }
  for (int a = 0; a < rr; a++) if (!ru[a]) { rcross.push_back(a); api.dims.push_back(rs.dims[a]); }
  if (api.dims.size() > 8) return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral: output rank %zu is not supported (max 8)", api.dims.size());

  // ---- dtype plan (dot.go:207-217, :340-372): half inputs accumulate in f32; another
  // accumulator dtype converts the inputs first; the result is converted to the API dtype.
  int32_t comp = in_dtype;
  if (acc_dtype && acc_dtype != in_dtype && !(is_half(in_dtype) && acc_dtype == CB_F32)) comp = acc_dtype;
  const bool comp_ok = comp == CB_F32 || comp == CB_F64 || comp == CB_BF16 || comp == CB_F16 || comp == CB_I32 || comp == CB_I64;
  if (!comp_ok || (comp != in_dtype && (!is_float(in_dtype) || !is_float(comp))))
    return fail(CB_ERR_NOT_IMPLEMENTED, "no DotGeneral implementation found for layout and dtypes=%s,%s", cb::dtype_name(in_dtype), cb::dtype_name(comp));
  if (cb::dtype_size(final_dtype) == 0 || final_dtype > CB_BF16)
    return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral: output dtype %s is not implemented", cb::dtype_name(final_dtype));
  cbg_value *l = lhs, *r = rhs;
  if (comp != in_dtype) { CB_TRY(convert_node(f, l, comp, &l)); CB_TRY(convert_node(f, r, comp, &r)); }

  // ---- normalisation to lhs [B,M,K], rhs [B,K,N] or [B,N,K] (dot.go:292-337)
  std::vector<int> lperm, rnn, rnt;
  for (int i = 0; i < n_batch; i++) lperm.push_back(lhs_batch[i]);
  for (int a : lcross) lperm.push_back(a);
  for (int i = 0; i < n_contract; i++) lperm.push_back(lhs_contract[i]);
  for (int i = 0; i < n_batch; i++) { rnn.push_back(rhs_batch[i]); rnt.push_back(rhs_batch[i]); }
  for (int i = 0; i < n_contract; i++) rnn.push_back(rhs_contract[i]);
  for (int a : rcross) { rnn.push_back(a); rnt.push_back(a); }
  for (int i = 0; i < n_contract; i++) rnt.push_back(rhs_contract[i]);
  auto identity = [](const std::vector<int>& p) { for (size_t i = 0; i < p.size(); i++) if (p[i] != (int)i) return false; return true; };
  int64_t B = 1, M = 1, N = 1, K = 1;
  for (int i = 0; i < n_batch; i++) B *= ls.dims[lhs_batch[i]];
  for (int a : lcross) M *= ls.dims[a];
  for (int a : rcross) N *= rs.dims[a];
  for (int i = 0; i < n_contract; i++) K *= ls.dims[lhs_contract[i]];
  l = transpose_node(f, l, lperm);
  bool transposed;
  // size-1 cross or contracting extents make both layouts the same memory
  if (identity(rnn) || N == 1 || K == 1) { if (!identity(rnn) && !identity(rnt)) r = transpose_node(f, r, rnn); transposed = false; }
  else if (identity(rnt)) transposed = true;
  else { r = transpose_node(f, r, rnt); transposed = true; }

  // the normalised op: integers keep their dtype, floats may store another float type
  int32_t dot_out = comp;
  if (is_float(comp)) {
    if (final_dtype == comp || final_dtype == CB_F32 || final_dtype == CB_F64) dot_out = final_dtype;
    else if (is_half(comp)) dot_out = CB_F32;     // reference: half inputs produce f32, converted afterwards
  }
  Shape ns;
  ns.dtype = dot_out;
  ns.dims = {B, M, N};
  cbg_value* d = add_node(f, N_DOT, ns, {l, r});
  d->dot.B = B; d->dot.M = M; d->dot.N = N; d->dot.K = K;
  d->dot.rhs_transposed = transposed ? 1 : 0;
  d->dot.in_dtype = comp;
  d->dot.out_dtype = dot_out;
  d->dot.variant = f->builder->be->fallback_only ? CB_DOT_GENERIC : CB_DOT_AUTO;
  cbg_value* res = d;
  if (dot_out != final_dtype) CB_TRY(convert_node(f, res, final_dtype, &res));
  res = reshape_node(f, res, api.dims);
  *v = res;
  return CB_OK;
}

static int check_small_dtype(const char* op, const cbg_value* x) {
  const int d = x->shape.dtype;
  if (d != CB_F32 && d != CB_F64 && d != CB_BF16 && d != CB_F16) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dtype %s", op, cb::dtype_name(d));
  return CB_OK;
}

// FusedOps.FusedSoftmax (fused_ops.go:318-323; internal/gobackend/fusedops/softmax.go:29-45): one non-negative axis.
int cbg_fn_fused_softmax(cbg_function* f, cbg_value* x, int axis, cbg_value** v) {
  const char* op = "FusedSoftmax";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x}));
  const int rank = (int)x->shape.dims.size();
  if (axis < 0 || axis >= rank) return fail(CB_ERR_INVALID_ARG, "%s: axis %d out of range for rank %d", op, axis, rank);
  CB_TRY(check_small_dtype(op, x));
  cbg_value* n = add_node(f, N_SOFTMAX, x->shape, {x});
  n->small_dims[0] = n->small_dims[2] = 1;
  for (int i = 0; i < axis; i++) n->small_dims[0] *= x->shape.dims[i];
  n->small_dims[1] = x->shape.dims[axis];
  for (int i = axis + 1; i < rank; i++) n->small_dims[2] *= x->shape.dims[i];
  *v = n;
  return CB_OK;
}

// FusedOps.FusedGelu (fused_ops.go:325-328; fusedops/gelu.go:31-41).
int cbg_fn_fused_gelu(cbg_function* f, cbg_value* x, int exact, cbg_value** v) {
  const char* op = "FusedGelu";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x}));
  CB_TRY(check_small_dtype(op, x));
  cbg_value* n = add_node(f, N_GELU, x->shape, {x});
  n->flags = exact ? 1 : 0;
  *v = n;
  return CB_OK;
}

// FusedOps.FusedLayerNorm (fused_ops.go:330-333; fusedops/layernorm.go:40-68, :96-127): negative axes count from
// the end; gamma and beta are indexed by the flat position inside the normalised axes, in the order given.  Axes
// that are not the trailing ones are moved there by a transposition and moved back afterwards.
int cbg_fn_fused_layer_norm(cbg_function* f, cbg_value* x, const int* axes, int n_axes, double epsilon, cbg_value* gamma,
                            cbg_value* beta, cbg_value** v) {
  const char* op = "FusedLayerNorm";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x}));
  if (gamma) CB_TRY(check_values(f, op, {gamma}));
  if (beta) CB_TRY(check_values(f, op, {beta}));
  const int rank = (int)x->shape.dims.size();
  if (n_axes < 0 || (n_axes > 0 && !axes)) return fail(CB_ERR_INVALID_ARG, "%s: axes are NULL", op);
  std::vector<int> norm;
  std::vector<bool> is_norm(rank, false);
  for (int i = 0; i < n_axes; i++) {
    int a = axes[i] < 0 ? axes[i] + rank : axes[i];
    if (a < 0 || a >= rank) return fail(CB_ERR_INVALID_ARG, "%s: axis %d out of range for rank %d", op, axes[i], rank);
    if (is_norm[a]) return fail(CB_ERR_INVALID_ARG, "%s: axis %d given more than once", op, axes[i]);
    is_norm[a] = true;
    norm.push_back(a);
  }
  CB_TRY(check_small_dtype(op, x));
  int64_t norm_size = 1;
  for (int a : norm) norm_size *= x->shape.dims[a];
  for (cbg_value* g : {gamma, beta})
    if (g && (g->shape.dtype != x->shape.dtype || g->shape.size() != norm_size))
      return fail(CB_ERR_INVALID_ARG, "%s: gamma and beta must have the dtype of x and %lld elements, got %s", op, (long long)norm_size, g->shape.str().c_str());
  std::vector<int> perm, inverse(rank);
  for (int a = 0; a < rank; a++) if (!is_norm[a]) perm.push_back(a);
  for (int a : norm) perm.push_back(a);
  for (int i = 0; i < rank; i++) inverse[perm[i]] = i;
  cbg_value* xt = transpose_node(f, x, perm);
  std::vector<cbg_value*> ins = {xt};
  if (gamma) ins.push_back(gamma);
  if (beta) ins.push_back(beta);
  cbg_value* n = add_node(f, N_LAYERNORM, xt->shape, ins);
  n->small_dims[0] = norm_size ? x->shape.size() / norm_size : 0;
  n->small_dims[1] = norm_size;
  n->small_dims[2] = 1;
  n->epsilon = epsilon;
  n->flags = (gamma ? 1 : 0) | (beta ? 2 : 0);
  *v = transpose_node(f, n, inverse);
  return CB_OK;
}

// FusedOps.FusedAttentionQKVProjection (fused_ops.go:437-461; internal/gobackend/fusedops/attentionqkv.go:38-96): one
// matmul x @ wQKV, then the three column ranges of the result, each with its optional bias.
int cbg_fn_fused_attention_qkv_projection(cbg_function* f, cbg_value* x, cbg_value* w_qkv, cbg_value* bias_q, cbg_value* bias_k,
                                          cbg_value* bias_v, int64_t query_dim, int64_t key_value_dim, cbg_value** query,
                                          cbg_value** key, cbg_value** value) {
  const char* op = "AttentionQKVProjection";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x, w_qkv}));
  for (cbg_value* b : {bias_q, bias_k, bias_v}) if (b) CB_TRY(check_values(f, op, {b}));
  const int xr = (int)x->shape.dims.size();
  if (xr < 1) return fail(CB_ERR_INVALID_ARG, "%s: x must have rank >= 1, got %d", op, xr);
  if (query_dim < 0 || key_value_dim < 0) return fail(CB_ERR_INVALID_ARG, "%s: negative projection dimension", op);
  const int64_t total = query_dim + 2 * key_value_dim;
  if (w_qkv->shape.dims.size() != 2 || w_qkv->shape.dims[0] != x->shape.dims.back() || w_qkv->shape.dims[1] != total)
    return fail(CB_ERR_INVALID_ARG, "%s: wQKV must be [%lld, %lld], got %s", op, (long long)x->shape.dims.back(), (long long)total, w_qkv->shape.str().c_str());
  if (w_qkv->shape.dtype != x->shape.dtype) return fail(CB_ERR_INVALID_ARG, "%s: x and wQKV must share one dtype", op);
  const int64_t widths[3] = {query_dim, key_value_dim, key_value_dim};
  cbg_value* biases[3] = {bias_q, bias_k, bias_v};
  for (int i = 0; i < 3; i++)
    if (biases[i] && (biases[i]->shape.dtype != x->shape.dtype || biases[i]->shape.dims != std::vector<int64_t>{widths[i]}))
      return fail(CB_ERR_INVALID_ARG, "%s: bias %d must be [%lld] of the dtype of x, got %s", op, i, (long long)widths[i], biases[i]->shape.str().c_str());
  // the reference executes Float32 and Float64 (attentionqkv.go:128-135); the half types are this backend's extension
  CB_TRY(check_small_dtype("FusedAttentionQKVProjection", x));
  const int lc = xr - 1, rc = 0;
  cbg_value* combined = nullptr;
  CB_TRY(cbg_fn_dot_general(f, x, &lc, 1, nullptr, 0, w_qkv, &rc, nullptr, 0, 0, &combined));
  const int64_t rows = total ? combined->shape.size() / total : x->shape.size() / std::max<int64_t>(1, x->shape.dims.back());
  cbg_value** outs[3] = {query, key, value};
  int64_t first = 0;
  for (int i = 0; i < 3; i++) {
    Shape s = x->shape;
    s.dims.back() = widths[i];
    std::vector<cbg_value*> ins = {combined};
    if (biases[i]) ins.push_back(biases[i]);
    cbg_value* n = add_node(f, N_COLS_BIAS, s, ins);
    n->small_dims[0] = rows; n->small_dims[1] = total; n->small_dims[2] = first; n->small_dims[3] = widths[i];
    n->flags = biases[i] ? 1 : 0;
    *outs[i] = n;
    first += widths[i];
  }
  return CB_OK;
}

// FusedOps.FusedDense (fused_ops.go:336-347; builder internal/gobackend/fusedops/dense.go:34-108): the matmul is a
// DotGeneral contracting x's last axis with the weight's first (InputOutputs) or last (OutputsInput) axis; bias and
// activation become the epilogue of that same kernel instead of a second pass over the result.
int cbg_fn_fused_dense(cbg_function* f, cbg_value* x, cbg_value* weight, cbg_value* bias, int activation, int weight_layout,
                       cbg_value** v) {
  const char* op = "FusedDense";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x, weight}));
  if (bias) CB_TRY(check_values(f, op, {bias}));
  const int xr = (int)x->shape.dims.size(), wr = (int)weight->shape.dims.size();
  if (xr < 1 || wr < 2)
    return fail(CB_ERR_INVALID_ARG, "%s: x must have rank >= 1 (got %d), weight must have rank >= 2 (got %d)", op, xr, wr);
  if (weight->shape.dtype != x->shape.dtype)
    return fail(CB_ERR_INVALID_ARG, "%s: x and weight must share one dtype, got %s and %s", op, cb::dtype_name(x->shape.dtype), cb::dtype_name(weight->shape.dtype));
  if (activation < CB_ACT_NONE || activation > CB_ACT_TANH) return fail(CB_ERR_INVALID_ARG, "%s: unknown activation %d", op, activation);
  const int64_t in_features = x->shape.dims.back();
  int w_axis;
  std::vector<int64_t> out_features;
  if (weight_layout == 0) {            // DenseLayoutInputOutputs: [in_features, out_features...]
    if (in_features != weight->shape.dims[0])
      return fail(CB_ERR_INVALID_ARG, "%s: x's last dim (%lld) must match weight's first dim (%lld) for DenseLayoutInputOutputs", op,
                  (long long)in_features, (long long)weight->shape.dims[0]);
    w_axis = 0;
    out_features.assign(weight->shape.dims.begin() + 1, weight->shape.dims.end());
  } else if (weight_layout == 1) {     // DenseLayoutOutputsInput: [out_features..., in_features]
    if (in_features != weight->shape.dims[wr - 1])
      return fail(CB_ERR_INVALID_ARG, "%s: x's last dim (%lld) must match weight's last dim (%lld) for DenseLayoutOutputsInput", op,
                  (long long)in_features, (long long)weight->shape.dims[wr - 1]);
    w_axis = wr - 1;
    out_features.assign(weight->shape.dims.begin(), weight->shape.dims.end() - 1);
  } else {
    return fail(CB_ERR_INVALID_ARG, "%s: unknown WeightLayout %d", op, weight_layout);
  }
  if (bias && (bias->shape.dtype != x->shape.dtype || bias->shape.dims != out_features))
    return fail(CB_ERR_INVALID_ARG, "%s: bias must have the dtype of x and the out-features shape, got %s", op, bias->shape.str().c_str());
  // the reference executes Float32 and Float64 (dense.go:149-163); the half types are this backend's extension
  if (x->shape.dtype != CB_F32 && x->shape.dtype != CB_F64 && x->shape.dtype != CB_BF16 && x->shape.dtype != CB_F16)
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dtype %s", op, cb::dtype_name(x->shape.dtype));
  const int lc = xr - 1;
  cbg_value* res = nullptr;
  CB_TRY(cbg_fn_dot_general(f, x, &lc, 1, nullptr, 0, weight, &w_axis, nullptr, 0, 0, &res));
  if (bias || activation != CB_ACT_NONE) {
    cbg_value* d = res;
    while (d->kind == N_RESHAPE) d = d->inputs[0];
    if (d->kind != N_DOT) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: the matmul did not lower to one kernel", op);
    d->dot.activation = activation;
    if (bias) {
      d->dot.has_bias = 1;
      d->inputs.push_back(bias);     // flat [N]: the out-feature axes in order, as the normalised rhs enumerates them
    }
  }
  *v = res;
  return CB_OK;
}

// validateGGMLTypeSupported and deriveGGMLK (internal/gobackend/fusedops/quantizeddense.go:145-176)
static int ggml_derive_k(const char* op, int64_t bytes_per_row, int ggml_type, int64_t* K) {
  int vpb = 0, bpb = 0;
  switch (ggml_type) {
    case CB_GGML_Q4_0: case CB_GGML_IQ4_NL: vpb = 32; bpb = 18; break;
    case CB_GGML_Q8_0: vpb = 32; bpb = 34; break;
    case CB_GGML_Q4_K: vpb = 256; bpb = 144; break;
    case CB_GGML_Q6_K: vpb = 256; bpb = 210; break;
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "%s: GGML type %d not supported in fused path", op, ggml_type);
  }
  if (bytes_per_row % bpb != 0)
    return fail(CB_ERR_INVALID_ARG, "%s: bytesPerRow %lld not divisible by bytesPerBlock %d", op, (long long)bytes_per_row, bpb);
  *K = bytes_per_row / bpb * vpb;
  return CB_OK;
}

// QuantizedEmbeddingLookup (internal/gobackend/fusedops/quantizeddense.go:250-321): data [vocab, bytesPerRow] Uint8 in a
// GGML block layout, indices integer with last dimension 1; the result replaces that dimension by K, Float32.
int cbg_fn_quantized_embedding_lookup(cbg_function* f, cbg_value* data, cbg_value* indices, int scheme, int ggml_type, cbg_value** v) {
  const char* op = "QuantizedEmbeddingLookup";
  CB_TRY(check_fn(f, op));
  if (scheme != CB_QUANT_GGML) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: only QuantGGML scheme is supported, got scheme %d", op, scheme);
  CB_TRY(check_values(f, op, {data, indices}));
  if (data->shape.dims.size() != 2 || data->shape.dtype != CB_U8)
    return fail(CB_ERR_INVALID_ARG, "%s: data must be [vocabSize, bytesPerRow] Uint8, got %s", op, data->shape.str().c_str());
  const int idt = indices->shape.dtype;
  const bool is_int = idt == CB_I8 || idt == CB_U8 || idt == CB_I32 || idt == CB_I64 || idt == CB_U32 || idt == CB_U64 || idt == CB_I16 || idt == CB_U16;
  if (!is_int) return fail(CB_ERR_INVALID_ARG, "%s: indices must be integer, got %s", op, cb::dtype_name(idt));
  if (indices->shape.dims.empty() || indices->shape.dims.back() != 1)
    return fail(CB_ERR_INVALID_ARG, "%s: indices last dim must be 1, got shape %s", op, indices->shape.str().c_str());
  int64_t K = 0;
  CB_TRY(ggml_derive_k(op, data->shape.dims[1], ggml_type, &K));
  if (idt != CB_I8 && idt != CB_U8 && idt != CB_I32 && idt != CB_I64)
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s: indices of dtype %s are not implemented", op, cb::dtype_name(idt));
  Shape s = indices->shape;
  s.dtype = CB_F32;
  s.dims.back() = K;
  cbg_value* n = add_node(f, N_EMBEDDING, s, {data, indices});
  n->axis = ggml_type;
  *v = n;
  return CB_OK;
}

// FusedQuantizedDense with compute.QuantGGML (internal/gobackend/fusedops/quantizeddense.go:181-248): weights
// [N, bytesPerRow] Uint8 in the native block layout; K follows from the row bytes and must equal x's last dimension.
int cbg_fn_fused_quantized_dense_ggml(cbg_function* f, cbg_value* x, cbg_value* weights, cbg_value* bias, int ggml_type,
                                      int activation, cbg_value** v) {
  const char* op = "FusedQuantizedDense(GGML)";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x, weights}));
  if (bias) CB_TRY(check_values(f, op, {bias}));
  if (x->shape.dtype != CB_F32 && x->shape.dtype != CB_BF16)
    return fail(CB_ERR_INVALID_ARG, "%s: x must be float32, got %s", op, cb::dtype_name(x->shape.dtype));
  if (x->shape.dims.size() < 1) return fail(CB_ERR_INVALID_ARG, "%s: x must have rank >= 1, got %zu", op, x->shape.dims.size());
  if (weights->shape.dims.size() != 2 || weights->shape.dtype != CB_U8)
    return fail(CB_ERR_INVALID_ARG, "%s: weights must be [N, bytesPerRow] Uint8, got %s", op, weights->shape.str().c_str());
  int64_t K = 0;
  CB_TRY(ggml_derive_k(op, weights->shape.dims[1], ggml_type, &K));
  const int64_t N = weights->shape.dims[0];
  if (x->shape.dims.back() != K)
    return fail(CB_ERR_INVALID_ARG, "%s: x's last dim (%lld) must match K=%lld derived from weights", op, (long long)x->shape.dims.back(), (long long)K);
  if (bias && (bias->shape.dtype != CB_F32 || bias->shape.dims != std::vector<int64_t>{N}))
    return fail(CB_ERR_INVALID_ARG, "%s: bias must be (Float32)[%lld], got %s", op, (long long)N, bias->shape.str().c_str());
  if (activation < CB_ACT_NONE || activation > CB_ACT_TANH) return fail(CB_ERR_INVALID_ARG, "%s: unknown activation %d", op, activation);
  Shape s = x->shape;
  s.dims.back() = N;
  std::vector<cbg_value*> ins = {x, weights};
  if (bias) ins.push_back(bias);
  cbg_value* n = add_node(f, N_QDENSE, s, ins);
  n->qd.M = K ? x->shape.size() / K : 0;
  n->qd.K = K; n->qd.N = N;
  n->qd.x_dtype = x->shape.dtype;
  n->qd.w_dtype = CB_U8;
  n->qd.scale_layout = CB_SCALE_CHANNEL;
  n->qd.has_bias = bias ? 1 : 0;
  n->qd.activation = activation;
  n->qd.scheme = CB_QUANT_GGML;
  n->qd.ggml_type = ggml_type;
  n->qd.variant = CB_QDENSE_GENERIC;
  *v = n;
  return CB_OK;
}

int cbg_fn_fused_quantized_dense(cbg_function* f, cbg_value* x, cbg_value* weights, cbg_value* bias, int scheme,
                                 cbg_value* scale, cbg_value* zero_point, int block_axis, int64_t block_size,
                                 int activation, cbg_value** v) {
  const char* op = "FusedQuantizedDense";
  CB_TRY(check_fn(f, op));
  if (scheme == 2) return fail(CB_ERR_INVALID_ARG, "%s: GGML weights go through cbg_fn_fused_quantized_dense_ggml", op);
  if (scheme != 0 && scheme != 1) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: unknown quantization scheme %d", op, scheme);
  CB_TRY(check_values(f, op, {x, weights, scale}));
  if (zero_point) CB_TRY(check_values(f, op, {zero_point}));
  if (bias) CB_TRY(check_values(f, op, {bias}));
  // x dtype: float32 in the reference (quantizeddense.go:93-95); bfloat16 is this backend's extension
  if (x->shape.dtype != CB_F32 && x->shape.dtype != CB_BF16)
    return fail(CB_ERR_INVALID_ARG, "%s: x must be float32, got %s", op, cb::dtype_name(x->shape.dtype));
  if (x->shape.dims.size() < 1) return fail(CB_ERR_INVALID_ARG, "%s: x must have rank >= 1, got %zu", op, x->shape.dims.size());
  const int64_t K = x->shape.dims.back();
  if (weights->shape.dims.size() != 2 || weights->shape.dims[0] != K)
    return fail(CB_ERR_INVALID_ARG, "%s: weights must be [%lld, N], got %s", op, (long long)K, weights->shape.str().c_str());
  const int64_t N = weights->shape.dims[1];
  // Int8 / Uint8, and the packed Int4 / Uint4 the reference unpacks first (quantizeddense.go:380-390; under NF4 the
  // nibbles are table indices, :392-409)
  const int wd = weights->shape.dtype;
  if (wd != CB_I8 && wd != CB_U8 && wd != CB_I4 && wd != CB_U4)
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s: %s unsupported weight type %s", op, scheme == 1 ? "NF4" : "Linear", cb::dtype_name(wd));
  // NF4 uses a fixed lookup table and takes no zero points (quantizeddense.go:126-129)
  if (scheme == 1 && zero_point) return fail(CB_ERR_INVALID_ARG, "%s: ZeroPoint must be nil for NF4 quantization scheme", op);
  if (block_size <= 0) return fail(CB_ERR_INVALID_ARG, "%s: BlockSize must be positive, got %lld", op, (long long)block_size);
  int layout;
  std::vector<int64_t> want;
  if (block_axis == 1) {
    layout = CB_SCALE_REF;
    want = {K, (N + block_size - 1) / block_size};
  } else if (block_axis == 0) {          // extension: blocks along the input-features axis
    want = {(K + block_size - 1) / block_size, N};
    layout = (want[0] <= 1) ? CB_SCALE_CHANNEL : CB_SCALE_KGROUP;
  } else {
    return fail(CB_ERR_INVALID_ARG, "%s: only Axis=1 is supported, got %d", op, block_axis);
  }
  if (scale->shape.dtype != CB_F32 || scale->shape.dims != want)
    return fail(CB_ERR_INVALID_ARG, "%s: scales must be (Float32)[%lld, %lld], got %s", op, (long long)want[0], (long long)want[1], scale->shape.str().c_str());
  if (zero_point && (zero_point->shape.dtype != CB_F32 || zero_point->shape.dims != want))
    return fail(CB_ERR_INVALID_ARG, "%s: zero points must be (Float32)[%lld, %lld], got %s", op, (long long)want[0], (long long)want[1], zero_point->shape.str().c_str());
  if (bias && (bias->shape.dtype != CB_F32 || bias->shape.dims != std::vector<int64_t>{N}))
    return fail(CB_ERR_INVALID_ARG, "%s: bias must be (Float32)[%lld], got %s", op, (long long)N, bias->shape.str().c_str());
  if (activation < CB_ACT_NONE || activation > CB_ACT_TANH) return fail(CB_ERR_INVALID_ARG, "%s: unknown activation %d", op, activation);
  // The reference expresses per-channel and K-group scales as [K, N] with BlockSize 1.  When such a scale is a
  // Constant whose rows repeat within groups of g rows, it is folded to the compact layout ([N], or [K/g, N]):
  // the same arithmetic element by element, and the layout the streaming kernels read.
  if (layout == CB_SCALE_REF && block_size == 1 && !zero_point && scheme == 0 && scale->kind == N_CONST &&
      (wd == CB_I8 || wd == CB_U8) && K > 1 && !f->builder->be->fallback_only) {
    const float* sd = reinterpret_cast<const float*>(scale->const_data.data());
    int64_t g = K;                                   // gcd of K and every row index where the row changes
    for (int64_t r = 1; r < K && g > 1; r++)
      if (memcmp(sd + r * N, sd + (r - 1) * N, (size_t)N * sizeof(float)) != 0) g = std::__gcd(g, r);
    if (g > 1) {
      Shape cs;
      cs.dtype = CB_F32;
      if (g == K) cs.dims = {N}; else cs.dims = {K / g, N};
      cbg_value* folded = add_node(f, N_CONST, cs, {});
      folded->const_data.resize(cs.bytes());
      float* out = reinterpret_cast<float*>(folded->const_data.data());
      for (int64_t r = 0; r < K / g; r++) memcpy(out + r * N, sd + r * g * N, (size_t)N * sizeof(float));
      scale = folded;
      layout = g == K ? CB_SCALE_CHANNEL : CB_SCALE_KGROUP;
      block_size = g;
    }
  }
  Shape s = x->shape;
  s.dims.back() = N;
  std::vector<cbg_value*> ins = {x, weights, scale};
  if (zero_point) ins.push_back(zero_point);
  if (bias) ins.push_back(bias);
  cbg_value* n = add_node(f, N_QDENSE, s, ins);
  n->qd.M = K ? x->shape.size() / K : 0;
  n->qd.K = K; n->qd.N = N;
  n->qd.x_dtype = x->shape.dtype;
  n->qd.w_dtype = weights->shape.dtype;
  n->qd.scale_layout = layout;
  n->qd.block_size = block_size;
  n->qd.has_zero_point = zero_point ? 1 : 0;
  n->qd.has_bias = bias ? 1 : 0;
  n->qd.activation = activation;
  n->qd.scheme = scheme;
  n->qd.variant = f->builder->be->fallback_only ? CB_QDENSE_GENERIC : CB_QDENSE_AUTO;
  *v = n;
  return CB_OK;
}

int cbg_fn_fused_sdpa(cbg_function* f, cbg_value* q, cbg_value* k, cbg_value* val, int axes_layout,
                      const cbg_sdpa_options* o, cbg_value** output) {
  const char* op = "FusedScaledDotProductAttention";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {q, k, val}));
  cbg_sdpa_options opt;
  memset(&opt, 0, sizeof(opt));
  if (o) opt = *o;
  if ((opt.query_seq_len != nullptr) != (opt.key_value_seq_len != nullptr))
    return fail(CB_ERR_INVALID_ARG, "%s: QuerySeqLen and KeyValueSeqLen must both be set or both nil", op);
  if (q->shape.dims.size() != 4) return fail(CB_ERR_INVALID_ARG, "%s: query must have rank 4, got %zu", op, q->shape.dims.size());
  if (k->shape.dims.size() != 4) return fail(CB_ERR_INVALID_ARG, "%s: key must have rank 4, got %zu", op, k->shape.dims.size());
  if (val->shape.dims != k->shape.dims) return fail(CB_ERR_INVALID_ARG, "%s: value shape %s must match key shape %s", op, val->shape.str().c_str(), k->shape.str().c_str());
  if (k->shape.dtype != q->shape.dtype || val->shape.dtype != q->shape.dtype)
    return fail(CB_ERR_INVALID_ARG, "%s: query, key and value must share one dtype", op);
  if (axes_layout != CB_LAYOUT_BHSD && axes_layout != CB_LAYOUT_BSHD) return fail(CB_ERR_INVALID_ARG, "%s: unknown axes layout %d", op, axes_layout);
  cb_sdpa_desc d;
  memset(&d, 0, sizeof(d));
  const int ha = axes_layout == CB_LAYOUT_BSHD ? 2 : 1, sa = axes_layout == CB_LAYOUT_BSHD ? 1 : 2;
  d.B = q->shape.dims[0]; d.Hq = q->shape.dims[ha]; d.S = q->shape.dims[sa]; d.D = q->shape.dims[3];
  d.Hkv = k->shape.dims[ha]; d.Skv = k->shape.dims[sa];
  if (k->shape.dims[0] != d.B || k->shape.dims[3] != d.D)
    return fail(CB_ERR_INVALID_ARG, "%s: key shape %s does not match query shape %s", op, k->shape.str().c_str(), q->shape.str().c_str());
  d.layout = axes_layout;
  d.dtype = q->shape.dtype;
  d.scale = opt.scale;
  d.causal = opt.causal ? 1 : 0;
  std::vector<cbg_value*> ins = {q, k, val};
  if (opt.mask) {
    CB_TRY(check_values(f, op, {opt.mask}));
    const Shape& ms = opt.mask->shape;
    if (ms.dtype == CB_BOOL) d.mask_kind = CB_MASK_BOOL;
    else if (ms.dtype == q->shape.dtype) d.mask_kind = CB_MASK_ADDITIVE;
    else return fail(CB_ERR_INVALID_ARG, "%s: mask must be Bool or %s, got %s", op, cb::dtype_name(q->shape.dtype), cb::dtype_name(ms.dtype));
    if (ms.dims.size() < 2 || ms.dims.size() > 4) return fail(CB_ERR_INVALID_ARG, "%s: mask must have rank 2, 3, or 4, got rank %zu", op, ms.dims.size());
    d.mask_rank = (int)ms.dims.size();
    for (size_t i = 0; i < ms.dims.size(); i++) d.mask_dims[i] = ms.dims[i];
    ins.push_back(opt.mask);
  }
  if (opt.query_seq_len) {
    CB_TRY(check_values(f, op, {opt.query_seq_len, opt.key_value_seq_len}));
    for (cbg_value* sl : {opt.query_seq_len, opt.key_value_seq_len})
      if (sl->shape.dtype != CB_I32 || sl->shape.dims != std::vector<int64_t>{d.B})
        return fail(CB_ERR_INVALID_ARG, "%s: QuerySeqLen / KeyValueSeqLen must be int32 with length batch (%lld), got %s", op, (long long)d.B, sl->shape.str().c_str());
    d.has_seq_lens = 1;
    ins.push_back(opt.query_seq_len);
    ins.push_back(opt.key_value_seq_len);
  }
  if (opt.bias) {
    CB_TRY(check_values(f, op, {opt.bias}));
    const Shape& bs = opt.bias->shape;
    if (!is_float(bs.dtype) || bs.dtype != q->shape.dtype)
      return fail(CB_ERR_INVALID_ARG, "%s: bias must be a float dtype matching the compute dtype, got %s", op, cb::dtype_name(bs.dtype));
    if (bs.dims.size() < 2 || bs.dims.size() > 4) return fail(CB_ERR_INVALID_ARG, "%s: bias must have rank 2, 3, or 4, got rank %zu", op, bs.dims.size());
    d.bias_rank = (int)bs.dims.size();
    for (size_t i = 0; i < bs.dims.size(); i++) d.bias_dims[i] = bs.dims[i];
    ins.push_back(opt.bias);
  }
  d.variant = f->builder->be->fallback_only ? CB_SDPA_GENERIC : CB_SDPA_AUTO;
  // plan once now so that dtype / head-count / broadcast errors surface at build time
  cb_plan* probe = nullptr;
  CB_TRY(cb_plan_sdpa(0, &d, &probe));
  cb_plan_destroy(probe);
  cbg_value* n = add_node(f, N_SDPA, q->shape, ins);
  n->sdpa = d;
  *output = n;
  return CB_OK;
}


// ---- element-wise and reduction ops of a decoder block (StandardOps, standard_ops.go:131-700)
static int binary_op(cbg_function* f, const char* op, int code, cbg_value* lhs, cbg_value* rhs, cbg_value** v) {
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {lhs, rhs}));
  const Shape &ls = lhs->shape, &rs = rhs->shape;
  // shapeinference.BinaryOp (shapeinference/shapeinference.go:219-300)
  if (ls.dtype != rs.dtype)
    return fail(CB_ERR_INVALID_ARG, "data types (DType) for BinaryOp %s must match, got %s and %s", op, ls.str().c_str(), rs.str().c_str());
  const bool is_flt = ls.dtype == CB_F32 || ls.dtype == CB_F64 || ls.dtype == CB_BF16 || ls.dtype == CB_F16;
  if (!is_flt && ls.dtype != CB_I32 && ls.dtype != CB_I64)
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dtype %s is not implemented by the cuda backend", op, cb::dtype_name(ls.dtype));
  Shape out;
  out.dtype = ls.dtype;
  if (ls.dims.empty()) out.dims = rs.dims;
  else if (rs.dims.empty()) out.dims = ls.dims;
  else {
    if (ls.dims.size() != rs.dims.size())
      return fail(CB_ERR_INVALID_ARG, "if operands are not scalars, their rank must match for BinaryOp (%s); got shapes %s and %s", op, ls.str().c_str(), rs.str().c_str());
    for (size_t a = 0; a < ls.dims.size(); a++) {
      const int64_t l = ls.dims[a], r = rs.dims[a];
      if (l != r && l != 1 && r != 1)
        return fail(CB_ERR_INVALID_ARG, "dimension of axis #%zu doesn't match and cannot be broadcast for BinaryOp (%s), got shapes %s and %s", a, op, ls.str().c_str(), rs.str().c_str());
      out.dims.push_back(l == 1 ? r : l);
    }
  }
  cbg_value* n = add_node(f, N_BINARY, out, {lhs, rhs});
  n->op = code;
  *v = n;
  return CB_OK;
}
int cbg_fn_add(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v) { return binary_op(f, "Add", CB_BIN_ADD, lhs, rhs, v); }
int cbg_fn_sub(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v) { return binary_op(f, "Sub", CB_BIN_SUB, lhs, rhs, v); }
int cbg_fn_mul(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v) { return binary_op(f, "Mul", CB_BIN_MUL, lhs, rhs, v); }
int cbg_fn_div(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v) { return binary_op(f, "Div", CB_BIN_DIV, lhs, rhs, v); }
int cbg_fn_max(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v) { return binary_op(f, "Max", CB_BIN_MAX, lhs, rhs, v); }
int cbg_fn_min(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v) { return binary_op(f, "Min", CB_BIN_MIN, lhs, rhs, v); }

static int unary_op(cbg_function* f, const char* op, int code, cbg_value* x, cbg_value** v) {
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x}));
  CB_TRY(check_small_dtype(op, x));
  cbg_value* n = add_node(f, N_UNARY, x->shape, {x});
  n->op = code;
  *v = n;
  return CB_OK;
}
int cbg_fn_neg(cbg_function* f, cbg_value* x, cbg_value** v) { return unary_op(f, "Neg", CB_UN_NEG, x, v); }
int cbg_fn_rsqrt(cbg_function* f, cbg_value* x, cbg_value** v) { return unary_op(f, "Rsqrt", CB_UN_RSQRT, x, v); }
int cbg_fn_sqrt(cbg_function* f, cbg_value* x, cbg_value** v) { return unary_op(f, "Sqrt", CB_UN_SQRT, x, v); }
int cbg_fn_exp(cbg_function* f, cbg_value* x, cbg_value** v) { return unary_op(f, "Exp", CB_UN_EXP, x, v); }
int cbg_fn_logistic(cbg_function* f, cbg_value* x, cbg_value** v) { return unary_op(f, "Logistic", CB_UN_LOGISTIC, x, v); }
int cbg_fn_tanh(cbg_function* f, cbg_value* x, cbg_value** v) { return unary_op(f, "Tanh", CB_UN_TANH, x, v); }

static int reduce_op(cbg_function* f, const char* op, int code, cbg_value* x, const int* axes, int n_axes, cbg_value** v) {
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x}));
  CB_TRY(check_small_dtype(op, x));
  const int rank = (int)x->shape.dims.size();
  std::vector<int32_t> flags(rank, 0);
  if (n_axes == 0) std::fill(flags.begin(), flags.end(), 1);     // no axes: reduce everything (standard_ops.go:660-682)
  for (int i = 0; i < n_axes; i++) {
    const int a = axes[i] < 0 ? axes[i] + rank : axes[i];
    if (a < 0 || a >= rank) return fail(CB_ERR_INVALID_ARG, "%s: axis %d out of range for rank %d", op, axes[i], rank);
    if (flags[a]) return fail(CB_ERR_INVALID_ARG, "%s: axis %d given more than once", op, axes[i]);
    flags[a] = 1;
  }
  Shape out;
  out.dtype = x->shape.dtype;
  for (int a = 0; a < rank; a++) if (!flags[a]) out.dims.push_back(x->shape.dims[a]);
  cbg_value* n = add_node(f, N_REDUCE, out, {x});
  n->op = code;
  n->axis_flags = flags;
  *v = n;
  return CB_OK;
}
int cbg_fn_reduce_sum(cbg_function* f, cbg_value* x, const int* axes, int n_axes, cbg_value** v) { return reduce_op(f, "ReduceSum", CB_REDUCE_SUM, x, axes, n_axes, v); }
int cbg_fn_reduce_max(cbg_function* f, cbg_value* x, const int* axes, int n_axes, cbg_value** v) { return reduce_op(f, "ReduceMax", CB_REDUCE_MAX, x, axes, n_axes, v); }

// StandardOps.BroadcastInDim (standard_ops.go:232-254)
int cbg_fn_broadcast_in_dim(cbg_function* f, cbg_value* x, int32_t dtype, int rank, const int64_t* dims, const int* broadcast_axes, cbg_value** v) {
  const char* op = "BroadcastInDim";
  CB_TRY(check_fn(f, op));
  CB_TRY(check_values(f, op, {x}));
  if (dtype != x->shape.dtype) return fail(CB_ERR_INVALID_ARG, "%s: output dtype %s differs from the operand's %s", op, cb::dtype_name(dtype), cb::dtype_name(x->shape.dtype));
  Shape out;
  out.dtype = dtype;
  CB_TRY(make_dims(op, rank, dims, &out.dims));
  const int xr = (int)x->shape.dims.size();
  int prev = -1;
  std::vector<int32_t> axes(xr);
  for (int a = 0; a < xr; a++) {
    const int t = broadcast_axes[a];
    if (t <= prev || t >= rank) return fail(CB_ERR_INVALID_ARG, "%s: broadcastAxes must be increasing and inside the output rank %d", op, rank);
    if (x->shape.dims[a] != 1 && x->shape.dims[a] != out.dims[t])
      return fail(CB_ERR_INVALID_ARG, "%s: operand axis %d (%lld) cannot be broadcast into output axis %d (%lld)", op, a, (long long)x->shape.dims[a], t, (long long)out.dims[t]);
    axes[a] = t;
    prev = t;
  }
  cbg_value* n = add_node(f, N_BROADCAST, out, {x});
  n->axis_flags = axes;
  *v = n;
  return CB_OK;
}

// ---- collectives (CollectiveOps.AllReduce collectiveops.go:10-20; the AllGather the interface sketches, :31-32)
// Replica groups are indices into the device assignment, as DeviceMesh.ComputeReplicaGroups produces them
// (distributed/devicemesh.go:224-293).  No groups = one group of all replicas; otherwise every replica belongs to
// exactly one group.  Validated against the replica count at Compile.
static int copy_groups(const char* op, const int* groups_flat, const int* group_sizes, int n_groups, std::vector<std::vector<int>>* out) {
  out->clear();
  if (n_groups < 0 || (n_groups > 0 && (!groups_flat || !group_sizes))) return fail(CB_ERR_INVALID_ARG, "%s: replica groups are NULL", op);
  int k = 0;
  for (int g = 0; g < n_groups; g++) {
    if (group_sizes[g] < 1) return fail(CB_ERR_INVALID_ARG, "%s: replica group %d is empty", op, g);
    out->emplace_back(groups_flat + k, groups_flat + k + group_sizes[g]);
    k += group_sizes[g];
  }
  return CB_OK;
}

int cbg_fn_all_reduce(cbg_function* f, cbg_value* const* operands, int n_operands, int reduce_type, const int* groups_flat,
                      const int* group_sizes, int n_groups, cbg_value** outputs) {
  const char* op = "AllReduce";
  CB_TRY(check_fn(f, op));
  if (n_operands < 1 || !operands || !outputs) return fail(CB_ERR_INVALID_ARG, "%s: no operands", op);
  // compute.ReduceOpType: Undefined 0, Sum 1, Product 2, Max 3, Min 4 (standard_ops.go:65-84)
  if (reduce_type < 1 || reduce_type > 4) return fail(CB_ERR_INVALID_ARG, "%s: reduction type %d is undefined", op, reduce_type);
  std::vector<std::vector<int>> groups;
  CB_TRY(copy_groups(op, groups_flat, group_sizes, n_groups, &groups));
  for (int i = 0; i < n_operands; i++) {
    CB_TRY(check_values(f, op, {operands[i]}));
    CB_TRY(check_small_dtype(op, operands[i]));
  }
  for (int i = 0; i < n_operands; i++) {
    cbg_value* n = add_node(f, N_ALLREDUCE, operands[i]->shape, {operands[i]});
    n->op = reduce_type - 1;      // cb_reduce_op
    n->replica_groups = groups;
    outputs[i] = n;
  }
  return CB_OK;
}

int cbg_fn_all_gather(cbg_function* f, cbg_value* const* operands, int n_operands, int gather_axis, const int* groups_flat,
                      const int* group_sizes, int n_groups, cbg_value** outputs) {
  const char* op = "AllGather";
  CB_TRY(check_fn(f, op));
  if (n_operands < 1 || !operands || !outputs) return fail(CB_ERR_INVALID_ARG, "%s: no operands", op);
  std::vector<std::vector<int>> groups;
  CB_TRY(copy_groups(op, groups_flat, group_sizes, n_groups, &groups));
  for (size_t g = 1; g < groups.size(); g++)
    if (groups[g].size() != groups[0].size()) return fail(CB_ERR_INVALID_ARG, "%s: all replica groups must have the same size", op);
  for (int i = 0; i < n_operands; i++) {
    CB_TRY(check_values(f, op, {operands[i]}));
    const int rank = (int)operands[i]->shape.dims.size();
    if (gather_axis < 0 || gather_axis >= rank) return fail(CB_ERR_INVALID_ARG, "%s: gather axis %d out of range for rank %d", op, gather_axis, rank);
  }
  const int spmd = f->builder->spmd > 0 ? f->builder->spmd : 1;
  const int64_t gsize = groups.empty() ? spmd : (int64_t)groups[0].size();
  for (int i = 0; i < n_operands; i++) {
    Shape out = operands[i]->shape;
    out.dims[gather_axis] *= gsize;
    cbg_value* n = add_node(f, N_ALLGATHER, out, {operands[i]});
    n->op = gather_axis;
    n->replica_groups = groups;
    outputs[i] = n;
  }
  return CB_OK;
}

// Function.Parameter with a ShardingSpec (function.go:57; distributed/shardingspec.go:43-110): one entry per tensor
// axis, each a comma-separated list of mesh axis names ("" = replicated).  The spec is validated as
// ShardingSpec.Validate does (known mesh axes, none used twice) and kept with the parameter; under SPMD every
// replica is given its own shard, so the declared shape is the shard's.
int cbg_fn_parameter_sharded(cbg_function* f, const char* name, int32_t dtype, int rank, const int64_t* dims,
                             const char* const* mesh_axis_names, const int* mesh_axis_sizes, int n_mesh_axes,
                             const char* const* axis_specs, int n_axis_specs, cbg_value** v) {
  const char* op = "Parameter";
  cb::clear_error();
  if (n_mesh_axes < 0 || n_axis_specs < 0 || (n_mesh_axes > 0 && (!mesh_axis_names || !mesh_axis_sizes)) || (n_axis_specs > 0 && !axis_specs))
    return fail(CB_ERR_INVALID_ARG, "%s: sharding spec is NULL", op);
  if (n_axis_specs > rank) return fail(CB_ERR_INVALID_ARG, "%s: ShardingSpec has %d axes, the parameter has rank %d", op, n_axis_specs, rank);
  std::vector<bool> used(n_mesh_axes, false);
  std::string text;                 // per tensor axis its mesh axes joined by ',', tensor axes joined by ';'
  bool sharded = false;
  for (int a = 0; a < n_axis_specs; a++) {
    std::stringstream ss(axis_specs[a] ? axis_specs[a] : "");
    std::string nm;
    if (a) text += ";";
    bool first = true;
    while (std::getline(ss, nm, ',')) {
      if (nm.empty()) continue;
      int idx = -1;
      for (int m = 0; m < n_mesh_axes; m++) if (nm == mesh_axis_names[m]) idx = m;
      if (idx < 0) return fail(CB_ERR_INVALID_ARG, "ShardingSpec axis #%d refers to unknown mesh axis \"%s\"", a, nm.c_str());
      if (used[idx]) return fail(CB_ERR_INVALID_ARG, "mesh axis \"%s\" used more than once in ShardingSpec", nm.c_str());
      used[idx] = true;
      text += (first ? "" : ",") + nm;
      first = false;
      sharded = true;
    }
  }
  CB_TRY(cbg_fn_parameter(f, name, dtype, rank, dims, v));
  (*v)->sharding = sharded ? text : "replicated";
  return CB_OK;
}

int cbg_exec_input_sharding(const cbg_exec* e, int i, char* buf, size_t n) {
  cb::clear_error();
  if (!e || !buf || n == 0 || i < 0 || i >= (int)e->fn->params.size()) return fail(CB_ERR_INVALID_ARG, "Executable.Inputs: index %d out of range", i);
  snprintf(buf, n, "%s", e->fn->params[i]->sharding.c_str());
  return CB_OK;
}

int cbg_fn_not_implemented(cbg_function* f, const char* op_name) {
  cb::clear_error();
  return fail(CB_ERR_NOT_IMPLEMENTED, "%s: not implemented by the cuda backend", op_name ? op_name : "op");
}

}  // extern "C"

// ---------------------------------------------------------------- Compile
namespace {

// the value of a one-element float constant, or false
bool scalar_constant(const cbg_value* v, double* out) {
  while (v->kind == N_RESHAPE || v->kind == N_BROADCAST) v = v->inputs[0];
  if (v->kind != N_CONST || v->shape.size() != 1) return false;
  const uint8_t* d = v->const_data.data();
  switch (v->shape.dtype) {
    case CB_F32: { float f; memcpy(&f, d, 4); *out = f; return true; }
    case CB_F64: { double f; memcpy(&f, d, 8); *out = f; return true; }
    case CB_BF16: { uint16_t h; memcpy(&h, d, 2); uint32_t b = (uint32_t)h << 16; float f; memcpy(&f, &b, 4); *out = f; return true; }
    default: return false;
  }
}

const cbg_value* through_reshape(const cbg_value* v) {
  while (v->kind == N_RESHAPE) v = v->inputs[0];
  return v;
}

// The decomposed RMS norm a caller of this interface writes (it has no fused one: FusedLayerNorm is mean-centred,
// internal/gobackend/fusedops/layernorm.go:102-137):
//     x * Reshape(Rsqrt(ReduceSum(x * x, last axis) * (1/H) + eps), [..., 1])  [ * gamma reshaped to [1..., H] ]
// with either operand order in every product and sum, or Div by H instead of Mul by 1/H.  Matches at the last
// product; returns x, gamma (or null) and eps.
bool match_rms_core(const cbg_value* n, const cbg_value** x_out, double* eps_out) {
  if (n->kind != N_BINARY || n->op != CB_BIN_MUL) return false;
  for (int o = 0; o < 2; o++) {
    const cbg_value* x = n->inputs[o];
    const cbg_value* rr = n->inputs[1 - o];
    if (x->shape.dims.empty()) continue;
    const int64_t H = x->shape.dims.back();
    std::vector<int64_t> want = x->shape.dims;
    want.back() = 1;
    if (rr->shape.dims != want) continue;
    const cbg_value* r = through_reshape(rr);
    if (r->kind != N_UNARY || r->op != CB_UN_RSQRT) continue;
    const cbg_value* me = r->inputs[0];
    if (me->kind != N_BINARY || me->op != CB_BIN_ADD) continue;
    for (int a = 0; a < 2; a++) {
      double eps = 0.0;
      if (!scalar_constant(me->inputs[1 - a], &eps)) continue;
      const cbg_value* ms = me->inputs[a];
      if (ms->kind != N_BINARY) continue;
      const cbg_value* ss = nullptr;
      double c = 0.0;
      if (ms->op == CB_BIN_MUL) {
        for (int b = 0; b < 2 && !ss; b++)
          if (scalar_constant(ms->inputs[1 - b], &c) && std::abs(c * (double)H - 1.0) < 1e-3) ss = ms->inputs[b];
      } else if (ms->op == CB_BIN_DIV) {
        if (scalar_constant(ms->inputs[1], &c) && std::abs(c - (double)H) < 1e-3 * (double)H) ss = ms->inputs[0];
      }
      if (!ss) continue;
      ss = through_reshape(ss);
      if (ss->kind != N_REDUCE || ss->op != CB_REDUCE_SUM) continue;
      const cbg_value* sq = ss->inputs[0];
      const int rank = (int)sq->shape.dims.size();
      bool last_only = rank >= 1;
      for (int d = 0; d < rank; d++) if ((ss->axis_flags[d] != 0) != (d == rank - 1)) last_only = false;
      if (!last_only) continue;
      if (sq->kind != N_BINARY || sq->op != CB_BIN_MUL || sq->inputs[0] != x || sq->inputs[1] != x) continue;
      *x_out = x;
      *eps_out = eps;
      return true;
    }
  }
  return false;
}

// Rewrites matching products into N_RMSNORM nodes (the nodes they replace become dead unless something else uses them).
void fuse_rms_norms(cbg_function* f) {
  // consumers first: the product with gamma is seen before the normalisation it scales
  for (size_t ni = f->nodes.size(); ni-- > 0;) {
    cbg_value* n = f->nodes[ni].get();
    const cbg_value* x = nullptr;
    double eps = 0.0;
    if (n->kind != N_BINARY || n->op != CB_BIN_MUL) continue;
    // with gamma: (x * rr) * g, g of H elements laid out along the last axis
    bool done = false;
    for (int o = 0; o < 2 && !done; o++) {
      cbg_value* core = n->inputs[o];
      cbg_value* g = n->inputs[1 - o];
      if (!match_rms_core(core, &x, &eps)) continue;
      const int64_t H = x->shape.dims.back();
      bool g_ok = g->shape.dtype == x->shape.dtype && g->shape.size() == H && !g->shape.dims.empty() && g->shape.dims.back() == H;
      if (!g_ok) continue;
      n->kind = N_RMSNORM;
      n->inputs = {const_cast<cbg_value*>(x), g};
      n->epsilon = eps;
      n->flags = 1;
      done = true;
    }
    if (done) continue;
    if (match_rms_core(n, &x, &eps)) {
      n->kind = N_RMSNORM;
      n->inputs = {const_cast<cbg_value*>(x)};
      n->epsilon = eps;
      n->flags = 0;
    }
  }
}

int check_replica_groups(const cbg_value* n, int replicas, const char* op) {
  std::vector<bool> seen(replicas, false);
  if (n->replica_groups.empty()) return CB_OK;
  for (const auto& g : n->replica_groups)
    for (int r : g) {
      if (r < 0 || r >= replicas) return fail(CB_ERR_INVALID_ARG, "%s: replica %d out of range for %d devices", op, r, replicas);
      if (seen[r]) return fail(CB_ERR_INVALID_ARG, "%s: replica %d appears in more than one replica group", op, r);
      seen[r] = true;
    }
  for (int r = 0; r < replicas; r++)
    if (!seen[r]) return fail(CB_ERR_INVALID_ARG, "%s: replica %d belongs to no replica group", op, r);
  return CB_OK;
}

bool same_decode_group(const cb_qdense_desc& a, const cb_qdense_desc& b) {
  return a.M == b.M && a.K == b.K && a.x_dtype == b.x_dtype && a.w_dtype == b.w_dtype && a.scale_layout == b.scale_layout &&
         (a.scale_layout == CB_SCALE_CHANNEL || a.block_size == b.block_size);
}

int build_dev_plans(cbg_exec* e, int dev, DevPlans* dp) {
  cbg_function* f = e->fn.get();
  const size_t nn = f->nodes.size();
  dp->plans.assign(nn, nullptr);
  dp->ws_bytes.assign(nn, 0);
  int st = CB_OK;
  for (size_t i = 0; i < nn && st == CB_OK; i++) {
    cbg_value* n = f->nodes[i].get();
    if (!e->live[i]) continue;
    cb_plan* p = nullptr;
    switch (n->kind) {
      case N_DOT: st = cb_plan_dot(dev, &n->dot, &p); break;
      case N_QDENSE:
        if (e->group_of[i] >= 0) {
          const std::vector<int>& members = e->groups[e->group_of[i]];
          if (members[0] != (int)i) break;                 // launched with the first member
          std::vector<cb_qdense_member> ms;
          for (int m : members) {
            const cb_qdense_desc& d = f->nodes[m]->qd;
            cb_qdense_member mm;
            mm.N = d.N; mm.has_bias = d.has_bias; mm.activation = d.activation;
            ms.push_back(mm);
          }
          st = cb_plan_qdense_group(dev, &n->qd, ms.data(), (int)ms.size(), &p);
        } else {
          st = cb_plan_qdense(dev, &n->qd, &p);
        }
        break;
      case N_SDPA: st = cb_plan_sdpa(dev, &n->sdpa, &p); break;
      case N_SLICE:
        st = cb_plan_slice(dev, n->shape.dtype, (int)n->inputs[0]->shape.dims.size(), n->inputs[0]->shape.dims.data(),
                           n->starts.data(), n->limits.data(), n->strides.data(), &p);
        break;
      case N_IOTA: st = cb_plan_iota(dev, n->shape.dtype, (int)n->shape.dims.size(), n->shape.dims.data(), n->axis, &p); break;
      case N_CONVERT: st = cb_plan_convert(dev, n->inputs[0]->shape.dtype, n->shape.dtype, n->shape.size(), &p); break;
      case N_GELU: st = cb_plan_gelu(dev, n->shape.dtype, n->shape.size(), n->flags, &p); break;
      case N_SOFTMAX: st = cb_plan_softmax(dev, n->shape.dtype, n->small_dims[0], n->small_dims[1], n->small_dims[2], &p); break;
      case N_COLS_BIAS:
        st = cb_plan_cols_bias(dev, n->shape.dtype, n->small_dims[0], n->small_dims[1], n->small_dims[2], n->small_dims[3], n->flags & 1, &p);
        break;
      case N_LAYERNORM:
        st = cb_plan_layernorm(dev, n->shape.dtype, n->small_dims[0], n->small_dims[1], n->epsilon, n->flags & 1, (n->flags & 2) ? 1 : 0, &p);
        break;
      case N_TRANSPOSE:
        st = cb_plan_transpose(dev, n->shape.dtype, (int)n->inputs[0]->shape.dims.size(), n->inputs[0]->shape.dims.data(), n->perm.data(), &p);
        break;
      case N_BINARY: {
        // both operands with the rank of the result (a scalar as all ones)
        const int r = (int)n->shape.dims.size();
        std::vector<int64_t> l(std::max(r, 1), 1), rr(std::max(r, 1), 1);
        if (!n->inputs[0]->shape.dims.empty()) l = n->inputs[0]->shape.dims;
        if (!n->inputs[1]->shape.dims.empty()) rr = n->inputs[1]->shape.dims;
        st = cb_plan_binary(dev, n->op, n->shape.dtype, r, l.data(), rr.data(), &p);
        break;
      }
      case N_UNARY: st = cb_plan_unary(dev, n->op, n->shape.dtype, n->shape.size(), &p); break;
      case N_REDUCE:
        st = cb_plan_reduce(dev, n->op, n->shape.dtype, (int)n->inputs[0]->shape.dims.size(), n->inputs[0]->shape.dims.data(), n->axis_flags.data(), &p);
        break;
      case N_BROADCAST:
        st = cb_plan_broadcast_in_dim(dev, n->shape.dtype, (int)n->inputs[0]->shape.dims.size(), n->inputs[0]->shape.dims.data(),
                                      (int)n->shape.dims.size(), n->shape.dims.data(), n->axis_flags.data(), &p);
        break;
      case N_RMSNORM: {
        const int64_t H = n->shape.dims.back();
        st = cb_plan_rms_norm(dev, n->shape.dtype, H ? n->shape.size() / H : 0, H, n->epsilon, n->flags & 1, &p);
        break;
      }
      case N_EMBEDDING:
        st = cb_plan_embedding_lookup(dev, n->inputs[0]->shape.dims[0], n->inputs[0]->shape.dims[1], n->inputs[1]->shape.size(),
                                      n->inputs[1]->shape.dtype, n->axis, &p);
        break;
      default: break;      // parameters, constants, reshapes, collectives
    }
    if (st == CB_OK && p) {
      dp->plans[i] = p;
      cb_plan_workspace_bytes(p, &dp->ws_bytes[i]);
    }
  }
  if (st != CB_OK) {
    for (cb_plan* p : dp->plans) if (p) cb_plan_destroy(p);
    dp->plans.clear();
  }
  return st;
}

}  // namespace

extern "C" {

int cbg_builder_compile(cbg_builder* bld, cbg_exec** exec) {
  cb::clear_error();
  if (!bld || !exec) return fail(CB_ERR_INVALID_ARG, "Builder.Compile: NULL argument");
  *exec = nullptr;
  if (bld->compiled || !bld->main) return fail(CB_ERR_INVALID_ARG, "Builder.Compile: builder %s was already compiled", bld->name.c_str());
  if (bld->be->finalized.load()) return fail(CB_ERR_INVALID_ARG, "Builder.Compile: backend has been finalized");
  cbg_function* f = bld->main.get();
  if (!f->returned) return fail(CB_ERR_INVALID_ARG, "Builder.Compile: Main function of %s has no Return", bld->name.c_str());
  auto e = std::make_unique<cbg_exec>();
  e->be = bld->be;
  e->name = bld->name;
  e->replicas = bld->spmd > 0 ? bld->spmd : 1;
  e->assignment = bld->assignment;
  if (e->assignment.empty()) for (int i = 0; i < e->replicas; i++) e->assignment.push_back(i);
  if ((int)e->assignment.size() != e->replicas)
    return fail(CB_ERR_INVALID_ARG, "Builder.Compile: device assignment has %zu devices, %d replicas requested", e->assignment.size(), e->replicas);
  for (size_t a = 0; a < e->assignment.size(); a++)
    for (size_t b = a + 1; b < e->assignment.size(); b++)
      if (e->assignment[a] == e->assignment[b]) return fail(CB_ERR_INVALID_ARG, "Builder.Compile: device %d assigned twice", e->assignment[a]);
  const size_t nn = f->nodes.size();
  for (size_t i = 0; i < nn; i++) {
    const cbg_value* n = f->nodes[i].get();
    if (n->kind == N_ALLREDUCE) CB_TRY(check_replica_groups(n, e->replicas, "AllReduce"));
    if (n->kind == N_ALLGATHER) {
      CB_TRY(check_replica_groups(n, e->replicas, "AllGather"));
      const int64_t gsize = n->replica_groups.empty() ? e->replicas : (int64_t)n->replica_groups[0].size();
      if (n->shape.dims[n->op] != n->inputs[0]->shape.dims[n->op] * gsize)
        return fail(CB_ERR_INVALID_ARG, "AllGather: the result shape was inferred for %lld replicas per group; call DistributedSPMD before building the op",
                    (long long)(n->inputs[0]->shape.dims[n->op] ? n->shape.dims[n->op] / n->inputs[0]->shape.dims[n->op] : 0));
    }
  }
  // ---- graph passes: the decomposed RMS norm becomes one row kernel; values nobody needs are not computed
  fuse_rms_norms(f);
  e->live.assign(nn, 0);
  for (cbg_value* o : f->outputs) e->live[o->index] = 1;
  for (size_t i = nn; i-- > 0;)
    if (e->live[i]) for (cbg_value* in : f->nodes[i]->inputs) e->live[in->index] = 1;
  for (cbg_value* prm : f->params) e->live[prm->index] = 1;
  // ---- independent decode-shaped FusedQuantizedDense nodes of one shape family become one grouped launch: a node
  // joins the open group when all its operands were already available where the group's first member stands.
  e->group_of.assign(nn, -1);
  if (!e->be->fallback_only) {
    std::vector<int> open;         // open groups (indices into e->groups)
    for (size_t i = 0; i < nn; i++) {
      cbg_value* n = f->nodes[i].get();
      if (!e->live[i] || n->kind != N_QDENSE) continue;
      cb_plan* probe = nullptr;
      if (cb_plan_qdense(0, &n->qd, &probe) != CB_OK) { cb::clear_error(); continue; }
      const bool decode_tc = std::string(cb_plan_kernel_name(probe)).rfind("qdense_decode_tc_", 0) == 0;
      cb_plan_destroy(probe);
      if (!decode_tc) continue;
      int joined = -1;
      for (int gi : open) {
        std::vector<int>& members = e->groups[gi];
        const cbg_value* first = f->nodes[members[0]].get();
        if ((int)members.size() >= CB_QDENSE_GROUP_MAX || !same_decode_group(first->qd, n->qd)) continue;
        bool ready = true;
        for (const cbg_value* in : n->inputs) {
          const cbg_value* root = through_reshape(in);       // parameters and constants exist from the start
          if (root->kind != N_PARAM && root->kind != N_CONST && in->index >= first->index) ready = false;
        }
        if (!ready) continue;
        joined = gi;
        break;
      }
      if (joined >= 0) { e->groups[joined].push_back((int)i); e->group_of[i] = joined; }
      else { e->groups.push_back({(int)i}); e->group_of[i] = (int)e->groups.size() - 1; open.push_back(e->group_of[i]); }
    }
    for (size_t gi = 0; gi < e->groups.size(); gi++)      // a group of one is an ordinary plan
      if (e->groups[gi].size() == 1) e->group_of[e->groups[gi][0]] = -1;
  }
  e->fn = std::move(bld->main);
  // plans for every assigned device (a plan carries its device: launches make that device current)
  int st = CB_OK;
  for (int dev : e->assignment) {
    st = build_dev_plans(e.get(), dev, &e->dev_plans[dev]);
    if (st != CB_OK) break;
  }
  if (st != CB_OK) {
    for (auto& kv : e->dev_plans) for (cb_plan* p : kv.second.plans) if (p) cb_plan_destroy(p);
    bld->main = std::move(e->fn);
    return st;
  }
  bld->compiled = true;
  *exec = e.release();
  return CB_OK;
}

// ---------------------------------------------------------------- Executable
int cbg_exec_num_inputs(const cbg_exec* e) { return e ? (int)e->fn->params.size() : 0; }
int cbg_exec_num_outputs(const cbg_exec* e) { return e ? (int)e->fn->outputs.size() : 0; }

int cbg_exec_input_info(const cbg_exec* e, int i, char* name, size_t name_len, int32_t* dtype, int* rank, int64_t* dims) {
  cb::clear_error();
  if (!e || i < 0 || i >= (int)e->fn->params.size()) return fail(CB_ERR_INVALID_ARG, "Executable.Inputs: index %d out of range", i);
  const cbg_value* p = e->fn->params[i];
  if (name && name_len) snprintf(name, name_len, "%s", p->name.c_str());
  return out_shape(p, dtype, rank, dims);
}

int cbg_exec_output_info(const cbg_exec* e, int i, int32_t* dtype, int* rank, int64_t* dims) {
  cb::clear_error();
  if (!e || i < 0 || i >= (int)e->fn->outputs.size()) return fail(CB_ERR_INVALID_ARG, "Executable.Outputs: index %d out of range", i);
  return out_shape(e->fn->outputs[i], dtype, rank, dims);
}

int cbg_exec_kernel_names(const cbg_exec* e, char* buf, size_t n) {
  cb::clear_error();
  if (!e || !buf || n == 0) return fail(CB_ERR_INVALID_ARG, "NULL argument");
  std::string s;
  auto it = e->dev_plans.find(e->assignment[0]);
  if (it != e->dev_plans.end())
    for (size_t i = 0; i < it->second.plans.size(); i++) {
      const cbg_value* nd = e->fn->nodes[i].get();
      if (it->second.plans[i]) { s += cb_plan_kernel_name(it->second.plans[i]); s += "\n"; }
      else if (e->live[i] && nd->kind == N_ALLREDUCE) s += "all_reduce\n";
      else if (e->live[i] && nd->kind == N_ALLGATHER) s += "all_gather\n";
    }
  snprintf(buf, n, "%s", s.c_str());
  return CB_OK;
}

int cbg_exec_graph_replays(cbg_exec* e) {
  if (!e) return 0;
  std::lock_guard<std::mutex> l(e->mu);
  return e->graph_replays;
}

int cbg_exec_last_trace(cbg_exec* e, char* buf, size_t n) {
  cb::clear_error();
  if (!e || !buf || n == 0) return fail(CB_ERR_INVALID_ARG, "NULL argument");
  std::lock_guard<std::mutex> l(e->mu);
  snprintf(buf, n, "%s", e->last_trace.c_str());
  return CB_OK;
}

}  // extern "C"

namespace {

// One replica of an Execute call.
struct Replica {
  int dev = 0;
  DevicePool* pool = nullptr;
  const DevPlans* dp = nullptr;
  cb_stream stream = nullptr;
  std::vector<void*> consts, ws, mem;
  std::vector<char> owned, taken;
  std::vector<std::pair<size_t, void*>> scratch;      // pool memory to give back after the final sync
  std::vector<cb_event> events;
  std::vector<std::pair<int, cb_event>> marks;        // tracing: (node, event recorded after its launch); node -1 = start
  cbg_buffer* const* inputs = nullptr;
  const uint8_t* donate = nullptr;
  std::vector<cbg_buffer*> outs;
};

int setup_replica(cbg_exec* e, Replica& r) {
  cbg_function* f = e->fn.get();
  const size_t nn = f->nodes.size();
  r.pool = e->be->pools[r.dev].get();
  {
    std::lock_guard<std::mutex> l(e->mu);
    auto pit = e->dev_plans.find(r.dev);
    if (pit == e->dev_plans.end()) {                    // a device chosen at Execute (defaultDevice) rather than at Compile
      DevPlans dp;
      CB_TRY(build_dev_plans(e, r.dev, &dp));
      pit = e->dev_plans.emplace(r.dev, std::move(dp)).first;
    }
    r.dp = &pit->second;
    auto it = e->const_dev.find(r.dev);
    if (it == e->const_dev.end()) {
      std::vector<void*> c(nn, nullptr);
      int st = CB_OK;
      for (size_t i = 0; i < nn && st == CB_OK; i++) {
        cbg_value* n = f->nodes[i].get();
        if (n->kind != N_CONST || !e->live[i]) continue;
        st = cb_alloc(r.dev, n->const_data.size(), &c[i]);
        if (st == CB_OK) st = cb_h2d(r.dev, c[i], n->const_data.data(), n->const_data.size(), nullptr);
      }
      if (st != CB_OK) { for (void* p : c) if (p) cb_free(r.dev, p); return st; }
      it = e->const_dev.emplace(r.dev, std::move(c)).first;
    }
    r.consts = it->second;
    auto& idle = e->idle_ws[r.dev];
    if (!idle.empty()) { r.ws = std::move(idle.back()); idle.pop_back(); }
  }
  if (r.ws.empty()) {
    r.ws.assign(nn, nullptr);
    int st = CB_OK;
    for (size_t i = 0; i < nn && st == CB_OK; i++) {
      if (!r.dp->plans[i] || r.dp->ws_bytes[i] == 0) continue;
      st = cb_alloc(r.dev, r.dp->ws_bytes[i], &r.ws[i]);
      if (st == CB_OK) st = cb_plan_prepare_workspace(r.dp->plans[i], r.ws[i], nullptr);
    }
    if (st == CB_OK) st = cb_stream_sync(r.dev, nullptr);
    if (st != CB_OK) { for (void* p : r.ws) if (p) cb_free(r.dev, p); r.ws.clear(); return st; }
  }
  CB_TRY(e->be->get_stream(r.dev, &r.stream));
  r.mem.assign(nn, nullptr);
  r.owned.assign(nn, 0);
  r.taken.assign(nn, 0);
  // parameters and constants exist from the start (a grouped launch may read operands declared after its first member)
  for (size_t i = 0; i < nn; i++) {
    const cbg_value* n = f->nodes[i].get();
    if (n->kind == N_PARAM) r.mem[i] = r.inputs[n->param_index]->ptr;
    else if (n->kind == N_CONST) r.mem[i] = r.consts[i];
  }
  return CB_OK;
}

// the memory of an operand; a Reshape shares its operand's
void* operand_ptr(const Replica& r, const cbg_value* v) {
  while (v->kind == N_RESHAPE) v = v->inputs[0];
  return r.mem[v->index];
}

int new_event(Replica& r, cb_event* ev) {
  CB_TRY(cb_event_create(r.dev, ev));
  r.events.push_back(*ev);
  return CB_OK;
}

// AllReduce / AllGather over the replicas of one Execute call (one process drives all devices): every member of a
// group pulls the operands of its peers with peer copies on its own stream, after an event that says the operand
// is ready, and reduces them in group order (so all members end with the same bits).  Operand buffers stay alive
// until the final sync of the call.
int run_collective(cbg_exec* e, cbg_value* n, std::vector<Replica>& reps) {
  const size_t idx = (size_t)n->index;
  const int in_idx = n->inputs[0]->index;
  const size_t bytes = n->inputs[0]->shape.bytes();
  std::vector<std::vector<int>> groups = n->replica_groups;
  if (groups.empty()) { groups.emplace_back(); for (int r = 0; r < (int)reps.size(); r++) groups[0].push_back(r); }
  std::vector<cb_event> ready(reps.size(), nullptr);
  for (size_t r = 0; r < reps.size(); r++) {
    CB_TRY(new_event(reps[r], &ready[r]));
    CB_TRY(cb_event_record(reps[r].dev, ready[r], reps[r].stream));
    CB_TRY(reps[r].pool->get(reps[r].dev, n->shape.bytes(), &reps[r].mem[idx]));
    reps[r].owned[idx] = 1;
  }
  for (const auto& g : groups) {
    const int gs = (int)g.size();
    for (int d : g) {
      Replica& me = reps[d];
      for (int src : g) if (src != d) CB_TRY(cb_stream_wait_event(me.dev, me.stream, ready[src]));
      if (n->kind == N_ALLREDUCE) {
        void* stack = nullptr;
        CB_TRY(me.pool->get(me.dev, bytes * gs, &stack));
        me.scratch.emplace_back(bytes * gs, stack);
        for (int k = 0; k < gs; k++)
          CB_TRY(cb_d2d(me.dev, (uint8_t*)stack + (size_t)k * bytes, reps[g[k]].dev, reps[g[k]].mem[in_idx], bytes, me.stream));
        CB_TRY(cb::set_device(me.dev));
        CB_TRY(cb::stacked_reduce_launch(n->shape.dtype, n->op, stack, gs, n->shape.size(), me.mem[idx], (cudaStream_t)me.stream));
      } else {
        // out viewed as [outer, group, chunk]: member k's operand fills [:, k, :]
        const Shape& is = n->inputs[0]->shape;
        int64_t outer = 1, chunk = cb::dtype_size(is.dtype);
        for (int a = 0; a < n->op; a++) outer *= is.dims[a];
        for (size_t a = (size_t)n->op; a < is.dims.size(); a++) chunk *= is.dims[a];
        for (int k = 0; k < gs; k++) {
          const Replica& src = reps[g[k]];
          if (outer == 1 || chunk == 0) {
            CB_TRY(cb_d2d(me.dev, (uint8_t*)me.mem[idx] + (size_t)k * chunk, src.dev, src.mem[in_idx], (size_t)chunk, me.stream));
          } else {
            CB_TRY(cb::set_device(me.dev));
            cudaMemcpy3DPeerParms pr;
            memset(&pr, 0, sizeof(pr));
            pr.srcDevice = src.dev;
            pr.dstDevice = me.dev;
            pr.srcPtr = make_cudaPitchedPtr(src.mem[in_idx], (size_t)chunk, (size_t)chunk, (size_t)outer);
            pr.dstPtr = make_cudaPitchedPtr((uint8_t*)me.mem[idx] + (size_t)k * chunk, (size_t)chunk * gs, (size_t)chunk * gs, (size_t)outer);
            pr.extent = make_cudaExtent((size_t)chunk, (size_t)outer, 1);
            CB_CUDA(cudaMemcpy3DPeerAsync(&pr, (cudaStream_t)me.stream));
          }
        }
      }
    }
  }
  return CB_OK;
}

int launch_node(cbg_exec* e, Replica& r, size_t i) {
  cbg_function* f = e->fn.get();
  cbg_value* n = f->nodes[i].get();
  switch (n->kind) {
    case N_PARAM: r.mem[i] = r.inputs[n->param_index]->ptr; return CB_OK;
    case N_CONST: r.mem[i] = r.consts[i]; return CB_OK;
    case N_RESHAPE: r.mem[i] = r.mem[n->inputs[0]->index]; return CB_OK;     // same bytes, new shape
    default: break;
  }
  if (n->kind == N_QDENSE && e->group_of[i] >= 0) {
    const std::vector<int>& members = e->groups[e->group_of[i]];
    if (members[0] != (int)i) return CB_OK;       // computed by the first member's launch
    std::vector<const void*> in;
    std::vector<void*> out;
    for (int m : members) {
      if (!r.mem[m]) {                            // (a graph instance brings its own memory)
        CB_TRY(r.pool->get(r.dev, f->nodes[m]->shape.bytes(), &r.mem[m]));
        r.owned[m] = 1;
      }
      for (const cbg_value* v : f->nodes[m]->inputs) in.push_back(operand_ptr(r, v));
      out.push_back(r.mem[m]);
    }
    return cb_launch(r.dp->plans[i], in.data(), (int)in.size(), out.data(), (int)out.size(), r.ws[i], r.stream);
  }
  if (!r.mem[i]) {
    CB_TRY(r.pool->get(r.dev, n->shape.bytes(), &r.mem[i]));
    r.owned[i] = 1;
  }
  const void* in[8];
  for (size_t k = 0; k < n->inputs.size(); k++) in[k] = operand_ptr(r, n->inputs[k]);
  void* out[1] = {r.mem[i]};
  // a kernel launch with zero elements is skipped inside cb_launch
  return cb_launch(r.dp->plans[i], in, (int)n->inputs.size(), out, 1, r.ws[i], r.stream);
}

int collect_outputs(cbg_exec* e, Replica& r) {
  cbg_function* f = e->fn.get();
  // results that must be copied (a replayed graph keeps its own memory; an output that is also a parameter) leave
  // together in one launch when there are several and their sizes allow 16-byte vectors
  std::vector<void*> cp_dst;
  std::vector<const void*> cp_src;
  std::vector<size_t> cp_bytes;
  int n_copies = 0;
  bool vectors = true;
  for (size_t o = 0; o < f->outputs.size(); o++) {
    const cbg_value* root = f->outputs[o];
    while (root->kind == N_RESHAPE) root = root->inputs[0];
    const bool donated_param = root->kind == N_PARAM && r.donate && r.donate[root->param_index];
    if (!(r.owned[root->index] || donated_param)) { n_copies++; vectors = vectors && f->outputs[o]->shape.bytes() % 16 == 0; }
  }
  const bool batch = n_copies >= 2 && n_copies <= cb::copy_many_max() && vectors;
  for (size_t o = 0; o < f->outputs.size(); o++) {
    cbg_value* n = f->outputs[o];
    // root of the aliasing chain (Reshape shares memory with its operand)
    cbg_value* root = n;
    while (root->kind == N_RESHAPE) root = root->inputs[0];
    auto buf = std::make_unique<cbg_buffer>();
    buf->be = e->be;
    buf->dev = r.dev;
    buf->shape = n->shape;
    const int ri = root->index;
    const bool donated_param = root->kind == N_PARAM && r.donate && r.donate[root->param_index];
    if ((r.owned[ri] || donated_param) && !r.taken[ri]) {
      buf->ptr = r.mem[ri];              // hand the memory over
      r.taken[ri] = 1;
    } else {
      CB_TRY(r.pool->get(r.dev, n->shape.bytes(), &buf->ptr));
      if (batch && n->shape.bytes() > 0 && (int)cp_dst.size() < cb::copy_many_max() && !((reinterpret_cast<uintptr_t>(buf->ptr) | reinterpret_cast<uintptr_t>(r.mem[ri])) & 15)) {
        cp_dst.push_back(buf->ptr); cp_src.push_back(r.mem[ri]); cp_bytes.push_back(n->shape.bytes());
      } else {
        int st = cb_d2d(r.dev, buf->ptr, r.dev, r.mem[ri], n->shape.bytes(), r.stream);
        if (st != CB_OK) { r.pool->put(n->shape.bytes(), buf->ptr); return st; }
      }
    }
    r.outs.push_back(buf.release());
  }
  if (!cp_dst.empty()) {
    CB_TRY(cb::set_device(r.dev));
    CB_TRY(cb::copy_many(cb::sm_count(r.dev), (int)cp_dst.size(), cp_dst.data(), cp_src.data(), cp_bytes.data(), (cudaStream_t)r.stream));
  }
  return CB_OK;
}


// ---------------------------------------------------------------- replay as a CUDA graph
bool graph_eligible(cbg_exec* e, const uint8_t* donate, int n_inputs) {
  if (e->replicas != 1 || e->be->trace || e->be->no_graphs || e->graphs_off) return false;
  if (donate) for (int i = 0; i < n_inputs; i++) if (donate[i]) return false;      // donation changes who owns the buffers
  cbg_function* f = e->fn.get();
  for (size_t i = 0; i < f->nodes.size(); i++) {
    if (!e->live[i]) continue;
    const NodeKind k = f->nodes[i]->kind;
    if (k == N_ALLREDUCE || k == N_ALLGATHER || k == N_EMBEDDING) return false;     // (the lookup reports through status words)
  }
  return true;
}

void graph_instance_free(cbg_exec::GraphInstance* g) {
  if (g->exec) cudaGraphExecDestroy(g->exec);
  for (void* p : g->owned_mem) if (p) cb_free(g->dev, p);
  for (void* p : g->ws) if (p) cb_free(g->dev, p);
  g->exec = nullptr; g->owned_mem.clear(); g->ws.clear(); g->mem.clear();
}

// Captures one pass over the nodes into a graph whose every buffer belongs to the instance.  On any failure the
// executable stays on the plain path for good (graphs_off) and the caller carries on there.
int graph_build(cbg_exec* e, cbg_exec::GraphInstance* g, cbg_buffer* const* inputs) {
  cbg_function* f = e->fn.get();
  const size_t nn = f->nodes.size();
  Replica r;
  r.dev = g->dev;
  r.inputs = inputs;
  CB_TRY(setup_replica(e, r));
  g->ws = std::move(r.ws);                      // stay with the instance: the kernels' parameters point into them
  r.ws = g->ws;
  int st = CB_OK;
  for (size_t i = 0; i < nn && st == CB_OK; i++) {
    const cbg_value* n = f->nodes[i].get();
    if (!e->live[i] || n->kind == N_PARAM || n->kind == N_CONST || n->kind == N_RESHAPE) continue;
    void* p = nullptr;
    st = cb_alloc(r.dev, std::max<size_t>(n->shape.bytes(), 16), &p);
    if (st == CB_OK) { r.mem[i] = p; g->owned_mem.push_back(p); }
  }
  cudaGraph_t graph = nullptr;
  bool capturing = false;
  if (st == CB_OK) {
    if (cudaStreamBeginCapture((cudaStream_t)r.stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) capturing = true;
    else st = fail(CB_ERR_CUDA, "graph capture could not begin");
  }
  for (size_t i = 0; i < nn && st == CB_OK; i++)
    if (e->live[i]) st = launch_node(e, r, i);
  if (capturing) {
    const cudaError_t ce = cudaStreamEndCapture((cudaStream_t)r.stream, &graph);
    if (ce != cudaSuccess || !graph) { if (st == CB_OK) st = fail(CB_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(ce)); }
  }
  if (st == CB_OK && cudaGraphInstantiate(&g->exec, graph, 0) != cudaSuccess) st = fail(CB_ERR_CUDA, "graph instantiation failed");
  if (graph) cudaGraphDestroy(graph);
  cudaGetLastError();                           // a failed capture leaves a sticky-looking error behind; it is not one
  e->be->put_stream(r.dev, r.stream);
  if (st != CB_OK) { graph_instance_free(g); return st; }
  g->mem = r.mem;
  return CB_OK;
}

// One Execute through an instance: launch, copy the results into fresh buffers, sync.
int graph_replay(cbg_exec* e, cbg_exec::GraphInstance* g, cbg_buffer* const* inputs, cbg_buffer** outputs) {
  cbg_function* f = e->fn.get();
  const size_t nn = f->nodes.size();
  Replica r;
  r.dev = g->dev;
  r.pool = e->be->pools[r.dev].get();
  r.inputs = inputs;
  r.mem = g->mem;
  r.owned.assign(nn, 0);
  r.taken.assign(nn, 0);
  {
    std::lock_guard<std::mutex> l(e->mu);
    r.dp = &e->dev_plans.find(r.dev)->second;
  }
  CB_TRY(e->be->get_stream(r.dev, &r.stream));
  const auto t_start = std::chrono::steady_clock::now();
  int st = cudaGraphLaunch(g->exec, (cudaStream_t)r.stream) == cudaSuccess ? CB_OK : fail(CB_ERR_CUDA, "graph launch failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (st == CB_OK) st = collect_outputs(e, r);
  const int sync_st = cb_stream_sync(r.dev, r.stream);
  if (st == CB_OK) st = sync_st;
  const double elapsed = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
  if (st == CB_OK && elapsed > 1.5)
    for (size_t i = 0; i < nn && st == CB_OK; i++)
      if (r.dp->plans[i] && g->ws[i]) st = cb_plan_check_status(r.dp->plans[i], g->ws[i]);
  e->be->put_stream(r.dev, r.stream);
  if (st != CB_OK) {
    for (cbg_buffer* b : r.outs) { r.pool->put(b->shape.bytes(), b->ptr); delete b; }
    return st;
  }
  for (size_t o = 0; o < f->outputs.size(); o++) outputs[o] = r.outs[o];
  return CB_OK;
}

}  // namespace

extern "C" {

int cbg_exec_execute(cbg_exec* e, cbg_buffer* const* inputs, int n_inputs, const uint8_t* donate,
                     int default_device, cbg_buffer** outputs, int n_outputs) {
  cb::clear_error();
  if (!e) return fail(CB_ERR_INVALID_ARG, "Execute: executable is NULL");
  if (e->finalized) return fail(CB_ERR_INVALID_ARG, "Execute: executable %s has been finalized", e->name.c_str());
  if (e->be->finalized.load()) return fail(CB_ERR_INVALID_ARG, "Execute: backend has been finalized");
  cbg_function* f = e->fn.get();
  const int np = (int)f->params.size(), no = (int)f->outputs.size();
  if (n_inputs != np * e->replicas)
    return fail(CB_ERR_INVALID_ARG, "Execute: %s expects %d inputs (%d parameters x %d devices), got %d", e->name.c_str(), np * e->replicas, np, e->replicas, n_inputs);
  if (n_outputs < no * e->replicas) return fail(CB_ERR_INVALID_ARG, "Execute: room for %d outputs, %d needed", n_outputs, no * e->replicas);
  std::vector<Replica> reps(e->replicas);
  for (int r = 0; r < e->replicas; r++) {
    const int dev = e->replicas == 1 ? (e->assignment.size() == 1 && e->assignment[0] != 0 ? e->assignment[0] : default_device) : e->assignment[r];
    if (dev < 0 || dev >= e->be->n_devices) return fail(CB_ERR_INVALID_ARG, "Execute: device %d out of range [0,%d)", dev, e->be->n_devices);
    for (int i = 0; i < np; i++) {
      const cbg_buffer* b = inputs[r * np + i];
      const cbg_value* p = f->params[i];
      if (!b) return fail(CB_ERR_INVALID_ARG, "Execute: input #%d (%s) is nil", i, p->name.c_str());
      if (!b->valid) return fail(CB_ERR_INVALID_ARG, "Execute: input #%d (%s) was finalized or donated", i, p->name.c_str());
      if (b->be != e->be) return fail(CB_ERR_INVALID_ARG, "Execute: input #%d (%s) belongs to another backend", i, p->name.c_str());
      if (!(b->shape == p->shape))
        return fail(CB_ERR_INVALID_ARG, "Execute: input #%d (%s) has shape %s, parameter wants %s", i, p->name.c_str(), b->shape.str().c_str(), p->shape.str().c_str());
      if (b->dev != dev) return fail(CB_ERR_INVALID_ARG, "Execute: input #%d (%s) is on device %d, execution is on device %d", i, p->name.c_str(), b->dev, dev);
    }
    reps[r].dev = dev;
    reps[r].inputs = inputs + r * np;
    reps[r].donate = donate ? donate + r * np : nullptr;
  }
  if (donate)       // a buffer donated twice would be handed to the pool twice
    for (int a = 0; a < n_inputs; a++)
      for (int b = a + 1; b < n_inputs; b++)
        if (donate[a] && donate[b] && inputs[a] == inputs[b])
          return fail(CB_ERR_INVALID_ARG, "Execute: the same buffer is donated as input #%d and input #%d", a, b);

  // ---- a call whose input buffers are those of an earlier call replays that call's CUDA graph
  if (graph_eligible(e, donate, n_inputs)) {
    const int dev = reps[0].dev;
    cbg_exec::GraphInstance* g = nullptr;
    bool build = false;
    {
      std::lock_guard<std::mutex> l(e->mu);
      for (auto& gi : e->graphs) {
        if (gi->dev != dev || (int)gi->key.size() != n_inputs) continue;
        bool same = true;
        for (int i = 0; i < n_inputs && same; i++) same = gi->key[i] == inputs[i]->ptr;
        if (same) { g = gi.get(); break; }
      }
      if (!g && e->graphs.size() < 8) {
        e->graphs.push_back(std::make_unique<cbg_exec::GraphInstance>());
        g = e->graphs.back().get();
        g->dev = dev;
        for (int i = 0; i < n_inputs; i++) g->key.push_back(inputs[i]->ptr);
      }
      if (g) {
        g->seen++;
        if (g->busy) g = nullptr;                         // another thread is inside this instance: plain path
        else if (g->exec) g->busy = true;
        else if (g->seen >= 2) { g->busy = true; build = true; }      // the first call ran plainly and configured every kernel
        else g = nullptr;
      }
    }
    if (g) {
      int gst = CB_OK;
      if (build) {
        gst = graph_build(e, g, inputs);
        if (gst != CB_OK) { cb::clear_error(); e->graphs_off = true; }
      }
      if (gst == CB_OK) {
        gst = graph_replay(e, g, inputs, outputs);
        std::lock_guard<std::mutex> l(e->mu);
        g->busy = false;
        g->launches++;
        e->graph_replays++;
        return gst;
      }
      std::lock_guard<std::mutex> l(e->mu);
      g->busy = false;
    }
  }

  // ---- launch: every replica is set up, then the nodes are walked once, each node launched on every replica
  // before the next (all launches are asynchronous, so the devices run side by side; collectives see the operands
  // of all replicas at their node); one sync per device at the end.
  const auto t_start = std::chrono::steady_clock::now();
  int st = CB_OK;
  int n_setup = 0;
  for (; n_setup < e->replicas && st == CB_OK; n_setup++) st = setup_replica(e, reps[n_setup]);
  if (st != CB_OK) n_setup--;                 // the one that failed set nothing up that needs returning
  const size_t nn = f->nodes.size();
  const bool trace = e->be->trace;
  auto mark = [&](Replica& rp, int node) {       // an event on the replica's stream after the launch of `node`
    cb_event ev = nullptr;
    int ms = cb_event_create(rp.dev, &ev);
    if (ms == CB_OK) ms = cb_event_record(rp.dev, ev, rp.stream);
    if (ms == CB_OK) { rp.marks.emplace_back(node, ev); rp.events.push_back(ev); }
    return ms;
  };
  if (trace) for (int r = 0; r < n_setup && st == CB_OK; r++) st = mark(reps[r], -1);
  for (size_t i = 0; i < nn && st == CB_OK; i++) {
    if (!e->live[i]) continue;
    cbg_value* n = f->nodes[i].get();
    if (n->kind == N_ALLREDUCE || n->kind == N_ALLGATHER) st = run_collective(e, n, reps);
    else for (int r = 0; r < e->replicas && st == CB_OK; r++) st = launch_node(e, reps[r], i);
    const bool launches = n->kind == N_ALLREDUCE || n->kind == N_ALLGATHER || (reps[0].dp->plans[i] && (e->group_of[i] < 0 || e->groups[e->group_of[i]][0] == (int)i));
    if (trace && launches) for (int r = 0; r < e->replicas && st == CB_OK; r++) st = mark(reps[r], (int)i);
  }
  for (int r = 0; r < e->replicas && st == CB_OK; r++) st = collect_outputs(e, reps[r]);
  for (int r = 0; r < n_setup; r++) {
    if (!reps[r].stream) continue;
    const int sync_st = cb_stream_sync(reps[r].dev, reps[r].stream);
    if (st == CB_OK) st = sync_st;
  }
  // an index outside the table is an error of the call (quantizeddense.go:487-489): the lookup's status words are read
  if (st == CB_OK)
    for (int r = 0; r < n_setup && st == CB_OK; r++)
      for (size_t i = 0; i < nn && st == CB_OK; i++)
        if (e->live[i] && f->nodes[i]->kind == N_EMBEDDING && reps[r].dp->plans[i] && reps[r].ws[i])
          st = cb_plan_check_status(reps[r].dp->plans[i], reps[r].ws[i]);
  if (trace && st == CB_OK) {
    // one line per launch: device time between the events after the previous launch and after this one
    std::string text;
    char line[512];
    for (int r = 0; r < n_setup; r++) {
      const Replica& rp = reps[r];
      for (size_t k = 1; k < rp.marks.size(); k++) {
        float ms = 0.0f;
        if (cb_event_elapsed_ms(rp.marks[k - 1].second, rp.marks[k].second, &ms) != CB_OK) continue;
        const int i = rp.marks[k].first;
        const cbg_value* nd = f->nodes[i].get();
        const char* kn = rp.dp->plans[i] ? cb_plan_kernel_name(rp.dp->plans[i]) : (nd->kind == N_ALLREDUCE ? "all_reduce" : "all_gather");
        snprintf(line, sizeof(line), "cudabackend trace: exec=%s device=%d node=%d kernel=%s out=%s us=%.2f\n",
                 e->name.c_str(), rp.dev, i, kn, nd->shape.str().c_str(), ms * 1e3);
        text += line;
      }
    }
    fputs(text.c_str(), stderr);
    std::lock_guard<std::mutex> l(e->mu);
    e->last_trace = std::move(text);
  }
  // Kernels with bounded waits report through a status word in their workspace; a wait gives up only after two
  // seconds, so the words are read (one small blocking copy per plan) only when the call took that long.
  const double elapsed = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
  if (st == CB_OK && elapsed > 1.5)
    for (int r = 0; r < n_setup && st == CB_OK; r++)
      for (size_t i = 0; i < nn && st == CB_OK; i++)
        if (reps[r].dp->plans[i] && reps[r].ws[i]) st = cb_plan_check_status(reps[r].dp->plans[i], reps[r].ws[i]);

  // ---- give everything back
  for (int r = 0; r < n_setup; r++) {
    Replica& rp = reps[r];
    for (cb_event ev : rp.events) cb_event_destroy(rp.dev, ev);
    if (rp.stream) e->be->put_stream(rp.dev, rp.stream);
    for (size_t i = 0; i < rp.mem.size(); i++)
      if (rp.owned[i] && !rp.taken[i]) rp.pool->put(f->nodes[i]->shape.bytes(), rp.mem[i]);
    for (auto& sc : rp.scratch) rp.pool->put(sc.first, sc.second);
    if (!rp.ws.empty()) {
      std::lock_guard<std::mutex> l(e->mu);
      e->idle_ws[rp.dev].push_back(std::move(rp.ws));
    }
    // donated inputs are consumed: their memory returns to the pool unless an output took it
    if (rp.donate)
      for (size_t p = 0; p < f->params.size(); p++)
        if (rp.donate[p]) {
          cbg_buffer* b = rp.inputs[p];
          if (!b->valid) continue;
          if (rp.taken.empty() || !rp.taken[f->params[p]->index]) rp.pool->put(b->shape.bytes(), b->ptr);
          b->ptr = nullptr;
          b->valid = false;
        }
  }
  if (st != CB_OK) {
    for (Replica& rp : reps) for (cbg_buffer* b : rp.outs) { rp.pool->put(b->shape.bytes(), b->ptr); delete b; }
    return st;
  }
  for (int r = 0; r < e->replicas; r++)
    for (int o = 0; o < no; o++) outputs[r * no + o] = reps[r].outs[o];
  return CB_OK;
}

int cbg_exec_finalize(cbg_exec* e) {
  cb::clear_error();
  if (!e) return CB_OK;
  for (auto& kv : e->dev_plans) for (cb_plan* p : kv.second.plans) if (p) cb_plan_destroy(p);
  for (auto& kv : e->const_dev) for (void* p : kv.second) if (p) cb_free(kv.first, p);
  for (auto& kv : e->idle_ws) for (auto& set : kv.second) for (void* p : set) if (p) cb_free(kv.first, p);
  for (auto& g : e->graphs) graph_instance_free(g.get());
  delete e;
  return CB_OK;
}

}  // extern "C"
