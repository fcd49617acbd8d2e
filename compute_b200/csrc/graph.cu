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
  size_t bytes() const { return (size_t)size() * cb::dtype_size(dtype); }
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
                N_GELU, N_SOFTMAX, N_LAYERNORM, N_COLS_BIAS };

bool is_float(int d) { return d == CB_F16 || d == CB_F32 || d == CB_F64 || d == CB_BF16 || d == CB_F8E4M3FN || d == CB_F8E5M2; }
bool is_half(int d) { return d == CB_F16 || d == CB_BF16; }

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

struct cbg_backend {
  int n_devices = 0;
  bool fallback_only = false;
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
  double epsilon = 0.0;               // layer norm
  int flags = 0;                      // gelu: exact; layer norm: 1 gamma, 2 beta
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

struct cbg_exec {
  cbg_backend* be = nullptr;
  std::string name;
  std::unique_ptr<cbg_function> fn;          // owns the nodes
  std::vector<cb_plan*> plans;               // per node (NULL for param/const/reshape)
  std::vector<size_t> ws_bytes;
  int replicas = 1;
  std::vector<int> assignment;
  std::mutex mu;
  std::map<int, std::vector<void*>> const_dev;                       // device -> per-node constant copy
  std::map<int, std::vector<std::vector<void*>>> idle_ws;            // device -> sets of prepared workspaces
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
    else if (item.rfind("devices=", 0) == 0) { /* accepted; device visibility is the process's */ }
    else return fail(CB_ERR_INVALID_ARG, "unknown configuration option \"%s\" for the cuda backend", item.c_str());
  }
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
  // OpType codes of optype.go: Parameter 1, Constant 2, DotGeneral 32, FusedSoftmax 116, FusedLayerNorm 117,
  // FusedGelu 118, FusedDense 119, FusedScaledDotProductAttention 120, FusedAttentionQKVProjection 122,
  // FusedQuantizedDense 123.  The helper ops
  // (Reshape, Slice, Iota, ConvertDType, Transpose) exist to serve DotGeneral and are
  // deliberately not advertised.
  static const int32_t k_ops[] = {1, 2, 32, 116, 117, 118, 119, 120, 122, 123};
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
  if (cb::dtype_size(dtype) == 0 || dtype > CB_BF16) return fail(CB_ERR_NOT_IMPLEMENTED, "BufferFromFlatData: dtype %s is not supported", cb::dtype_name(dtype));
  auto buf = std::make_unique<cbg_buffer>();
  buf->be = b;
  buf->dev = dev;
  buf->shape.dtype = dtype;
  CB_TRY(make_dims("BufferFromFlatData", rank, dims, &buf->shape.dims));
  if (buf->shape.bytes() > 0 && !host_flat) return fail(CB_ERR_INVALID_ARG, "BufferFromFlatData: flat data is NULL");
  CB_TRY(b->pools[dev]->get(dev, buf->shape.bytes(), &buf->ptr));
  int st = cb_h2d(dev, buf->ptr, host_flat, buf->shape.bytes(), nullptr);
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
  return cb_d2h(buf->dev, host_flat, buf->ptr, n_bytes, nullptr);
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
  if (cb::dtype_size(dtype) == 0 || dtype > CB_BF16) return fail(CB_ERR_NOT_IMPLEMENTED, "Parameter: dtype %s is not supported", cb::dtype_name(dtype));
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
  if (cb::dtype_size(dtype) == 0 || dtype > CB_BF16) return fail(CB_ERR_NOT_IMPLEMENTED, "Constant: dtype %s is not supported", cb::dtype_name(dtype));
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
  if (ggml_type != CB_GGML_Q4_0 && ggml_type != CB_GGML_Q8_0)
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s: GGML type %d not yet supported in fused path", op, ggml_type);
  const int64_t N = weights->shape.dims[0], bytes_per_row = weights->shape.dims[1];
  const int64_t block_bytes = ggml_type == CB_GGML_Q8_0 ? 34 : 18;
  if (bytes_per_row % block_bytes != 0)
    return fail(CB_ERR_INVALID_ARG, "%s: bytesPerRow=%lld is not a multiple of the %lld-byte block", op, (long long)bytes_per_row, (long long)block_bytes);
  const int64_t K = bytes_per_row / block_bytes * 32;
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
  if (weights->shape.dtype != CB_I8 && weights->shape.dtype != CB_U8)
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s: %s unsupported weight type %s", op, scheme == 1 ? "NF4" : "Linear", cb::dtype_name(weights->shape.dtype));
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

int cbg_fn_not_implemented(cbg_function* f, const char* op_name) {
  cb::clear_error();
  return fail(CB_ERR_NOT_IMPLEMENTED, "%s: not implemented by the cuda backend", op_name ? op_name : "op");
}

// ---------------------------------------------------------------- Compile
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
  e->plans.assign(f->nodes.size(), nullptr);
  e->ws_bytes.assign(f->nodes.size(), 0);
  int st = CB_OK;
  for (size_t i = 0; i < f->nodes.size() && st == CB_OK; i++) {
    cbg_value* n = f->nodes[i].get();
    cb_plan* p = nullptr;
    const int dev = e->assignment[0];   // plans hold no device state beyond the SM count
    switch (n->kind) {
      case N_DOT: st = cb_plan_dot(dev, &n->dot, &p); break;
      case N_QDENSE: st = cb_plan_qdense(dev, &n->qd, &p); break;
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
      default: break;
    }
    if (st == CB_OK && p) {
      e->plans[i] = p;
      cb_plan_workspace_bytes(p, &e->ws_bytes[i]);
    }
  }
  if (st != CB_OK) {
    for (cb_plan* p : e->plans) if (p) cb_plan_destroy(p);
    return st;
  }
  e->fn = std::move(bld->main);
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
  for (cb_plan* p : e->plans) if (p) { s += cb_plan_kernel_name(p); s += "\n"; }
  snprintf(buf, n, "%s", s.c_str());
  return CB_OK;
}

static int run_replica(cbg_exec* e, int dev, cbg_buffer* const* inputs, const uint8_t* donate, cbg_buffer** outputs) {
  cbg_function* f = e->fn.get();
  cbg_backend* be = e->be;
  DevicePool& pool = *be->pools[dev];
  const size_t nn = f->nodes.size();
  // constants of this device and a set of prepared workspaces
  std::vector<void*> consts, ws;
  {
    std::lock_guard<std::mutex> l(e->mu);
    auto it = e->const_dev.find(dev);
    if (it == e->const_dev.end()) {
      std::vector<void*> c(nn, nullptr);
      for (size_t i = 0; i < nn; i++) {
        cbg_value* n = f->nodes[i].get();
        if (n->kind != N_CONST) continue;
        CB_TRY(cb_alloc(dev, n->const_data.size(), &c[i]));
        CB_TRY(cb_h2d(dev, c[i], n->const_data.data(), n->const_data.size(), nullptr));
      }
      it = e->const_dev.emplace(dev, std::move(c)).first;
    }
    consts = it->second;
    auto& idle = e->idle_ws[dev];
    if (!idle.empty()) { ws = std::move(idle.back()); idle.pop_back(); }
  }
  if (ws.empty()) {
    ws.assign(nn, nullptr);
    for (size_t i = 0; i < nn; i++) {
      if (!e->plans[i] || e->ws_bytes[i] == 0) continue;
      CB_TRY(cb_alloc(dev, e->ws_bytes[i], &ws[i]));
      CB_TRY(cb_plan_prepare_workspace(e->plans[i], ws[i], nullptr));
    }
    CB_TRY(cb_stream_sync(dev, nullptr));
  }
  cb_stream stream = nullptr;
  CB_TRY(be->get_stream(dev, &stream));

  std::vector<void*> mem(nn, nullptr);      // device pointer of every node's value
  std::vector<bool> owned(nn, false);       // allocated from the pool by this call
  int st = CB_OK;
  for (size_t i = 0; i < nn && st == CB_OK; i++) {
    cbg_value* n = f->nodes[i].get();
    switch (n->kind) {
      case N_PARAM: mem[i] = inputs[n->param_index]->ptr; break;
      case N_CONST: mem[i] = consts[i]; break;
      case N_RESHAPE: mem[i] = mem[n->inputs[0]->index]; break;     // same bytes, new shape
      default: {
        st = pool.get(dev, n->shape.bytes(), &mem[i]);
        if (st != CB_OK) break;
        owned[i] = true;
        const void* in[8];
        for (size_t k = 0; k < n->inputs.size(); k++) in[k] = mem[n->inputs[k]->index];
        void* out[1] = {mem[i]};
        // a kernel launch with zero elements is skipped inside cb_launch
        st = cb_launch(e->plans[i], in, (int)n->inputs.size(), out, 1, ws[i], stream);
      }
    }
  }
  // outputs: every output is a distinct buffer owned by the caller
  std::vector<bool> taken(nn, false);
  std::vector<cbg_buffer*> outs;
  for (size_t o = 0; o < f->outputs.size() && st == CB_OK; o++) {
    cbg_value* n = f->outputs[o];
    // root of the aliasing chain (Reshape shares memory with its operand)
    cbg_value* root = n;
    while (root->kind == N_RESHAPE) root = root->inputs[0];
    auto buf = std::make_unique<cbg_buffer>();
    buf->be = be;
    buf->dev = dev;
    buf->shape = n->shape;
    const int ri = root->index;
    const bool donated_param = root->kind == N_PARAM && donate && donate[root->param_index];
    if ((owned[ri] || donated_param) && !taken[ri]) {
      buf->ptr = mem[ri];              // hand the memory over
      taken[ri] = true;
    } else {
      st = pool.get(dev, n->shape.bytes(), &buf->ptr);
      if (st == CB_OK) st = cb_d2d(dev, buf->ptr, dev, mem[ri], n->shape.bytes(), stream);
    }
    if (st == CB_OK) outs.push_back(buf.release());
  }
  int sync_st = cb_stream_sync(dev, stream);
  if (st == CB_OK) st = sync_st;
  for (size_t i = 0; i < nn && st == CB_OK; i++)
    if (e->plans[i] && ws[i]) st = cb_plan_check_status(e->plans[i], ws[i]);
  be->put_stream(dev, stream);
  for (size_t i = 0; i < nn; i++)
    if (owned[i] && !taken[i]) pool.put(f->nodes[i]->shape.bytes(), mem[i]);
  {
    std::lock_guard<std::mutex> l(e->mu);
    e->idle_ws[dev].push_back(std::move(ws));
  }
  // donated inputs are consumed: their memory returns to the pool unless an output took it
  if (donate)
    for (size_t p = 0; p < f->params.size(); p++)
      if (donate[p]) {
        cbg_buffer* b = inputs[p];
        if (!taken[f->params[p]->index]) pool.put(b->shape.bytes(), b->ptr);
        b->ptr = nullptr;
        b->valid = false;
      }
  if (st != CB_OK) {
    for (cbg_buffer* b : outs) { pool.put(b->shape.bytes(), b->ptr); delete b; }
    return st;
  }
  for (size_t o = 0; o < outs.size(); o++) outputs[o] = outs[o];
  return CB_OK;
}

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
  }
  for (int r = 0; r < e->replicas; r++) {
    const int dev = e->replicas == 1 ? (e->assignment.size() == 1 && e->assignment[0] != 0 ? e->assignment[0] : default_device) : e->assignment[r];
    CB_TRY(run_replica(e, dev, inputs + r * np, donate ? donate + r * np : nullptr, outputs + r * no));
  }
  return CB_OK;
}

int cbg_exec_finalize(cbg_exec* e) {
  cb::clear_error();
  if (!e) return CB_OK;
  for (cb_plan* p : e->plans) if (p) cb_plan_destroy(p);
  for (auto& kv : e->const_dev) for (void* p : kv.second) if (p) cb_free(kv.first, p);
  for (auto& kv : e->idle_ws) for (auto& set : kv.second) for (void* p : set) if (p) cb_free(kv.first, p);
  delete e;
  return CB_OK;
}

}  // extern "C"
