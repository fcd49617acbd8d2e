// Process/device/buffer/stream entry points of the C ABI and the plan object's
// life cycle.  Replaces, for the accelerated path, the host-memory runtime of
// the reference's CPU backend (internal/gobackend/gobackend.go, buffers.go).
#include "common.cuh"

#include <stdarg.h>
#include <string.h>
#include <map>
#include <mutex>
#include <vector>

namespace cb {

static thread_local char g_err[1024] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}
void clear_error() { g_err[0] = 0; }

static std::once_flag g_init_once;
static int g_ndev = -1;
static std::vector<int> g_sm;

static void do_init() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
  g_ndev = n;
  g_sm.assign(n, 0);
  for (int d = 0; d < n; d++) {
    int sm = 0;
    cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, d);
    g_sm[d] = sm;
  }
}

int set_device(int dev) {
  std::call_once(g_init_once, do_init);
  if (g_ndev <= 0) return fail(CB_ERR_NO_DEVICE, "no CUDA device is visible to this process");
  if (dev < 0 || dev >= g_ndev) return fail(CB_ERR_INVALID_ARG, "device %d out of range [0,%d)", dev, g_ndev);
  CB_CUDA(cudaSetDevice(dev));
  return CB_OK;
}

int sm_count(int dev) {
  std::call_once(g_init_once, do_init);
  return (dev >= 0 && dev < g_ndev) ? g_sm[dev] : 0;
}

encode_tiled_fn tensor_map_encoder() {
  static encode_tiled_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_tiled_fn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

const char* dtype_name(int d) {
  switch (d) {
    case CB_BOOL: return "Bool"; case CB_I8: return "Int8"; case CB_I16: return "Int16";
    case CB_I32: return "Int32"; case CB_I64: return "Int64"; case CB_U8: return "Uint8";
    case CB_U16: return "Uint16"; case CB_U32: return "Uint32"; case CB_U64: return "Uint64";
    case CB_F16: return "Float16"; case CB_F32: return "Float32"; case CB_F64: return "Float64";
    case CB_BF16: return "BFloat16"; case CB_F8E5M2: return "F8E5M2"; case CB_F8E4M3FN: return "F8E4M3FN";
    case CB_I4: return "Int4"; case CB_U4: return "Uint4";
    default: return "InvalidDType";
  }
}

// The page-locked ranges this library handed out, so that a transfer from one of them needs no query of the driver.
static std::mutex g_host_mu;
static std::map<uintptr_t, size_t> g_host_ranges;      // base -> bytes
void host_range_add(const void* p, size_t bytes) {
  std::lock_guard<std::mutex> l(g_host_mu);
  g_host_ranges[reinterpret_cast<uintptr_t>(p)] = bytes;
}
void host_range_remove(const void* p) {
  std::lock_guard<std::mutex> l(g_host_mu);
  g_host_ranges.erase(reinterpret_cast<uintptr_t>(p));
}
bool host_range_is_page_locked(const void* p, size_t bytes) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  std::lock_guard<std::mutex> l(g_host_mu);
  auto it = g_host_ranges.upper_bound(a);
  if (it == g_host_ranges.begin()) return false;
  --it;
  return a >= it->first && a + bytes <= it->first + it->second;
}

}  // namespace cb

using namespace cb;

extern "C" {

int cb_init(int* n_devices) {
  clear_error();
  std::call_once(g_init_once, do_init);
  if (n_devices) *n_devices = g_ndev < 0 ? 0 : g_ndev;
  if (g_ndev <= 0) return fail(CB_ERR_NO_DEVICE, "no CUDA device is visible to this process");
  return CB_OK;
}

int cb_device_desc(int dev, char* buf, size_t buf_len) {
  CB_TRY(set_device(dev));
  cudaDeviceProp p;
  CB_CUDA(cudaGetDeviceProperties(&p, dev));
  snprintf(buf, buf_len, "cuda:%d %s sm_%d%d %d SMs %.1f GiB", dev, p.name, p.major, p.minor,
           p.multiProcessorCount, (double)p.totalGlobalMem / (1024.0 * 1024.0 * 1024.0));
  return CB_OK;
}

int cb_device_sm_count(int dev, int* n_sm) {
  CB_TRY(set_device(dev));
  *n_sm = sm_count(dev);
  return CB_OK;
}

const char* cb_last_error(void) { return g_err; }

const char* cb_status_name(int s) {
  switch (s) {
    case CB_OK: return "ok";
    case CB_ERR_INVALID_ARG: return "invalid argument";
    case CB_ERR_NOT_IMPLEMENTED: return "not implemented";
    case CB_ERR_OOM: return "out of device memory";
    case CB_ERR_CUDA: return "CUDA error";
    case CB_ERR_TIMEOUT: return "device-side wait timed out";
    case CB_ERR_NO_DEVICE: return "no CUDA device";
    default: return "unknown status";
  }
}

int cb_alloc(int dev, size_t bytes, void** dptr) {
  CB_TRY(set_device(dev));
  if (!dptr) return fail(CB_ERR_INVALID_ARG, "cb_alloc: dptr is NULL");
  *dptr = nullptr;
  // Zero-sized tensors still get a distinct, valid pointer.
  CB_CUDA(cudaMalloc(dptr, bytes ? bytes : 16));
  return CB_OK;
}

int cb_free(int dev, void* dptr) {
  if (!dptr) return CB_OK;
  CB_TRY(set_device(dev));
  CB_CUDA(cudaFree(dptr));
  return CB_OK;
}

int cb_memset(int dev, void* dptr, int value, size_t bytes, cb_stream stream) {
  CB_TRY(set_device(dev));
  if (bytes == 0) return CB_OK;
  CB_CUDA(cudaMemsetAsync(dptr, value, bytes, (cudaStream_t)stream));
  if (!stream) CB_CUDA(cudaStreamSynchronize(nullptr));
  return CB_OK;
}

int cb_h2d(int dev, void* dst, const void* host_src, size_t bytes, cb_stream stream) {
  CB_TRY(set_device(dev));
  if (bytes == 0) return CB_OK;
  if (stream) {
    CB_CUDA(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  } else {
    // A copy from pageable memory may return once the data are staged, before the transfer to the
    // device has finished, and the streams of this library do not wait for the default stream:
    // complete it here, so that "synchronous" holds for work on any stream.
    CB_CUDA(cudaMemcpy(dst, host_src, bytes, cudaMemcpyHostToDevice));
    CB_CUDA(cudaStreamSynchronize(nullptr));
  }
  return CB_OK;
}

int cb_d2h(int dev, void* host_dst, const void* src, size_t bytes, cb_stream stream) {
  CB_TRY(set_device(dev));
  if (bytes == 0) return CB_OK;
  if (stream) CB_CUDA(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  else CB_CUDA(cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost));
  return CB_OK;
}

int cb_d2d(int dst_dev, void* dst, int src_dev, const void* src, size_t bytes, cb_stream stream) {
  CB_TRY(set_device(dst_dev));
  if (bytes == 0) return CB_OK;
  if (dst_dev == src_dev) {
    CB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  } else {
    CB_CUDA(cudaMemcpyPeerAsync(dst, dst_dev, src, src_dev, bytes, (cudaStream_t)stream));
  }
  if (!stream) CB_CUDA(cudaStreamSynchronize(nullptr));
  return CB_OK;
}

int cb_host_alloc(size_t bytes, void** host_ptr) {
  clear_error();
  const size_t n = bytes ? bytes : 16;
  CB_CUDA(cudaMallocHost(host_ptr, n));
  cb::host_range_add(*host_ptr, n);
  return CB_OK;
}

int cb_host_free(void* host_ptr) {
  if (!host_ptr) return CB_OK;
  cb::host_range_remove(host_ptr);
  CB_CUDA(cudaFreeHost(host_ptr));
  return CB_OK;
}

int cb_stream_create(int dev, cb_stream* stream) {
  CB_TRY(set_device(dev));
  cudaStream_t s;
  CB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = (cb_stream)s;
  return CB_OK;
}

int cb_stream_sync(int dev, cb_stream stream) {
  CB_TRY(set_device(dev));
  CB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return CB_OK;
}

int cb_stream_destroy(int dev, cb_stream stream) {
  CB_TRY(set_device(dev));
  if (stream) CB_CUDA(cudaStreamDestroy((cudaStream_t)stream));
  return CB_OK;
}

int cb_event_create(int dev, cb_event* ev) {
  CB_TRY(set_device(dev));
  cudaEvent_t e;
  CB_CUDA(cudaEventCreate(&e));
  *ev = (cb_event)e;
  return CB_OK;
}

int cb_event_record(int dev, cb_event ev, cb_stream stream) {
  CB_TRY(set_device(dev));
  CB_CUDA(cudaEventRecord((cudaEvent_t)ev, (cudaStream_t)stream));
  return CB_OK;
}

int cb_ipc_export(int dev, const void* dptr, unsigned char* handle) {
  CB_TRY(set_device(dev));
  if (!dptr || !handle) return fail(CB_ERR_INVALID_ARG, "cb_ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == CB_IPC_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  CB_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(dptr)));
  memcpy(handle, &h, sizeof(h));
  return CB_OK;
}

int cb_ipc_open(int dev, const unsigned char* handle, void** dptr) {
  CB_TRY(set_device(dev));
  if (!dptr || !handle) return fail(CB_ERR_INVALID_ARG, "cb_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  CB_CUDA(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
  return CB_OK;
}

int cb_ipc_close(int dev, void* dptr) {
  CB_TRY(set_device(dev));
  if (!dptr) return CB_OK;
  CB_CUDA(cudaIpcCloseMemHandle(dptr));
  return CB_OK;
}

int cb_peer_signal(int dev, void* const* flags, int n_ranks, int slot, cb_stream stream) {
  CB_TRY(set_device(dev));
  if (!flags) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal: null argument");
  if (slot < 0 || slot >= 32) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal: slot %d", slot);
  for (int r = 0; r < n_ranks && r < 8; r++)
    if (!flags[r]) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal: null flag array for rank %d", r);
  return cb::peer_signal_launch(flags, n_ranks, slot, (cudaStream_t)stream);
}

int cb_peer_wait(int dev, const void* flags, int n_flags, uint32_t target, void* status_word, cb_stream stream) {
  CB_TRY(set_device(dev));
  if (!flags || !status_word) return fail(CB_ERR_INVALID_ARG, "cb_peer_wait: null argument");
  if (n_flags < 1 || n_flags > 32) return fail(CB_ERR_INVALID_ARG, "cb_peer_wait: %d flags", n_flags);
  return cb::peer_wait_launch((const unsigned*)flags, n_flags, target, (unsigned*)status_word, (cudaStream_t)stream);
}

int cb_peer_signal_wait(int dev, void* const* flags, int n_ranks, int slot, const void* local_flags, uint32_t target,
                        void* status_word, cb_stream stream) {
  CB_TRY(set_device(dev));
  if (!flags || !local_flags || !status_word) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal_wait: null argument");
  if (slot < 0 || slot >= 32) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal_wait: slot %d", slot);
  for (int r = 0; r < n_ranks && r < 8; r++)
    if (!flags[r]) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal_wait: null flag array for rank %d", r);
  return cb::peer_signal_wait_launch(flags, n_ranks, slot, (const unsigned*)local_flags, target, (unsigned*)status_word, (cudaStream_t)stream);
}

int cb_stream_wait_event(int dev, cb_stream stream, cb_event ev) {
  CB_TRY(set_device(dev));
  CB_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)ev, 0));
  return CB_OK;
}

int cb_event_elapsed_ms(cb_event start, cb_event stop, float* ms) {
  clear_error();
  CB_CUDA(cudaEventSynchronize((cudaEvent_t)stop));
  CB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return CB_OK;
}

int cb_event_destroy(int dev, cb_event ev) {
  CB_TRY(set_device(dev));
  if (ev) CB_CUDA(cudaEventDestroy((cudaEvent_t)ev));
  return CB_OK;
}

// ---- plans --------------------------------------------------------------------

static int new_plan(int dev, int kind, cb_plan** out, cb_plan** tmp) {
  clear_error();
  if (!out) return fail(CB_ERR_INVALID_ARG, "plan output pointer is NULL");
  *out = nullptr;
  // Plans can be built without touching the device (shape/dtype selection only),
  // so a missing GPU is not an error here; launches check it.
  cb_plan* p = new cb_plan();
  p->kind = kind;
  p->dev = dev;
  p->n_sm = sm_count(dev);
  if (p->n_sm <= 0) p->n_sm = 148;   // B200; used only to size grids when planning off-device
  *tmp = p;
  return CB_OK;
}

static int finish_plan(int status, cb_plan* p, cb_plan** out) {
  if (status != CB_OK) { delete p; return status; }
  *out = p;
  return CB_OK;
}

int cb_plan_qdense(int dev, const cb_qdense_desc* desc, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_QDENSE, plan, &p));
  if (!desc) { delete p; return fail(CB_ERR_INVALID_ARG, "desc is NULL"); }
  p->qd = *desc;
  return finish_plan(qdense_plan(p), p, plan);
}

int cb_plan_qdense_group(int dev, const cb_qdense_desc* shared, const cb_qdense_member* members, int n_members,
                         cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_QDENSE, plan, &p));
  if (!shared || !members || n_members < 1) { delete p; return fail(CB_ERR_INVALID_ARG, "cb_plan_qdense_group: NULL or empty argument"); }
  p->qd = *shared;
  p->group.assign(members, members + n_members);
  return finish_plan(qdense_group_plan(p), p, plan);
}

int cb_plan_dot(int dev, const cb_dot_desc* desc, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_DOT, plan, &p));
  if (!desc) { delete p; return fail(CB_ERR_INVALID_ARG, "desc is NULL"); }
  p->dot = *desc;
  return finish_plan(dot_plan(p), p, plan);
}

int cb_plan_sdpa(int dev, const cb_sdpa_desc* desc, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_SDPA, plan, &p));
  if (!desc) { delete p; return fail(CB_ERR_INVALID_ARG, "desc is NULL"); }
  p->sdpa = *desc;
  return finish_plan(sdpa_plan(p), p, plan);
}

int cb_plan_copy(int dev, int32_t dtype, int64_t n, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_COPY, plan, &p));
  p->helper.dtype = dtype;
  p->helper.n = n;
  return finish_plan(helper_plan(p), p, plan);
}

int cb_plan_convert(int dev, int32_t from, int32_t to, int64_t n, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_CONVERT, plan, &p));
  p->helper.dtype = from;
  p->helper.dtype_to = to;
  p->helper.n = n;
  return finish_plan(helper_plan(p), p, plan);
}

int cb_plan_iota(int dev, int32_t dtype, int32_t rank, const int64_t* dims, int32_t axis, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_IOTA, plan, &p));
  if (rank < 0 || rank > 8 || (rank > 0 && !dims)) { delete p; return fail(CB_ERR_INVALID_ARG, "iota: rank %d unsupported", rank); }
  p->helper.dtype = dtype;
  p->helper.rank = rank;
  p->helper.axis = axis;
  for (int i = 0; i < rank; i++) p->helper.dims[i] = dims[i];
  return finish_plan(helper_plan(p), p, plan);
}

int cb_plan_slice(int dev, int32_t dtype, int32_t rank, const int64_t* dims, const int64_t* starts,
                  const int64_t* limits, const int64_t* strides, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_SLICE, plan, &p));
  if (rank < 0 || rank > 8) { delete p; return fail(CB_ERR_INVALID_ARG, "slice: rank %d unsupported", rank); }
  p->helper.dtype = dtype;
  p->helper.rank = rank;
  for (int i = 0; i < rank; i++) {
    int64_t st = strides ? strides[i] : 1;
    if (st < 1 || starts[i] < 0 || limits[i] > dims[i] || starts[i] > limits[i]) {
      delete p;
      return fail(CB_ERR_INVALID_ARG, "slice: axis %d start=%lld limit=%lld stride=%lld invalid for dim %lld", i,
                  (long long)starts[i], (long long)limits[i], (long long)st, (long long)dims[i]);
    }
    p->helper.dims[i] = dims[i];
    p->helper.starts[i] = starts[i];
    p->helper.strides[i] = st;
    p->helper.out_dims[i] = (limits[i] - starts[i] + st - 1) / st;
  }
  return finish_plan(helper_plan(p), p, plan);
}

int cb_plan_transpose(int dev, int32_t dtype, int32_t rank, const int64_t* dims,
                      const int32_t* permutation, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_TRANSPOSE, plan, &p));
  if (rank < 0 || rank > 8) { delete p; return fail(CB_ERR_INVALID_ARG, "transpose: rank %d unsupported", rank); }
  p->helper.dtype = dtype;
  p->helper.rank = rank;
  bool seen[8] = {false};
  for (int i = 0; i < rank; i++) {
    int a = permutation[i];
    if (a < 0 || a >= rank || seen[a]) { delete p; return fail(CB_ERR_INVALID_ARG, "transpose: invalid permutation"); }
    seen[a] = true;
    p->helper.dims[i] = dims[i];
    p->helper.perm[i] = a;
    p->helper.out_dims[i] = dims[a];
  }
  return finish_plan(helper_plan(p), p, plan);
}

int cb_plan_gelu(int dev, int32_t dtype, int64_t n, int32_t exact, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_GELU, plan, &p));
  p->helper.dtype = dtype;
  p->helper.n = n;
  p->helper.axis = exact ? 1 : 0;
  return finish_plan(fused_small_plan(p), p, plan);
}

int cb_plan_softmax(int dev, int32_t dtype, int64_t outer, int64_t axis_size, int64_t inner, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_SOFTMAX, plan, &p));
  p->helper.dtype = dtype;
  p->helper.dims[0] = outer; p->helper.dims[1] = axis_size; p->helper.dims[2] = inner;
  return finish_plan(fused_small_plan(p), p, plan);
}

int cb_plan_layernorm(int dev, int32_t dtype, int64_t rows, int64_t norm_size, double epsilon, int32_t has_gamma,
                      int32_t has_beta, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_LAYERNORM, plan, &p));
  p->helper.dtype = dtype;
  p->helper.dims[0] = rows; p->helper.dims[1] = norm_size; p->helper.dims[2] = 1;
  p->helper.eps = epsilon;
  p->helper.flags = (has_gamma ? 1 : 0) | (has_beta ? 2 : 0);
  return finish_plan(fused_small_plan(p), p, plan);
}

int cb_plan_cols_bias(int dev, int32_t dtype, int64_t rows, int64_t total_cols, int64_t first_col, int64_t n_cols,
                      int32_t has_bias, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_COLS_BIAS, plan, &p));
  p->helper.dtype = dtype;
  p->helper.dims[0] = rows; p->helper.dims[1] = total_cols; p->helper.dims[2] = first_col; p->helper.dims[3] = n_cols;
  p->helper.flags = has_bias ? 1 : 0;
  return finish_plan(fused_small_plan(p), p, plan);
}

int cb_plan_binary(int dev, int32_t op, int32_t dtype, int32_t rank, const int64_t* lhs_dims, const int64_t* rhs_dims, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_BINARY, plan, &p));
  if (rank < 0 || rank > 8 || (rank > 0 && (!lhs_dims || !rhs_dims))) { delete p; return fail(CB_ERR_INVALID_ARG, "binary op: rank %d unsupported", rank); }
  p->helper.dtype = dtype;
  p->helper.rank = rank;
  p->helper.axis = op;
  for (int i = 0; i < rank; i++) { p->helper.dims[i] = lhs_dims[i]; p->helper.starts[i] = rhs_dims[i]; }
  return finish_plan(elementwise_plan(p), p, plan);
}

int cb_plan_unary(int dev, int32_t op, int32_t dtype, int64_t n, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_UNARY, plan, &p));
  p->helper.dtype = dtype;
  p->helper.axis = op;
  p->helper.n = n;
  return finish_plan(elementwise_plan(p), p, plan);
}

int cb_plan_reduce(int dev, int32_t reduce_op, int32_t dtype, int32_t rank, const int64_t* dims, const int32_t* reduced_axis_flags,
                   cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_REDUCE, plan, &p));
  if (rank < 0 || rank > 8 || (rank > 0 && (!dims || !reduced_axis_flags))) { delete p; return fail(CB_ERR_INVALID_ARG, "reduce: rank %d unsupported", rank); }
  p->helper.dtype = dtype;
  p->helper.rank = rank;
  p->helper.axis = reduce_op;
  for (int i = 0; i < rank; i++) { p->helper.dims[i] = dims[i]; p->helper.perm[i] = reduced_axis_flags[i] ? 1 : 0; }
  return finish_plan(elementwise_plan(p), p, plan);
}

int cb_plan_broadcast_in_dim(int dev, int32_t dtype, int32_t rank, const int64_t* dims, int32_t out_rank, const int64_t* out_dims,
                             const int32_t* broadcast_axes, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_BROADCAST, plan, &p));
  if (rank < 0 || rank > 8 || out_rank < 0 || out_rank > 8 || rank > out_rank) { delete p; return fail(CB_ERR_INVALID_ARG, "BroadcastInDim: ranks %d -> %d unsupported", rank, out_rank); }
  p->helper.dtype = dtype;
  p->helper.rank = rank;
  p->helper.strides[0] = out_rank;
  for (int i = 0; i < rank; i++) { p->helper.dims[i] = dims[i]; p->helper.perm[i] = broadcast_axes[i]; }
  for (int i = 0; i < out_rank; i++) p->helper.out_dims[i] = out_dims[i];
  return finish_plan(elementwise_plan(p), p, plan);
}

int cb_plan_rms_norm(int dev, int32_t dtype, int64_t rows, int64_t row_size, double epsilon, int32_t has_gamma, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_RMSNORM, plan, &p));
  if (rows < 0 || row_size < 1) { delete p; return fail(CB_ERR_INVALID_ARG, "rms norm: rows %lld of %lld elements", (long long)rows, (long long)row_size); }
  p->helper.dtype = dtype;
  p->helper.dims[0] = rows; p->helper.dims[1] = row_size;
  p->helper.eps = epsilon;
  p->helper.flags = has_gamma ? 1 : 0;
  return finish_plan(elementwise_plan(p), p, plan);
}

int cb_plan_embedding_lookup(int dev, int64_t vocab, int64_t bytes_per_row, int64_t n_indices, int32_t index_dtype, int32_t ggml_type, cb_plan** plan) {
  cb_plan* p;
  CB_TRY(new_plan(dev, PLAN_EMBEDDING, plan, &p));
  p->helper.dtype = index_dtype;
  p->helper.dims[0] = vocab; p->helper.dims[1] = bytes_per_row;
  p->helper.n = n_indices;
  p->helper.axis = ggml_type;
  return finish_plan(embedding_lookup_plan(p), p, plan);
}

int cb_plan_workspace_bytes(const cb_plan* plan, size_t* bytes) {
  clear_error();
  if (!plan || !bytes) return fail(CB_ERR_INVALID_ARG, "NULL argument");
  *bytes = plan->workspace_bytes;
  return CB_OK;
}

int cb_plan_prepare_workspace(const cb_plan* plan, void* workspace, cb_stream stream) {
  clear_error();
  if (!plan) return fail(CB_ERR_INVALID_ARG, "plan is NULL");
  if (plan->counter_bytes == 0) return CB_OK;
  if (!workspace) return fail(CB_ERR_INVALID_ARG, "plan %s needs %zu bytes of workspace", plan->name.c_str(), plan->workspace_bytes);
  CB_TRY(set_device(plan->dev));
  CB_CUDA(cudaMemsetAsync(workspace, 0, plan->counter_bytes, (cudaStream_t)stream));
  return CB_OK;
}

const char* cb_plan_kernel_name(const cb_plan* plan) { return plan ? plan->name.c_str() : ""; }

int cb_plan_grid(const cb_plan* plan, int* blocks, int* threads, int* dyn_smem_bytes) {
  clear_error();
  if (!plan) return fail(CB_ERR_INVALID_ARG, "plan is NULL");
  if (blocks) *blocks = plan->blocks;
  if (threads) *threads = plan->threads;
  if (dyn_smem_bytes) *dyn_smem_bytes = plan->dyn_smem;
  return CB_OK;
}

static int check_launch_args(const cb_plan* plan, const void* const* inputs, int n_inputs, void* const* outputs, int n_outputs,
                             const void* workspace);
static int launch_checked(const cb_plan* plan, const void* const* inputs, void* const* outputs, void* workspace, cudaStream_t s);

int cb_launch(const cb_plan* plan, const void* const* inputs, int n_inputs,
              void* const* outputs, int n_outputs, void* workspace, cb_stream stream) {
  clear_error();
  CB_TRY(check_launch_args(plan, inputs, n_inputs, outputs, n_outputs, workspace));
  CB_TRY(set_device(plan->dev));
  return launch_checked(plan, inputs, outputs, workspace, (cudaStream_t)stream);
}

static int check_launch_args(const cb_plan* plan, const void* const* inputs, int n_inputs, void* const* outputs, int n_outputs,
                             const void* workspace) {
  if (!plan) return fail(CB_ERR_INVALID_ARG, "plan is NULL");
  if (n_inputs != plan->n_inputs)
    return fail(CB_ERR_INVALID_ARG, "%s expects %d inputs, got %d", plan->name.c_str(), plan->n_inputs, n_inputs);
  if (n_outputs != plan->n_outputs)
    return fail(CB_ERR_INVALID_ARG, "%s produces %d outputs, got %d", plan->name.c_str(), plan->n_outputs, n_outputs);
  for (int i = 0; i < n_inputs; i++)
    if (!inputs[i]) return fail(CB_ERR_INVALID_ARG, "%s: input %d is NULL", plan->name.c_str(), i);
  for (int i = 0; i < n_outputs; i++)
    if (!outputs[i]) return fail(CB_ERR_INVALID_ARG, "%s: output %d is NULL", plan->name.c_str(), i);
  if (plan->workspace_bytes && !workspace)
    return fail(CB_ERR_INVALID_ARG, "%s needs %zu bytes of workspace", plan->name.c_str(), plan->workspace_bytes);
  return CB_OK;
}

static int launch_checked(const cb_plan* plan, const void* const* inputs, void* const* outputs, void* workspace, cudaStream_t s) {
  switch (plan->kind) {
    case PLAN_QDENSE: return qdense_launch(plan, inputs, outputs, workspace, s);
    case PLAN_DOT: return dot_launch(plan, inputs, outputs, workspace, s);
    case PLAN_SDPA: return sdpa_launch(plan, inputs, outputs, workspace, s);
    case PLAN_GELU: case PLAN_SOFTMAX: case PLAN_LAYERNORM: case PLAN_COLS_BIAS: return fused_small_launch(plan, inputs, outputs, workspace, s);
    case PLAN_BINARY: case PLAN_UNARY: case PLAN_REDUCE: case PLAN_BROADCAST: case PLAN_RMSNORM: return elementwise_launch(plan, inputs, outputs, workspace, s);
    case PLAN_EMBEDDING: return embedding_lookup_launch(plan, inputs, outputs, workspace, s);
    default: return helper_launch(plan, inputs, outputs, workspace, s);
  }
}

}  // extern "C"

// A plan with its buffers fixed.  The tensor-core decode plan keeps its prepared launch arguments
// (encoded tensor maps, problem table already in the workspace); every other plan keeps the
// pointer lists and goes through its ordinary launch.
struct cb_bound {
  const cb_plan* plan = nullptr;
  std::vector<const void*> in;
  std::vector<void*> out;
  void* ws = nullptr;
  void* decode_tc = nullptr;
};

extern "C" {

int cb_plan_bind(const cb_plan* plan, const void* const* inputs, int n_inputs, void* const* outputs, int n_outputs,
                 void* workspace, cb_bound** bound) {
  clear_error();
  if (!bound) return fail(CB_ERR_INVALID_ARG, "cb_plan_bind: bound is NULL");
  *bound = nullptr;
  CB_TRY(check_launch_args(plan, inputs, n_inputs, outputs, n_outputs, workspace));
  CB_TRY(set_device(plan->dev));
  cb_bound* b = new cb_bound();
  b->plan = plan;
  b->in.assign(inputs, inputs + n_inputs);
  b->out.assign(outputs, outputs + n_outputs);
  b->ws = workspace;
  if (plan->kind == PLAN_QDENSE && plan->variant == CB_QDENSE_DECODE_TC) {
    const int st = qdense_decode_tc_bind(plan, b->in.data(), b->out.data(), workspace, &b->decode_tc);
    if (st != CB_OK) { delete b; return st; }
  }
  *bound = b;
  return CB_OK;
}

static int bound_launch(const cb_bound* b, cudaStream_t s) {
  if (b->decode_tc) return qdense_decode_tc_launch_bound(b->plan, b->decode_tc, s);
  return launch_checked(b->plan, b->in.data(), b->out.data(), b->ws, s);
}

int cb_bound_launch(const cb_bound* bound, cb_stream stream) {
  clear_error();
  if (!bound) return fail(CB_ERR_INVALID_ARG, "cb_bound_launch: bound is NULL");
  CB_TRY(set_device(bound->plan->dev));
  return bound_launch(bound, (cudaStream_t)stream);
}

int cb_bound_launch_many(const cb_bound* const* bounds, int n_bounds, cb_stream stream) {
  clear_error();
  if (n_bounds < 0 || (n_bounds > 0 && !bounds)) return fail(CB_ERR_INVALID_ARG, "cb_bound_launch_many: NULL argument");
  int dev = -1;
  for (int i = 0; i < n_bounds; i++) {
    if (!bounds[i]) return fail(CB_ERR_INVALID_ARG, "cb_bound_launch_many: bound %d is NULL", i);
    if (bounds[i]->plan->dev != dev) { dev = bounds[i]->plan->dev; CB_TRY(set_device(dev)); }
    CB_TRY(bound_launch(bounds[i], (cudaStream_t)stream));
  }
  return CB_OK;
}

int cb_bound_destroy(cb_bound* bound) {
  if (!bound) return CB_OK;
  if (bound->decode_tc) qdense_decode_tc_unbind(bound->decode_tc);
  delete bound;
  return CB_OK;
}

int cb_plan_check_status(const cb_plan* plan, const void* workspace) {
  clear_error();
  if (!plan) return fail(CB_ERR_INVALID_ARG, "plan is NULL");
  if (plan->kind == PLAN_EMBEDDING && workspace) { CB_TRY(set_device(plan->dev)); return embedding_lookup_check(plan, workspace); }
  if (!plan->has_status || !workspace) return CB_OK;
  CB_TRY(set_device(plan->dev));
  unsigned int word[2] = {0, 0};
  CB_CUDA(cudaMemcpy(word, workspace, sizeof(word), cudaMemcpyDeviceToHost));
  if (word[0] != 0)
    return fail(CB_ERR_TIMEOUT, "%s: a bounded device-side wait gave up (code %u, detail %u)",
                plan->name.c_str(), word[0], word[1]);
  return CB_OK;
}

int cb_plan_destroy(cb_plan* plan) {
  delete plan;
  return CB_OK;
}

}  // extern "C"
