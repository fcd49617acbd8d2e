// Shared declarations of libcudabackend's translation units: error plumbing,
// the plan object, dtype helpers and the device-side scalar conversions that
// must follow the reference's rounding rules.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>

#include "../../include/cudabackend.h"

namespace cb {

// ---- errors -----------------------------------------------------------------
int fail(int status, const char* fmt, ...);   // records the thread-local message, returns status
void clear_error();

#define CB_CUDA(expr)                                                                      \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess) {                                                               \
      (void)cudaGetLastError();                                                            \
      return cb::fail(_e == cudaErrorMemoryAllocation ? CB_ERR_OOM : CB_ERR_CUDA,          \
                      "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__,    \
                      __LINE__);                                                           \
    }                                                                                      \
  } while (0)

#define CB_TRY(expr)            \
  do {                          \
    int _s = (expr);            \
    if (_s != CB_OK) return _s; \
  } while (0)

// Makes `dev` current for the calling thread (cgo calls may land on any OS thread).
int set_device(int dev);
int sm_count(int dev);
bool host_range_is_page_locked(const void* p, size_t bytes);   // inside a range cb_host_alloc returned
// several same-device copies as one kernel launch (elementwise.cu): pointers and sizes multiples of 16 bytes
int copy_many_max();
int copy_many(int n_sm, int n, void* const* dst, const void* const* src, const size_t* bytes, cudaStream_t s);

// cuTensorMapEncodeTiled resolved through the runtime (no link-time libcuda dependency).
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn tensor_map_encoder();

// ---- dtypes -----------------------------------------------------------------
inline size_t dtype_size(int d) {
  switch (d) {
    case CB_BOOL: case CB_I8: case CB_U8: case CB_F8E5M2: case CB_F8E4M3FN: return 1;
    case CB_I16: case CB_U16: case CB_F16: case CB_BF16: return 2;
    case CB_I32: case CB_U32: case CB_F32: return 4;
    case CB_I64: case CB_U64: case CB_F64: return 8;
    default: return 0;
  }
}
const char* dtype_name(int d);

// ---- plans ------------------------------------------------------------------
enum PlanKind { PLAN_QDENSE = 1, PLAN_DOT, PLAN_SDPA, PLAN_COPY, PLAN_CONVERT, PLAN_IOTA,
                PLAN_SLICE, PLAN_TRANSPOSE, PLAN_GELU, PLAN_SOFTMAX, PLAN_LAYERNORM, PLAN_COLS_BIAS,
                PLAN_BINARY, PLAN_UNARY, PLAN_REDUCE, PLAN_BROADCAST, PLAN_RMSNORM, PLAN_EMBEDDING };

struct HelperDesc {
  int32_t dtype = 0, dtype_to = 0, rank = 0, axis = 0;
  int64_t n = 0;
  int64_t dims[8] = {0}, starts[8] = {0}, strides[8] = {0}, out_dims[8] = {0};
  int32_t perm[8] = {0};
  double eps = 0.0;        // layer norm
  int32_t flags = 0;       // layer norm: 1 = gamma, 2 = beta
};

}  // namespace cb

struct cb_plan {
  int kind = 0;
  int dev = 0;
  int variant = 0;
  int n_inputs = 0;
  int n_outputs = 1;
  int n_sm = 0;
  size_t workspace_bytes = 0;
  size_t counter_bytes = 0;       // leading region of the workspace zeroed by prepare
  int blocks = 0, threads = 0, dyn_smem = 0;
  bool has_status = false;        // kernel keeps a status word at workspace offset 0
  bool w4_stream = false;         // quantized dense on packed 4-bit weights: the streaming decode kernel, not the generic one
  bool whole_tiles = false;       // decode tensor-core plan: every CTA takes whole column tiles (nothing is split or parked)
  int tile_cluster = 0;           // decode tensor-core plan: CTAs per column tile when these form a thread-block cluster (0: no clusters)
  std::string name;
  cb_qdense_desc qd{};
  std::vector<cb_qdense_member> group;   // members of a grouped decode plan (one entry for an ordinary plan)
  cb_dot_desc dot{};
  cb_sdpa_desc sdpa{};
  cb::HelperDesc helper{};
};

namespace cb {

int qdense_plan(cb_plan* p);
int qdense_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int qdense_group_plan(cb_plan* p);
// Bound form of the tensor-core decode plan: everything a launch needs, prepared once.
int qdense_decode_tc_bind(const cb_plan* p, const void* const* in, void* const* out, void* ws, void** impl);
int qdense_decode_tc_launch_bound(const cb_plan* p, const void* impl, cudaStream_t s);
void qdense_decode_tc_unbind(void* impl);
int dot_plan(cb_plan* p);
int dot_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int sdpa_plan(cb_plan* p);
int sdpa_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int helper_plan(cb_plan* p);
int helper_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int fused_small_plan(cb_plan* p);
int fused_small_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int elementwise_plan(cb_plan* p);
int qdense_ggml_plan(cb_plan* p);
int qdense_ggml_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
bool qdense_w4_supports(const cb_qdense_desc& d);
void qdense_w4_plan(cb_plan* p);
int qdense_w4_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
bool qdense_ggml_mma_supports(const cb_qdense_desc& d);
void qdense_ggml_mma_plan(cb_plan* p, const char* type_name);
int qdense_ggml_mma_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int embedding_lookup_plan(cb_plan* p);
int embedding_lookup_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int embedding_lookup_check(const cb_plan* p, const void* ws);
int elementwise_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
// out[i] = reduction over r of stacked[r][i], r in rank order (the local step of AllReduce)
int stacked_reduce_launch(int dtype, int op, const void* stacked, int g, int64_t n, void* out, cudaStream_t s);
int peer_signal_launch(void* const* flags, int n_ranks, int slot, cudaStream_t s);
int peer_signal_wait_launch(void* const* flags, int n_ranks, int slot, const unsigned* local, uint32_t target, unsigned* status_word, cudaStream_t s);
int peer_wait_launch(const unsigned* flags, int n_flags, uint32_t target, unsigned* status_word, cudaStream_t s);

// ---- device scalar helpers --------------------------------------------------
// bf16 <-> f32 exactly as dtypes/bfloat16/bfloat16.go:25-39 of the reference:
// round to nearest even; NaN/Inf keep their top 16 bits.
__host__ __device__ inline uint16_t f32_to_bf16_bits(float x) {
#ifdef __CUDA_ARCH__
  uint32_t b = __float_as_uint(x);
#else
  uint32_t b; memcpy(&b, &x, 4);
#endif
  if ((b & 0x7F800000u) == 0x7F800000u) return (uint16_t)(b >> 16);
  b += 0x7FFFu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}
__device__ inline float bf16_bits_to_f32(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }

template <typename T> struct Scalar;   // load as compute type / store from compute type
template <> struct Scalar<float> {
  typedef float acc_t;
  __device__ static float load(const float* p, int64_t i) { return p[i]; }
  __device__ static void store(float* p, int64_t i, float v) { p[i] = v; }
};
template <> struct Scalar<double> {
  typedef double acc_t;
  __device__ static double load(const double* p, int64_t i) { return p[i]; }
  __device__ static void store(double* p, int64_t i, double v) { p[i] = v; }
};
template <> struct Scalar<__nv_bfloat16> {
  typedef float acc_t;
  __device__ static float load(const __nv_bfloat16* p, int64_t i) {
    return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p)[i]);
  }
  __device__ static void store(__nv_bfloat16* p, int64_t i, float v) {
    reinterpret_cast<uint16_t*>(p)[i] = f32_to_bf16_bits(v);
  }
};
template <> struct Scalar<__half> {
  typedef float acc_t;
  __device__ static float load(const __half* p, int64_t i) { return __half2float(p[i]); }
  __device__ static void store(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }
};

// A launch that may be scheduled while the kernel before it in the stream is still running (programmatic dependent
// launch): the kernel must execute pdl_enter() before it reads or writes memory.  pdl_enter also lets the kernel after
// this one be scheduled early, under the same condition.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename Kernel, typename... Args>
inline cudaError_t launch_dependent(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// fusedDenseApplyActivation (internal/gobackend/fusedops/dense.go:176-205) in f32.
__device__ inline float apply_activation(float x, int act) {
  switch (act) {
    case CB_ACT_GELU: return (x * 0.5f) * (1.0f + erff(x * 0.70710678118654752440f));
    case CB_ACT_RELU: return x < 0.0f ? 0.0f : x;
    case CB_ACT_SILU: return x / (1.0f + expf(-x));
    case CB_ACT_HARDSWISH: {
      float g = fminf(fmaxf(__fadd_rn(__fmul_rn(x, (float)(1.0 / 6.0)), 0.5f), 0.0f), 1.0f);
      return __fmul_rn(x, g);
    }
    case CB_ACT_TANH: return tanhf(x);
    default: return x;
  }
}

}  // namespace cb
