// Element-wise and reduction ops a decoder block needs around its projections and attention:
// binary ops with the reference's broadcasting rule, unary ops, ReduceSum / ReduceMax,
// BroadcastInDim, the stacked reduction behind AllReduce, and a fused RMS-norm row kernel that
// the graph compiler substitutes for the decomposed form (the interface has no fused RMS norm).
// Reference behaviour: StandardOps (standard_ops.go:131-700: Add / Sub / Mul / Div / Max / Min,
// Neg / Exp / Rsqrt / Sqrt / Logistic / Tanh, ReduceSum / ReduceMax, BroadcastInDim :232-254),
// shape rule shapeinference.BinaryOp (shapeinference/shapeinference.go:219-300: equal ranks,
// each dimension equal or 1; a scalar takes the other side's shape), executors
// internal/gobackend/ops.  Half types compute in float32 and round once.
#include "common.cuh"

#include <algorithm>

namespace cb {

struct Idx8 { int64_t v[8]; };

template <typename T> struct EwT { typedef T acc; };
template <> struct EwT<__nv_bfloat16> { typedef float acc; };
template <> struct EwT<__half> { typedef float acc; };

template <typename A> __device__ __forceinline__ A ew_binary(A a, A b, int op) {
  switch (op) {
    case CB_BIN_ADD: return a + b;
    case CB_BIN_SUB: return a - b;
    case CB_BIN_MUL: return a * b;
    case CB_BIN_DIV: return a / b;
    case CB_BIN_MAX: return a > b ? a : (b > a ? b : (a != a ? a : b));     // NaN propagates, as Go's max
    default: return a < b ? a : (b < a ? b : (a != a ? a : b));
  }
}

template <typename A> __device__ __forceinline__ A ew_unary_f(A x, int op) {
  switch (op) {
    case CB_UN_NEG: return -x;
    case CB_UN_RSQRT: return (A)1 / sqrt(x);
    case CB_UN_SQRT: return sqrt(x);
    case CB_UN_EXP: return exp(x);
    case CB_UN_LOGISTIC: return (A)1 / ((A)1 + exp(-x));
    default: return tanh(x);
  }
}

// out[i] = lhs[bcast(i)] op rhs[bcast(i)]; strides are 0 along broadcast axes.
template <typename T>
__global__ void binary_kernel(const T* __restrict__ lhs, const T* __restrict__ rhs, T* __restrict__ out, int rank,
                              Idx8 out_dims, Idx8 ls, Idx8 rs, int64_t n, int op, int same) {
  pdl_enter();
  typedef typename EwT<T>::acc A;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t li = i, ri = i;
    if (!same) {
      int64_t rem = i;
      li = ri = 0;
      for (int a = rank - 1; a >= 0; a--) {
        const int64_t c = rem % out_dims.v[a];
        rem /= out_dims.v[a];
        li += c * ls.v[a];
        ri += c * rs.v[a];
      }
    }
    const A a = (A)Scalar<T>::load(lhs, li), b = (A)Scalar<T>::load(rhs, ri);
    Scalar<T>::store(out, i, ew_binary<A>(a, b, op));
  }
}
// Both operands of the output's shape, 16-byte aligned, a whole number of 16-byte vectors: a thread takes whole vectors,
// all its loads issued before the first use.  The arithmetic is the scalar kernel's (same conversions, same rounding).
template <typename T>
__global__ void __launch_bounds__(256)
binary_vec_kernel(const T* __restrict__ lhs, const T* __restrict__ rhs, T* __restrict__ out, int64_t n_vec, int op) {
  pdl_enter();
  typedef typename EwT<T>::acc A;
  constexpr int VEC = 16 / (int)sizeof(T);
  union V { uint4 u; T e[VEC]; };
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    V a, b, r;
    a.u = __ldg(reinterpret_cast<const uint4*>(lhs) + i);
    b.u = __ldg(reinterpret_cast<const uint4*>(rhs) + i);
#pragma unroll
    for (int e = 0; e < VEC; e++) Scalar<T>::store(r.e, e, ew_binary<A>((A)Scalar<T>::load(a.e, e), (A)Scalar<T>::load(b.e, e), op));
    reinterpret_cast<uint4*>(out)[i] = r.u;
  }
}
// integer flavour: no Scalar<> specialisations exist for the integer types
template <typename T>
__global__ void binary_int_kernel(const T* __restrict__ lhs, const T* __restrict__ rhs, T* __restrict__ out, int rank,
                                  Idx8 out_dims, Idx8 ls, Idx8 rs, int64_t n, int op) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, li = 0, ri = 0;
    for (int a = rank - 1; a >= 0; a--) {
      const int64_t c = rem % out_dims.v[a];
      rem /= out_dims.v[a];
      li += c * ls.v[a];
      ri += c * rs.v[a];
    }
    const T a = lhs[li], b = rhs[ri];
    T r;
    switch (op) {
      case CB_BIN_ADD: r = a + b; break;
      case CB_BIN_SUB: r = a - b; break;
      case CB_BIN_MUL: r = a * b; break;
      case CB_BIN_DIV: r = b != 0 ? a / b : 0; break;
      case CB_BIN_MAX: r = a > b ? a : b; break;
      default: r = a < b ? a : b; break;
    }
    out[i] = r;
  }
}

template <typename T>
__global__ void unary_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n, int op) {
  pdl_enter();
  typedef typename EwT<T>::acc A;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    Scalar<T>::store(out, i, ew_unary_f<A>((A)Scalar<T>::load(x, i), op));
}

// One warp per output element: the kept axes give the base offset, the lanes stride over the
// reduced index space.  op: cb_reduce_op.
template <typename T>
__global__ void reduce_kernel(const T* __restrict__ x, T* __restrict__ out, int kept_rank, Idx8 kept_dims, Idx8 kept_strides,
                              int red_rank, Idx8 red_dims, Idx8 red_strides, int64_t n_out, int64_t n_red, int op) {
  typedef typename EwT<T>::acc A;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t o = warp; o < n_out; o += n_warps) {
    int64_t rem = o, base = 0;
    for (int a = kept_rank - 1; a >= 0; a--) {
      base += (rem % kept_dims.v[a]) * kept_strides.v[a];
      rem /= kept_dims.v[a];
    }
    A acc = op == CB_REDUCE_SUM ? (A)0 : (op == CB_REDUCE_PRODUCT ? (A)1 : (A)Scalar<T>::load(x, base));
    for (int64_t r = lane; r < n_red; r += 32) {
      int64_t rr = r, off = base;
      for (int a = red_rank - 1; a >= 0; a--) {
        off += (rr % red_dims.v[a]) * red_strides.v[a];
        rr /= red_dims.v[a];
      }
      const A v = (A)Scalar<T>::load(x, off);
      acc = op == CB_REDUCE_SUM ? acc + v : (op == CB_REDUCE_PRODUCT ? acc * v : (op == CB_REDUCE_MAX ? ew_binary<A>(acc, v, CB_BIN_MAX) : ew_binary<A>(acc, v, CB_BIN_MIN)));
    }
    for (int d = 16; d > 0; d >>= 1) {
      const A v = __shfl_xor_sync(0xFFFFFFFFu, acc, d);
      acc = op == CB_REDUCE_SUM ? acc + v : (op == CB_REDUCE_PRODUCT ? acc * v : (op == CB_REDUCE_MAX ? ew_binary<A>(acc, v, CB_BIN_MAX) : ew_binary<A>(acc, v, CB_BIN_MIN)));
    }
    if (lane == 0) Scalar<T>::store(out, o, acc);
  }
}

template <typename T>
__global__ void broadcast_kernel(const T* __restrict__ x, T* __restrict__ out, int rank, Idx8 out_dims, Idx8 in_strides, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, src = 0;
    for (int a = rank - 1; a >= 0; a--) {
      src += (rem % out_dims.v[a]) * in_strides.v[a];
      rem /= out_dims.v[a];
    }
    out[i] = x[src];
  }
}

// out[i] = reduce over r of stacked[r][i], in rank order (every replica reduces in the same order,
// so all replicas of an AllReduce hold the same bits).
template <typename T>
__global__ void stacked_reduce_kernel(const T* __restrict__ stacked, T* __restrict__ out, int64_t n, int g, int op) {
  typedef typename EwT<T>::acc A;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    A acc = (A)Scalar<T>::load(stacked, i);
    for (int r = 1; r < g; r++) {
      const A v = (A)Scalar<T>::load(stacked, (int64_t)r * n + i);
      acc = op == CB_REDUCE_SUM ? acc + v : (op == CB_REDUCE_PRODUCT ? acc * v : (op == CB_REDUCE_MAX ? ew_binary<A>(acc, v, CB_BIN_MAX) : ew_binary<A>(acc, v, CB_BIN_MIN)));
    }
    Scalar<T>::store(out, i, acc);
  }
}

// y[row, :] = x[row, :] * rsqrt(mean(x[row, :]^2) + eps) (* gamma).  One block per row; the row is
// read once into registers (up to 8 elements per thread) or re-read when longer.
constexpr int RMS_THREADS = 256;
template <typename T>
__global__ void __launch_bounds__(RMS_THREADS)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ gamma, T* __restrict__ out, int64_t rows, int64_t L, float eps) {
  pdl_enter();
  __shared__ float s_part[RMS_THREADS / 32];
  __shared__ float s_inv;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * L;
    float v[8];
    float ss = 0.0f;
    const bool in_regs = L <= (int64_t)RMS_THREADS * 8;
    if (in_regs) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int64_t c = threadIdx.x + (int64_t)j * RMS_THREADS;
        v[j] = c < L ? (float)Scalar<T>::load(xr, c) : 0.0f;
        ss += v[j] * v[j];
      }
    } else {
      for (int64_t c = threadIdx.x; c < L; c += RMS_THREADS) { const float t = (float)Scalar<T>::load(xr, c); ss += t * t; }
    }
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int w = 0; w < RMS_THREADS / 32; w++) t += s_part[w];
      s_inv = rsqrtf(t / (float)L + eps);
    }
    __syncthreads();
    const float inv = s_inv;
    if (in_regs) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int64_t c = threadIdx.x + (int64_t)j * RMS_THREADS;
        if (c < L) Scalar<T>::store(out + row * L, c, v[j] * inv * (gamma ? (float)Scalar<T>::load(gamma, c) : 1.0f));
      }
    } else {
      for (int64_t c = threadIdx.x; c < L; c += RMS_THREADS)
        Scalar<T>::store(out + row * L, c, (float)Scalar<T>::load(xr, c) * inv * (gamma ? (float)Scalar<T>::load(gamma, c) : 1.0f));
    }
    __syncthreads();      // s_part / s_inv are rewritten for the next row
  }
}
// The streaming form for rows whose bytes are a multiple of 16: WPR warps per row (1 for short rows, 4 from 128 vectors
// up, so that a few thousand rows still fill the SMs with loads in flight), the row read once with 16-byte loads into
// registers (NV vectors per lane), reduced by shuffles and, for WPR > 1, one exchange through shared memory, written
// with 16-byte stores.  Rows are taken block-wide in a grid-stride loop, so every thread reaches every barrier.
template <typename T, int NV, int WPR>
__global__ void __launch_bounds__(RMS_THREADS)
rmsnorm_vec_kernel(const T* __restrict__ x, const T* __restrict__ gamma, T* __restrict__ out, int64_t rows, int64_t L, float eps) {
  pdl_enter();
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int RPB = RMS_THREADS / 32 / WPR;             // rows per block and pass
  __shared__ float s_part[RPB][WPR];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r_in = warp / WPR, w_in = warp % WPR;
  const int64_t n_vec = L / VEC;
  for (int64_t row0 = (int64_t)blockIdx.x * RPB; row0 < rows; row0 += (int64_t)gridDim.x * RPB) {
    const int64_t row = row0 + r_in;
    const bool live = row < rows;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * L);
    uint4 raw[NV];
#pragma unroll
    for (int j = 0; j < NV; j++) {
      const int64_t c = (int64_t)(j * WPR + w_in) * 32 + lane;
      raw[j] = (live && c < n_vec) ? __ldg(xr + c) : make_uint4(0, 0, 0, 0);
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; j++) {
      const T* e = reinterpret_cast<const T*>(&raw[j]);
#pragma unroll
      for (int i = 0; i < VEC; i++) { const float t = (float)e[i]; ss = fmaf(t, t, ss); }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
    if (WPR > 1) {
      if (lane == 0) s_part[r_in][w_in] = ss;
      __syncthreads();
      ss = 0.0f;
#pragma unroll
      for (int k = 0; k < WPR; k++) ss += s_part[r_in][k];
      __syncthreads();                      // the partials are rewritten in the next pass
    }
    const float inv = rsqrtf(ss / (float)L + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + row * L);
#pragma unroll
    for (int j = 0; j < NV; j++) {
      const int64_t c = (int64_t)(j * WPR + w_in) * 32 + lane;
      if (live && c < n_vec) {
        uint4 gv = make_uint4(0, 0, 0, 0);
        if (gamma) gv = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
        const T* e = reinterpret_cast<const T*>(&raw[j]);
        const T* ge = reinterpret_cast<const T*>(&gv);
        uint4 ov;
        T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int i = 0; i < VEC; i++) oe[i] = (T)((float)e[i] * inv * (gamma ? (float)ge[i] : 1.0f));
        orow[c] = ov;
      }
    }
  }
}
template <>
__global__ void __launch_bounds__(RMS_THREADS)
rmsnorm_kernel<double>(const double* __restrict__ x, const double* __restrict__ gamma, double* __restrict__ out, int64_t rows, int64_t L, float eps) {
  pdl_enter();
  __shared__ double s_part[RMS_THREADS / 32];
  __shared__ double s_inv;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const double* xr = x + row * L;
    double ss = 0.0;
    for (int64_t c = threadIdx.x; c < L; c += RMS_THREADS) ss += xr[c] * xr[c];
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      double t = 0.0;
      for (int w = 0; w < RMS_THREADS / 32; w++) t += s_part[w];
      s_inv = 1.0 / sqrt(t / (double)L + (double)eps);
    }
    __syncthreads();
    for (int64_t c = threadIdx.x; c < L; c += RMS_THREADS) out[row * L + c] = xr[c] * s_inv * (gamma ? gamma[c] : 1.0);
    __syncthreads();
  }
}

static int ew_grid(int64_t n) { return (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, 148 * 8)); }

template <typename F>
static int by_float(int dtype, const char* op, F&& f) {
  switch (dtype) {
    case CB_F32: return f((float*)nullptr);
    case CB_F64: return f((double*)nullptr);
    case CB_BF16: return f((__nv_bfloat16*)nullptr);
    case CB_F16: return f((__half*)nullptr);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dtype %s is not implemented", op, dtype_name(dtype));
  }
}

static const char* bin_name(int op) {
  static const char* n[] = {"add", "sub", "mul", "div", "max", "min"};
  return n[op];
}
static const char* un_name(int op) {
  static const char* n[] = {"neg", "rsqrt", "sqrt", "exp", "logistic", "tanh"};
  return n[op];
}
static const char* red_name(int op) {
  static const char* n[] = {"sum", "product", "max", "min"};
  return n[op];
}

// HelperDesc use: binary: dims = lhs dims, starts = rhs dims, out_dims, axis = op; unary: n, axis = op;
// reduce: dims = operand dims, perm[a] = 1 for reduced axes, axis = op; broadcast: dims = operand dims
// (rank flags), out_dims, perm = broadcast axes; rms norm: dims[0] rows, dims[1] row length, eps, flags bit 0 gamma.
int elementwise_plan(cb_plan* p) {
  HelperDesc& h = p->helper;
  p->n_outputs = 1;
  p->threads = 256;
  const bool is_flt = h.dtype == CB_F32 || h.dtype == CB_F64 || h.dtype == CB_BF16 || h.dtype == CB_F16;
  const bool is_int = h.dtype == CB_I32 || h.dtype == CB_I64;
  switch (p->kind) {
    case PLAN_BINARY: {
      if (h.axis < CB_BIN_ADD || h.axis > CB_BIN_MIN) return fail(CB_ERR_INVALID_ARG, "binary op %d unknown", h.axis);
      if (!is_flt && !is_int) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dtype %s is not implemented", bin_name(h.axis), dtype_name(h.dtype));
      h.n = 1;
      for (int a = 0; a < h.rank; a++) {
        const int64_t l = h.dims[a], r = h.starts[a];
        if (l != r && l != 1 && r != 1)
          return fail(CB_ERR_INVALID_ARG, "dimension of axis #%d doesn't match and cannot be broadcast for BinaryOp (%s), got %lld and %lld",
                      a, bin_name(h.axis), (long long)l, (long long)r);
        h.out_dims[a] = l == 1 ? r : l;
        h.n *= h.out_dims[a];
      }
      p->n_inputs = 2;
      p->name = std::string("binary_") + bin_name(h.axis) + "_" + dtype_name(h.dtype);
      break;
    }
    case PLAN_UNARY:
      if (h.axis < CB_UN_NEG || h.axis > CB_UN_TANH) return fail(CB_ERR_INVALID_ARG, "unary op %d unknown", h.axis);
      if (!is_flt) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dtype %s is not implemented", un_name(h.axis), dtype_name(h.dtype));
      p->n_inputs = 1;
      p->name = std::string("unary_") + un_name(h.axis) + "_" + dtype_name(h.dtype);
      break;
    case PLAN_REDUCE: {
      if (h.axis < CB_REDUCE_SUM || h.axis > CB_REDUCE_MIN) return fail(CB_ERR_INVALID_ARG, "reduce op %d unknown", h.axis);
      if (!is_flt) return fail(CB_ERR_NOT_IMPLEMENTED, "Reduce%s: dtype %s is not implemented", red_name(h.axis), dtype_name(h.dtype));
      h.n = 1;
      for (int a = 0; a < h.rank; a++) if (!h.perm[a]) h.n *= h.dims[a];
      p->n_inputs = 1;
      p->name = std::string("reduce_") + red_name(h.axis) + "_" + dtype_name(h.dtype);
      break;
    }
    case PLAN_BROADCAST: {
      if (dtype_size(h.dtype) == 0) return fail(CB_ERR_NOT_IMPLEMENTED, "BroadcastInDim: dtype %s is not implemented", dtype_name(h.dtype));
      h.n = 1;
      const int out_rank = (int)h.strides[0];
      for (int a = 0; a < out_rank; a++) h.n *= h.out_dims[a];
      int prev = -1;
      for (int a = 0; a < h.rank; a++) {
        const int t = h.perm[a];
        if (t <= prev || t >= out_rank) return fail(CB_ERR_INVALID_ARG, "BroadcastInDim: broadcastAxes must be increasing and inside the output rank");
        if (h.dims[a] != 1 && h.dims[a] != h.out_dims[t])
          return fail(CB_ERR_INVALID_ARG, "BroadcastInDim: operand axis %d (%lld) cannot be broadcast into output axis %d (%lld)", a,
                      (long long)h.dims[a], t, (long long)h.out_dims[t]);
        prev = t;
      }
      p->n_inputs = 1;
      p->name = "broadcast_in_dim";
      break;
    }
    case PLAN_RMSNORM:
      if (!is_flt) return fail(CB_ERR_NOT_IMPLEMENTED, "rms norm: dtype %s is not implemented", dtype_name(h.dtype));
      h.n = h.dims[0] * h.dims[1];
      p->n_inputs = 1 + (h.flags & 1);
      p->name = std::string("rms_norm_") + dtype_name(h.dtype);
      p->blocks = (int)std::max<int64_t>(1, std::min<int64_t>(h.dims[0], 148 * 8));
      p->threads = RMS_THREADS;
      return CB_OK;
    default: return fail(CB_ERR_INVALID_ARG, "unknown element-wise plan kind %d", p->kind);
  }
  if (h.n < 0) return fail(CB_ERR_INVALID_ARG, "negative element count");
  p->blocks = ew_grid(h.n);
  return CB_OK;
}

static void row_major_strides(int rank, const int64_t* dims, int64_t* strides) {
  int64_t mul = 1;
  for (int a = rank - 1; a >= 0; a--) { strides[a] = mul; mul *= dims[a]; }
}

int elementwise_launch(const cb_plan* p, const void* const* in, void* const* out, void*, cudaStream_t s) {
  const HelperDesc& h = p->helper;
  if (h.n == 0) return CB_OK;
  switch (p->kind) {
    case PLAN_BINARY: {
      Idx8 od, ls, rs;
      int64_t lst[8], rst[8];
      row_major_strides(h.rank, h.dims, lst);
      row_major_strides(h.rank, h.starts, rst);
      bool same = true;
      for (int a = 0; a < 8; a++) {
        od.v[a] = a < h.rank ? h.out_dims[a] : 1;
        ls.v[a] = a < h.rank && h.dims[a] != 1 ? lst[a] : 0;
        rs.v[a] = a < h.rank && h.starts[a] != 1 ? rst[a] : 0;
        if (a < h.rank && (h.dims[a] != h.out_dims[a] || h.starts[a] != h.out_dims[a])) same = false;
      }
      if (h.dtype == CB_I32) binary_int_kernel<int32_t><<<p->blocks, 256, 0, s>>>((const int32_t*)in[0], (const int32_t*)in[1], (int32_t*)out[0], h.rank, od, ls, rs, h.n, h.axis);
      else if (h.dtype == CB_I64) binary_int_kernel<int64_t><<<p->blocks, 256, 0, s>>>((const int64_t*)in[0], (const int64_t*)in[1], (int64_t*)out[0], h.rank, od, ls, rs, h.n, h.axis);
      else CB_TRY(by_float(h.dtype, "binary op", [&](auto* t) {
        typedef typename std::remove_pointer<decltype(t)>::type T;
        constexpr int VEC = 16 / (int)sizeof(T);
        const bool aligned = !((reinterpret_cast<uintptr_t>(in[0]) | reinterpret_cast<uintptr_t>(in[1]) | reinterpret_cast<uintptr_t>(out[0])) & 15);
        if (same && aligned && h.n % VEC == 0 && h.n > 0) {
          const int64_t n_vec = h.n / VEC;
          CB_CUDA(launch_dependent(binary_vec_kernel<T>, dim3((unsigned)ew_grid(n_vec)), dim3(256), 0, s, (const T*)in[0], (const T*)in[1], (T*)out[0], n_vec,
                                   (int)h.axis));
          return (int)CB_OK;
        }
        CB_CUDA(launch_dependent(binary_kernel<T>, dim3(p->blocks), dim3(256), 0, s, (const T*)in[0], (const T*)in[1], (T*)out[0], (int)h.rank, od, ls, rs,
                                 (int64_t)h.n, (int)h.axis, same ? 1 : 0));
        return (int)CB_OK;
      }));
      break;
    }
    case PLAN_UNARY:
      CB_TRY(by_float(h.dtype, "unary op", [&](auto* t) {
        typedef typename std::remove_pointer<decltype(t)>::type T;
        CB_CUDA(launch_dependent(unary_kernel<T>, dim3(p->blocks), dim3(256), 0, s, (const T*)in[0], (T*)out[0], (int64_t)h.n, (int)h.axis));
        return (int)CB_OK;
      }));
      break;
    case PLAN_REDUCE: {
      int64_t st[8];
      row_major_strides(h.rank, h.dims, st);
      Idx8 kd, ks, rd, rs;
      int kr = 0, rr = 0;
      int64_t n_red = 1;
      for (int a = 0; a < 8; a++) { kd.v[a] = rd.v[a] = 1; ks.v[a] = rs.v[a] = 0; }
      for (int a = 0; a < h.rank; a++) {
        if (h.perm[a]) { rd.v[rr] = h.dims[a]; rs.v[rr] = st[a]; rr++; n_red *= h.dims[a]; }
        else { kd.v[kr] = h.dims[a]; ks.v[kr] = st[a]; kr++; }
      }
      const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((h.n + 7) / 8, 148 * 8));
      CB_TRY(by_float(h.dtype, "reduce", [&](auto* t) {
        typedef typename std::remove_pointer<decltype(t)>::type T;
        reduce_kernel<T><<<blocks, 256, 0, s>>>((const T*)in[0], (T*)out[0], kr, kd, ks, rr, rd, rs, h.n, n_red, h.axis);
        return (int)CB_OK;
      }));
      break;
    }
    case PLAN_BROADCAST: {
      const int out_rank = (int)h.strides[0];
      int64_t st[8];
      row_major_strides(h.rank, h.dims, st);
      Idx8 od, is;
      for (int a = 0; a < 8; a++) { od.v[a] = a < out_rank ? h.out_dims[a] : 1; is.v[a] = 0; }
      for (int a = 0; a < h.rank; a++) if (h.dims[a] != 1) is.v[h.perm[a]] = st[a];
      switch (dtype_size(h.dtype)) {
        case 1: broadcast_kernel<uint8_t><<<p->blocks, 256, 0, s>>>((const uint8_t*)in[0], (uint8_t*)out[0], out_rank, od, is, h.n); break;
        case 2: broadcast_kernel<uint16_t><<<p->blocks, 256, 0, s>>>((const uint16_t*)in[0], (uint16_t*)out[0], out_rank, od, is, h.n); break;
        case 4: broadcast_kernel<uint32_t><<<p->blocks, 256, 0, s>>>((const uint32_t*)in[0], (uint32_t*)out[0], out_rank, od, is, h.n); break;
        default: broadcast_kernel<uint64_t><<<p->blocks, 256, 0, s>>>((const uint64_t*)in[0], (uint64_t*)out[0], out_rank, od, is, h.n); break;
      }
      break;
    }
    case PLAN_RMSNORM:
      CB_TRY(by_float(h.dtype, "rms norm", [&](auto* t) {
        typedef typename std::remove_pointer<decltype(t)>::type T;
        const T* g = (h.flags & 1) ? (const T*)in[1] : nullptr;
        if constexpr (sizeof(T) <= 4) {
          constexpr int VEC = 16 / (int)sizeof(T);
          const int64_t L = h.dims[1], n_vec = L / VEC;
          const bool aligned = !((reinterpret_cast<uintptr_t>(in[0]) | reinterpret_cast<uintptr_t>(out[0]) | reinterpret_cast<uintptr_t>(g)) & 15);
          const int wpr = n_vec >= 128 ? 4 : 1;
          const int64_t per_lane = (n_vec + 32 * wpr - 1) / (32 * wpr);
          if (L % VEC == 0 && per_lane <= 8 && aligned) {
            const int rpb = RMS_THREADS / 32 / wpr;
            const int64_t want = (h.dims[0] + rpb - 1) / rpb;
            const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)p->n_sm * 8));
            auto go = [&](auto nv, auto w) {
              launch_dependent(rmsnorm_vec_kernel<T, decltype(nv)::value, decltype(w)::value>, dim3(grid), dim3(RMS_THREADS), 0, s, (const T*)in[0], g, (T*)out[0],
                               (int64_t)h.dims[0], L, (float)h.eps);
            };
            auto by_nv = [&](auto w) {
              if (per_lane <= 1) go(std::integral_constant<int, 1>(), w); else if (per_lane <= 2) go(std::integral_constant<int, 2>(), w);
              else if (per_lane <= 4) go(std::integral_constant<int, 4>(), w); else go(std::integral_constant<int, 8>(), w);
            };
            if (wpr == 4) by_nv(std::integral_constant<int, 4>()); else by_nv(std::integral_constant<int, 1>());
            return (int)CB_OK;
          }
        }
        CB_CUDA(launch_dependent(rmsnorm_kernel<T>, dim3(p->blocks), dim3(RMS_THREADS), 0, s, (const T*)in[0], g, (T*)out[0], (int64_t)h.dims[0], (int64_t)h.dims[1],
                                 (float)h.eps));
        return (int)CB_OK;
      }));
      break;
    default: return fail(CB_ERR_INVALID_ARG, "unknown element-wise plan kind %d", p->kind);
  }
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

int stacked_reduce_launch(int dtype, int op, const void* stacked, int g, int64_t n, void* out, cudaStream_t s) {
  if (n == 0) return CB_OK;
  if (op < CB_REDUCE_SUM || op > CB_REDUCE_MIN) return fail(CB_ERR_INVALID_ARG, "AllReduce: unknown reduction %d", op);
  CB_TRY(by_float(dtype, "AllReduce", [&](auto* t) {
    typedef typename std::remove_pointer<decltype(t)>::type T;
    stacked_reduce_kernel<T><<<ew_grid(n), 256, 0, s>>>((const T*)stacked, (T*)out, n, g, op);
    return (int)CB_OK;
  }));
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}


// ---------------------------------------------------------------------------
// several device-to-device copies as one launch
// ---------------------------------------------------------------------------
// The results of a replayed graph live in the graph's own memory and are handed to the caller as fresh buffers: one
// launch copies all of them (16-byte vectors, every pointer 16-byte aligned) instead of one copy engine call each.
constexpr int COPY_MANY_MAX = 16;
struct CopyMany {
  const uint4* src[COPY_MANY_MAX];
  uint4* dst[COPY_MANY_MAX];
  unsigned long long vecs[COPY_MANY_MAX];      // 16-byte vectors per copy
  int n;
};
__global__ void __launch_bounds__(256) copy_many_kernel(const CopyMany c) {
  for (int k = 0; k < c.n; k++) {
    const uint4* s = c.src[k];
    uint4* d = c.dst[k];
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < c.vecs[k]; i += (unsigned long long)gridDim.x * blockDim.x)
      d[i] = s[i];
  }
}

int copy_many_max() { return COPY_MANY_MAX; }

// n <= copy_many_max() copies of bytes[k] from src[k] to dst[k] on one device; every pointer and size a multiple of 16
int copy_many(int n_sm, int n, void* const* dst, const void* const* src, const size_t* bytes, cudaStream_t s) {
  if (n <= 0) return CB_OK;
  if (n > COPY_MANY_MAX) return fail(CB_ERR_INVALID_ARG, "copy_many: %d copies, at most %d", n, COPY_MANY_MAX);
  CopyMany c;
  memset(&c, 0, sizeof(c));
  c.n = n;
  unsigned long long total = 0;
  for (int k = 0; k < n; k++) {
    if ((reinterpret_cast<uintptr_t>(dst[k]) | reinterpret_cast<uintptr_t>(src[k]) | bytes[k]) & 15)
      return fail(CB_ERR_INVALID_ARG, "copy_many: pointers and sizes must be multiples of 16 bytes");
    c.src[k] = reinterpret_cast<const uint4*>(src[k]);
    c.dst[k] = reinterpret_cast<uint4*>(dst[k]);
    c.vecs[k] = bytes[k] / 16;
    total += c.vecs[k];
  }
  if (total == 0) return CB_OK;
  const unsigned long long want = (total + 256 * 4 - 1) / (256 * 4);          // about four vectors per thread
  const unsigned blocks = (unsigned)std::min<unsigned long long>(std::max<unsigned long long>(want, 1), (unsigned long long)(n_sm > 0 ? n_sm : 148) * 8);
  copy_many_kernel<<<blocks, 256, 0, s>>>(c);        // an ordinary launch: it may follow a graph launch
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

}  // namespace cb
