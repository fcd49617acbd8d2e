// FusedGelu, FusedSoftmax and FusedLayerNorm (FusedOps, fused_ops.go:318-334): the bandwidth-bound
// companions of the dense ops.  One pass over HBM each: a row (softmax axis / normalised extent) is
// staged in shared memory, reduced by its CTA, and written once.
//   gelu       internal/gobackend/fusedops/gelu.go:113-126 (exact: erf; approximate: tanh)
//   softmax    internal/gobackend/fusedops/softmax.go:83-118 (max, exp(x - max), sum, scale)
//   layer norm internal/gobackend/fusedops/layernorm.go:129-168 (mean, variance of the differences,
//              1 / sqrt(var + eps), gamma, beta) over trailing axes; other axis sets are transposed
//              to trailing ones by the graph layer
// Float32 and Float64 as in the reference, BFloat16 / Float16 computed in f32 (gelu: as the reference's
// half-precision path gelu.go:128-145; softmax and layer norm: an extension).
#include "common.cuh"

namespace cb {

constexpr int FS_THREADS = 256;
constexpr int FS_SMEM_BYTES = 40 * 1024;      // row cache; longer rows are re-read from L2 / HBM

// FAST (16-bit element types): the hardware exponential, whose error is far below one unit of the output type.
template <typename A, bool FAST = false> __device__ __forceinline__ A fs_exp(A x);
template <> __device__ __forceinline__ float fs_exp<float, false>(float x) { return expf(x); }
template <> __device__ __forceinline__ float fs_exp<float, true>(float x) { return __expf(x); }
template <> __device__ __forceinline__ double fs_exp<double, false>(double x) { return exp(x); }

template <typename A> __device__ __forceinline__ A fs_gelu(A x, bool exact);
template <> __device__ __forceinline__ float fs_gelu<float>(float x, bool exact) {
  if (exact) return (x * 0.5f) * (1.0f + erff(x * 0.70710678118654752440f));
  const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return (x * 0.5f) * (1.0f + tanhf(inner));
}
template <> __device__ __forceinline__ double fs_gelu<double>(double x, bool exact) {
  if (exact) return (x * 0.5) * (1.0 + erf(x * 0.70710678118654752440));
  const double inner = 0.7978845608028654 * (x + 0.044715 * x * x * x);
  return (x * 0.5) * (1.0 + tanh(inner));
}

template <typename T> __device__ __forceinline__ uint32_t fs_pack2(float a, float b) { return 0; }
template <> __device__ __forceinline__ uint32_t fs_pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t fs_pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Elements move in 16-byte pieces when the extent allows it (VEC), one at a time otherwise.
template <typename T, bool VEC> struct Chunk {
  typedef typename Scalar<T>::acc_t A;
  static constexpr int N = VEC ? 16 / (int)sizeof(T) : 1;
  static __device__ __forceinline__ void load(const T* p, int64_t i, A (&v)[N]) {
    if (VEC) {
      union { uint4 raw; T e[16 / sizeof(T)]; } u;
      u.raw = *reinterpret_cast<const uint4*>(p + i);
#pragma unroll
      for (int j = 0; j < N; j++) v[j] = Scalar<T>::load(u.e, j);
    } else {
      v[0] = Scalar<T>::load(p, i);
    }
  }
  static __device__ __forceinline__ void store(T* p, int64_t i, const A (&v)[N]) {
    if (VEC && sizeof(T) == 2 && N == 8) {
      // two elements per conversion instruction (round to nearest even; a NaN becomes the canonical NaN)
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; j++) w[j] = fs_pack2<T>((float)v[2 * j], (float)v[2 * j + 1]);
      *reinterpret_cast<uint4*>(p + i) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if (VEC) {
      union { uint4 raw; T e[16 / sizeof(T)]; } u;
#pragma unroll
      for (int j = 0; j < N; j++) Scalar<T>::store(u.e, j, v[j]);
      *reinterpret_cast<uint4*>(p + i) = u.raw;
    } else {
      Scalar<T>::store(p, i, v[0]);
    }
  }
};

template <typename T, bool VEC>
__global__ void __launch_bounds__(FS_THREADS) gelu_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n, int exact) {
  typedef Chunk<T, VEC> Ch;
  typedef typename Ch::A A;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * Ch::N; i < n; i += (int64_t)gridDim.x * blockDim.x * Ch::N) {
    A v[Ch::N];
    Ch::load(x, i, v);
#pragma unroll
    for (int j = 0; j < Ch::N; j++) v[j] = fs_gelu<A>(v[j], exact != 0);
    Ch::store(y, i, v);
  }
}

// ---- block reductions (256 threads) -----------------------------------------
template <typename A, bool MAX>
__device__ __forceinline__ A fs_block_reduce(A v, A* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const A w = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = MAX ? (w > v ? w : v) : v + w;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  A r = scratch[0];
#pragma unroll
  for (int w = 1; w < FS_THREADS / 32; w++) r = MAX ? (scratch[w] > r ? scratch[w] : r) : r + scratch[w];
  return r;
}

// Softmax over the last axis (inner == 1): one CTA per row, rows taken grid-stride.
template <typename T, bool VEC>
__global__ void __launch_bounds__(FS_THREADS)
softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t L, int cached) {
  typedef Chunk<T, VEC> Ch;
  typedef typename Ch::A A;
  constexpr int N = Ch::N;
  extern __shared__ __align__(16) uint8_t fs_smem[];
  A* row = reinterpret_cast<A*>(fs_smem);
  __shared__ A scratch[FS_THREADS / 32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * L;
    T* yr = y + r * L;
    A mx = -INFINITY;
    for (int64_t i = (int64_t)threadIdx.x * N; i < L; i += FS_THREADS * N) {
      A v[N];
      Ch::load(xr, i, v);
#pragma unroll
      for (int j = 0; j < N; j++) { if (cached) row[i + j] = v[j]; if (v[j] > mx) mx = v[j]; }
    }
    mx = fs_block_reduce<A, true>(mx, scratch);
    A sum = 0;
    for (int64_t i = (int64_t)threadIdx.x * N; i < L; i += FS_THREADS * N) {
      A v[N];
      if (!cached) Ch::load(xr, i, v);
#pragma unroll
      for (int j = 0; j < N; j++) {
        const A e = fs_exp<A, sizeof(T) == 2>((cached ? row[i + j] : v[j]) - mx);
        if (cached) row[i + j] = e;
        sum += e;
      }
    }
    sum = fs_block_reduce<A, false>(sum, scratch);
    const A inv = (A)1 / sum;
    for (int64_t i = (int64_t)threadIdx.x * N; i < L; i += FS_THREADS * N) {
      A v[N];
      if (!cached) Ch::load(xr, i, v);
#pragma unroll
      for (int j = 0; j < N; j++) v[j] = (cached ? row[i + j] : fs_exp<A, sizeof(T) == 2>(v[j] - mx)) * inv;
      Ch::store(yr, i, v);
    }
    __syncthreads();                     // the row cache is rewritten by the next row
  }
}

// Rows short enough to live in registers (at most FS_REG_CHUNKS 16-byte pieces per thread): every load
// of a row is in flight before the first use, nothing is staged in shared memory.
constexpr int FS_REG_CHUNKS = 4;

template <typename T>
__global__ void __launch_bounds__(FS_THREADS)
softmax_rows_reg_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t L) {
  typedef Chunk<T, true> Ch;
  typedef typename Ch::A A;
  constexpr int N = Ch::N, R = FS_REG_CHUNKS;
  __shared__ A scratch[FS_THREADS / 32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * L;
    T* yr = y + r * L;
    A v[R][N];
#pragma unroll
    for (int c = 0; c < R; c++) {
      const int64_t i = ((int64_t)c * FS_THREADS + threadIdx.x) * N;
      if (i < L) Ch::load(xr, i, v[c]);
      else {
#pragma unroll
        for (int j = 0; j < N; j++) v[c][j] = -INFINITY;
      }
    }
    A mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < R; c++)
#pragma unroll
      for (int j = 0; j < N; j++) mx = v[c][j] > mx ? v[c][j] : mx;
    mx = fs_block_reduce<A, true>(mx, scratch);
    A sum = 0;
#pragma unroll
    for (int c = 0; c < R; c++)
#pragma unroll
      for (int j = 0; j < N; j++) { v[c][j] = fs_exp<A, sizeof(T) == 2>(v[c][j] - mx); sum += v[c][j]; }     // exp(-inf) = 0 beyond the row
    sum = fs_block_reduce<A, false>(sum, scratch);
    const A inv = (A)1 / sum;
#pragma unroll
    for (int c = 0; c < R; c++) {
      const int64_t i = ((int64_t)c * FS_THREADS + threadIdx.x) * N;
      if (i < L) {
#pragma unroll
        for (int j = 0; j < N; j++) v[c][j] *= inv;
        Ch::store(yr, i, v[c]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(FS_THREADS)
layernorm_rows_reg_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                          int64_t rows, int64_t L, double eps) {
  typedef Chunk<T, true> Ch;
  typedef typename Ch::A A;
  constexpr int N = Ch::N, R = FS_REG_CHUNKS;
  __shared__ A scratch[FS_THREADS / 32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * L;
    T* yr = y + r * L;
    A v[R][N];
#pragma unroll
    for (int c = 0; c < R; c++) {
      const int64_t i = ((int64_t)c * FS_THREADS + threadIdx.x) * N;
      if (i < L) Ch::load(xr, i, v[c]);
      else {
#pragma unroll
        for (int j = 0; j < N; j++) v[c][j] = 0;
      }
    }
    A sum = 0;
#pragma unroll
    for (int c = 0; c < R; c++)
#pragma unroll
      for (int j = 0; j < N; j++) sum += v[c][j];
    const A mean = fs_block_reduce<A, false>(sum, scratch) / (A)L;
    A vs = 0;
#pragma unroll
    for (int c = 0; c < R; c++) {
      const int64_t i = ((int64_t)c * FS_THREADS + threadIdx.x) * N;
      if (i < L) {
#pragma unroll
        for (int j = 0; j < N; j++) { const A d = v[c][j] - mean; vs += d * d; }
      }
    }
    const A var = fs_block_reduce<A, false>(vs, scratch) / (A)L;
    const A inv_std = (A)(1.0 / sqrt((double)var + eps));        // layernorm.go:150
#pragma unroll
    for (int c = 0; c < R; c++) {
      const int64_t i = ((int64_t)c * FS_THREADS + threadIdx.x) * N;
      if (i < L) {
        A g[N], bt[N];
        if (gamma) Ch::load(gamma, i, g);
        if (beta) Ch::load(beta, i, bt);
#pragma unroll
        for (int j = 0; j < N; j++) {
          A o = (v[c][j] - mean) * inv_std;
          if (gamma) o *= g[j];
          if (beta) o += bt[j];
          v[c][j] = o;
        }
        Ch::store(yr, i, v[c]);
      }
    }
  }
}

// Softmax over an inner axis: one thread per (outer, inner) line; neighbouring threads read
// neighbouring addresses at every step along the axis.
template <typename T>
__global__ void __launch_bounds__(FS_THREADS)
softmax_lines_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t outer, int64_t L, int64_t inner) {
  typedef typename Scalar<T>::acc_t A;
  const int64_t lines = outer * inner;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < lines; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = t / inner, in = t - o * inner;
    const int64_t base = o * L * inner + in;
    A mx = -INFINITY;
    for (int64_t i = 0; i < L; i++) { const A v = Scalar<T>::load(x, base + i * inner); if (v > mx) mx = v; }
    A sum = 0;
    for (int64_t i = 0; i < L; i++) sum += fs_exp<A>((A)Scalar<T>::load(x, base + i * inner) - mx);
    const A inv = (A)1 / sum;
    for (int64_t i = 0; i < L; i++) Scalar<T>::store(y, base + i * inner, fs_exp<A>((A)Scalar<T>::load(x, base + i * inner) - mx) * inv);
  }
}

// Layer norm over the trailing L elements of every row.
template <typename T, bool VEC>
__global__ void __launch_bounds__(FS_THREADS)
layernorm_rows_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                      int64_t rows, int64_t L, double eps, int cached) {
  typedef Chunk<T, VEC> Ch;
  typedef typename Ch::A A;
  constexpr int N = Ch::N;
  extern __shared__ __align__(16) uint8_t fs_smem[];
  A* row = reinterpret_cast<A*>(fs_smem);
  __shared__ A scratch[FS_THREADS / 32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * L;
    T* yr = y + r * L;
    A sum = 0;
    for (int64_t i = (int64_t)threadIdx.x * N; i < L; i += FS_THREADS * N) {
      A v[N];
      Ch::load(xr, i, v);
#pragma unroll
      for (int j = 0; j < N; j++) { if (cached) row[i + j] = v[j]; sum += v[j]; }
    }
    const A mean = fs_block_reduce<A, false>(sum, scratch) / (A)L;
    A vs = 0;
    for (int64_t i = (int64_t)threadIdx.x * N; i < L; i += FS_THREADS * N) {
      A v[N];
      if (!cached) Ch::load(xr, i, v);
#pragma unroll
      for (int j = 0; j < N; j++) { const A d = (cached ? row[i + j] : v[j]) - mean; vs += d * d; }
    }
    const A var = fs_block_reduce<A, false>(vs, scratch) / (A)L;
    const A inv_std = (A)(1.0 / sqrt((double)var + eps));        // layernorm.go:150
    for (int64_t i = (int64_t)threadIdx.x * N; i < L; i += FS_THREADS * N) {
      A v[N], g[N], bt[N];
      if (!cached) Ch::load(xr, i, v);
      if (gamma) Ch::load(gamma, i, g);
      if (beta) Ch::load(beta, i, bt);
#pragma unroll
      for (int j = 0; j < N; j++) {
        A o = ((cached ? row[i + j] : v[j]) - mean) * inv_std;
        if (gamma) o *= g[j];
        if (beta) o += bt[j];
        v[j] = o;
      }
      Ch::store(yr, i, v);
    }
    __syncthreads();
  }
}

// Columns [first, first + width) of a [rows, total] matrix, plus an optional bias[width]: the scatter half of
// FusedAttentionQKVProjection (internal/gobackend/fusedops/attentionqkv.go:140-199).
template <typename T>
__global__ void __launch_bounds__(FS_THREADS)
cols_bias_kernel(const T* __restrict__ src, const T* __restrict__ bias, T* __restrict__ out, int64_t rows, int64_t total,
                 int64_t first, int64_t width) {
  typedef typename Scalar<T>::acc_t A;
  const int64_t n = rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i - r * width;
    A v = Scalar<T>::load(src, r * total + first + c);
    if (bias) v += (A)Scalar<T>::load(bias, c);
    Scalar<T>::store(out, i, v);
  }
}

// ---- plans ------------------------------------------------------------------
static bool fs_float(int d) { return d == CB_F32 || d == CB_F64 || d == CB_BF16 || d == CB_F16; }
static size_t fs_acc_size(int d) { return d == CB_F64 ? 8 : 4; }

int fused_small_plan(cb_plan* p) {
  HelperDesc& h = p->helper;
  const char* op = p->kind == PLAN_GELU ? "FusedGelu" : (p->kind == PLAN_SOFTMAX ? "FusedSoftmax" : (p->kind == PLAN_COLS_BIAS ? "FusedAttentionQKVProjection" : "FusedLayerNorm"));
  if (!fs_float(h.dtype)) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: dtype %s", op, dtype_name(h.dtype));
  p->n_outputs = 1;
  p->threads = FS_THREADS;
  const int64_t per_sm = 8;
  if (p->kind == PLAN_GELU) {
    if (h.n < 0) return fail(CB_ERR_INVALID_ARG, "%s: negative element count", op);
    p->n_inputs = 1;
    p->blocks = (int)std::max<int64_t>(1, std::min<int64_t>((h.n + FS_THREADS - 1) / FS_THREADS, (int64_t)p->n_sm * per_sm));
    p->name = std::string("gelu_") + (h.axis ? "exact_" : "tanh_") + dtype_name(h.dtype);
    return CB_OK;
  }
  if (p->kind == PLAN_COLS_BIAS) {
    const int64_t rows = h.dims[0], total = h.dims[1], first = h.dims[2], width = h.dims[3];
    if (rows < 0 || total < 0 || first < 0 || width < 0 || first + width > total)
      return fail(CB_ERR_INVALID_ARG, "%s: columns [%lld, %lld) do not lie inside %lld", op, (long long)first, (long long)(first + width), (long long)total);
    h.n = rows * width;
    p->n_inputs = 1 + ((h.flags & 1) ? 1 : 0);
    p->blocks = (int)std::max<int64_t>(1, std::min<int64_t>((h.n + FS_THREADS - 1) / FS_THREADS, (int64_t)p->n_sm * per_sm));
    p->name = std::string("cols_bias_") + dtype_name(h.dtype);
    return CB_OK;
  }
  const int64_t outer = h.dims[0], L = h.dims[1], inner = h.dims[2];
  if (outer < 0 || L < 0 || inner < 0) return fail(CB_ERR_INVALID_ARG, "%s: negative dimension", op);
  h.n = outer * L * inner;
  const bool cached = (size_t)L * fs_acc_size(h.dtype) <= (size_t)FS_SMEM_BYTES;
  if (p->kind == PLAN_SOFTMAX) {
    p->n_inputs = 1;
    if (inner == 1) {
      p->blocks = (int)std::max<int64_t>(1, std::min<int64_t>(outer, (int64_t)p->n_sm * per_sm));
      p->dyn_smem = cached ? (int)((size_t)L * fs_acc_size(h.dtype)) : 0;
      p->name = std::string("softmax_rows_") + dtype_name(h.dtype);
    } else {
      p->blocks = (int)std::max<int64_t>(1, std::min<int64_t>((outer * inner + FS_THREADS - 1) / FS_THREADS, (int64_t)p->n_sm * per_sm));
      p->name = std::string("softmax_lines_") + dtype_name(h.dtype);
    }
    return CB_OK;
  }
  if (inner != 1) return fail(CB_ERR_INVALID_ARG, "%s: the normalised axes must be trailing", op);
  p->n_inputs = 1 + ((h.flags & 1) ? 1 : 0) + ((h.flags & 2) ? 1 : 0);
  p->blocks = (int)std::max<int64_t>(1, std::min<int64_t>(outer, (int64_t)p->n_sm * per_sm));
  p->dyn_smem = cached ? (int)((size_t)L * fs_acc_size(h.dtype)) : 0;
  p->name = std::string("layernorm_rows_") + dtype_name(h.dtype);
  return CB_OK;
}

template <typename F>
static int fs_by_dtype(int dtype, F&& f) {
  switch (dtype) {
    case CB_F32: return f((float*)nullptr);
    case CB_F64: return f((double*)nullptr);
    case CB_BF16: return f((__nv_bfloat16*)nullptr);
    case CB_F16: return f((__half*)nullptr);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "dtype %s", dtype_name(dtype));
  }
}

int fused_small_launch(const cb_plan* p, const void* const* in, void* const* out, void*, cudaStream_t s) {
  const HelperDesc& h = p->helper;
  if (h.n == 0) return CB_OK;
  const int64_t outer = h.dims[0], L = h.dims[1], inner = h.dims[2];
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  int st = fs_by_dtype(h.dtype, [&](auto* t) {
    typedef typename std::remove_pointer<decltype(t)>::type T;
    constexpr int64_t VN = 16 / (int64_t)sizeof(T);
    if (p->kind == PLAN_COLS_BIAS) {
      cols_bias_kernel<T><<<p->blocks, FS_THREADS, 0, s>>>((const T*)in[0], (h.flags & 1) ? (const T*)in[1] : nullptr, (T*)out[0],
                                                         h.dims[0], h.dims[1], h.dims[2], h.dims[3]);
    } else if (p->kind == PLAN_GELU) {
      if (h.n % VN == 0 && aligned(in[0]) && aligned(out[0]))
        gelu_kernel<T, true><<<p->blocks, FS_THREADS, 0, s>>>((const T*)in[0], (T*)out[0], h.n, h.axis);
      else
        gelu_kernel<T, false><<<p->blocks, FS_THREADS, 0, s>>>((const T*)in[0], (T*)out[0], h.n, h.axis);
    } else if (p->kind == PLAN_SOFTMAX) {
      if (inner != 1) softmax_lines_kernel<T><<<p->blocks, FS_THREADS, 0, s>>>((const T*)in[0], (T*)out[0], outer, L, inner);
      else if (L % VN == 0 && aligned(in[0]) && aligned(out[0]) && L <= (int64_t)FS_THREADS * VN * FS_REG_CHUNKS)
        softmax_rows_reg_kernel<T><<<p->blocks, FS_THREADS, 0, s>>>((const T*)in[0], (T*)out[0], outer, L);
      else if (L % VN == 0 && aligned(in[0]) && aligned(out[0]))
        softmax_rows_kernel<T, true><<<p->blocks, FS_THREADS, p->dyn_smem, s>>>((const T*)in[0], (T*)out[0], outer, L, p->dyn_smem > 0);
      else
        softmax_rows_kernel<T, false><<<p->blocks, FS_THREADS, p->dyn_smem, s>>>((const T*)in[0], (T*)out[0], outer, L, p->dyn_smem > 0);
    } else {
      int idx = 1;
      const T* gamma = (h.flags & 1) ? (const T*)in[idx++] : nullptr;
      const T* beta = (h.flags & 2) ? (const T*)in[idx++] : nullptr;
      const bool vec = L % VN == 0 && aligned(in[0]) && aligned(out[0]) && aligned(gamma) && aligned(beta);
      if (vec && L <= (int64_t)FS_THREADS * VN * FS_REG_CHUNKS)
        layernorm_rows_reg_kernel<T><<<p->blocks, FS_THREADS, 0, s>>>((const T*)in[0], gamma, beta, (T*)out[0], outer, L, h.eps);
      else if (vec)
        layernorm_rows_kernel<T, true><<<p->blocks, FS_THREADS, p->dyn_smem, s>>>((const T*)in[0], gamma, beta, (T*)out[0], outer, L, h.eps, p->dyn_smem > 0);
      else
        layernorm_rows_kernel<T, false><<<p->blocks, FS_THREADS, p->dyn_smem, s>>>((const T*)in[0], gamma, beta, (T*)out[0], outer, L, h.eps, p->dyn_smem > 0);
    }
    return (int)CB_OK;
  });
  CB_TRY(st);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

}  // namespace cb
