// DotGeneral in normalised form, generic CUDA-core kernel:
//   out[B,M,N] = lhs[B,M,K] x rhs[B,K,N]      (rhs_transposed = 0)
//   out[B,M,N] = lhs[B,M,K] x rhs[B,N,K]^T    (rhs_transposed = 1)
// for every dtype the path supports (f32, f64, bf16, f16, i32, i64).  Half inputs
// accumulate in f32 (internal/gobackend/dot/dot.go:207-210 of the reference); each
// output is a plain k-ascending dot product, like the reference's unpacked small
// kernels (dot/matmul/nosimd_small.go).  Any shape, no alignment requirements.
#include "common.cuh"

namespace cb {

template <typename T> struct DotAcc { typedef T type; };
template <> struct DotAcc<__nv_bfloat16> { typedef float type; };
template <> struct DotAcc<__half> { typedef float type; };

template <typename T, typename A> struct DotIO {
  __device__ static A load(const T* p, int64_t i) { return (A)p[i]; }
};
template <> struct DotIO<__nv_bfloat16, float> {
  __device__ static float load(const __nv_bfloat16* p, int64_t i) { return Scalar<__nv_bfloat16>::load(p, i); }
};
template <> struct DotIO<__half, float> {
  __device__ static float load(const __half* p, int64_t i) { return __half2float(p[i]); }
};
template <typename A, typename O> struct DotStore {
  __device__ static void store(O* p, int64_t i, A v) { p[i] = (O)v; }
};
template <typename A> struct DotStore<A, __nv_bfloat16> {
  __device__ static void store(__nv_bfloat16* p, int64_t i, A v) { Scalar<__nv_bfloat16>::store(p, i, (float)v); }
};
template <typename A> struct DotStore<A, __half> {
  __device__ static void store(__half* p, int64_t i, A v) { p[i] = __float2half_rn((float)v); }
};

constexpr int DG_TILE = 64;
constexpr int DG_KT = 16;

// FusedDense epilogue (internal/gobackend/fusedops/dense.go:111-205): bias[n] added to the matmul
// result, then the activation, in the accumulator's type (f64 for f64, f32 otherwise).  Integer
// dot products have no epilogue.
__device__ inline double apply_activation_f64(double x, int act) {
  switch (act) {
    case CB_ACT_GELU: return x * 0.5 * (1.0 + erf(x * (1.0 / 1.4142135623730951)));     // gelu.go:113-118
    case CB_ACT_RELU: return x < 0.0 ? 0.0 : x;
    case CB_ACT_SILU: return x / (1.0 + exp(-x));
    case CB_ACT_HARDSWISH: { const double g = fmin(fmax(x * (1.0 / 6.0) + 0.5, 0.0), 1.0); return x * g; }
    case CB_ACT_TANH: return tanh(x);
    default: return x;
  }
}
template <typename T, typename A> struct DenseEpilogue {
  static __device__ __forceinline__ A apply(A v, const T*, int64_t, int) { return v; }
};
template <typename T> struct DenseEpilogue<T, float> {
  static __device__ __forceinline__ float apply(float v, const T* bias, int64_t n, int act) {
    if (bias) v = __fadd_rn(v, DotIO<T, float>::load(bias, n));
    return apply_activation(v, act);
  }
};
template <> struct DenseEpilogue<double, double> {
  static __device__ __forceinline__ double apply(double v, const double* bias, int64_t n, int act) {
    if (bias) v = v + bias[n];
    return apply_activation_f64(v, act);
  }
};

template <typename T, typename O>
__global__ void __launch_bounds__(256)
dot_generic_kernel(const T* __restrict__ lhs, const T* __restrict__ rhs, const T* __restrict__ bias, O* __restrict__ out,
                   int64_t M, int64_t N, int64_t K, int rhs_transposed, int act) {
  typedef typename DotAcc<T>::type A;
  __shared__ A As[DG_KT][DG_TILE + 1];
  __shared__ A Bs[DG_KT][DG_TILE + 1];
  const int64_t b = blockIdx.z;
  const int64_t m0 = (int64_t)blockIdx.y * DG_TILE, n0 = (int64_t)blockIdx.x * DG_TILE;
  const T* L = lhs + b * M * K;
  const T* R = rhs + b * K * N;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  A acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = (A)0;
  for (int64_t k0 = 0; k0 < K; k0 += DG_KT) {
    for (int idx = threadIdx.x; idx < DG_TILE * DG_KT; idx += 256) {
      {  // lhs tile: rows m, k contiguous
        const int r = idx / DG_KT, c = idx % DG_KT;
        const int64_t m = m0 + r, k = k0 + c;
        As[c][r] = (m < M && k < K) ? DotIO<T, A>::load(L, m * K + k) : (A)0;
      }
      if (rhs_transposed) {
        const int r = idx / DG_KT, c = idx % DG_KT;
        const int64_t n = n0 + r, k = k0 + c;
        Bs[c][r] = (n < N && k < K) ? DotIO<T, A>::load(R, n * K + k) : (A)0;
      } else {
        const int c = idx / DG_TILE, r = idx % DG_TILE;
        const int64_t n = n0 + r, k = k0 + c;
        Bs[c][r] = (n < N && k < K) ? DotIO<T, A>::load(R, k * N + n) : (A)0;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < DG_KT; kk++) {
      A a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bb[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * bb[j];
    }
    __syncthreads();
  }
  O* C = out + b * M * N;
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int64_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) DotStore<A, O>::store(C, m * N + n, DenseEpilogue<T, A>::apply(acc[i][j], bias, n, act));
    }
}

template <typename T, typename O>
static int launch_t(const cb_dot_desc& d, const void* const* in, void* const* out, cudaStream_t s) {
  dim3 grid((unsigned)((d.N + DG_TILE - 1) / DG_TILE), (unsigned)((d.M + DG_TILE - 1) / DG_TILE), (unsigned)d.B);
  dot_generic_kernel<T, O><<<grid, 256, 0, s>>>((const T*)in[0], (const T*)in[1], d.has_bias ? (const T*)in[2] : nullptr, (O*)out[0],
                                                d.M, d.N, d.K, d.rhs_transposed, d.activation);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

template <typename T>
static int launch_out(const cb_dot_desc& d, int od, const void* const* in, void* const* out, cudaStream_t s) {
  if (od == d.in_dtype) return launch_t<T, T>(d, in, out, s);
  if (od == CB_F32) return launch_t<T, float>(d, in, out, s);
  if (od == CB_F64) return launch_t<T, double>(d, in, out, s);
  return fail(CB_ERR_NOT_IMPLEMENTED, "no DotGeneral implementation found for layout and dtypes=%s,%s",
              dtype_name(d.in_dtype), dtype_name(od));
}

bool dot_generic_supports_epilogue(int in_dtype) {
  return in_dtype == CB_F32 || in_dtype == CB_F64 || in_dtype == CB_BF16 || in_dtype == CB_F16;
}

bool dot_generic_supports(int in_dtype, int out_dtype) {
  const bool in_ok = in_dtype == CB_F32 || in_dtype == CB_F64 || in_dtype == CB_BF16 || in_dtype == CB_F16 ||
                     in_dtype == CB_I32 || in_dtype == CB_I64;
  if (!in_ok) return false;
  if (out_dtype == in_dtype) return true;
  const bool in_float = in_dtype != CB_I32 && in_dtype != CB_I64;
  return in_float && (out_dtype == CB_F32 || out_dtype == CB_F64);
}

int dot_generic_launch(const cb_dot_desc& d, const void* const* in, void* const* out, cudaStream_t s) {
  const int od = d.out_dtype ? d.out_dtype : d.in_dtype;
  if (d.B == 0 || d.M == 0 || d.N == 0) return CB_OK;
  if (d.B > 65535 || (d.M + DG_TILE - 1) / DG_TILE > 65535)
    return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral generic kernel: batch or M too large for one launch");
  switch (d.in_dtype) {
    case CB_F32: return launch_out<float>(d, od, in, out, s);
    case CB_F64: return launch_out<double>(d, od, in, out, s);
    case CB_BF16: return launch_out<__nv_bfloat16>(d, od, in, out, s);
    case CB_F16: return launch_out<__half>(d, od, in, out, s);
    case CB_I32: return launch_t<int32_t, int32_t>(d, in, out, s);
    case CB_I64: return launch_t<int64_t, int64_t>(d, in, out, s);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral: dtype %s is not implemented", dtype_name(d.in_dtype));
  }
}

}  // namespace cb
