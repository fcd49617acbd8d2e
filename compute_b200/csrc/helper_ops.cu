// The handful of data-movement ops the DotGeneral path needs around the GEMM:
// Reshape (a copy), ConvertDType, Iota, Slice, Transpose.  Reference behaviour:
// internal/gobackend/ops/{reshape,convertdtype,iota,slice,transpose}.go.
#include "common.cuh"

namespace cb {

struct Dims8 { int64_t v[8]; };
struct Perm8 { int32_t v[8]; };

template <typename T>
__global__ void slice_kernel(const T* __restrict__ in, T* __restrict__ out, int rank, Dims8 in_dims, Dims8 out_dims,
                             Dims8 starts, Dims8 strides, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, src = 0, mul = 1;
    for (int a = rank - 1; a >= 0; a--) {
      const int64_t c = rem % out_dims.v[a];
      rem /= out_dims.v[a];
      src += (starts.v[a] + c * strides.v[a]) * mul;
      mul *= in_dims.v[a];
    }
    out[i] = in[src];
  }
}

template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int rank, Dims8 in_strides,
                                 Dims8 out_dims, Perm8 perm, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, src = 0;
    for (int a = rank - 1; a >= 0; a--) {
      const int64_t c = rem % out_dims.v[a];
      rem /= out_dims.v[a];
      src += c * in_strides.v[perm.v[a]];
    }
    out[i] = in[src];
  }
}

// Compute-type round trip used by Iota and ConvertDType.
template <typename T> struct Conv {
  __device__ static double get(const T* p, int64_t i) { return (double)p[i]; }
  __device__ static void put(T* p, int64_t i, double v) { p[i] = (T)v; }
  __device__ static void put_i(T* p, int64_t i, int64_t v) { p[i] = (T)v; }
  __device__ static int64_t get_i(const T* p, int64_t i) { return (int64_t)p[i]; }
  static constexpr bool is_float = false;
};
template <> struct Conv<float> {
  __device__ static double get(const float* p, int64_t i) { return (double)p[i]; }
  __device__ static void put(float* p, int64_t i, double v) { p[i] = (float)v; }
  __device__ static void put_i(float* p, int64_t i, int64_t v) { p[i] = (float)v; }
  __device__ static int64_t get_i(const float* p, int64_t i) { return (int64_t)p[i]; }
  static constexpr bool is_float = true;
};
template <> struct Conv<double> {
  __device__ static double get(const double* p, int64_t i) { return p[i]; }
  __device__ static void put(double* p, int64_t i, double v) { p[i] = v; }
  __device__ static void put_i(double* p, int64_t i, int64_t v) { p[i] = (double)v; }
  __device__ static int64_t get_i(const double* p, int64_t i) { return (int64_t)p[i]; }
  static constexpr bool is_float = true;
};
template <> struct Conv<__nv_bfloat16> {
  __device__ static double get(const __nv_bfloat16* p, int64_t i) { return (double)Scalar<__nv_bfloat16>::load(p, i); }
  __device__ static void put(__nv_bfloat16* p, int64_t i, double v) { Scalar<__nv_bfloat16>::store(p, i, (float)v); }
  __device__ static void put_i(__nv_bfloat16* p, int64_t i, int64_t v) { Scalar<__nv_bfloat16>::store(p, i, (float)v); }
  __device__ static int64_t get_i(const __nv_bfloat16* p, int64_t i) { return (int64_t)Scalar<__nv_bfloat16>::load(p, i); }
  static constexpr bool is_float = true;
};
template <> struct Conv<__half> {
  __device__ static double get(const __half* p, int64_t i) { return (double)__half2float(p[i]); }
  __device__ static void put(__half* p, int64_t i, double v) { p[i] = __float2half_rn((float)v); }
  __device__ static void put_i(__half* p, int64_t i, int64_t v) { p[i] = __float2half_rn((float)v); }
  __device__ static int64_t get_i(const __half* p, int64_t i) { return (int64_t)__half2float(p[i]); }
  static constexpr bool is_float = true;
};
struct BoolT { uint8_t v; };
template <> struct Conv<BoolT> {
  __device__ static double get(const BoolT* p, int64_t i) { return p[i].v ? 1.0 : 0.0; }
  __device__ static void put(BoolT* p, int64_t i, double v) { p[i].v = (v != 0.0) ? 1 : 0; }
  __device__ static void put_i(BoolT* p, int64_t i, int64_t v) { p[i].v = (v != 0) ? 1 : 0; }
  __device__ static int64_t get_i(const BoolT* p, int64_t i) { return p[i].v ? 1 : 0; }
  static constexpr bool is_float = false;
};

template <typename FROM, typename TO>
__global__ void convert_kernel(const FROM* __restrict__ in, TO* __restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    if (Conv<FROM>::is_float) Conv<TO>::put(out, i, Conv<FROM>::get(in, i));
    else Conv<TO>::put_i(out, i, Conv<FROM>::get_i(in, i));
  }
}

template <typename T>
__global__ void iota_kernel(T* __restrict__ out, int64_t n, int64_t axis_dim, int64_t inner) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    Conv<T>::put_i(out, i, (i / inner) % axis_dim);
}

static int grid_for(int64_t n) { return (int)std::min<int64_t>((n + 255) / 256, 148 * 8); }

template <typename F>
static int by_dtype(int dtype, F&& f) {
  switch (dtype) {
    case CB_BOOL: return f((BoolT*)nullptr);
    case CB_I8: return f((int8_t*)nullptr);
    case CB_U8: return f((uint8_t*)nullptr);
    case CB_I16: return f((int16_t*)nullptr);
    case CB_U16: return f((uint16_t*)nullptr);
    case CB_I32: return f((int32_t*)nullptr);
    case CB_U32: return f((uint32_t*)nullptr);
    case CB_I64: return f((int64_t*)nullptr);
    case CB_U64: return f((uint64_t*)nullptr);
    case CB_F16: return f((__half*)nullptr);
    case CB_BF16: return f((__nv_bfloat16*)nullptr);
    case CB_F32: return f((float*)nullptr);
    case CB_F64: return f((double*)nullptr);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "dtype %s is not implemented", dtype_name(dtype));
  }
}

template <typename F>
static int by_size(int dtype, F&& f) {
  switch (dtype_size(dtype)) {
    case 1: return f((uint8_t*)nullptr);
    case 2: return f((uint16_t*)nullptr);
    case 4: return f((uint32_t*)nullptr);
    case 8: return f((uint64_t*)nullptr);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "dtype %s is not implemented", dtype_name(dtype));
  }
}

int helper_plan(cb_plan* p) {
  HelperDesc& h = p->helper;
  if (dtype_size(h.dtype) == 0) return fail(CB_ERR_NOT_IMPLEMENTED, "dtype %s is not implemented", dtype_name(h.dtype));
  p->n_outputs = 1;
  p->threads = 256;
  switch (p->kind) {
    case PLAN_COPY: p->n_inputs = 1; p->name = "copy"; break;
    case PLAN_CONVERT:
      if (dtype_size(h.dtype_to) == 0 || h.dtype_to > CB_BF16 || h.dtype > CB_BF16)
        return fail(CB_ERR_NOT_IMPLEMENTED, "ConvertDType %s -> %s is not implemented", dtype_name(h.dtype), dtype_name(h.dtype_to));
      p->n_inputs = 1; p->name = "convert_dtype"; break;
    case PLAN_IOTA: {
      if (h.rank < 1 || h.axis < 0 || h.axis >= h.rank) return fail(CB_ERR_INVALID_ARG, "Iota: axis %d out of range for rank %d", h.axis, h.rank);
      if (h.dtype == CB_BOOL) return fail(CB_ERR_INVALID_ARG, "Iota: Bool is not a numeric dtype");
      h.n = 1;
      for (int i = 0; i < h.rank; i++) h.n *= h.dims[i];
      p->n_inputs = 0; p->name = "iota"; break;
    }
    case PLAN_SLICE:
      h.n = 1;
      for (int i = 0; i < h.rank; i++) h.n *= h.out_dims[i];
      p->n_inputs = 1; p->name = "slice"; break;
    case PLAN_TRANSPOSE:
      h.n = 1;
      for (int i = 0; i < h.rank; i++) h.n *= h.out_dims[i];
      p->n_inputs = 1; p->name = "transpose"; break;
    default: return fail(CB_ERR_INVALID_ARG, "unknown helper plan kind %d", p->kind);
  }
  if (h.n < 0) return fail(CB_ERR_INVALID_ARG, "negative element count");
  p->blocks = grid_for(h.n > 0 ? h.n : 1);
  return CB_OK;
}

int helper_launch(const cb_plan* p, const void* const* in, void* const* out, void*, cudaStream_t s) {
  const HelperDesc& h = p->helper;
  if (h.n == 0) return CB_OK;
  const int grid = p->blocks;
  switch (p->kind) {
    case PLAN_COPY:
      CB_CUDA(cudaMemcpyAsync(out[0], in[0], (size_t)h.n * dtype_size(h.dtype), cudaMemcpyDeviceToDevice, s));
      return CB_OK;
    case PLAN_CONVERT: {
      int st = by_dtype(h.dtype, [&](auto* from) {
        typedef typename std::remove_pointer<decltype(from)>::type F;
        return by_dtype(h.dtype_to, [&](auto* to) {
          typedef typename std::remove_pointer<decltype(to)>::type T;
          convert_kernel<F, T><<<grid, 256, 0, s>>>((const F*)in[0], (T*)out[0], h.n);
          return (int)CB_OK;
        });
      });
      CB_TRY(st);
      break;
    }
    case PLAN_IOTA: {
      int64_t inner = 1;
      for (int i = h.axis + 1; i < h.rank; i++) inner *= h.dims[i];
      int st = by_dtype(h.dtype, [&](auto* t) {
        typedef typename std::remove_pointer<decltype(t)>::type T;
        iota_kernel<T><<<grid, 256, 0, s>>>((T*)out[0], h.n, h.dims[h.axis], inner);
        return (int)CB_OK;
      });
      CB_TRY(st);
      break;
    }
    case PLAN_SLICE: {
      Dims8 id, od, st8, sr;
      for (int i = 0; i < 8; i++) { id.v[i] = h.dims[i]; od.v[i] = h.out_dims[i]; st8.v[i] = h.starts[i]; sr.v[i] = h.strides[i]; }
      int st = by_size(h.dtype, [&](auto* t) {
        typedef typename std::remove_pointer<decltype(t)>::type T;
        slice_kernel<T><<<grid, 256, 0, s>>>((const T*)in[0], (T*)out[0], h.rank, id, od, st8, sr, h.n);
        return (int)CB_OK;
      });
      CB_TRY(st);
      break;
    }
    case PLAN_TRANSPOSE: {
      Dims8 is, od;
      Perm8 pm;
      int64_t mul = 1;
      for (int i = 0; i < 8; i++) { is.v[i] = 0; od.v[i] = 1; pm.v[i] = 0; }
      for (int a = h.rank - 1; a >= 0; a--) { is.v[a] = mul; mul *= h.dims[a]; }
      for (int i = 0; i < h.rank; i++) { od.v[i] = h.out_dims[i]; pm.v[i] = h.perm[i]; }
      int st = by_size(h.dtype, [&](auto* t) {
        typedef typename std::remove_pointer<decltype(t)>::type T;
        transpose_kernel<T><<<grid, 256, 0, s>>>((const T*)in[0], (T*)out[0], h.rank, is, od, pm, h.n);
        return (int)CB_OK;
      });
      CB_TRY(st);
      break;
    }
    default: return fail(CB_ERR_INVALID_ARG, "unknown helper plan kind %d", p->kind);
  }
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

}  // namespace cb
