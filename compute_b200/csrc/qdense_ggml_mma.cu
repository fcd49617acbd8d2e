// GGML block formats on the integer tensor cores, for decode shapes (M <= 16, K a multiple of 256): Q4_0, Q8_0,
// IQ4_NL and Q4_K.  Reference arithmetic: internal/gobackend/fusedops/quantizeddense_ggml.go:98-260 (per output the
// weight row is dequantised block by block and multiplied with x).
//
// The CUDA-core kernel of qdense_ggml.cu spends five to seven lane-operations on every weight value (extract, convert,
// scale, multiply-add), which is what bounds it.  Here the integers inside the blocks go to mma.sync m16n8k32 (s8) as
// they are, against x in block fixed point:
//   x[m, k] = unit[m] * (d0 + 128 d1 + 16384 d2),  signed base-128 digits, unit[m] a power of two from the largest |x| of
//   the row (20 bits below it: an error of at most 2^-21 of the row's maximum per element);
// one MMA forms, for 16 weight rows and one 32-value block, the exact integer dot products with eight (digit plane, x
// row) columns, and the block's own scale is applied to that integer in float32:
//   Q8_0    d * sum(q x)                      Q4_0    d * (sum(n x) - 8 sum(x))       n = nibble
//   IQ4_NL  d * sum(table[n] x)               Q4_K    (d sc) * sum(n x) - (dmin m) * sum(x)
// sum(x) per block comes from the digit kernel.  The k index of the product is permuted (lane t of a quad owns the
// values 8t..8t+7 of the block, for the weights and for the digits alike), so every operand fragment is eight
// contiguous bytes.
//
// A CTA owns 64 weight rows: warps 0-3 take 16 rows each over the first half of K, warps 4-7 the same rows over the second
// half; every warp streams its rows through a private three-stage ring of 256-value steps filled by cp.async.  At the
// end the halves and the digit planes are combined through shared memory, bias and activation applied, results stored.
#include "common.cuh"

#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <string>

namespace cb {
namespace {

constexpr int GM_WARPS = 8;
constexpr int GM_ROWS = 64;                 // weight rows per CTA
constexpr int GM_STEP = 256;                // values per ring stage and row
constexpr int GM_STAGES = 3;
constexpr int GM_MAX_COLS = 48;             // 3 digit planes x 16 rows of x

__host__ __device__ constexpr int gm_block_bytes(int t) { return t == CB_GGML_Q8_0 ? 34 : t == CB_GGML_Q4_K ? 144 : 18; }
__host__ __device__ constexpr int gm_seg(int t) { return t == CB_GGML_Q4_K ? 144 : 8 * gm_block_bytes(t); }   // bytes of 256 values
__host__ __device__ constexpr int gm_pitch(int t) { return gm_seg(t) + 16; }
__host__ __device__ constexpr int gm_stage_bytes(int t) { return 16 * gm_pitch(t); }

__device__ __forceinline__ void gm_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Eight bytes starting at shared address `a` (a multiple of 2): three aligned words and two funnel shifts.
__device__ __forceinline__ void gm_lds8(uint32_t a, uint32_t& w0, uint32_t& w1) {
  const uint32_t base = a & ~3u, sh = (a & 2u) * 8u;
  uint32_t x0, x1, x2;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x0) : "r"(base));
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x1) : "r"(base + 4));
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x2) : "r"(base + 8));
  w0 = __funnelshift_r(x0, x1, sh);
  w1 = __funnelshift_r(x1, x2, sh);
}
__device__ __forceinline__ float gm_lds_f16(uint32_t a) {
  unsigned short h;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(a));
  return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ uint32_t gm_lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}

// compute.IQ4NLLookupTable (fused_ops.go:127-130) as int8, four entries per word
__device__ __forceinline__ uint32_t gm_iq4nl(uint32_t nibbles) {      // four bytes holding 0..15 -> their table values
  constexpr uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;   // -127,-104,-83,-65 | -49,-35,-22,-10 | 1,13,25,38 | 53,69,89,113
  const uint32_t t = nibbles | (nibbles >> 4);
  const uint32_t sel = __byte_perm(t, 0, 0x4420);                      // b0 | b1 << 4 | b2 << 8 | b3 << 12
  const uint32_t lo = __byte_perm(T0, T1, sel & 0x7777u), hi = __byte_perm(T2, T3, sel & 0x7777u);
  const uint32_t mask = __byte_perm(0x0000FF00u, 0, (sel >> 3) & 0x1111u);
  return (lo & ~mask) | (hi & mask);
}

// ---- x -> digits, one block per row of x
constexpr int GD_THREADS = 256;
template <typename XT> __device__ __forceinline__ float gd_x(const XT* p, int64_t i);
template <> __device__ __forceinline__ float gd_x<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <> __device__ __forceinline__ float gd_x<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// digits [3][M][K] int8, dsum [3][M][K / 32] int32 (sum of a block's digits), units [M] float
template <typename XT>
__global__ void __launch_bounds__(GD_THREADS)
ggml_row_digits_kernel(const XT* __restrict__ x, int M, int64_t K, int8_t* __restrict__ digits, int* __restrict__ dsum, float* __restrict__ units) {
  __shared__ uint32_t s_mx[GD_THREADS / 32];
  __shared__ int s_bad;
  const int m = blockIdx.x;
  const XT* xr = x + (int64_t)m * K;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  uint32_t mx = 0;
  bool bad = false;
  for (int64_t k = threadIdx.x; k < K; k += GD_THREADS) {
    const uint32_t a = __float_as_uint(gd_x<XT>(xr, k)) & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) bad = true; else mx = max(mx, a);
  }
  mx = __reduce_max_sync(0xFFFFFFFFu, mx);
  if (__any_sync(0xFFFFFFFFu, bad) && (threadIdx.x & 31) == 0) atomicExch(&s_bad, 1);
  if ((threadIdx.x & 31) == 0) s_mx[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = 0;
  for (int w = 0; w < GD_THREADS / 32; w++) mx = max(mx, s_mx[w]);
  // |x| < 2^ex; shift so that |x| * 2^shift <= 2^20 (three signed base-128 digits)
  const int ef = (int)(mx >> 23);
  const int ex = ef > 0 ? ef - 126 : (32 - __clz(mx)) - 149;
  const int shift = min(20 - ex, 149);
  const int sh1 = shift / 2, sh2 = shift - sh1;
  const float p1 = __int_as_float((127 + sh1) << 23), p2 = __int_as_float((127 + sh2) << 23);
  if (threadIdx.x == 0) {
    float unit = shift <= 126 ? __int_as_float((127 - shift) << 23) : __int_as_float(1 << (149 - shift));
    if (s_bad) unit = __int_as_float(0x7FC00000);      // a row holding inf or NaN comes back NaN
    units[m] = unit;
  }
  const int64_t U = K / 32;
  // a thread converts 4 consecutive values; the 8 threads of a 32-value block add their digit sums by shuffles
  for (int64_t k = (int64_t)threadIdx.x * 4; k < K; k += GD_THREADS * 4) {
    uint32_t w0 = 0, w1 = 0, w2 = 0;
    int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      float v = gd_x<XT>(xr, k + e);
      if ((__float_as_uint(v) & 0x7FFFFFFFu) >= 0x7F800000u) v = 0.0f;
      const int q = (int)(__float_as_uint(fmaf(v * p1, p2, 12582912.0f)) - 0x4B400000u);     // round to nearest, |q| <= 2^20
      const int a = ((q + 64) & 127) - 64;
      const int q1 = (q - a) >> 7;
      const int b = ((q1 + 64) & 127) - 64;
      const int c = (q1 - b) >> 7;
      w0 |= (uint32_t)(a & 0xFF) << (8 * e); w1 |= (uint32_t)(b & 0xFF) << (8 * e); w2 |= (uint32_t)(c & 0xFF) << (8 * e);
      s0 += a; s1 += b; s2 += c;
    }
    *reinterpret_cast<uint32_t*>(digits + ((int64_t)0 * M + m) * K + k) = w0;
    *reinterpret_cast<uint32_t*>(digits + ((int64_t)1 * M + m) * K + k) = w1;
    *reinterpret_cast<uint32_t*>(digits + ((int64_t)2 * M + m) * K + k) = w2;
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
      s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, d); s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, d); s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, d);
    }
    if ((threadIdx.x & 7) == 0) {
      const int64_t u = k / 32;
      dsum[((int64_t)0 * M + m) * U + u] = s0; dsum[((int64_t)1 * M + m) * U + u] = s1; dsum[((int64_t)2 * M + m) * U + u] = s2;
    }
  }
}

// ---- the products.  NT = 8-column tiles of (plane, row) columns: column c = plane * M + m, 3 M columns in all.
template <typename XT, int GGML, int NT>
__global__ void __launch_bounds__(GM_WARPS * 32, 2)
ggml_mma_kernel(const uint8_t* __restrict__ w, const int8_t* __restrict__ digits, const int* __restrict__ dsum, const float* __restrict__ units,
                const float* __restrict__ bias, XT* __restrict__ out, int M, int64_t K, int64_t N, int act) {
  constexpr int BB = gm_block_bytes(GGML), SEG = gm_seg(GGML), PITCH = gm_pitch(GGML), STAGE = gm_stage_bytes(GGML);
  extern __shared__ __align__(16) unsigned char gm_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int half = warp >> 2;                                  // which half of K
  const int64_t row0 = (int64_t)blockIdx.x * GM_ROWS + (warp & 3) * 16;
  const int64_t U = K / 32, steps_all = K / GM_STEP;
  const int64_t step0 = half == 0 ? 0 : (steps_all + 1) / 2, step1 = half == 0 ? (steps_all + 1) / 2 : steps_all;
  const int n_steps = (int)(step1 - step0);
  const int64_t bytes_per_row = K / (GGML == CB_GGML_Q4_K ? 256 : 32) * BB;
  const int ncols = 3 * M;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(gm_smem) + warp * GM_STAGES * STAGE;

  // this warp's 16 rows, 16 bytes per copy: SEG / 16 copies per row and stage
  auto fill = [&](int s) {
    if (s < n_steps) {
      const uint32_t st = ring + (s % GM_STAGES) * STAGE;
      constexpr int VPR = SEG / 16;
      for (int id = lane; id < 16 * VPR; id += 32) {
        const int r = id / VPR, v = id % VPR;
        const int64_t row = min(row0 + r, N - 1);             // rows past N repeat the last one; their results are not stored
        const uint8_t* src = w + row * bytes_per_row + (step0 + s) * SEG + v * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(st + r * PITCH + v * 16), "l"(src) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int s = 0; s < GM_STAGES - 1; s++) fill(s);

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f; }
  // the digit rows and block sums this lane reads: B fragment column 8j + g, C columns 8j + 2t and 8j + 2t + 1
  const int8_t* dcol[NT];
  const int* scol0[NT];
  const int* scol1[NT];
#pragma unroll
  for (int j = 0; j < NT; j++) {
    const int cb = 8 * j + g, c0 = 8 * j + 2 * t, c1 = c0 + 1;
    dcol[j] = cb < ncols ? digits + (int64_t)cb * K : nullptr;
    scol0[j] = c0 < ncols ? dsum + (int64_t)c0 * U : nullptr;
    scol1[j] = c1 < ncols ? dsum + (int64_t)c1 * U : nullptr;
  }

  for (int s = 0; s < n_steps; s++) {
    asm volatile("cp.async.wait_group %0;" :: "n"(GM_STAGES - 2) : "memory");
    __syncwarp();
    fill(s + GM_STAGES - 1);
    const uint32_t st = ring + (s % GM_STAGES) * STAGE;
    const uint32_t rlo = st + g * PITCH, rhi = st + (g + 8) * PITCH;
    const int64_t u0 = (step0 + s) * 8;                       // first 32-value block of this step
#pragma unroll
    for (int u = 0; u < 8; u++) {
      // ---- A fragments: rows g and g + 8, the block's values 8t .. 8t + 7
      uint32_t a0, a1, a2, a3;
      float dl, dh, ml = 0.0f, mh = 0.0f;                       // scale (and, Q4_K, min term) of the two rows
      if (GGML == CB_GGML_Q8_0) {
        gm_lds8(rlo + u * 34 + 2 + 8 * t, a0, a2);
        gm_lds8(rhi + u * 34 + 2 + 8 * t, a1, a3);
        dl = gm_lds_f16(rlo + u * 34); dh = gm_lds_f16(rhi + u * 34);
      } else if (GGML == CB_GGML_Q4_0 || GGML == CB_GGML_IQ4_NL) {
        uint32_t l0, l1, h0, h1;
        gm_lds8(rlo + u * 18 + 2 + 8 * (t & 1), l0, l1);
        gm_lds8(rhi + u * 18 + 2 + 8 * (t & 1), h0, h1);
        const int sh = 4 * (t >> 1);                            // values 0-15 are the low nibbles, 16-31 the high ones
        a0 = (l0 >> sh) & 0x0F0F0F0Fu; a2 = (l1 >> sh) & 0x0F0F0F0Fu;
        a1 = (h0 >> sh) & 0x0F0F0F0Fu; a3 = (h1 >> sh) & 0x0F0F0F0Fu;
        if (GGML == CB_GGML_IQ4_NL) { a0 = gm_iq4nl(a0); a1 = gm_iq4nl(a1); a2 = gm_iq4nl(a2); a3 = gm_iq4nl(a3); }
        dl = gm_lds_f16(rlo + u * 18); dh = gm_lds_f16(rhi + u * 18);
      } else {  // Q4_K: sub-block u of the row's block: bytes 16 + 32 (u / 2) + 8t .., low nibbles for even u, high for odd
        uint2 l, h;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(l.x), "=r"(l.y) : "r"(rlo + 16 + 32 * (u >> 1) + 8 * t));
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(h.x), "=r"(h.y) : "r"(rhi + 16 + 32 * (u >> 1) + 8 * t));
        const int sh = 4 * (u & 1);
        a0 = (l.x >> sh) & 0x0F0F0F0Fu; a2 = (l.y >> sh) & 0x0F0F0F0Fu;
        a1 = (h.x >> sh) & 0x0F0F0F0Fu; a3 = (h.y >> sh) & 0x0F0F0F0Fu;
        // getScaleMinK4 (quantizeddense_ggml.go:219-228) on the 12 packed bytes at offset 4
        auto scale_min = [&](uint32_t rowa, float& dsc, float& dmn) {
          uint32_t sc, mn;
          if (u < 4) { sc = gm_lds_u8(rowa + 4 + u) & 63u; mn = gm_lds_u8(rowa + 8 + u) & 63u; }
          else {
            const uint32_t x4 = gm_lds_u8(rowa + 8 + u), xa = gm_lds_u8(rowa + u), xb = gm_lds_u8(rowa + 4 + u);
            sc = (x4 & 0xFu) | ((xa >> 6) << 4);
            mn = (x4 >> 4) | ((xb >> 6) << 4);
          }
          dsc = __fmul_rn(gm_lds_f16(rowa), (float)sc);
          dmn = __fmul_rn(gm_lds_f16(rowa + 2), (float)mn);
        };
        scale_min(rlo, dl, ml);
        scale_min(rhi, dh, mh);
      }
      const int64_t ub = u0 + u;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        uint2 b = make_uint2(0u, 0u);
        if (dcol[j]) b = __ldg(reinterpret_cast<const uint2*>(dcol[j] + ub * 32 + 8 * t));
        int c[4];
        gm_mma(c, a0, a1, a2, a3, b.x, b.y);
        if (GGML == CB_GGML_Q8_0 || GGML == CB_GGML_IQ4_NL) {
          acc[j][0] = fmaf(dl, (float)c[0], acc[j][0]); acc[j][1] = fmaf(dl, (float)c[1], acc[j][1]);
          acc[j][2] = fmaf(dh, (float)c[2], acc[j][2]); acc[j][3] = fmaf(dh, (float)c[3], acc[j][3]);
        } else {
          const int x0 = scol0[j] ? __ldg(scol0[j] + ub) : 0, x1 = scol1[j] ? __ldg(scol1[j] + ub) : 0;   // sum of the block's digits
          if (GGML == CB_GGML_Q4_0) {
            acc[j][0] = fmaf(dl, (float)(c[0] - 8 * x0), acc[j][0]); acc[j][1] = fmaf(dl, (float)(c[1] - 8 * x1), acc[j][1]);
            acc[j][2] = fmaf(dh, (float)(c[2] - 8 * x0), acc[j][2]); acc[j][3] = fmaf(dh, (float)(c[3] - 8 * x1), acc[j][3]);
          } else {
            const float f0 = (float)x0, f1 = (float)x1;
            acc[j][0] += fmaf(dl, (float)c[0], -ml * f0); acc[j][1] += fmaf(dl, (float)c[1], -ml * f1);
            acc[j][2] += fmaf(dh, (float)c[2], -mh * f0); acc[j][3] += fmaf(dh, (float)c[3], -mh * f1);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                             // the rings are free: they become the exchange buffer
  // ---- halves of K and digit planes meet in shared memory: part[half][row][column]
  float* part = reinterpret_cast<float*>(gm_smem);
  const int rl = (warp & 3) * 16 + g;
#pragma unroll
  for (int j = 0; j < NT; j++) {
    const int c0 = 8 * j + 2 * t;
    float* p0 = part + ((half * GM_ROWS + rl) * GM_MAX_COLS), *p1 = part + ((half * GM_ROWS + rl + 8) * GM_MAX_COLS);
    if (c0 < ncols) { p0[c0] = acc[j][0]; p1[c0] = acc[j][2]; }
    if (c0 + 1 < ncols) { p0[c0 + 1] = acc[j][1]; p1[c0 + 1] = acc[j][3]; }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GM_ROWS * M; idx += GM_WARPS * 32) {
    const int m = idx / GM_ROWS, r = idx % GM_ROWS;            // consecutive threads write consecutive columns of out
    const int64_t n = (int64_t)blockIdx.x * GM_ROWS + r;
    if (n >= N) continue;
    float v = 0.0f;
#pragma unroll
    for (int pl = 2; pl >= 0; pl--) {                          // smallest plane last: unit * (A0 + 128 A1 + 16384 A2)
      const int c = pl * M + m;
      const float a = part[(0 * GM_ROWS + r) * GM_MAX_COLS + c] + part[(1 * GM_ROWS + r) * GM_MAX_COLS + c];
      v = fmaf(v, 128.0f, a);
    }
    v *= units[m];
    if (bias) v = __fadd_rn(v, bias[n]);
    Scalar<XT>::store(out, (int64_t)m * N + n, apply_activation(v, act));
  }
}

size_t gm_smem_bytes(int ggml) {
  return std::max((size_t)GM_WARPS * GM_STAGES * gm_stage_bytes(ggml), (size_t)2 * GM_ROWS * GM_MAX_COLS * sizeof(float));
}

static size_t gm_align(size_t b) { return (b + 255) & ~(size_t)255; }
struct GmLayout { size_t off_digits, off_dsum, off_units, total; };
GmLayout gm_layout(int64_t M, int64_t K) {
  GmLayout l;
  l.off_digits = 0;
  l.off_dsum = gm_align((size_t)(3 * M * K));
  l.off_units = l.off_dsum + gm_align((size_t)(3 * M * (K / 32)) * 4);
  l.total = l.off_units + 256;
  return l;
}

template <typename XT, int GGML, int NT>
int gm_launch_k(const cb_qdense_desc& d, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  int dev = 0;
  CB_CUDA(cudaGetDevice(&dev));
  const size_t smem = gm_smem_bytes(GGML);
  if (dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(ggml_mma_kernel<XT, GGML, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  const GmLayout l = gm_layout(d.M, d.K);
  uint8_t* w8 = (uint8_t*)ws;
  int8_t* digits = (int8_t*)(w8 + l.off_digits);
  int* dsum = (int*)(w8 + l.off_dsum);
  float* units = (float*)(w8 + l.off_units);
  ggml_row_digits_kernel<XT><<<(unsigned)d.M, GD_THREADS, 0, s>>>((const XT*)in[0], (int)d.M, d.K, digits, dsum, units);
  CB_CUDA(cudaGetLastError());
  const float* bias = d.has_bias ? (const float*)in[2] : nullptr;
  ggml_mma_kernel<XT, GGML, NT><<<(unsigned)((d.N + GM_ROWS - 1) / GM_ROWS), GM_WARPS * 32, smem, s>>>(
      (const uint8_t*)in[1], digits, dsum, units, bias, (XT*)out[0], (int)d.M, d.K, d.N, d.activation);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

template <typename XT, int GGML>
int gm_launch_n(const cb_qdense_desc& d, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const int ncols = 3 * (int)d.M;
  if (ncols <= 8) return gm_launch_k<XT, GGML, 1>(d, in, out, ws, s);
  if (ncols <= 16) return gm_launch_k<XT, GGML, 2>(d, in, out, ws, s);
  return gm_launch_k<XT, GGML, 6>(d, in, out, ws, s);
}

template <typename XT>
int gm_launch_t(const cb_qdense_desc& d, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  switch (d.ggml_type) {
    case CB_GGML_Q4_0: return gm_launch_n<XT, CB_GGML_Q4_0>(d, in, out, ws, s);
    case CB_GGML_Q8_0: return gm_launch_n<XT, CB_GGML_Q8_0>(d, in, out, ws, s);
    case CB_GGML_IQ4_NL: return gm_launch_n<XT, CB_GGML_IQ4_NL>(d, in, out, ws, s);
    default: return gm_launch_n<XT, CB_GGML_Q4_K>(d, in, out, ws, s);
  }
}

}  // namespace

bool qdense_ggml_mma_supports(const cb_qdense_desc& d) {
  if (d.scheme != CB_QUANT_GGML || d.variant == CB_QDENSE_GENERIC) return false;
  if (d.ggml_type != CB_GGML_Q4_0 && d.ggml_type != CB_GGML_Q8_0 && d.ggml_type != CB_GGML_IQ4_NL && d.ggml_type != CB_GGML_Q4_K) return false;
  return d.M >= 1 && d.M <= 16 && d.K >= 256 && d.K % 256 == 0 && d.N >= 1 && (d.N + GM_ROWS - 1) / GM_ROWS <= 0x7FFFFFFFLL;
}

void qdense_ggml_mma_plan(cb_plan* p, const char* type_name) {
  const cb_qdense_desc& d = p->qd;
  p->blocks = (int)((d.N + GM_ROWS - 1) / GM_ROWS);
  p->threads = GM_WARPS * 32;
  p->dyn_smem = (int)gm_smem_bytes(d.ggml_type);
  p->workspace_bytes = gm_layout(d.M, d.K).total;
  p->counter_bytes = 0;
  p->name = std::string("qdense_ggml_mma_") + (d.x_dtype == CB_BF16 ? "bf16_" : "f32_") + type_name;
}

int qdense_ggml_mma_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  return d.x_dtype == CB_BF16 ? gm_launch_t<__nv_bfloat16>(d, in, out, ws, s) : gm_launch_t<float>(d, in, out, ws, s);
}

}  // namespace cb
