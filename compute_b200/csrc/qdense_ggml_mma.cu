// GGML block formats on the integer tensor cores, for decode shapes (M <= 16, K a multiple of 256): Q4_0, Q8_0,
// IQ4_NL and Q4_K.  Reference arithmetic: internal/gobackend/fusedops/quantizeddense_ggml.go:98-260 (per output the
// weight row is dequantised block by block and multiplied with x).
//
// The CUDA-core kernel of qdense_ggml.cu spends five to seven lane-operations on every weight value (extract, convert,
// scale, multiply-add), which is what bounds it.  Here the integers inside the blocks go to mma.sync m16n8k32 (s8) as
// they are, against x in block fixed point:
//   x[m, k] = unit[m] * (d0 + 128 d1 + 16384 d2),  signed base-128 digits, unit[m] a power of two from the largest |x| of
//   the row (20 bits below it: an error of at most 2^-21 of the row's maximum per element; bfloat16 x takes two digits,
//   13 bits);
// one MMA forms, for 16 weight rows and one 32-value block, the exact integer dot products with eight (digit plane, x
// row) columns, and the block's own scale is applied to that integer in float32:
//   Q8_0    d * sum(q x)                      Q4_0    (d / 16) * sum(16 (n - 8) x)    n = nibble
//   IQ4_NL  d * sum(table[n] x)               Q4_K    d * sum over the super-block of sc * sum(n x)  -  (dmin m) * sum(x)
// sum(x) per block comes from the digit kernel.  The k index of the product is permuted (lane t of a quad owns the
// values 8t..8t+7 of the block, for the weights and for the digits alike), so every operand fragment is eight
// contiguous bytes.
//
// A CTA owns up to 64 weight rows: warps 0-3 take 16 rows each over the first half of K, warps 4-7 the same rows over the second
// half; every warp streams its rows through a private three-stage ring of 256-value steps, each stage one TMA tile
// (16 rows x the step's bytes) announced on the warp's own mbarrier.  At the end the halves and the digit planes are
// combined through shared memory, bias and activation applied, results stored.  Every wait is bounded: a stage that does
// not arrive within two seconds ends the kernel with a status word set, which cb_plan_check_status reports.
#include "tc_common.cuh"

#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <string>

namespace cb {
namespace {

constexpr int GM_WARPS = 8;
constexpr int GM_ROWS = 64;                 // weight rows per CTA
constexpr int GM_STEP = 256;                // values per ring stage and row
constexpr int GM_STAGES = 3;
constexpr int GM_MAX_COLS = 48;             // 3 digit planes x 16 rows of x
// Up to this many rows of x the kernel runs once per 16 rows: four runs of 37 us beat expanding the weights to bf16 planes
// for the GEMM (176 us whatever M on the 4096 x 14336 projection).
constexpr int GM_MAX_M = 64;
constexpr int GM_BAR_BYTES = 256;           // the stages' barriers (8 warps x 3) and the digits' one
static_assert((GM_WARPS * GM_STAGES + 1) * 8 <= GM_BAR_BYTES, "barrier area");
constexpr int GM_DPAD = 32;                 // bytes between two columns of digits in shared memory, past K
// A CTA asks for at least this much shared memory, so that no more than two fit an SM.  With three, the CTAs of the
// next launch of a decode loop (scheduled early, as dependents) settle beside the running ones and both slow down:
// IQ4_NL at M = 4 took 28 us with the floor and 49 us without.
constexpr size_t GM_SMEM_FLOOR = 78 * 1024;
// CTAs of a launch: two per SM when W has the row groups for it, never more than four groups per CTA.  With the fixed
// 64 rows per CTA that this replaces, 14336 rows gave 224 CTAs: 76 SMs with two and 72 with one.
__host__ inline int gm_grid(int64_t N, int n_sm) {
  const int64_t G = (N + 15) / 16;
  return (int)std::max((G + 3) / 4, std::min<int64_t>(2 * (int64_t)std::max(n_sm, 1), G));
}
constexpr size_t GM_SMEM_CTA = 112 * 1024;  // what a CTA may use while two still fit an SM (227 KB, 1 KB reserved per CTA)

__host__ __device__ constexpr int gm_block_bytes(int t) { return t == CB_GGML_Q8_0 ? 34 : t == CB_GGML_Q4_K ? 144 : 18; }
__host__ __device__ constexpr int gm_seg(int t) { return t == CB_GGML_Q4_K ? 144 : 8 * gm_block_bytes(t); }   // bytes of 256 values
// Row pitch in the ring = the inner extent of the TMA box.  18-byte blocks: the step's 144 bytes = 36 words, so the eight
// rows of a fragment read start in banks 0, 4, .., 28 and the two 8-byte halves a row is read in fill the gaps.  Q4_K:
// 160 bytes (the box takes 16 bytes of the next step along): the four rows of a half-warp's 64-bit reads start 8 banks
// apart.  Q8_0: the step's 272 bytes.
__host__ __device__ constexpr int gm_pitch(int t) { return t == CB_GGML_Q4_K ? 160 : gm_seg(t); }
__host__ __device__ constexpr int gm_stage_bytes(int t) { return 16 * gm_pitch(t); }
// Digit planes of x: three for float32 (20 bits below the row's largest value), two for bfloat16 (13 bits: its own
// elements carry 8).
template <typename XT> __host__ __device__ constexpr int gm_planes_of() { return sizeof(XT) == 2 ? 2 : 3; }
__host__ inline int gm_planes(const cb_qdense_desc& d) { return d.x_dtype == CB_BF16 ? 2 : 3; }
__host__ __device__ constexpr int gm_tiles(int M, int planes) { return (planes * M + 7) / 8; }   // 8-column tiles of (plane, row) columns

__device__ __forceinline__ void gm_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Eight bytes at p + off.  p is 8-byte aligned and off is a constant once the caller's loop is unrolled, so the choice
// below is made by the compiler: one 64-bit read, two 32-bit reads, or (off = 2 mod 4) three words and two funnel shifts.
__device__ __forceinline__ void gm_ld8(const unsigned char* p, int off, uint32_t& w0, uint32_t& w1) {
  if (off % 8 == 0) {
    const uint2 v = *reinterpret_cast<const uint2*>(p + off);
    w0 = v.x; w1 = v.y;
  } else if (off % 4 == 0) {
    w0 = *reinterpret_cast<const uint32_t*>(p + off); w1 = *reinterpret_cast<const uint32_t*>(p + off + 4);
  } else {
    const uint32_t x0 = *reinterpret_cast<const uint32_t*>(p + off - 2), x1 = *reinterpret_cast<const uint32_t*>(p + off + 2),
                   x2 = *reinterpret_cast<const uint32_t*>(p + off + 6);
    w0 = __funnelshift_r(x0, x1, 16); w1 = __funnelshift_r(x1, x2, 16);
  }
}
// int -> float for |c| < 2^22 with an integer add and a float add (the conversion instruction shares its issue queue
// with the shared-memory reads, which is what this kernel waits on)
__device__ __forceinline__ float gm_i2f(int c) { return __int_as_float(0x4B400000 + c) - 12582912.0f; }
__device__ __forceinline__ float gm_f16(const unsigned char* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }

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
constexpr int GD_CACHE = 4;                 // a thread keeps its first 16 values in registers between the two passes
template <typename XT> __device__ __forceinline__ float4 gd_x4(const XT* p, int64_t i);
template <> __device__ __forceinline__ float4 gd_x4<float>(const float* p, int64_t i) { return __ldg(reinterpret_cast<const float4*>(p + i)); }
template <> __device__ __forceinline__ float4 gd_x4<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(p + i));
  return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
}

// digits [cols][K] int8 with column = plane * M + m; dsum [K / 32][cols] float = the sum of a block's digits (written
// when the format has a per-block minimum); units [M] float.  `cols` is (planes x M) rounded up to whole 8-column tiles: the
// columns past planes x M are never written and whatever they hold only reaches results that are dropped.
template <typename XT>
__global__ void __launch_bounds__(GD_THREADS)
ggml_row_digits_kernel(const XT* __restrict__ x, int M, int64_t K, int cols, int8_t* __restrict__ digits, float* __restrict__ dsum, float* __restrict__ units) {
  // The product kernel may be scheduled now (it requests weights, then waits for this grid); this grid may itself
  // have been scheduled while the kernel before it, which may produce x or still read the digits, was running.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ uint32_t s_mx[GD_THREADS / 32];
  __shared__ int s_bad;
  const int m = blockIdx.x;
  const XT* xr = x + (int64_t)m * K;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  uint32_t mx = 0;
  bool bad = false;
  float4 cache[GD_CACHE];
  auto look = [&](const float4& v) {
    const uint32_t a[4] = {__float_as_uint(v.x) & 0x7FFFFFFFu, __float_as_uint(v.y) & 0x7FFFFFFFu, __float_as_uint(v.z) & 0x7FFFFFFFu,
                           __float_as_uint(v.w) & 0x7FFFFFFFu};
#pragma unroll
    for (int e = 0; e < 4; e++) { if (a[e] >= 0x7F800000u) bad = true; else mx = max(mx, a[e]); }
  };
#pragma unroll
  for (int i = 0; i < GD_CACHE; i++) {
    const int64_t k = ((int64_t)i * GD_THREADS + threadIdx.x) * 4;
    cache[i] = k < K ? gd_x4<XT>(xr, k) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < GD_CACHE; i++) look(cache[i]);
  for (int64_t k = ((int64_t)GD_CACHE * GD_THREADS + threadIdx.x) * 4; k < K; k += GD_THREADS * 4) look(gd_x4<XT>(xr, k));
  mx = __reduce_max_sync(0xFFFFFFFFu, mx);
  if (__any_sync(0xFFFFFFFFu, bad) && (threadIdx.x & 31) == 0) atomicExch(&s_bad, 1);
  if ((threadIdx.x & 31) == 0) s_mx[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = 0;
  for (int w = 0; w < GD_THREADS / 32; w++) mx = max(mx, s_mx[w]);
  // |x| < 2^ex; shift so that |x| * 2^shift <= 2^QBITS (PL signed base-128 digits)
  constexpr int PL = gm_planes_of<XT>(), QBITS = 7 * PL - 1;
  const int ef = (int)(mx >> 23);
  const int ex = ef > 0 ? ef - 126 : (32 - __clz(mx)) - 149;
  const int shift = min(QBITS - ex, 149);
  const int sh1 = shift / 2, sh2 = shift - sh1;
  const float p1 = __int_as_float((127 + sh1) << 23), p2 = __int_as_float((127 + sh2) << 23);
  if (threadIdx.x == 0) {
    float unit = shift <= 126 ? __int_as_float((127 - shift) << 23) : __int_as_float(1 << (149 - shift));
    if (s_bad) unit = __int_as_float(0x7FC00000);      // a row holding inf or NaN comes back NaN
    units[m] = unit;
  }
  // a thread converts 4 consecutive values; the 8 threads of a 32-value block add their digit sums by shuffles
  auto convert = [&](const float4& v4, int64_t k) {
    const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
    uint32_t w0 = 0, w1 = 0, w2 = 0;
    int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      float v = vv[e];
      if ((__float_as_uint(v) & 0x7FFFFFFFu) >= 0x7F800000u) v = 0.0f;
      const int q = (int)(__float_as_uint(fmaf(v * p1, p2, 12582912.0f)) - 0x4B400000u);     // round to nearest, |q| <= 2^QBITS
      const int a = ((q + 64) & 127) - 64;
      const int q1 = (q - a) >> 7;
      const int b = PL == 2 ? q1 : ((q1 + 64) & 127) - 64;    // two planes: |q1| <= 64 is the top digit
      const int c = PL == 2 ? 0 : (q1 - b) >> 7;
      w0 |= (uint32_t)(a & 0xFF) << (8 * e); w1 |= (uint32_t)(b & 0xFF) << (8 * e); w2 |= (uint32_t)(c & 0xFF) << (8 * e);
      s0 += a; s1 += b; s2 += c;
    }
    *reinterpret_cast<uint32_t*>(digits + ((int64_t)0 * M + m) * K + k) = w0;
    *reinterpret_cast<uint32_t*>(digits + ((int64_t)1 * M + m) * K + k) = w1;
    if (PL == 3) *reinterpret_cast<uint32_t*>(digits + ((int64_t)2 * M + m) * K + k) = w2;
    if (dsum) {
#pragma unroll
      for (int d = 1; d < 8; d <<= 1) {
        s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, d); s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, d); s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, d);
      }
      if ((threadIdx.x & 7) == 0) {
        float* o = dsum + (k / 32) * cols;
        o[0 * M + m] = (float)s0; o[1 * M + m] = (float)s1;
        if (PL == 3) o[2 * M + m] = (float)s2;
      }
    }
  };
#pragma unroll
  for (int i = 0; i < GD_CACHE; i++) {
    const int64_t k = ((int64_t)i * GD_THREADS + threadIdx.x) * 4;
    if (k < K) convert(cache[i], k);                      // K is a multiple of 256: whole warps take this branch together
  }
  for (int64_t k = ((int64_t)GD_CACHE * GD_THREADS + threadIdx.x) * 4; k < K; k += GD_THREADS * 4) convert(gd_x4<XT>(xr, k), k);
}

// ---- the products.  NT = 8-column tiles of (plane, row) columns: column c = plane * M + m, 3 M columns in all.
// BSMEM: the digits of all columns are brought into shared memory once per CTA (small M); otherwise every block's B
// fragments come through L1, requested one block ahead.
template <typename XT, int GGML, int NT, bool BSMEM>
__global__ void __launch_bounds__(GM_WARPS * 32, 2)
ggml_mma_kernel(const __grid_constant__ CUtensorMap tmap_w, const int8_t* __restrict__ digits, const float* __restrict__ dsum,
                const float* __restrict__ units, const float* __restrict__ bias, XT* __restrict__ out, int M, int64_t K, int64_t N, int act,
                unsigned* __restrict__ status) {
  constexpr int SEG = gm_seg(GGML), PITCH = gm_pitch(GGML), STAGE = gm_stage_bytes(GGML);
  constexpr int COLS = 8 * NT;
  extern __shared__ __align__(1024) unsigned char gm_smem[];
  // a following digit kernel of this library may be scheduled early: it waits for this grid before it touches anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int half = warp >> 2;                                  // which half of K
  // The 16-row groups of W are dealt out evenly: CTA b takes groups [b G / grid, (b + 1) G / grid), at most four (the
  // host sizes the grid so); warp pairs without a group only take part in the barriers.
  const int64_t G = (N + 15) / 16;
  const int64_t g_begin = (int64_t)blockIdx.x * G / gridDim.x;
  const int n_groups = (int)(((int64_t)blockIdx.x + 1) * G / gridDim.x - g_begin);
  const int64_t row_base = g_begin * 16;
  const int64_t row0 = row_base + (warp & 3) * 16;
  const int64_t steps_all = K / GM_STEP;
  const int64_t step0 = half == 0 ? 0 : (steps_all + 1) / 2, step1 = half == 0 ? (steps_all + 1) / 2 : steps_all;
  const int n_steps = (warp & 3) < n_groups ? (int)(step1 - step0) : 0;
  unsigned char* ring = gm_smem + warp * GM_STAGES * STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(gm_smem + GM_WARPS * GM_STAGES * STAGE) + warp * GM_STAGES;
  uint64_t* bar_digits = reinterpret_cast<uint64_t*>(gm_smem + GM_WARPS * GM_STAGES * STAGE) + GM_WARPS * GM_STAGES;
  unsigned char* dsm = gm_smem + GM_WARPS * GM_STAGES * STAGE + GM_BAR_BYTES;     // [3 M columns][K + 32] when BSMEM
  constexpr int PL = gm_planes_of<XT>();
  const int ncols = PL * M;
  const int64_t dpitch = K + GM_DPAD;

  // The ring: lane 0 asks for one tile per step - the warp's 16 rows by the step's bytes of each - and the stage's
  // barrier completes when all of it has landed.  Rows past N come back as zeros (scale 0); their results are not stored.
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < GM_STAGES; k++) tc::mbar_init(&bars[k], 1);
    if (BSMEM && warp == 0) tc::mbar_init(bar_digits, 1);
    tc::fence_barrier_init();
  }
  if (BSMEM) __syncthreads(); else __syncwarp();
  auto fill = [&](int s, int slot) {
    if (s < n_steps && lane == 0) {
      tc::mbar_expect_tx(&bars[slot], STAGE);
      tc::tma_load_2d(ring + slot * STAGE, &tmap_w, (int)((step0 + s) * (SEG / 4)), (int)row0, &bars[slot]);
    }
  };
#pragma unroll
  for (int s = 0; s < GM_STAGES - 1; s++) fill(s, s);

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f; }

  // weights do not come from the digit kernel; everything below reads what it wrote
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // B fragment of tile j: column 8 j + g, the block's values 8 t .. 8 t + 7; C columns 8 j + 2 t and 8 j + 2 t + 1.
  // Columns from 3 M on do not exist: in shared memory their fragments are zero, in global memory they are whatever
  // the padded digit buffer holds (their products are dropped).
  const int8_t* bp = digits + (int64_t)g * K + step0 * GM_STEP + 8 * t;
  const unsigned char* bs = dsm + (int64_t)g * dpitch + step0 * GM_STEP + 8 * t;
  const float* sp = dsum + step0 * 8 * COLS + 2 * t;
  const int64_t tile_stride = 8 * (BSMEM ? dpitch : K);
  bool colv[NT];
#pragma unroll
  for (int j = 0; j < NT; j++) colv[j] = 8 * j + g < ncols;
  uint2 bnext[NT];
  bool failed = false;
  if (BSMEM) {
    // one bulk copy per column, K bytes each, rows K + 32 bytes apart: the four columns a half-warp reads 64 bits of
    // start 8 banks apart
    if (threadIdx.x == 0) {
      tc::mbar_expect_tx(bar_digits, (uint32_t)(ncols * K));
      for (int c = 0; c < ncols; c++)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(tc::smem_u32(dsm + c * dpitch)), "l"(digits + (int64_t)c * K), "r"((uint32_t)K), "r"(tc::smem_u32(bar_digits)) : "memory");
    }
    const bool ok = tc::mbar_wait(bar_digits, 0);
    if (!__all_sync(0xFFFFFFFFu, ok)) failed = true;
  } else {
#pragma unroll
    for (int j = 0; j < NT; j++)
      bnext[j] = n_steps > 0 ? __ldg(reinterpret_cast<const uint2*>(bp + j * tile_stride)) : make_uint2(0u, 0u);
  }

  int slot = 0;
  uint32_t phase = 0;
  int consumed = 0;                                            // steps whose stage has been waited for
  for (int s = 0; s < n_steps && !failed; s++) {
    const bool ok = tc::mbar_wait(&bars[slot], phase);
    if (!__all_sync(0xFFFFFFFFu, ok)) { failed = true; break; }
    consumed = s + 1;
    // every lane has passed the vote, so the stage read in the previous step is free
    fill(s + GM_STAGES - 1, slot == 0 ? GM_STAGES - 1 : slot - 1);
    const unsigned char* rlo = ring + slot * STAGE + g * PITCH;
    const unsigned char* rhi = rlo + 8 * PITCH;
    if (++slot == GM_STAGES) { slot = 0; phase ^= 1u; }
    const bool last_step = s + 1 == n_steps;

    // Q4_K: the super-block's header, once per step and row
    float dl = 0.f, dh = 0.f, ml = 0.f, mh = 0.f;
    uint32_t ql0 = 0, ql1 = 0, ql2 = 0, qh0 = 0, qh1 = 0, qh2 = 0;
    int isum[NT][4];
    if (GGML == CB_GGML_Q4_K) {
      dl = gm_f16(rlo); ml = gm_f16(rlo + 2); dh = gm_f16(rhi); mh = gm_f16(rhi + 2);
      ql0 = *reinterpret_cast<const uint32_t*>(rlo + 4); ql1 = *reinterpret_cast<const uint32_t*>(rlo + 8); ql2 = *reinterpret_cast<const uint32_t*>(rlo + 12);
      qh0 = *reinterpret_cast<const uint32_t*>(rhi + 4); qh1 = *reinterpret_cast<const uint32_t*>(rhi + 8); qh2 = *reinterpret_cast<const uint32_t*>(rhi + 12);
#pragma unroll
      for (int j = 0; j < NT; j++) { isum[j][0] = isum[j][1] = isum[j][2] = isum[j][3] = 0; }
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      // ---- B fragments: from shared memory, or requested one block ago (and the next block's requested now)
      uint2 b[NT];
      if (BSMEM) {
#pragma unroll
        for (int j = 0; j < NT; j++)
          b[j] = colv[j] ? *reinterpret_cast<const uint2*>(bs + j * tile_stride + (s * 8 + u) * 32) : make_uint2(0u, 0u);
      } else {
#pragma unroll
        for (int j = 0; j < NT; j++) b[j] = bnext[j];
        if (!(last_step && u == 7)) {
          const int8_t* nb = bp + ((int64_t)s * 8 + u + 1) * 32;
#pragma unroll
          for (int j = 0; j < NT; j++) bnext[j] = __ldg(reinterpret_cast<const uint2*>(nb + j * tile_stride));
        }
      }
      // ---- A fragments: rows g and g + 8, the block's values 8t .. 8t + 7
      uint32_t a0, a1, a2, a3;
      if (GGML == CB_GGML_Q8_0) {
        gm_ld8(rlo + 8 * t, u * 34 + 2, a0, a2);
        gm_ld8(rhi + 8 * t, u * 34 + 2, a1, a3);
        dl = gm_f16(rlo + u * 34); dh = gm_f16(rhi + u * 34);
      } else if (GGML == CB_GGML_Q4_0 || GGML == CB_GGML_IQ4_NL) {
        uint32_t l0, l1, h0, h1;
        gm_ld8(rlo + 8 * (t & 1), u * 18 + 2, l0, l1);
        gm_ld8(rhi + 8 * (t & 1), u * 18 + 2, h0, h1);
        dl = gm_f16(rlo + u * 18); dh = gm_f16(rhi + u * 18);
        if (GGML == CB_GGML_IQ4_NL) {
          const int sh = 4 * (t >> 1);                          // values 0-15 are the low nibbles, 16-31 the high ones
          a0 = gm_iq4nl((l0 >> sh) & 0x0F0F0F0Fu); a2 = gm_iq4nl((l1 >> sh) & 0x0F0F0F0Fu);
          a1 = gm_iq4nl((h0 >> sh) & 0x0F0F0F0Fu); a3 = gm_iq4nl((h1 >> sh) & 0x0F0F0F0Fu);
        } else {
          // the nibble goes to the top of its byte with its top bit flipped: as int8 that is 16 (n - 8), and the 1/16 goes
          // into the block's scale (exact: a power of two)
          const int sh = 4 - 4 * (t >> 1);
          a0 = ((l0 << sh) & 0xF0F0F0F0u) ^ 0x80808080u; a2 = ((l1 << sh) & 0xF0F0F0F0u) ^ 0x80808080u;
          a1 = ((h0 << sh) & 0xF0F0F0F0u) ^ 0x80808080u; a3 = ((h1 << sh) & 0xF0F0F0F0u) ^ 0x80808080u;
          dl *= 0.0625f; dh *= 0.0625f;
        }
      } else {  // Q4_K: sub-block u of the super-block: bytes 16 + 32 (u / 2) + 8t .., low nibbles for even u, high for odd
        const uint2 l = *reinterpret_cast<const uint2*>(rlo + 16 + 32 * (u >> 1) + 8 * t);
        const uint2 h = *reinterpret_cast<const uint2*>(rhi + 16 + 32 * (u >> 1) + 8 * t);
        const int sh = 4 * (u & 1);
        a0 = (l.x >> sh) & 0x0F0F0F0Fu; a2 = (l.y >> sh) & 0x0F0F0F0Fu;
        a1 = (h.x >> sh) & 0x0F0F0F0Fu; a3 = (h.y >> sh) & 0x0F0F0F0Fu;
      }
      // getScaleMinK4 (quantizeddense_ggml.go:219-228) on the 12 packed bytes q[0..11] = words q0, q1, q2
      int scl = 0, sch = 0;
      float mnl = 0.f, mnh = 0.f;
      if (GGML == CB_GGML_Q4_K) {
        auto scale_min = [&](uint32_t q0, uint32_t q1, uint32_t q2, int& sc, int& mn) {
          if (u < 4) { sc = (q0 >> (8 * u)) & 63; mn = (q1 >> (8 * u)) & 63; }
          else {
            const int v = u - 4;
            const uint32_t x4 = (q2 >> (8 * v)) & 0xFFu, xa = (q0 >> (8 * v)) & 0xFFu, xb = (q1 >> (8 * v)) & 0xFFu;
            sc = (int)((x4 & 0xFu) | ((xa >> 6) << 4));
            mn = (int)((x4 >> 4) | ((xb >> 6) << 4));
          }
        };
        int mn_l, mn_h;
        scale_min(ql0, ql1, ql2, scl, mn_l);
        scale_min(qh0, qh1, qh2, sch, mn_h);
        mnl = ml * (float)mn_l; mnh = mh * (float)mn_h;       // dmin * m, exact: 11 x 6 bits
      }
#pragma unroll
      for (int j = 0; j < NT; j++) {
        int c[4];
        gm_mma(c, a0, a1, a2, a3, b[j].x, b[j].y);
        if (GGML == CB_GGML_Q4_K) {
          // the 6-bit scales multiply the integer sums; the super-block's d comes once per step.  The minimum takes
          // the block's digit sums of the two columns.
          isum[j][0] += scl * c[0]; isum[j][1] += scl * c[1]; isum[j][2] += sch * c[2]; isum[j][3] += sch * c[3];
          const float2 x = __ldg(reinterpret_cast<const float2*>(sp + ((int64_t)s * 8 + u) * COLS + 8 * j));
          acc[j][0] = fmaf(-mnl, x.x, acc[j][0]); acc[j][1] = fmaf(-mnl, x.y, acc[j][1]);
          acc[j][2] = fmaf(-mnh, x.x, acc[j][2]); acc[j][3] = fmaf(-mnh, x.y, acc[j][3]);
        } else {
          // |c| <= 32 * 127 * 64 < 2^22
          acc[j][0] = fmaf(dl, gm_i2f(c[0]), acc[j][0]); acc[j][1] = fmaf(dl, gm_i2f(c[1]), acc[j][1]);
          acc[j][2] = fmaf(dh, gm_i2f(c[2]), acc[j][2]); acc[j][3] = fmaf(dh, gm_i2f(c[3]), acc[j][3]);
        }
      }
    }
    if (GGML == CB_GGML_Q4_K) {
#pragma unroll
      for (int j = 0; j < NT; j++) {
        acc[j][0] = fmaf(dl, (float)isum[j][0], acc[j][0]); acc[j][1] = fmaf(dl, (float)isum[j][1], acc[j][1]);
        acc[j][2] = fmaf(dh, (float)isum[j][2], acc[j][2]); acc[j][3] = fmaf(dh, (float)isum[j][3], acc[j][3]);
      }
    }
  }
  if (failed) {
    // A stage did not arrive.  Tiles that were asked for may still land: give each one more bounded wait before the
    // shared memory is given up, record the failure, and leave the outputs alone.
    if (lane == 0) {
      const int issued = min(n_steps, consumed + GM_STAGES - 1);
      for (int s = consumed; s < issued; s++) tc::mbar_wait(&bars[s % GM_STAGES], (uint32_t)((s / GM_STAGES) & 1));
      if (BSMEM && threadIdx.x == 0) tc::mbar_wait(bar_digits, 0);
      if (atomicCAS(&status[0], 0u, 1u) == 0u) atomicExch(&status[1], (unsigned)blockIdx.x << 8 | (unsigned)warp);
    }
  }
  const int any_failed = __syncthreads_or(failed ? 1 : 0);     // the rings are free: they become the exchange buffer
  if (any_failed) return;
  // ---- halves of K and digit planes meet in shared memory: part[half][row][column]
  float* part = reinterpret_cast<float*>(gm_smem);
  const int rl = (warp & 3) * 16 + g;
#pragma unroll
  for (int j = 0; j < NT; j++) {
    const int c0 = 8 * j + 2 * t;
    float* p0 = part + ((half * GM_ROWS + rl) * GM_MAX_COLS), *p1 = part + ((half * GM_ROWS + rl + 8) * GM_MAX_COLS);
    *reinterpret_cast<float2*>(p0 + c0) = make_float2(acc[j][0], acc[j][1]);
    *reinterpret_cast<float2*>(p1 + c0) = make_float2(acc[j][2], acc[j][3]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GM_ROWS * M; idx += GM_WARPS * 32) {
    const int m = idx / GM_ROWS, r = idx % GM_ROWS;            // consecutive threads write consecutive columns of out
    const int64_t n = row_base + r;
    if (r >= 16 * n_groups || n >= N) continue;
    float v = 0.0f;
#pragma unroll
    for (int pl = PL - 1; pl >= 0; pl--) {                     // smallest plane last: unit * (A0 + 128 A1 (+ 16384 A2))
      const int c = pl * M + m;
      const float a = part[(0 * GM_ROWS + r) * GM_MAX_COLS + c] + part[(1 * GM_ROWS + r) * GM_MAX_COLS + c];
      v = fmaf(v, 128.0f, a);
    }
    v *= units[m];
    if (bias) v = __fadd_rn(v, bias[n]);
    Scalar<XT>::store(out, (int64_t)m * N + n, apply_activation(v, act));
  }
}

size_t gm_smem_bytes(int ggml) {      // the rings and their barriers; the exchange buffer lies over the rings
  static_assert((size_t)GM_WARPS * GM_STAGES * gm_stage_bytes(CB_GGML_Q4_0) >= (size_t)2 * GM_ROWS * GM_MAX_COLS * sizeof(float), "exchange buffer");
  return (size_t)GM_WARPS * GM_STAGES * gm_stage_bytes(ggml) + GM_BAR_BYTES;
}
size_t gm_digit_smem(int64_t M, int64_t K, int planes) { return (size_t)(planes * M) * (size_t)(K + GM_DPAD); }
bool gm_digits_resident(int ggml, int64_t M, int64_t K, int planes) { return gm_smem_bytes(ggml) + gm_digit_smem(M, K, planes) <= GM_SMEM_CTA; }

// The weights as a matrix of 32-bit words [N rows][bytes per row / 4], in boxes of 16 rows by one step (plus, for Q4_K,
// four words of the next).  Encoding is a pure function of its arguments and a decode loop asks for the same few maps
// on every launch, so the last ones are remembered per thread.
int gm_encode(CUtensorMap* m, const void* ptr, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes) {
  struct Entry { const void* ptr; uint64_t row_bytes, rows; uint32_t box_bytes; bool valid; CUtensorMap map; };
  constexpr int SLOTS = 64;
  static thread_local Entry cache[SLOTS];
  const uintptr_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull;
  Entry& e = cache[(h >> 40) % SLOTS];
  if (e.valid && e.ptr == ptr && e.row_bytes == row_bytes && e.rows == rows && e.box_bytes == box_bytes) { *m = e.map; return CB_OK; }
  encode_tiled_fn enc = tensor_map_encoder();
  if (!enc) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {row_bytes / 4, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes / 4, 16};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  e.ptr = ptr; e.row_bytes = row_bytes; e.rows = rows; e.box_bytes = box_bytes; e.map = *m; e.valid = true;
  return CB_OK;
}

static size_t gm_align(size_t b) { return (b + 255) & ~(size_t)255; }
// The digit kernel's outputs in the plan's workspace.  Each array is followed by at least 256 spare bytes: the product
// kernel requests the digits of the block after the one it works on.
// The first 256 bytes hold the status words (zeroed when the workspace is prepared).
constexpr size_t GM_HEADER = 256;
struct GmLayout { size_t off_digits, off_dsum, off_units, total; };
GmLayout gm_layout(int64_t M, int64_t K, int planes) {
  const size_t cols = 8 * (size_t)gm_tiles((int)M, planes);
  GmLayout l;
  l.off_digits = GM_HEADER;
  l.off_dsum = l.off_digits + gm_align(cols * (size_t)K) + 256;
  l.off_units = l.off_dsum + gm_align(cols * (size_t)(K / 32) * 4) + 256;
  l.total = l.off_units + 256;
  return l;
}

template <typename K_, typename... Args>
int gm_launch_pdl(K_ kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  return CB_OK;
}

template <typename XT, int GGML, int NT, bool BSMEM>
int gm_launch_k(const cb_qdense_desc& d, int n_sm, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  int dev = 0;
  CB_CUDA(cudaGetDevice(&dev));
  const size_t smem = std::max(gm_smem_bytes(GGML) + (BSMEM ? gm_digit_smem(d.M, d.K, gm_planes(d)) : 0), GM_SMEM_FLOOR);
  if (dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(ggml_mma_kernel<XT, GGML, NT, BSMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GM_SMEM_CTA));
    if (dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  const GmLayout l = gm_layout(d.M, d.K, gm_planes(d));
  CUtensorMap tmap;
  CB_TRY(gm_encode(&tmap, in[1], (uint64_t)(d.K / (GGML == CB_GGML_Q4_K ? 256 : 32) * gm_block_bytes(GGML)), (uint64_t)d.N, (uint32_t)gm_pitch(GGML)));
  uint8_t* w8 = (uint8_t*)ws;
  int8_t* digits = (int8_t*)(w8 + l.off_digits);
  float* dsum = (float*)(w8 + l.off_dsum);
  float* units = (float*)(w8 + l.off_units);
  int rc = gm_launch_pdl(ggml_row_digits_kernel<XT>, dim3((unsigned)d.M), dim3(GD_THREADS), 0, s, (const XT*)in[0], (int)d.M, (int64_t)d.K, 8 * NT,
                         digits, GGML == CB_GGML_Q4_K ? dsum : (float*)nullptr, units);
  if (rc != CB_OK) return rc;
  const float* bias = d.has_bias ? (const float*)in[2] : nullptr;
  return gm_launch_pdl(ggml_mma_kernel<XT, GGML, NT, BSMEM>, dim3((unsigned)gm_grid(d.N, n_sm)), dim3(GM_WARPS * 32), smem, s,
                       tmap, (const int8_t*)digits, (const float*)dsum, (const float*)units, bias, (XT*)out[0], (int)d.M,
                       (int64_t)d.K, (int64_t)d.N, (int)d.activation, (unsigned*)w8);
}

template <typename XT, int GGML>
int gm_launch_n(const cb_qdense_desc& d, int n_sm, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const bool resident = gm_digits_resident(GGML, d.M, d.K, gm_planes(d));
  switch (gm_tiles((int)d.M, gm_planes(d))) {
    case 1: return resident ? gm_launch_k<XT, GGML, 1, true>(d, n_sm, in, out, ws, s) : gm_launch_k<XT, GGML, 1, false>(d, n_sm, in, out, ws, s);
    case 2: return resident ? gm_launch_k<XT, GGML, 2, true>(d, n_sm, in, out, ws, s) : gm_launch_k<XT, GGML, 2, false>(d, n_sm, in, out, ws, s);
    case 3: return gm_launch_k<XT, GGML, 3, false>(d, n_sm, in, out, ws, s);
    case 4: return gm_launch_k<XT, GGML, 4, false>(d, n_sm, in, out, ws, s);
    case 5: return gm_launch_k<XT, GGML, 5, false>(d, n_sm, in, out, ws, s);
    default: return gm_launch_k<XT, GGML, 6, false>(d, n_sm, in, out, ws, s);
  }
}

template <typename XT>
int gm_launch_t(const cb_qdense_desc& d, int n_sm, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  switch (d.ggml_type) {
    case CB_GGML_Q4_0: return gm_launch_n<XT, CB_GGML_Q4_0>(d, n_sm, in, out, ws, s);
    case CB_GGML_Q8_0: return gm_launch_n<XT, CB_GGML_Q8_0>(d, n_sm, in, out, ws, s);
    case CB_GGML_IQ4_NL: return gm_launch_n<XT, CB_GGML_IQ4_NL>(d, n_sm, in, out, ws, s);
    default: return gm_launch_n<XT, CB_GGML_Q4_K>(d, n_sm, in, out, ws, s);
  }
}

}  // namespace

bool qdense_ggml_mma_supports(const cb_qdense_desc& d) {
  if (d.scheme != CB_QUANT_GGML || d.variant != CB_QDENSE_AUTO) return false;    // by name: the CUDA-core kernel or the prefill path
  if (d.ggml_type != CB_GGML_Q4_0 && d.ggml_type != CB_GGML_Q8_0 && d.ggml_type != CB_GGML_IQ4_NL && d.ggml_type != CB_GGML_Q4_K) return false;
  return d.M >= 1 && d.M <= GM_MAX_M && d.K >= 256 && d.K % 256 == 0 && d.K <= (1 << 24) && d.N >= 1 && (d.N + GM_ROWS - 1) / GM_ROWS <= 0x7FFFFFFFLL;
}

void qdense_ggml_mma_plan(cb_plan* p, const char* type_name) {
  const cb_qdense_desc& d = p->qd;
  p->blocks = gm_grid(d.N, p->n_sm);
  p->threads = GM_WARPS * 32;
  const int64_t m16 = std::min<int64_t>(d.M, 16);
  const int pl = gm_planes(d);
  p->dyn_smem = (int)std::max(gm_smem_bytes(d.ggml_type) + (gm_tiles((int)m16, pl) <= 2 && gm_digits_resident(d.ggml_type, m16, d.K, pl) ? gm_digit_smem(m16, d.K, pl) : 0),
                              GM_SMEM_FLOOR);
  p->workspace_bytes = gm_layout(std::min<int64_t>(d.M, 16), d.K, gm_planes(d)).total;
  p->counter_bytes = GM_HEADER;
  p->has_status = true;
  p->name = std::string("qdense_ggml_mma_") + (d.x_dtype == CB_BF16 ? "bf16_" : "f32_") + type_name;
}

int qdense_ggml_mma_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  // 16 rows of x per run; the runs follow each other on the stream and share the workspace
  const size_t esz = p->qd.x_dtype == CB_BF16 ? 2 : 4;
  for (int64_t m0 = 0; m0 < p->qd.M; m0 += 16) {
    cb_qdense_desc d = p->qd;
    d.M = std::min<int64_t>(16, p->qd.M - m0);
    const void* cin[3] = {(const uint8_t*)in[0] + (size_t)m0 * d.K * esz, in[1], d.has_bias ? in[2] : nullptr};
    void* cout[1] = {(uint8_t*)out[0] + (size_t)m0 * d.N * esz};
    CB_TRY(d.x_dtype == CB_BF16 ? gm_launch_t<__nv_bfloat16>(d, p->n_sm, cin, cout, ws, s) : gm_launch_t<float>(d, p->n_sm, cin, cout, ws, s));
  }
  return CB_OK;
}

}  // namespace cb
