// FusedQuantizedDense, Linear scheme, 8-bit weights:
//   y[M,N] = act( x[M,K] @ (W[K,N] * scale (+ zero_point)) + bias[N] )
// Reference semantics: internal/gobackend/fusedops/quantizeddense.go:330-418, :616-650
// and the activation epilogue fusedops/dense.go:176-205 of gomlx/compute.
//
// Two kernels:
//  * qdense_generic_kernel — CUDA cores, every scale layout, zero points, any
//    shape.  One thread owns one output column and sums k ascending with
//    un-fused f32 multiplies/adds, i.e. the reference's own summation order.
//  * qdense_decode_kernel — the HBM-bound decode path (M <= 16, compact
//    scales).  W is streamed exactly once: a stream-K partition gives every SM
//    the same number of [64 x 128] int8 chunks, an elected producer thread
//    keeps a ring of TMA loads (128B-swizzled) in flight, consumer warps
//    convert int8 -> f16 in registers (exact) and feed mma.sync with x (rows
//    pre-scaled by an exact power of two, then f16) as the 8-wide operand,
//    accumulate in f32, apply the per-group scale per chunk,
//    reduce across warps in shared memory and across SMs through a small
//    workspace with per-tile arrival counters (deterministic order).
#include "common.cuh"

#include <stdlib.h>
#include <string.h>
#include <atomic>
#include <mutex>

namespace cb {

// ---------------------------------------------------------------------------
// generic kernel
// ---------------------------------------------------------------------------
constexpr int QG_COLS = 128;
constexpr int QG_ROWS = 8;
constexpr int QG_KT = 256;

// Weight element (k, n) as a float.  8-bit types are read as they are; Int4 / Uint4 are packed two
// per byte over the flat element order, low nibble first, Int4 nibbles 8..15 meaning -8..-1
// (internal/gobackend/ops/convertdtype.go:199-226).  Under the NF4 scheme the low four bits of the
// element index the NormalFloat4 table of QLoRA (fused_ops.go:114-121; quantizeddense.go:586-609).
struct PackedI4 {};
struct PackedU4 {};
__constant__ float kNf4Table[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
template <typename WT> struct WeightAt {
  static __device__ __forceinline__ int get(const void* w, int64_t e) { return (int)reinterpret_cast<const WT*>(w)[e]; }
};
template <> struct WeightAt<PackedU4> {
  static __device__ __forceinline__ int get(const void* w, int64_t e) {
    const int b = reinterpret_cast<const uint8_t*>(w)[e >> 1];
    return (e & 1) ? (b >> 4) : (b & 0x0F);
  }
};
template <> struct WeightAt<PackedI4> {
  static __device__ __forceinline__ int get(const void* w, int64_t e) {
    const int v = WeightAt<PackedU4>::get(w, e);
    return v >= 8 ? v - 16 : v;
  }
};

template <typename XT, typename WT, bool NF4>
__global__ void __launch_bounds__(QG_COLS)
qdense_generic_kernel(const XT* __restrict__ x, const void* __restrict__ w, const float* __restrict__ scales,
                      const float* __restrict__ zps, const float* __restrict__ bias, XT* __restrict__ out,
                      int64_t M, int64_t K, int64_t N, int layout, int64_t block, int act) {
  __shared__ float xs[QG_ROWS][QG_KT];
  const int64_t n = (int64_t)blockIdx.x * QG_COLS + threadIdx.x;
  const int64_t m0 = (int64_t)blockIdx.y * QG_ROWS;
  const int64_t nblk = (layout == CB_SCALE_REF) ? (N + block - 1) / block : 0;
  float acc[QG_ROWS];
  const float b = (bias != nullptr && n < N) ? bias[n] : 0.0f;
#pragma unroll
  for (int i = 0; i < QG_ROWS; i++) acc[i] = b;
  for (int64_t kb = 0; kb < K; kb += QG_KT) {
    const int kt = (int)min((int64_t)QG_KT, K - kb);
    __syncthreads();
    for (int idx = threadIdx.x; idx < QG_ROWS * QG_KT; idx += QG_COLS) {
      const int r = idx / QG_KT, c = idx % QG_KT;
      xs[r][c] = (m0 + r < M && c < kt) ? (float)Scalar<XT>::load(x, (m0 + r) * K + kb + c) : 0.0f;
    }
    __syncthreads();
    if (n < N) {
      for (int kk = 0; kk < kt; kk++) {
        const int64_t k = kb + kk;
        const int wi = WeightAt<WT>::get(w, k * N + n);
        const float wf = NF4 ? kNf4Table[wi & 0x0F] : (float)wi;
        int64_t si;
        if (layout == CB_SCALE_REF) si = k * nblk + n / block;
        else if (layout == CB_SCALE_CHANNEL) si = n;
        else si = (k / block) * N + n;
        const float s = scales[si];
        if (zps != nullptr) {
          const float dq = __fadd_rn(__fmul_rn(wf, s), zps[si]);
#pragma unroll
          for (int i = 0; i < QG_ROWS; i++) acc[i] = __fadd_rn(acc[i], __fmul_rn(xs[i][kk], dq));
        } else {
#pragma unroll
          for (int i = 0; i < QG_ROWS; i++)
            acc[i] = __fadd_rn(acc[i], __fmul_rn(__fmul_rn(xs[i][kk], wf), s));
        }
      }
    }
  }
  if (n < N) {
#pragma unroll
    for (int i = 0; i < QG_ROWS; i++)
      if (m0 + i < M) Scalar<XT>::store(out, (m0 + i) * N + n, apply_activation(acc[i], act));
  }
}

// ---------------------------------------------------------------------------
// decode kernel
// ---------------------------------------------------------------------------
constexpr int QD_TILE_N = 64;                  // columns per tile
constexpr int QD_CHUNK_K = 64;                 // rows per chunk
constexpr int QD_PITCH = 80;                   // shared-memory row pitch: 64 data bytes + 16 pad (conflict-free 8-byte reads)
constexpr int QD_STEP_BYTES = 16 * QD_PITCH;    // copy unit: one k-step (16 rows)
constexpr int QD_RING_STEPS = 8;               // k-steps in each warp's ring: one in use, seven in flight
constexpr int QD_WARPS = 16;
constexpr int QD_THREADS = QD_WARPS * 32;
constexpr int QD_WS_HEADER = 64;               // status words live in the first 64 bytes

struct QdParams {
  const void* x;
  const uint8_t* w;
  const float* scales;
  const float* bias;
  void* out;
  unsigned* status;     // [0] error code, [1] detail (reserved; this kernel has no device-side waits)
  unsigned* counters;   // arrivals per stream-K tile
  float* partials;      // [grid][2][MT*8*64]
  int M, K, N;
  int n_tiles, cpt;     // column tiles, chunks per tile
  int sk_tiles;         // tiles [0, sk_tiles) are split across CTAs; the rest are owned whole
  int dp_per_cta;       // whole tiles per CTA
  long long sk_total;   // sk_tiles * cpt
  int scale_group;      // rows per scale row; 0 = one scale per column
  int activation;
  unsigned long long* dbg;   // per-CTA phase time stamps (16 per CTA) in builds with -DCB_QD_STAMPS, else NULL
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// int8 -> f16 without arithmetic.  0x64uu is the f16 number 1024 + uu, so two bytes dropped
// under 0x64 high bytes are the (biased) weights plus a constant: w + 1152 for int8 (bytes
// xor 0x80), w + 1024 for uint8, both exact.  The constant is taken out again per chunk as
// constant * sum_k x, which one extra MMA against an all-ones operand provides.
// X and Y are the same four columns of two consecutive k rows; H[b] = {X.b, Y.b} as f16x2.
__device__ __forceinline__ void bytes_to_f16x2(uint32_t X, uint32_t Y, uint32_t (&H)[4]) {
  const uint32_t ra = __byte_perm(X, Y, 0x5140);   // X.0 Y.0 X.1 Y.1
  const uint32_t rb = __byte_perm(X, Y, 0x7362);   // X.2 Y.2 X.3 Y.3
  H[0] = __byte_perm(ra, 0x64646464u, 0x4140);
  H[1] = __byte_perm(ra, 0x64646464u, 0x4342);
  H[2] = __byte_perm(rb, 0x64646464u, 0x4140);
  H[3] = __byte_perm(rb, 0x64646464u, 0x4342);
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Activation operand of one k-step and row tile.  Rows are pre-multiplied by a power of
// two (exact) that brings the row's largest magnitude to [2^14, 2^15), so the f16
// conversion cannot overflow and keeps every value within 2^-28 of the row maximum.
template <typename XT> struct XFrag;
template <> struct XFrag<__nv_bfloat16> {
  static constexpr int SPLITS = 1;     // bf16 has 8 significant bits: one f16 term is exact
  uint32_t raw[2];
  __device__ __forceinline__ void load(const uint8_t* ptr) {     // elements k, k+1 and k+8, k+9
    raw[0] = __ldg(reinterpret_cast<const uint32_t*>(ptr));
    raw[1] = __ldg(reinterpret_cast<const uint32_t*>(ptr + 16));
  }
  __device__ __forceinline__ void operands(float mul, uint32_t (&b0)[1], uint32_t (&b1)[1]) const {
    b0[0] = pack_f16x2(__uint_as_float(raw[0] << 16) * mul, __uint_as_float(raw[0] & 0xFFFF0000u) * mul);
    b1[0] = pack_f16x2(__uint_as_float(raw[1] << 16) * mul, __uint_as_float(raw[1] & 0xFFFF0000u) * mul);
  }
};
template <> struct XFrag<float> {
  static constexpr int SPLITS = 2;     // hi + lo f16 terms carry 22 significant bits
  float2 raw[2];
  __device__ __forceinline__ void load(const uint8_t* ptr) {     // elements k, k+1 and k+8, k+9
    raw[0] = __ldg(reinterpret_cast<const float2*>(ptr));
    raw[1] = __ldg(reinterpret_cast<const float2*>(ptr + 32));
  }
  __device__ __forceinline__ static void split(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(h);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = pack_f16x2(a - hf.x, b - hf.y);
  }
  __device__ __forceinline__ void operands(float mul, uint32_t (&b0)[2], uint32_t (&b1)[2]) const {
    split(raw[0].x * mul, raw[0].y * mul, b0[0], b0[1]);
    split(raw[1].x * mul, raw[1].y * mul, b1[0], b1[1]);
  }
};

// Per-row power-of-two multiplier from the row's largest magnitude (biased exponent E):
// 2^(141-E) puts the maximum in [2^14, 2^15).  Zero / denormal rows and non-finite rows
// are left unscaled (non-finite values then propagate as inf/NaN, as in f32 arithmetic).
__device__ __forceinline__ float row_multiplier(uint32_t biased_exp) {
  if (biased_exp == 0u || biased_exp == 255u) return 1.0f;
  int e = 268 - (int)biased_exp;
  e = e > 254 ? 254 : e;
  return __uint_as_float((uint32_t)e << 23);
}

// Work list of one CTA: first its share of the stream-K region (chunks of tiles that are
// split across CTAs, so their cross-CTA sums finish early), then the tiles it owns whole.
struct QdSched {
  unsigned c0;         // first stream-K chunk of this CTA (chunk counts fit 32 bits: checked at plan time)
  int n_sk, n_local;   // stream-K chunks, all chunks
  unsigned cpt;
  int sk_tiles, G, cta;
  __device__ __forceinline__ void coords(int i, int& tile, int& kc) const {
    if (i < n_sk) {
      const unsigned ch = c0 + (unsigned)i;
      const unsigned q = ch / cpt;
      tile = (int)q;
      kc = (int)(ch - q * cpt);
    } else {
      const unsigned j = (unsigned)(i - n_sk);
      const unsigned q = j / cpt;
      tile = sk_tiles + (int)q * G + cta;
      kc = (int)(j - q * cpt);
    }
  }
};

template <typename XT, int MT, bool WUNSIGNED>
__global__ void __launch_bounds__(QD_THREADS, 1)
qdense_decode_kernel(const QdParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr int RED_FLOATS = MT * 8 * QD_TILE_N;   // one [rows x 64] partial tile
  uint8_t* ring = smem_raw;
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)QD_WARPS * QD_RING_STEPS * QD_STEP_BYTES);
  __shared__ unsigned s_last[2];
  __shared__ unsigned s_rowmax[16];
  __shared__ float s_mul[16], s_inv[16];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = gridDim.x, cta = blockIdx.x;
  QdSched sched;
  sched.cpt = (unsigned)p.cpt; sched.sk_tiles = p.sk_tiles; sched.G = G; sched.cta = cta;
  // the stream-K region is shared by the first Gsk CTAs (all of them unless it is tiny)
  const int Gsk = (int)min((long long)G, p.sk_total);
  sched.c0 = cta < Gsk ? (unsigned)((long long)cta * p.sk_total / Gsk) : 0u;
  sched.n_sk = cta < Gsk ? (int)((long long)(cta + 1) * p.sk_total / Gsk - sched.c0) : 0;
  sched.n_local = sched.n_sk + p.dp_per_cta * p.cpt;
  const int n_local = sched.n_local;
  const int ksteps_tile = p.K / 16;                      // k-steps (16 rows) per column tile
  const int gsteps = p.scale_group ? p.scale_group / 16 : 0;   // k-steps per scale group (0: one scale per column)

  int dbg_n = 0;
#ifdef CB_QD_STAMPS
#define QD_STAMP() do { if (p.dbg && tid == 0 && dbg_n < 16) p.dbg[cta * 16 + dbg_n++] = global_ns(); } while (0)
#else
#define QD_STAMP() do { (void)dbg_n; } while (0)
#endif
  QD_STAMP();

  // ---- copy cursor: walks this warp's k-steps through all segments, QD_RING_STEPS ahead of the math.
  // Within a segment (one column tile, a run of chunks) the 16 warps take contiguous, equal shares
  // of the k-steps, so they reach the segment's reduction together.
  int cp_ks = 0, cp_end = 0, cp_next_seg = 0;   // next / end k-step of the share, next segment's first chunk
  const uint8_t* cp_src = p.w;                   // this lane's source address for the next k-step
  uint32_t cp_size = 16;                         // 0 for column pieces outside the matrix (zero fill)
  auto seg_share = [&](int seg_begin, int& tile, int& s0, int& s1) {   // this warp's k-steps [s0,s1) of a segment
    int kc0;
    sched.coords(seg_begin, tile, kc0);
    const int seg_end = seg_begin < sched.n_sk ? min(sched.n_sk, seg_begin + p.cpt - kc0) : seg_begin + p.cpt;
    const int a = kc0 * 4, b = min(ksteps_tile, (kc0 + seg_end - seg_begin) * 4);
    s0 = a + (b - a) * warp / QD_WARPS;
    s1 = a + (b - a) * (warp + 1) / QD_WARPS;
    return seg_end;
  };
  auto cp_issue = [&](uint8_t* slot) {           // copy one k-step (16 rows x 64 bytes), or close an empty group
    while (cp_ks >= cp_end && cp_next_seg < n_local) {
      int tile;
      cp_next_seg = seg_share(cp_next_seg, tile, cp_ks, cp_end);
      const int col = tile * QD_TILE_N + 16 * (lane & 3);
      cp_size = col < p.N ? 16u : 0u;
      cp_src = p.w + (size_t)(cp_ks * 16 + (lane >> 2)) * p.N + (cp_size ? col : 0);
    }
    if (cp_ks < cp_end) {
      const uint32_t dst = smem_u32(slot + (lane >> 2) * QD_PITCH + 16 * (lane & 3));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(cp_src), "r"(cp_size) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + 8 * QD_PITCH), "l"(cp_src + (size_t)8 * p.N), "r"(cp_size) : "memory");
      cp_src += (size_t)16 * p.N;
      cp_ks++;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // start streaming before anything else
  uint8_t* my_ring = ring + (size_t)warp * QD_RING_STEPS * QD_STEP_BYTES;
#pragma unroll 1
  for (int d = 0; d < QD_RING_STEPS; d++) cp_issue(my_ring + d * QD_STEP_BYTES);
  QD_STAMP();   // [1] first copies issued

  // Row maxima of x (every CTA computes the same values, so partial sums of different
  // CTAs share one scaling); one warp per row, all loads of a row issued together.
  if (tid < 16) s_rowmax[tid] = 0;
  __syncthreads();
  {
    constexpr int PER16 = 16 / (int)sizeof(XT);             // elements per 16-byte load
    const int vec_per_row = p.K / PER16;
    for (int m = warp; m < p.M; m += QD_WARPS) {
      uint32_t mx = 0;
      const uint4* row = reinterpret_cast<const uint4*>(reinterpret_cast<const XT*>(p.x) + (int64_t)m * p.K);
      for (int v0 = 0; v0 < vec_per_row; v0 += 32 * 8) {
        uint4 q[8];      // eight independent loads in flight per lane
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const int v = v0 + u * 32 + lane;
          q[u] = v < vec_per_row ? __ldg(row + v) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
          if (sizeof(XT) == 2) {
            const uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
            for (int e = 0; e < 4; e++) mx = max(mx, max((w[e] & 0x7FFFu) << 16, w[e] & 0x7FFF0000u));
          } else {
            mx = max(max(mx, q[u].x & 0x7FFFFFFFu), max(max(q[u].y & 0x7FFFFFFFu, q[u].z & 0x7FFFFFFFu), q[u].w & 0x7FFFFFFFu));
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) s_rowmax[m] = mx;
    }
    __syncthreads();
    if (tid < 16) {
      const float mul = row_multiplier(s_rowmax[tid] >> 23);
      s_mul[tid] = mul;
      s_inv[tid] = 1.0f / mul;
    }
    __syncthreads();
  }
  QD_STAMP();   // [2] prologue done

  float mul[MT];
  const uint8_t* xrow[MT];   // this lane's x operands; rows past M read row M-1 with weight 0
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
    const int m = mt * 8 + g;
    mul[mt] = m < p.M ? s_mul[m] : 0.0f;
    xrow[mt] = reinterpret_cast<const uint8_t*>(p.x) + ((size_t)min(m, p.M - 1) * p.K + 2 * t) * sizeof(XT);
  }
  const float wbias = WUNSIGNED ? 1024.0f : 1152.0f;   // constant carried by the converted weights

  float tot[4][MT][4];
#pragma unroll
  for (int j = 0; j < 4; j++)
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
      for (int c = 0; c < 4; c++) tot[j][mt][c] = 0.0f;

  int n_done = 0;        // k-steps this warp has consumed (selects its ring slot)
  int pend_tile[2], n_pend = 0;       // split tiles whose arrival ticket is checked at the end
  unsigned pend_ticket[2] = {0u, 0u}; // meaningful in thread 0 only
  int seg_begin = 0;
  while (seg_begin < n_local) {
    int tile, ks0, ks1;
    const int seg_end = seg_share(seg_begin, tile, ks0, ks1);
    int kc0;
    { int tt; sched.coords(seg_begin, tt, kc0); }
    const int colbase = tile * QD_TILE_N;
    const bool cols_ok = colbase + 8 * g < p.N;     // N is a multiple of 16

    // blocks of up to 8 k-steps that stay inside one scale group
    for (int ks = ks0; ks < ks1;) {
      int cnt = min(8, ks1 - ks);
      if (gsteps) cnt = min(cnt, gsteps - ks % gsteps);
      // scales of the block's group for the thread's 8 columns, x operands of its k-steps
      float sc[8];
      {
        const float* sp = p.scales + (size_t)(gsteps ? ks / gsteps : 0) * p.N + colbase + 8 * g;
#pragma unroll
        for (int q = 0; q < 2; q++) {
          const float4 v = cols_ok ? __ldg(reinterpret_cast<const float4*>(sp) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
          sc[4 * q] = v.x; sc[4 * q + 1] = v.y; sc[4 * q + 2] = v.z; sc[4 * q + 3] = v.w;
        }
      }
      XFrag<XT> xf[8][MT];
#pragma unroll
      for (int s = 0; s < 8; s++)
        if (s < cnt) {
#pragma unroll
          for (int mt = 0; mt < MT; mt++) xf[s][mt].load(xrow[mt] + (size_t)(ks + s) * 16 * sizeof(XT));
        }

      float acc[4][MT][4], xsum[MT][4];     // xsum: sum_k x of the block, per row, from the all-ones MMA
#pragma unroll
      for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int c = 0; c < 4; c++) {
          xsum[mt][c] = 0.0f;
#pragma unroll
          for (int j = 0; j < 4; j++) acc[j][mt][c] = 0.0f;
        }

#pragma unroll
      for (int s = 0; s < 8; s++) {
        if (s < cnt) {
          // the k-step about to be used is the oldest of this warp's open copy groups
          uint8_t* slot = my_ring + (n_done % QD_RING_STEPS) * QD_STEP_BYTES;
          asm volatile("cp.async.wait_group %0;" ::"n"(QD_RING_STEPS - 1) : "memory");
          __syncwarp();
          {
            // rows 2t, 2t+1, 2t+8, 2t+9: exactly the k indices the mma fragment assigns to lane t;
            // the 80-byte pitch makes the loads conflict-free.
            uint32_t L[4][2];
#pragma unroll
            for (int r = 0; r < 4; r++) {
              const int row = 2 * t + (r & 1) + 8 * (r >> 1);
              const uint2 v = *reinterpret_cast<const uint2*>(slot + row * QD_PITCH + 8 * g);
              L[r][0] = v.x; L[r][1] = v.y;
              if (!WUNSIGNED) { L[r][0] ^= 0x80808080u; L[r][1] ^= 0x80808080u; }
            }
            uint32_t xb0[MT][XFrag<XT>::SPLITS], xb1[MT][XFrag<XT>::SPLITS];
#pragma unroll
            for (int mt = 0; mt < MT; mt++) xf[s][mt].operands(mul[mt], xb0[mt], xb1[mt]);
            // H*[b]: columns b (lo) and 4+b (hi) of the thread's 8, for k rows (2t,2t+1) and (2t+8,2t+9)
            uint32_t Hlo01[4], Hhi01[4], Hlo23[4], Hhi23[4];
            bytes_to_f16x2(L[0][0], L[1][0], Hlo01);
            bytes_to_f16x2(L[0][1], L[1][1], Hhi01);
            bytes_to_f16x2(L[2][0], L[3][0], Hlo23);
            bytes_to_f16x2(L[2][1], L[3][1], Hhi23);
            {
              const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};   // f16 1.0
#pragma unroll
              for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int sp = 0; sp < XFrag<XT>::SPLITS; sp++) mma_f16_16816(xsum[mt], ones, xb0[mt][sp], xb1[mt][sp]);
            }
#pragma unroll
            for (int b = 0; b < 4; b++) {
              const uint32_t a[4] = {Hlo01[b], Hhi01[b], Hlo23[b], Hhi23[b]};
#pragma unroll
              for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int sp = 0; sp < XFrag<XT>::SPLITS; sp++)
                  mma_f16_16816(acc[b][mt], a, xb0[mt][sp], xb1[mt][sp]);
            }
          }
          __syncwarp();     // every lane is done reading the slot: refill it
          cp_issue(slot);
          n_done++;
        }
      }
      // column of acc[b][*][0..1] is 8g+b, of acc[b][*][2..3] is 8g+4+b
#pragma unroll
      for (int b = 0; b < 4; b++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
          tot[b][mt][0] = fmaf(fmaf(-wbias, xsum[mt][0], acc[b][mt][0]), sc[b], tot[b][mt][0]);
          tot[b][mt][1] = fmaf(fmaf(-wbias, xsum[mt][1], acc[b][mt][1]), sc[b], tot[b][mt][1]);
          tot[b][mt][2] = fmaf(fmaf(-wbias, xsum[mt][2], acc[b][mt][2]), sc[4 + b], tot[b][mt][2]);
          tot[b][mt][3] = fmaf(fmaf(-wbias, xsum[mt][3], acc[b][mt][3]), sc[4 + b], tot[b][mt][3]);
        }
      ks += cnt;
    }
    QD_STAMP();

    // ---- cross-warp reduction of this segment -------------------------
    float* mine = red + warp * RED_FLOATS;
#pragma unroll
    for (int b = 0; b < 4; b++)
#pragma unroll
      for (int mt = 0; mt < MT; mt++) {
        const int m = mt * 8 + 2 * t;
        mine[m * QD_TILE_N + 8 * g + b] = tot[b][mt][0];
        mine[(m + 1) * QD_TILE_N + 8 * g + b] = tot[b][mt][1];
        mine[m * QD_TILE_N + 8 * g + 4 + b] = tot[b][mt][2];
        mine[(m + 1) * QD_TILE_N + 8 * g + 4 + b] = tot[b][mt][3];
        tot[b][mt][0] = tot[b][mt][1] = tot[b][mt][2] = tot[b][mt][3] = 0.0f;
      }
    __syncthreads();
    QD_STAMP();   // after deposit barrier

    constexpr int PER_THREAD = RED_FLOATS / QD_THREADS;
    float sum[PER_THREAD];
#pragma unroll
    for (int e = 0; e < PER_THREAD; e++) {
      const int idx = tid + e * QD_THREADS;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < QD_WARPS; w++) v += red[w * RED_FLOATS + idx];
      sum[e] = v;
    }

    const bool whole_tile = (kc0 == 0) && (seg_end - seg_begin == p.cpt);
    bool finalize = whole_tile;
    if (!whole_tile) {
      // partial tile: park the CTA's sum, then see whether every contributor has arrived
      const long long tile_begin = (long long)tile * p.cpt, tile_end = tile_begin + p.cpt;
      const int slot = (kc0 > 0) ? 0 : 1;
      float* dst = p.partials + ((size_t)cta * 2 + slot) * RED_FLOATS;
#pragma unroll
      for (int e = 0; e < PER_THREAD; e++) dst[tid + e * QD_THREADS] = sum[e];
      __syncthreads();
      // Arrive on the tile's counter now, look at the ticket only when the CTA has finished all
      // its chunks: by then every contributor has parked its sum, and nobody waits in between.
      pend_tile[n_pend] = tile;
      if (tid == 0) {
        __threadfence();
        pend_ticket[n_pend] = atomicAdd(&p.counters[tile], 1u);
      }
      n_pend++;
    }
    if (finalize) {
#pragma unroll
      for (int e = 0; e < PER_THREAD; e++) {
        const int idx = tid + e * QD_THREADS;
        const int m = idx / QD_TILE_N, col = colbase + idx % QD_TILE_N;
        if (m < p.M && col < p.N) {
          float v = sum[e] * s_inv[m];           // undo the row's power-of-two scaling (exact)
          if (p.bias) v += __ldg(p.bias + col);
          v = apply_activation(v, p.activation);
          Scalar<XT>::store(reinterpret_cast<XT*>(p.out), (int64_t)m * p.N + col, v);
        }
      }
    }
    __syncthreads();   // red[] is reused by the next segment
    QD_STAMP();
    seg_begin = seg_end;
  }
  asm volatile("cp.async.wait_all;" ::: "memory");

  // ---- split tiles this CTA contributed to: the last arriver sums the parked partials ----
  if (tid == 0) {
    __threadfence();     // the tickets came back long ago; order the reads below after them
    for (int i = 0; i < 2; i++) {
      unsigned last = 0u;
      if (i < n_pend) {
        const int tile = pend_tile[i];
        const long long tile_begin = (long long)tile * p.cpt, tile_end = tile_begin + p.cpt;
        const int cf = (int)(((tile_begin + 1) * Gsk - 1) / p.sk_total);
        const int cl = (int)((tile_end * Gsk - 1) / p.sk_total);
        last = (pend_ticket[i] == (unsigned)(cl - cf)) ? 1u : 0u;
        if (last) p.counters[tile] = 0;      // leave the workspace prepared for the next launch
      }
      s_last[i] = last;
    }
  }
  __syncthreads();
  for (int i = 0; i < n_pend; i++) {
    if (s_last[i] == 0) continue;
    const int tile = pend_tile[i];
    const long long tile_begin = (long long)tile * p.cpt, tile_end = tile_begin + p.cpt;
    const int cf = (int)(((tile_begin + 1) * Gsk - 1) / p.sk_total);
    const int cl = (int)((tile_end * Gsk - 1) / p.sk_total);
    constexpr int PER_THREAD = RED_FLOATS / QD_THREADS;
    float sum[PER_THREAD];
#pragma unroll
    for (int e = 0; e < PER_THREAD; e++) sum[e] = 0.0f;
    for (int c0 = cf; c0 <= cl; c0 += 4) {   // fixed order: results do not depend on arrival order
      float v[4][PER_THREAD];                // four contributors' loads in flight together
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int c = min(c0 + u, cl);
        const long long cs = (long long)c * p.sk_total / Gsk;
        const float* src = p.partials + ((size_t)c * 2 + (cs > tile_begin ? 0 : 1)) * RED_FLOATS;
#pragma unroll
        for (int e = 0; e < PER_THREAD; e++) v[u][e] = __ldcg(src + tid + e * QD_THREADS);
      }
#pragma unroll
      for (int u = 0; u < 4; u++)
        if (c0 + u <= cl) {
#pragma unroll
          for (int e = 0; e < PER_THREAD; e++) sum[e] += v[u][e];
        }
    }
    const int colbase = tile * QD_TILE_N;
#pragma unroll
    for (int e = 0; e < PER_THREAD; e++) {
      const int idx = tid + e * QD_THREADS;
      const int m = idx / QD_TILE_N, col = colbase + idx % QD_TILE_N;
      if (m < p.M && col < p.N) {
        float v = sum[e] * s_inv[m];
        if (p.bias) v += __ldg(p.bias + col);
        v = apply_activation(v, p.activation);
        Scalar<XT>::store(reinterpret_cast<XT*>(p.out), (int64_t)m * p.N + col, v);
      }
    }
  }
  QD_STAMP();
#undef QD_STAMP
}

// ---------------------------------------------------------------------------
// planning and launch
// ---------------------------------------------------------------------------
static size_t decode_smem(int mt) {
  return (size_t)QD_WARPS * QD_RING_STEPS * QD_STEP_BYTES + (size_t)QD_WARPS * mt * 8 * QD_TILE_N * 4;
}

// Tiles split across CTAs (stream-K) and tiles owned whole, for `tiles` column tiles on `grid` CTAs.
static void decode_schedule(long long tiles, int grid, int* sk_tiles, int* dp_per_cta) {
  *dp_per_cta = (int)(tiles / grid);
  *sk_tiles = (int)(tiles - (long long)*dp_per_cta * grid);
}

static bool decode_eligible(const cb_qdense_desc& d, std::string* why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  if (d.M < 1 || d.M > 16) return no("M must be in [1,16]");
  if (d.has_zero_point) return no("zero points are handled by the generic kernel");
  if (d.scale_layout == CB_SCALE_REF) return no("reference [K, N/block] scales are handled by the generic kernel");
  if (d.K < 16 || d.K % 16 != 0) return no("K must be a positive multiple of 16");
  if (d.N < 16 || d.N % 16 != 0) return no("N must be a positive multiple of 16");
  if (d.scale_layout == CB_SCALE_KGROUP && (d.block_size <= 0 || d.block_size % QD_CHUNK_K != 0))
    return no("K-group size must be a multiple of 64");
  if (d.K > (1 << 30) || d.N > (1 << 30)) return no("dimension too large");
  if (((d.K + QD_CHUNK_K - 1) / QD_CHUNK_K) * ((d.N + QD_TILE_N - 1) / QD_TILE_N) >= (1ll << 31)) return no("too many chunks");
  return true;
}

bool qdense_prefill_eligible(const cb_qdense_desc& d, std::string* why);
int qdense_prefill_plan(cb_plan* p);
int qdense_prefill_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
bool qdense_decode_tc_eligible(const cb_qdense_desc& d, std::string* why);
int qdense_decode_tc_plan(cb_plan* p);
int qdense_decode_tc_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);

int qdense_plan(cb_plan* p) {
  cb_qdense_desc& d = p->qd;
  if (d.M < 0 || d.K < 0 || d.N < 0) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: negative dimension");
  if (d.x_dtype != CB_F32 && d.x_dtype != CB_BF16)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: x must be float32 (or bfloat16), got %s", dtype_name(d.x_dtype));
  if (d.scheme == CB_QUANT_GGML) return qdense_ggml_plan(p);
  if (d.scheme != CB_QUANT_LINEAR && d.scheme != CB_QUANT_NF4)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense: unknown quantization scheme %d", d.scheme);
  if (d.w_dtype != CB_I8 && d.w_dtype != CB_U8 && d.w_dtype != CB_I4 && d.w_dtype != CB_U4)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense: %s unsupported weight type %s", d.scheme == CB_QUANT_NF4 ? "NF4" : "Linear", dtype_name(d.w_dtype));
  if (d.scheme == CB_QUANT_NF4 && d.has_zero_point)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: ZeroPoint must be nil for NF4 quantization scheme");
  // the streaming and tensor-core kernels read int8 / uint8 Linear weights; everything else is the generic kernel's
  const bool generic_only = d.scheme != CB_QUANT_LINEAR || d.w_dtype == CB_I4 || d.w_dtype == CB_U4;
  if (d.scale_layout < CB_SCALE_REF || d.scale_layout > CB_SCALE_KGROUP)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown scale layout %d", d.scale_layout);
  if (d.scale_layout != CB_SCALE_CHANNEL && d.block_size <= 0)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: block size must be positive, got %lld", (long long)d.block_size);
  if (d.activation < CB_ACT_NONE || d.activation > CB_ACT_TANH)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown activation %d", d.activation);
  p->n_inputs = 3 + (d.has_zero_point ? 1 : 0) + (d.has_bias ? 1 : 0);
  p->n_outputs = 1;
  if (d.gather_ranks < 0) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: gather_ranks must not be negative");

  int variant = d.variant;
  std::string why;
  const bool can_decode = !generic_only && decode_eligible(d, &why);
  if (generic_only) why = "packed 4-bit weights and the NF4 scheme run on the generic kernel";
  std::string why_prefill, why_tc;
  const bool can_decode_tc = !generic_only && qdense_decode_tc_eligible(d, &why_tc);
  // the prefill path expands every weight format of the Linear and NF4 schemes to bf16 planes
  const bool can_prefill = qdense_prefill_eligible(d, &why_prefill);
  if (generic_only) why_tc = why;
  if (d.gather_ranks > 1) {          // the fused all-gather exists in the tensor-core decode kernel only
    if (variant != CB_QDENSE_AUTO && variant != CB_QDENSE_DECODE_TC)
      return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense: a gathered plan needs the tensor-core decode kernel");
    variant = CB_QDENSE_DECODE_TC;
  }
  if (variant == CB_QDENSE_AUTO) {
    // decode shapes stream W once; beyond 16 rows the tensor-core GEMM wins as soon as the
    // problem is large enough to pay for expanding the weights (small ones stay on the
    // CUDA-core kernel, which also keeps the reference's summation order)
    if (can_decode_tc) variant = CB_QDENSE_DECODE_TC;
    else if (can_decode) variant = CB_QDENSE_DECODE_MMA;
    else if (can_prefill && d.M > 16 && (double)d.M * d.K * d.N >= 64.0 * 1024 * 1024 && !qdense_w4_supports(d)) variant = CB_QDENSE_PREFILL;
    else variant = CB_QDENSE_GENERIC;
  }
  if (variant == CB_QDENSE_DECODE_MMA && !can_decode)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense decode kernel: %s", why.c_str());
  if (variant == CB_QDENSE_PREFILL && !can_prefill)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense prefill kernel: %s", why_prefill.c_str());
  if (variant == CB_QDENSE_DECODE_TC && !can_decode_tc)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense tensor-core decode kernel: %s", why_tc.c_str());
  if (variant < CB_QDENSE_AUTO || variant > CB_QDENSE_DECODE_TC)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown kernel variant %d", variant);
  p->variant = variant;
  if (variant == CB_QDENSE_PREFILL) return qdense_prefill_plan(p);
  if (variant == CB_QDENSE_DECODE_TC) return qdense_decode_tc_plan(p);

  if (variant == CB_QDENSE_GENERIC && qdense_w4_supports(d)) {   // decode shapes of the packed 4-bit formats
    p->w4_stream = true;
    qdense_w4_plan(p);
    return CB_OK;
  }
  if (variant == CB_QDENSE_GENERIC) {
    p->blocks = (int)(((d.N + QG_COLS - 1) / QG_COLS) * ((d.M + QG_ROWS - 1) / QG_ROWS));
    p->threads = QG_COLS;
    p->dyn_smem = 0;
    p->workspace_bytes = 0;
    const char* wn = d.w_dtype == CB_U8 ? "_u8" : (d.w_dtype == CB_I8 ? "_i8" : (d.w_dtype == CB_U4 ? "_u4" : "_i4"));
    p->name = std::string("qdense_generic_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") + wn + (d.scheme == CB_QUANT_NF4 ? "_nf4" : "");
    return CB_OK;
  }
  const int mt = d.M <= 8 ? 1 : 2;
  const long long n_tiles = (d.N + QD_TILE_N - 1) / QD_TILE_N;
  const long long cpt = (d.K + QD_CHUNK_K - 1) / QD_CHUNK_K;
  p->blocks = (int)std::min<long long>(p->n_sm, n_tiles * cpt);
  p->threads = QD_THREADS;
  p->dyn_smem = (int)decode_smem(mt);
  p->counter_bytes = (QD_WS_HEADER + (size_t)n_tiles * 4 + 255) & ~(size_t)255;
  p->workspace_bytes = p->counter_bytes + (size_t)p->blocks * 2 * mt * 8 * QD_TILE_N * 4 + (size_t)p->blocks * 16 * 8;
  p->has_status = false;
  p->name = std::string("qdense_decode_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") + (mt == 1 ? "_m8" : "_m16") +
            (d.w_dtype == CB_U8 ? "_u8" : "_i8");
  return CB_OK;
}

template <typename XT, typename WT, bool NF4>
static int launch_generic(const cb_plan* p, const void* const* in, void* const* out, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (d.M == 0 || d.N == 0) return CB_OK;
  int idx = 3;
  const float* zp = d.has_zero_point ? (const float*)in[idx++] : nullptr;
  const float* bias = d.has_bias ? (const float*)in[idx++] : nullptr;
  dim3 grid((unsigned)((d.N + QG_COLS - 1) / QG_COLS), (unsigned)((d.M + QG_ROWS - 1) / QG_ROWS));
  qdense_generic_kernel<XT, WT, NF4><<<grid, QG_COLS, 0, s>>>((const XT*)in[0], in[1], (const float*)in[2], zp,
                                                         bias, (XT*)out[0], d.M, d.K, d.N, d.scale_layout,
                                                         d.block_size > 0 ? d.block_size : 1, d.activation);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

template <typename XT, int MT, bool WU>
static int launch_decode_t(const cb_plan* p, const QdParams& prm, cudaStream_t s) {
  // The attribute is per device: set it once for each device this process launches on.
  static std::atomic<bool> configured[64];
  if (p->dev >= 64 || !configured[p->dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(qdense_decode_kernel<XT, MT, WU>, cudaFuncAttributeMaxDynamicSharedMemorySize, p->dyn_smem));
    if (p->dev < 64) configured[p->dev].store(true, std::memory_order_release);
  }
  qdense_decode_kernel<XT, MT, WU><<<p->blocks, QD_THREADS, p->dyn_smem, s>>>(prm);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

static int launch_decode(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  QdParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.x = in[0];
  prm.w = (const uint8_t*)in[1];
  prm.scales = (const float*)in[2];
  prm.bias = d.has_bias ? (const float*)in[3] : nullptr;
  prm.out = out[0];
  uint8_t* w8 = (uint8_t*)ws;
  const int mt = d.M <= 8 ? 1 : 2;
  prm.status = (unsigned*)w8;
  prm.counters = (unsigned*)(w8 + QD_WS_HEADER);
  prm.partials = (float*)(w8 + p->counter_bytes);
  prm.M = (int)d.M; prm.K = (int)d.K; prm.N = (int)d.N;
  prm.n_tiles = (int)((d.N + QD_TILE_N - 1) / QD_TILE_N);
  prm.cpt = (int)((d.K + QD_CHUNK_K - 1) / QD_CHUNK_K);
  decode_schedule(prm.n_tiles, p->blocks, &prm.sk_tiles, &prm.dp_per_cta);
  prm.sk_total = (long long)prm.sk_tiles * prm.cpt;
  prm.scale_group = d.scale_layout == CB_SCALE_KGROUP ? (int)d.block_size : 0;
  prm.activation = d.activation;
#ifdef CB_QD_STAMPS
  prm.dbg = (unsigned long long*)(w8 + p->counter_bytes + (size_t)p->blocks * 2 * mt * 8 * QD_TILE_N * 4);
#else
  prm.dbg = nullptr;
#endif
  if ((reinterpret_cast<uintptr_t>(in[0]) & 15) || (reinterpret_cast<uintptr_t>(in[1]) & 15) || (reinterpret_cast<uintptr_t>(in[2]) & 15))
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: x, weights and scales must be 16-byte aligned");
  const bool bf = d.x_dtype == CB_BF16, wu = d.w_dtype == CB_U8;
#define QD_DISPATCH(XT)                                                                       \
  (mt == 1 ? (wu ? launch_decode_t<XT, 1, true>(p, prm, s) : launch_decode_t<XT, 1, false>(p, prm, s)) \
           : (wu ? launch_decode_t<XT, 2, true>(p, prm, s) : launch_decode_t<XT, 2, false>(p, prm, s)))
  return bf ? QD_DISPATCH(__nv_bfloat16) : QD_DISPATCH(float);
#undef QD_DISPATCH
}

int qdense_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (d.scheme == CB_QUANT_GGML) return qdense_ggml_launch(p, in, out, ws, s);
  if (p->w4_stream) return qdense_w4_launch(p, in, out, ws, s);
  if (p->variant == CB_QDENSE_DECODE_MMA) return launch_decode(p, in, out, ws, s);
  if (p->variant == CB_QDENSE_PREFILL) return qdense_prefill_launch(p, in, out, ws, s);
  if (p->variant == CB_QDENSE_DECODE_TC) return qdense_decode_tc_launch(p, in, out, ws, s);
  const bool bf = d.x_dtype == CB_BF16, wu = d.w_dtype == CB_U8;
  (void)wu;
  const bool nf4 = d.scheme == CB_QUANT_NF4;
#define QG_DISPATCH_W(XT, WT) (nf4 ? launch_generic<XT, WT, true>(p, in, out, s) : launch_generic<XT, WT, false>(p, in, out, s))
#define QG_DISPATCH(XT)                                                     \
  (d.w_dtype == CB_U8 ? QG_DISPATCH_W(XT, uint8_t)                          \
   : d.w_dtype == CB_I8 ? QG_DISPATCH_W(XT, int8_t)                         \
   : d.w_dtype == CB_U4 ? QG_DISPATCH_W(XT, PackedU4) : QG_DISPATCH_W(XT, PackedI4))
  return bf ? QG_DISPATCH(__nv_bfloat16) : QG_DISPATCH(float);
#undef QG_DISPATCH
#undef QG_DISPATCH_W
}


// ---------------------------------------------------------------------------
// Decode kernel without any allocation: the scratch lives in the library image.
// ---------------------------------------------------------------------------
// Some hosts of this library may not allocate device memory at the moment they need a
// projection: an inference server that has handed every byte of HBM to its own arena, a
// plugin running inside another framework's stream callback or graph-replay window, a
// process whose allocator is locked down after start-up.  For them the stream-K scratch
// (arrival counters + parked partial tiles) is a fixed array in device memory that every
// GPU loading the library holds until the process exits.
constexpr size_t QD_STATIC_SCRATCH_BYTES = 2u << 20;   // 2 MiB per device
static __device__ __align__(256) unsigned char g_qd_static_scratch[QD_STATIC_SCRATCH_BYTES];

// In host code `g_qd_static_scratch` is only a handle for the runtime, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, per device.
static std::mutex g_qd_static_mu;
static void* g_qd_static_ptr[64];

static int qd_static_scratch(int dev, void** ptr) {
  if (dev < 0 || dev >= 64) return fail(CB_ERR_INVALID_ARG, "device %d out of range for the static scratch", dev);
  std::lock_guard<std::mutex> l(g_qd_static_mu);
  if (!g_qd_static_ptr[dev]) {
    void* p = nullptr;
    CB_CUDA(cudaGetSymbolAddress(&p, g_qd_static_scratch));   // `dev` is current: set_device ran just before
    g_qd_static_ptr[dev] = p;
  }
  *ptr = g_qd_static_ptr[dev];
  return CB_OK;
}

template <typename XT, int MT, bool WU>
static int launch_decode_static_t(int dev, int blocks, int dyn_smem, const QdParams& prm, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  if (!configured[dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(qdense_decode_kernel<XT, MT, WU>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem));
    configured[dev].store(true, std::memory_order_release);
  }
  qdense_decode_kernel<XT, MT, WU><<<blocks, QD_THREADS, dyn_smem, s>>>(prm);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

}  // namespace cb

extern "C" int cb_qdense_decode_static(int dev, const cb_qdense_desc* desc, const void* x, const void* weights,
                                       const void* scales, const void* bias, void* out, cb_stream stream) {
  using namespace cb;
  clear_error();
  if (!desc || !x || !weights || !scales || !out) return fail(CB_ERR_INVALID_ARG, "cb_qdense_decode_static: NULL argument");
  const cb_qdense_desc& d = *desc;
  std::string why;
  if (d.x_dtype != CB_F32 && d.x_dtype != CB_BF16) return fail(CB_ERR_INVALID_ARG, "cb_qdense_decode_static: x must be float32 or bfloat16");
  if (d.w_dtype != CB_I8 && d.w_dtype != CB_U8) return fail(CB_ERR_NOT_IMPLEMENTED, "cb_qdense_decode_static: weights must be int8 or uint8");
  if (d.scheme != CB_QUANT_LINEAR) return fail(CB_ERR_NOT_IMPLEMENTED, "cb_qdense_decode_static: only the Linear scheme");
  if (!decode_eligible(d, &why)) return fail(CB_ERR_NOT_IMPLEMENTED, "cb_qdense_decode_static: %s", why.c_str());
  if (d.has_bias && !bias) return fail(CB_ERR_INVALID_ARG, "cb_qdense_decode_static: bias is NULL");
  if (d.activation < CB_ACT_NONE || d.activation > CB_ACT_TANH)
    return fail(CB_ERR_INVALID_ARG, "cb_qdense_decode_static: unknown activation %d", d.activation);
  if (d.gather_ranks > 1)
    return fail(CB_ERR_NOT_IMPLEMENTED, "cb_qdense_decode_static: a gathered plan needs the tensor-core decode kernel (cb_plan_qdense)");
  CB_TRY(set_device(dev));
  const int mt = d.M <= 8 ? 1 : 2;
  const long long n_tiles = (d.N + QD_TILE_N - 1) / QD_TILE_N;
  const long long cpt = (d.K + QD_CHUNK_K - 1) / QD_CHUNK_K;
  int n_sm = sm_count(dev);
  if (n_sm <= 0) n_sm = 148;
  const int blocks = (int)std::min<long long>(n_sm, n_tiles * cpt);
  const size_t counter_bytes = (QD_WS_HEADER + (size_t)n_tiles * 4 + 255) & ~(size_t)255;
  const size_t need = counter_bytes + (size_t)blocks * 2 * mt * 8 * QD_TILE_N * 4;
  if (need > QD_STATIC_SCRATCH_BYTES)
    return fail(CB_ERR_INVALID_ARG,
                "cb_qdense_decode_static: this shape needs %zu bytes of scratch, the built-in scratch holds %zu "
                "(use cb_plan_qdense with a caller-owned workspace)", need, QD_STATIC_SCRATCH_BYTES);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(weights) & 15) || (reinterpret_cast<uintptr_t>(scales) & 15))
    return fail(CB_ERR_INVALID_ARG, "cb_qdense_decode_static: x, weights and scales must be 16-byte aligned");
  void* scratch = nullptr;
  CB_TRY(qd_static_scratch(dev, &scratch));
  cudaStream_t s = (cudaStream_t)stream;
  // The array keeps whatever the previous call left: the arrival counters must start at zero.
  CB_CUDA(cudaMemsetAsync(scratch, 0, counter_bytes, s));
  QdParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.x = x;
  prm.w = (const uint8_t*)weights;
  prm.scales = (const float*)scales;
  prm.bias = d.has_bias ? (const float*)bias : nullptr;
  prm.out = out;
  uint8_t* w8 = (uint8_t*)scratch;
  prm.status = (unsigned*)w8;
  prm.counters = (unsigned*)(w8 + QD_WS_HEADER);
  prm.partials = (float*)(w8 + counter_bytes);
  prm.M = (int)d.M; prm.K = (int)d.K; prm.N = (int)d.N;
  prm.n_tiles = (int)n_tiles;
  prm.cpt = (int)cpt;
  decode_schedule(prm.n_tiles, blocks, &prm.sk_tiles, &prm.dp_per_cta);
  prm.sk_total = (long long)prm.sk_tiles * prm.cpt;
  prm.scale_group = d.scale_layout == CB_SCALE_KGROUP ? (int)d.block_size : 0;
  prm.activation = d.activation;
  const int smem = (int)decode_smem(mt);
  const bool bf = d.x_dtype == CB_BF16, wu = d.w_dtype == CB_U8;
#define QD_DISPATCH(XT)                                                                                     \
  (mt == 1 ? (wu ? launch_decode_static_t<XT, 1, true>(dev, blocks, smem, prm, s) : launch_decode_static_t<XT, 1, false>(dev, blocks, smem, prm, s)) \
           : (wu ? launch_decode_static_t<XT, 2, true>(dev, blocks, smem, prm, s) : launch_decode_static_t<XT, 2, false>(dev, blocks, smem, prm, s)))
  return bf ? QD_DISPATCH(__nv_bfloat16) : QD_DISPATCH(float);
#undef QD_DISPATCH
}
