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
//    convert int8 -> bf16 in registers (exact) and feed mma.sync with x as the
//    8-wide operand, accumulate in f32, apply the per-group scale per chunk,
//    reduce across warps in shared memory and across SMs through a small
//    workspace with per-tile arrival counters (deterministic order).
#include "common.cuh"

#include <string.h>
#include <mutex>

namespace cb {

// ---------------------------------------------------------------------------
// generic kernel
// ---------------------------------------------------------------------------
constexpr int QG_COLS = 128;
constexpr int QG_ROWS = 8;
constexpr int QG_KT = 256;

template <typename XT, typename WT>
__global__ void __launch_bounds__(QG_COLS)
qdense_generic_kernel(const XT* __restrict__ x, const WT* __restrict__ w, const float* __restrict__ scales,
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
        const float wf = (float)w[k * N + n];
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
constexpr int QD_TILE_N = 128;                 // columns per chunk = one swizzled 128-byte row
constexpr int QD_CHUNK_K = 64;                 // rows per chunk
constexpr int QD_STAGE_BYTES = QD_TILE_N * QD_CHUNK_K;
constexpr int QD_CONSUMERS = 8;                // consumer warps (two warpgroups)
constexpr int QD_THREADS = (QD_CONSUMERS + 4) * 32;   // + one producer warpgroup (one lane works)
constexpr int QD_WS_HEADER = 64;               // status words live in the first 64 bytes
constexpr unsigned long long QD_WAIT_NS = 1000000000ull;   // every barrier wait gives up after 1 s

enum { QD_ERR_FULL_WAIT = 1, QD_ERR_EMPTY_WAIT = 2 };

struct QdParams {
  const void* x;
  const float* scales;
  const float* bias;
  void* out;
  unsigned* status;     // [0] error code, [1] detail
  unsigned* counters;   // per column tile
  float* partials;      // [grid][2][MT*8*128]
  int M, K, N;
  int n_tiles, cpt;     // column tiles, chunks per tile
  long long total;      // n_tiles * cpt
  int scale_group;      // rows per scale row; 0 = one scale per column
  int activation;
  int stages;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false once QD_WAIT_NS elapsed without the phase completing.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > QD_WAIT_NS) return false;
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte `b` of `word` (already biased to unsigned) -> exact f32 integer value.
// 0x4B0000uu is 2^23 + uu; subtracting the magic removes 2^23 and the +128 bias.
template <int B>
__device__ __forceinline__ float byte_to_f32(uint32_t word, float magic) {
  return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540 + B)) - magic;
}
// Two exact small-integer floats -> packed bf16x2 (their upper halves; no rounding happens).
__device__ __forceinline__ uint32_t pack_hi16(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename XT> struct XFrag;
// bf16 activations: one operand register pair per k-step and row tile.
template <> struct XFrag<__nv_bfloat16> {
  static constexpr int SPLITS = 1;
  uint32_t b0[1], b1[1];
  __device__ __forceinline__ void load(const void* x, int64_t row_off, int k, bool ok) {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(x) + row_off + k;
    b0[0] = ok ? *reinterpret_cast<const uint32_t*>(p) : 0u;
    b1[0] = ok ? *reinterpret_cast<const uint32_t*>(p + 8) : 0u;
  }
};
// f32 activations: split every value into three bf16 terms (hi + mid + lo carries
// all 24 significand bits), so the products with the exact bf16 weights are exact.
template <> struct XFrag<float> {
  static constexpr int SPLITS = 3;
  uint32_t b0[3], b1[3];
  __device__ __forceinline__ static void split(float a, float b, uint32_t* out, int stride) {
    float ah = __bfloat162float(__float2bfloat16_rn(a)), bh = __bfloat162float(__float2bfloat16_rn(b));
    float ar = a - ah, br = b - bh;
    float am = __bfloat162float(__float2bfloat16_rn(ar)), bm = __bfloat162float(__float2bfloat16_rn(br));
    float al = ar - am, bl = br - bm;
    out[0] = pack_hi16(ah, bh);
    out[stride] = pack_hi16(am, bm);
    out[2 * stride] = pack_bf16x2(al, bl);
  }
  __device__ __forceinline__ void load(const void* x, int64_t row_off, int k, bool ok) {
    const float* p = reinterpret_cast<const float*>(x) + row_off + k;
    float2 lo = ok ? *reinterpret_cast<const float2*>(p) : make_float2(0.f, 0.f);
    float2 hi = ok ? *reinterpret_cast<const float2*>(p + 8) : make_float2(0.f, 0.f);
    split(lo.x, lo.y, b0, 1);
    split(hi.x, hi.y, b1, 1);
  }
};

template <typename XT, int MT, bool WUNSIGNED>
__global__ void __launch_bounds__(QD_THREADS, 1)
qdense_decode_kernel(const __grid_constant__ CUtensorMap tmap, const QdParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int RED_FLOATS = MT * 8 * QD_TILE_N;   // one [rows x 128] partial tile
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = base;
  float* red = reinterpret_cast<float*>(base + (size_t)p.stages * QD_STAGE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(red + QD_CONSUMERS * RED_FLOATS);
  uint64_t* empty = full + p.stages;
  __shared__ unsigned s_flag;
  __shared__ unsigned s_failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const long long c0 = (long long)cta * p.total / G;
  const long long c1 = (long long)(cta + 1) * p.total / G;
  const int n_local = (int)(c1 - c0);

  if (tid == 0) {
    for (int s = 0; s < p.stages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp >= QD_CONSUMERS) {
    // ---------------- producer warpgroup: keep the TMA ring full ---------
    // Registers move from this warpgroup to the two consumer warpgroups
    // (384 x 168 = 128 x 40 + 256 x 232).
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == QD_CONSUMERS && lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap) : "memory");
      for (int i = 0; i < n_local; i++) {
        const int s = i % p.stages;
        if (i >= p.stages) {
          if (!mbar_wait_bounded(&empty[s], (uint32_t)((i / p.stages - 1) & 1))) {
            atomicExch(&p.status[0], (unsigned)QD_ERR_EMPTY_WAIT);
            atomicExch(&p.status[1], (unsigned)i);
            atomicExch(&s_failed, 1u);
            break;
          }
        }
        if (*reinterpret_cast<volatile unsigned*>(&s_failed)) break;
        const long long chunk = c0 + i;
        const int ct = (int)(chunk / p.cpt), kc = (int)(chunk % p.cpt);
        mbar_expect_tx(&full[s], QD_STAGE_BYTES);
        tma_load_2d(ring + (size_t)s * QD_STAGE_BYTES, &tmap, ct * QD_TILE_N, kc * QD_CHUNK_K, &full[s]);
      }
    }
    return;   // consumers only use named barrier 1 from here on
  }

  // -------------------- consumers -------------------------------------
  asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
  const int g = lane >> 2, t = lane & 3;
  const float magic = WUNSIGNED ? 8388608.0f : 8388736.0f;
  float tot[8][MT][4];
#pragma unroll
  for (int j = 0; j < 8; j++)
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
      for (int c = 0; c < 4; c++) tot[j][mt][c] = 0.0f;

  bool failed = false;
  int seg_begin = 0;
  while (seg_begin < n_local) {
    const long long first_chunk = c0 + seg_begin;
    const int ct = (int)(first_chunk / p.cpt);
    const long long tile_begin = (long long)ct * p.cpt, tile_end = tile_begin + p.cpt;
    const int seg_end = (int)min((long long)n_local, tile_end - c0);
    const int colbase = ct * QD_TILE_N;

    // first local chunk index >= seg_begin that belongs to this warp
    int i = seg_begin + ((warp - seg_begin) % QD_CONSUMERS + QD_CONSUMERS) % QD_CONSUMERS;
    for (; i < seg_end; i += QD_CONSUMERS) {
      const int s = i % p.stages;
      const int kc = (int)((c0 + i) % p.cpt);
      const int k0 = kc * QD_CHUNK_K;
      // scales of this chunk's group for the thread's 16 columns
      float sc[16];
      {
        const int srow = p.scale_group ? k0 / p.scale_group : 0;
        const float* sp = p.scales + (int64_t)srow * p.N + colbase + 16 * g;
        const bool ok = colbase + 16 * g < p.N;     // N is a multiple of 16
#pragma unroll
        for (int q = 0; q < 4; q++) {
          float4 v = ok ? __ldg(reinterpret_cast<const float4*>(sp) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
          sc[4 * q] = v.x; sc[4 * q + 1] = v.y; sc[4 * q + 2] = v.z; sc[4 * q + 3] = v.w;
        }
      }
      // activation operands for the four k-steps of the chunk
      XFrag<XT> xf[4][MT];
#pragma unroll
      for (int ks = 0; ks < 4; ks++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
          const int m = mt * 8 + g, k = k0 + 16 * ks + 2 * t;
          xf[ks][mt].load(p.x, (int64_t)m * p.K, k, m < p.M && k0 + 16 * ks < p.K);
        }
      if (!failed && !mbar_wait_bounded(&full[s], (uint32_t)((i / p.stages) & 1))) {
        failed = true;
        atomicExch(&p.status[0], (unsigned)QD_ERR_FULL_WAIT);
        atomicExch(&p.status[1], (unsigned)i);
        atomicExch(&s_failed, 1u);
      }
      if (failed) continue;

      float acc[8][MT][4];
#pragma unroll
      for (int j = 0; j < 8; j++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
          for (int c = 0; c < 4; c++) acc[j][mt][c] = 0.0f;

      const uint8_t* stage = ring + (size_t)s * QD_STAGE_BYTES;
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        // rows 2t, 2t+1, 2t+8, 2t+9 of this k-step: exactly the k indices the mma
        // fragment assigns to lane t; the 128B swizzle makes the loads conflict-free.
        uint32_t L[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
          const int row = 16 * ks + 2 * t + (r & 1) + 8 * (r >> 1);
          const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 128 + ((g ^ (row & 7)) << 4));
          L[r][0] = v.x; L[r][1] = v.y; L[r][2] = v.z; L[r][3] = v.w;
          if (!WUNSIGNED) {
#pragma unroll
            for (int q = 0; q < 4; q++) L[r][q] ^= 0x80808080u;
          }
        }
#pragma unroll
        for (int qh = 0; qh < 2; qh++) {
#define QD_BYTE_STEP(B)                                                                             \
  {                                                                                                 \
    uint32_t a[4];                                                                                  \
    a[0] = pack_hi16(byte_to_f32<B>(L[0][qh], magic), byte_to_f32<B>(L[1][qh], magic));             \
    a[1] = pack_hi16(byte_to_f32<B>(L[0][2 + qh], magic), byte_to_f32<B>(L[1][2 + qh], magic));     \
    a[2] = pack_hi16(byte_to_f32<B>(L[2][qh], magic), byte_to_f32<B>(L[3][qh], magic));             \
    a[3] = pack_hi16(byte_to_f32<B>(L[2][2 + qh], magic), byte_to_f32<B>(L[3][2 + qh], magic));     \
    _Pragma("unroll") for (int mt = 0; mt < MT; mt++) {                                             \
      _Pragma("unroll") for (int sp = 0; sp < XFrag<XT>::SPLITS; sp++)                              \
          mma_bf16_16816(acc[4 * qh + B][mt], a, xf[ks][mt].b0[sp], xf[ks][mt].b1[sp]);             \
    }                                                                                               \
  }
          QD_BYTE_STEP(0) QD_BYTE_STEP(1) QD_BYTE_STEP(2) QD_BYTE_STEP(3)
#undef QD_BYTE_STEP
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);   // stage may be refilled

      // column of acc[j][*][0..1] is 16g+j, of acc[j][*][2..3] is 16g+8+j
#pragma unroll
      for (int j = 0; j < 8; j++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
          tot[j][mt][0] = fmaf(acc[j][mt][0], sc[j], tot[j][mt][0]);
          tot[j][mt][1] = fmaf(acc[j][mt][1], sc[j], tot[j][mt][1]);
          tot[j][mt][2] = fmaf(acc[j][mt][2], sc[8 + j], tot[j][mt][2]);
          tot[j][mt][3] = fmaf(acc[j][mt][3], sc[8 + j], tot[j][mt][3]);
        }
    }

    // ---- cross-warp reduction of this segment -------------------------
    float* mine = red + warp * RED_FLOATS;
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int mt = 0; mt < MT; mt++) {
        const int m = mt * 8 + 2 * t;
        mine[m * QD_TILE_N + 16 * g + j] = tot[j][mt][0];
        mine[(m + 1) * QD_TILE_N + 16 * g + j] = tot[j][mt][1];
        mine[m * QD_TILE_N + 16 * g + 8 + j] = tot[j][mt][2];
        mine[(m + 1) * QD_TILE_N + 16 * g + 8 + j] = tot[j][mt][3];
        tot[j][mt][0] = tot[j][mt][1] = tot[j][mt][2] = tot[j][mt][3] = 0.0f;
      }
    asm volatile("bar.sync 1, %0;" ::"n"(QD_CONSUMERS * 32) : "memory");

    constexpr int PER_THREAD = RED_FLOATS / (QD_CONSUMERS * 32);
    float sum[PER_THREAD];
#pragma unroll
    for (int e = 0; e < PER_THREAD; e++) {
      const int idx = tid + e * QD_CONSUMERS * 32;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < QD_CONSUMERS; w++) v += red[w * RED_FLOATS + idx];
      sum[e] = v;
    }

    const bool whole_tile = (first_chunk == tile_begin) && (c0 + seg_end == tile_end);
    bool finalize = whole_tile;
    if (!whole_tile) {
      // partial tile: park the CTA's sum, then see whether every contributor has arrived
      const int slot = (first_chunk > tile_begin) ? 0 : 1;
      float* dst = p.partials + ((size_t)cta * 2 + slot) * RED_FLOATS;
#pragma unroll
      for (int e = 0; e < PER_THREAD; e++) dst[tid + e * QD_CONSUMERS * 32] = sum[e];
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(QD_CONSUMERS * 32) : "memory");
      const int cf = (int)(((tile_begin + 1) * G - 1) / p.total);
      const int cl = (int)((tile_end * G - 1) / p.total);
      if (tid == 0) {
        const unsigned old = atomicAdd(&p.counters[ct], 1u);
        const unsigned last = (old == (unsigned)(cl - cf)) ? 1u : 0u;
        if (last) p.counters[ct] = 0;      // leave the workspace prepared for the next launch
        s_flag = last;
        __threadfence();
      }
      asm volatile("bar.sync 1, %0;" ::"n"(QD_CONSUMERS * 32) : "memory");
      finalize = (s_flag != 0);
      if (finalize) {
#pragma unroll
        for (int e = 0; e < PER_THREAD; e++) sum[e] = 0.0f;
        for (int c = cf; c <= cl; c++) {       // fixed order: results do not depend on arrival order
          const long long cs = (long long)c * p.total / G;
          const float* src = p.partials + ((size_t)c * 2 + (cs > tile_begin ? 0 : 1)) * RED_FLOATS;
#pragma unroll
          for (int e = 0; e < PER_THREAD; e++) sum[e] += __ldcg(src + tid + e * QD_CONSUMERS * 32);
        }
      }
    }
    if (finalize && !*reinterpret_cast<volatile unsigned*>(&s_failed)) {
#pragma unroll
      for (int e = 0; e < PER_THREAD; e++) {
        const int idx = tid + e * QD_CONSUMERS * 32;
        const int m = idx / QD_TILE_N, col = colbase + idx % QD_TILE_N;
        if (m < p.M && col < p.N) {
          float v = sum[e];
          if (p.bias) v += __ldg(p.bias + col);
          v = apply_activation(v, p.activation);
          Scalar<XT>::store(reinterpret_cast<XT*>(p.out), (int64_t)m * p.N + col, v);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(QD_CONSUMERS * 32) : "memory");   // red[] is reused
    seg_begin = seg_end;
  }
}

// ---------------------------------------------------------------------------
// planning and launch
// ---------------------------------------------------------------------------
static int decode_stages(int mt) { return mt == 1 ? 24 : 20; }
static size_t decode_smem(int mt) {
  return 1024 + (size_t)decode_stages(mt) * QD_STAGE_BYTES + (size_t)QD_CONSUMERS * mt * 8 * QD_TILE_N * 4 +
         (size_t)2 * decode_stages(mt) * 8;
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
  return true;
}

int qdense_plan(cb_plan* p) {
  cb_qdense_desc& d = p->qd;
  if (d.M < 0 || d.K < 0 || d.N < 0) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: negative dimension");
  if (d.x_dtype != CB_F32 && d.x_dtype != CB_BF16)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: x must be float32 (or bfloat16), got %s", dtype_name(d.x_dtype));
  if (d.w_dtype != CB_I8 && d.w_dtype != CB_U8)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense: Linear unsupported weight type %s", dtype_name(d.w_dtype));
  if (d.scale_layout < CB_SCALE_REF || d.scale_layout > CB_SCALE_KGROUP)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown scale layout %d", d.scale_layout);
  if (d.scale_layout != CB_SCALE_CHANNEL && d.block_size <= 0)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: block size must be positive, got %lld", (long long)d.block_size);
  if (d.activation < CB_ACT_NONE || d.activation > CB_ACT_TANH)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown activation %d", d.activation);
  p->n_inputs = 3 + (d.has_zero_point ? 1 : 0) + (d.has_bias ? 1 : 0);
  p->n_outputs = 1;

  int variant = d.variant;
  std::string why;
  const bool can_decode = decode_eligible(d, &why);
  if (variant == CB_QDENSE_AUTO) variant = can_decode ? CB_QDENSE_DECODE_MMA : CB_QDENSE_GENERIC;
  if (variant == CB_QDENSE_DECODE_MMA && !can_decode)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense decode kernel: %s", why.c_str());
  if (variant == CB_QDENSE_PREFILL)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense prefill kernel is not built yet");
  p->variant = variant;

  if (variant == CB_QDENSE_GENERIC) {
    p->blocks = (int)(((d.N + QG_COLS - 1) / QG_COLS) * ((d.M + QG_ROWS - 1) / QG_ROWS));
    p->threads = QG_COLS;
    p->dyn_smem = 0;
    p->workspace_bytes = 0;
    p->name = std::string("qdense_generic_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") + (d.w_dtype == CB_U8 ? "_u8" : "_i8");
    return CB_OK;
  }
  const int mt = d.M <= 8 ? 1 : 2;
  const long long n_tiles = (d.N + QD_TILE_N - 1) / QD_TILE_N;
  const long long cpt = (d.K + QD_CHUNK_K - 1) / QD_CHUNK_K;
  const long long total = n_tiles * cpt;
  p->blocks = (int)std::min<long long>(p->n_sm, total);
  p->threads = QD_THREADS;
  p->dyn_smem = (int)decode_smem(mt);
  p->counter_bytes = (QD_WS_HEADER + (size_t)n_tiles * 4 + 255) & ~(size_t)255;
  p->workspace_bytes = p->counter_bytes + (size_t)p->blocks * 2 * mt * 8 * QD_TILE_N * 4;
  p->has_status = true;
  p->name = std::string("qdense_decode_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") + (mt == 1 ? "_m8" : "_m16") +
            (d.w_dtype == CB_U8 ? "_u8" : "_i8");
  return CB_OK;
}

template <typename XT, typename WT>
static int launch_generic(const cb_plan* p, const void* const* in, void* const* out, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (d.M == 0 || d.N == 0) return CB_OK;
  int idx = 3;
  const float* zp = d.has_zero_point ? (const float*)in[idx++] : nullptr;
  const float* bias = d.has_bias ? (const float*)in[idx++] : nullptr;
  dim3 grid((unsigned)((d.N + QG_COLS - 1) / QG_COLS), (unsigned)((d.M + QG_ROWS - 1) / QG_ROWS));
  qdense_generic_kernel<XT, WT><<<grid, QG_COLS, 0, s>>>((const XT*)in[0], (const WT*)in[1], (const float*)in[2], zp,
                                                         bias, (XT*)out[0], d.M, d.K, d.N, d.scale_layout,
                                                         d.block_size > 0 ? d.block_size : 1, d.activation);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

// Encoded tensor maps are cached per (device, weights pointer, shape): a resident
// weight matrix is encoded once, not on every launch.
struct MapCacheEntry { int dev; const void* w; int64_t K, N; CUtensorMap map; };
static std::mutex g_map_mu;
static MapCacheEntry g_map_cache[64];
static int g_map_next = 0, g_map_count = 0;

static int weight_tensor_map(int dev, const void* w, int64_t K, int64_t N, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mu);
  for (int i = 0; i < g_map_count; i++) {
    const MapCacheEntry& e = g_map_cache[i];
    if (e.dev == dev && e.w == w && e.K == K && e.N == N) { *out = e.map; return CB_OK; }
  }
  encode_tiled_fn enc = tensor_map_encoder();
  if (!enc) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(w) & 15) != 0)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: weights must be 16-byte aligned");
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
  cuuint64_t strides[1] = {(cuuint64_t)N};
  cuuint32_t box[2] = {QD_TILE_N, QD_CHUNK_K};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  MapCacheEntry& e = g_map_cache[g_map_next];
  e.dev = dev; e.w = w; e.K = K; e.N = N; e.map = m;
  g_map_next = (g_map_next + 1) % 64;
  if (g_map_count < 64) g_map_count++;
  *out = m;
  return CB_OK;
}

template <typename XT, int MT, bool WU>
static int launch_decode_t(const cb_plan* p, const CUtensorMap& map, const QdParams& prm, cudaStream_t s) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  // The attribute is per device; setting it again is cheap and keeps multi-GPU processes correct.
  attr_err = cudaFuncSetAttribute(qdense_decode_kernel<XT, MT, WU>, cudaFuncAttributeMaxDynamicSharedMemorySize, p->dyn_smem);
  (void)once;
  CB_CUDA(attr_err);
  qdense_decode_kernel<XT, MT, WU><<<p->blocks, QD_THREADS, p->dyn_smem, s>>>(map, prm);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

static int launch_decode(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  CUtensorMap map;
  CB_TRY(weight_tensor_map(p->dev, in[1], d.K, d.N, &map));
  QdParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.x = in[0];
  prm.scales = (const float*)in[2];
  prm.bias = d.has_bias ? (const float*)in[3] : nullptr;
  prm.out = out[0];
  uint8_t* w8 = (uint8_t*)ws;
  prm.status = (unsigned*)w8;
  prm.counters = (unsigned*)(w8 + QD_WS_HEADER);
  prm.partials = (float*)(w8 + p->counter_bytes);
  prm.M = (int)d.M; prm.K = (int)d.K; prm.N = (int)d.N;
  prm.n_tiles = (int)((d.N + QD_TILE_N - 1) / QD_TILE_N);
  prm.cpt = (int)((d.K + QD_CHUNK_K - 1) / QD_CHUNK_K);
  prm.total = (long long)prm.n_tiles * prm.cpt;
  prm.scale_group = d.scale_layout == CB_SCALE_KGROUP ? (int)d.block_size : 0;
  prm.activation = d.activation;
  const int mt = d.M <= 8 ? 1 : 2;
  prm.stages = decode_stages(mt);
  if ((reinterpret_cast<uintptr_t>(in[0]) & 7) || (reinterpret_cast<uintptr_t>(in[2]) & 15))
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: x must be 8-byte and scales 16-byte aligned");
  const bool bf = d.x_dtype == CB_BF16, wu = d.w_dtype == CB_U8;
#define QD_DISPATCH(XT)                                                                       \
  (mt == 1 ? (wu ? launch_decode_t<XT, 1, true>(p, map, prm, s) : launch_decode_t<XT, 1, false>(p, map, prm, s)) \
           : (wu ? launch_decode_t<XT, 2, true>(p, map, prm, s) : launch_decode_t<XT, 2, false>(p, map, prm, s)))
  return bf ? QD_DISPATCH(__nv_bfloat16) : QD_DISPATCH(float);
#undef QD_DISPATCH
}

int qdense_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (p->variant == CB_QDENSE_DECODE_MMA) return launch_decode(p, in, out, ws, s);
  const bool bf = d.x_dtype == CB_BF16, wu = d.w_dtype == CB_U8;
  if (bf) return wu ? launch_generic<__nv_bfloat16, uint8_t>(p, in, out, s) : launch_generic<__nv_bfloat16, int8_t>(p, in, out, s);
  return wu ? launch_generic<float, uint8_t>(p, in, out, s) : launch_generic<float, int8_t>(p, in, out, s);
}

}  // namespace cb
