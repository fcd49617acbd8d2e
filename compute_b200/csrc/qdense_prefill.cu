// FusedQuantizedDense for prefill-shaped inputs (M > 16) on the tcgen05 GEMM.
//
//   y[M,N] = act( x[M,K] @ dq(W)[K,N] + bias[N] ),   dq(W) = W * scale (+ zero_point)
// (reference semantics: internal/gobackend/fusedops/quantizeddense.go:330-418 of gomlx/compute).
//
// Two launches (three for float32 x):
//   1. qdense_planes_kernel expands the weights (8-bit, packed 4-bit, NF4 indices) to bf16 planes in the workspace.
//      Per-channel scales without zero points: one plane holding bf16(W) exactly, the scale is
//      applied to the f32 accumulator in the GEMM epilogue.  Every other layout (K-group scales,
//      the reference's [K, N/block] scales, zero points): dq(W) in f32, split into 2 planes
//      (16 mantissa bits: bfloat16 x, and the 4-bit families) or 3 planes (24 bits: 8-bit weights with float32 x).
//   2. float32 x is split into as many bf16 planes.
//   3. The GEMM accumulates the plane products in f32 in tensor memory and applies
//      scale, bias and activation before the store.
// With M in the thousands the weight expansion (1 byte read, 2-6 written per weight) is a
// small fraction of the GEMM; near M = 17 it dominates, which is still several times faster
// than the CUDA-core kernel.
#include "gemm_tc.h"

#include <algorithm>
#include <stdlib.h>

namespace cb {

// One thread owns 8 adjacent columns and a run of consecutive rows (grid.y splits the rows), so
// K-group scales are fetched once per group.  Bytes become floats without the conversion unit:
// 0x4B0000bb is 2^23 + bb, and signed bytes are biased by 128 first.  WKIND: how the eight weights are stored - one
// byte each (unsigned or signed), or as the eight nibbles of one 32-bit word (packed Uint4 / Int4: element (k, n) is
// nibble n & 1 of byte (k N + n) / 2, internal/gobackend/ops/convertdtype.go:199-226).  NF4: the low four bits of a
// weight index the NormalFloat4 table (quantizeddense.go:586-609).
enum { QP_U8 = 0, QP_I8 = 1, QP_U4 = 2, QP_I4 = 3 };
__constant__ float kPrefillNf4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
template <int WKIND, int NPLANES, bool RAW, bool NF4>
__global__ void __launch_bounds__(256)
qdense_planes_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scales, const float* __restrict__ zps,
                     uint16_t* __restrict__ planes, int64_t K, int64_t N, int layout, int64_t block, int rows_per_cta) {
  constexpr bool WUNSIGNED = WKIND == QP_U8 || WKIND == QP_U4;
  constexpr bool PACKED = WKIND == QP_U4 || WKIND == QP_I4;
  // the table is read with a different index in every lane: from shared memory (16 banks), not from the constant cache
  __shared__ float s_nf4[16];
  if (NF4) {
    if (threadIdx.x < 16) s_nf4[threadIdx.x] = kPrefillNf4[threadIdx.x];
    __syncthreads();
  }
  // the GEMM that consumes the planes may set itself up meanwhile; it waits for this grid before it loads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t n = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (n >= N) return;
  const int64_t nblk = (layout == CB_SCALE_REF) ? (N + block - 1) / block : 0;
  const size_t plane_elems = (size_t)K * N;
  const int64_t k0 = (int64_t)blockIdx.y * rows_per_cta, k1 = min(K, k0 + rows_per_cta);
  const float magic = WUNSIGNED ? 8388608.0f : 8388736.0f;
  float sc[8], zp[8];
#pragma unroll
  for (int e = 0; e < 8; e++) { sc[e] = 1.0f; zp[e] = 0.0f; }
  int64_t loaded = -1;                       // scale row currently in registers
  for (int64_t krow = k0; krow < k1; krow++) {
    if (!RAW) {
      const int64_t srow = layout == CB_SCALE_CHANNEL ? 0 : (layout == CB_SCALE_KGROUP ? krow / block : krow);
      if (srow != loaded) {
        loaded = srow;
#pragma unroll
        for (int e = 0; e < 8; e++) {
          const int64_t si = layout == CB_SCALE_REF ? srow * nblk + (n + e) / block : srow * N + n + e;
          sc[e] = __ldg(scales + si);
          if (zps) zp[e] = __ldg(zps + si);
        }
      }
    }
    float v[8];
    if (PACKED) {
      const uint32_t word = *reinterpret_cast<const uint32_t*>(w + (krow * N + n) / 2);
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const uint32_t nib = (word >> (4 * e)) & 0xFu;
        v[e] = NF4 ? s_nf4[nib] : __uint_as_float(0x4B000000u | (WUNSIGNED ? nib : (nib ^ 8u))) - (WUNSIGNED ? 8388608.0f : 8388616.0f);
      }
    } else {
      uint2 raw8 = *reinterpret_cast<const uint2*>(w + krow * N + n);
      if (NF4) {
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = s_nf4[((e < 4 ? raw8.x : raw8.y) >> (8 * (e & 3))) & 0xFu];
      } else {
        if (!WUNSIGNED) { raw8.x ^= 0x80808080u; raw8.y ^= 0x80808080u; }
#pragma unroll
        for (int e = 0; e < 8; e++)
          v[e] = __uint_as_float(__byte_perm(e < 4 ? raw8.x : raw8.y, 0x4B000000u, 0x7650u | (e & 3))) - magic;
      }
    }
    uint32_t pl[3][4];
    if (RAW) {                               // |w| <= 255 has at most 8 significant bits: bf16(w) is exact
#pragma unroll
      for (int e2 = 0; e2 < 4; e2++)
        pl[0][e2] = __byte_perm(__float_as_uint(v[2 * e2]), __float_as_uint(v[2 * e2 + 1]), 0x7632u);
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) {
        v[e] = __fmul_rn(v[e], sc[e]);
        if (zps) v[e] = __fadd_rn(v[e], zp[e]);
      }
#pragma unroll
      for (int q = 0; q < NPLANES; q++) {
#pragma unroll
        for (int e2 = 0; e2 < 4; e2++) {
          const uint32_t packed = (uint32_t)f32_to_bf16_bits(v[2 * e2]) | ((uint32_t)f32_to_bf16_bits(v[2 * e2 + 1]) << 16);
          pl[q][e2] = packed;
          // what the planes so far leave over (nothing for non-finite values)
          const float h0 = __uint_as_float(packed << 16), h1 = __uint_as_float(packed & 0xFFFF0000u);
          v[2 * e2] = isfinite(v[2 * e2]) ? v[2 * e2] - h0 : 0.0f;
          v[2 * e2 + 1] = isfinite(v[2 * e2 + 1]) ? v[2 * e2 + 1] - h1 : 0.0f;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < NPLANES; q++)
      *reinterpret_cast<uint4*>(planes + (size_t)q * plane_elems + (size_t)krow * N + n) = make_uint4(pl[q][0], pl[q][1], pl[q][2], pl[q][3]);
  }
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static bool prefill_raw(const cb_qdense_desc& d) {
  return d.scale_layout == CB_SCALE_CHANNEL && !d.has_zero_point && d.scheme == CB_QUANT_LINEAR;   // NF4 values are not 8-bit integers
}
// Planes per operand.  8-bit weights with float32 x: three planes each (all 24 mantissa bits; six plane products).
// The 4-bit families (packed Int4 / Uint4, NF4 indices) with float32 x: two planes each and the three products
// a0 b0 + a0 b1 + a1 b0, which leaves out terms of 2^-16 relative size, as the float32 DotGeneral does by default
// (2e-5 normalised in the tests, against a bar of 1e-4) - half the time of six products.  bfloat16 x: one plane of
// x, two of the weights.
static bool prefill_four_bit(const cb_qdense_desc& d) { return d.scheme == CB_QUANT_NF4 || d.w_dtype == CB_I4 || d.w_dtype == CB_U4; }
static int prefill_x_planes(const cb_qdense_desc& d) { return d.x_dtype != CB_F32 ? 1 : prefill_four_bit(d) ? 2 : 3; }
static int prefill_w_planes(const cb_qdense_desc& d) { return prefill_raw(d) ? 1 : (d.x_dtype == CB_F32 && !prefill_four_bit(d) ? 3 : 2); }

bool qdense_prefill_eligible(const cb_qdense_desc& d, std::string* why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  if (d.M < 1) return no("empty x");
  if (d.K < 8 || d.K % 8 != 0) return no("K must be a positive multiple of 8");
  if (d.N < 8 || d.N % 8 != 0) return no("N must be a positive multiple of 8");
  if (d.M > (1 << 30) || d.K > (1 << 30) || d.N > (1 << 30)) return no("dimension too large");
  return true;
}

int qdense_prefill_plan(cb_plan* p) {
  const cb_qdense_desc& d = p->qd;
  p->blocks = gemm_tc_blocks(p->n_sm, 1, d.M, d.N);
  p->threads = gemm_tc_threads();
  p->dyn_smem = gemm_tc_smem();
  p->counter_bytes = 256;
  p->workspace_bytes = 256 + align256((size_t)prefill_w_planes(d) * d.K * d.N * 2) +
                       (d.x_dtype == CB_F32 ? align256((size_t)prefill_x_planes(d) * d.M * d.K * 2) : 0);
  p->has_status = true;
  p->name = std::string("qdense_prefill_tcgen05_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") +
            (d.w_dtype == CB_U8 ? "_u8" : d.w_dtype == CB_I8 ? "_i8" : d.w_dtype == CB_U4 ? "_u4" : "_i4") + (d.scheme == CB_QUANT_NF4 ? "_nf4" : "");
  return CB_OK;
}

int qdense_prefill_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (d.M == 0 || d.N == 0) return CB_OK;
  int idx = 3;
  const float* zp = d.has_zero_point ? (const float*)in[idx++] : nullptr;
  const float* bias = d.has_bias ? (const float*)in[idx++] : nullptr;
  const bool packed = d.w_dtype == CB_I4 || d.w_dtype == CB_U4;
  if ((reinterpret_cast<uintptr_t>(in[0]) & 15) || (reinterpret_cast<uintptr_t>(in[1]) & (packed ? 3 : 7)))
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense prefill kernel: x must be 16-byte and weights 8-byte (packed 4-bit: 4-byte) aligned");
  uint8_t* w8 = (uint8_t*)ws;
  const int wp = prefill_w_planes(d);
  const bool raw = prefill_raw(d);
  uint16_t* wplanes = (uint16_t*)(w8 + 256);
  uint16_t* xplanes = (uint16_t*)(w8 + 256 + align256((size_t)wp * d.K * d.N * 2));

  const int64_t block = d.block_size > 0 ? d.block_size : 1;
  const unsigned gx = (unsigned)((d.N / 8 + 255) / 256);
  const int64_t want_y = std::max<int64_t>(1, std::min<int64_t>(d.K, ((int64_t)p->n_sm * 8 + gx - 1) / gx));
  const int rows_per_cta = (int)((d.K + want_y - 1) / want_y);
  const dim3 grid(gx, (unsigned)((d.K + rows_per_cta - 1) / rows_per_cta));
  const uint8_t* wq = (const uint8_t*)in[1];
  const float* sc = (const float*)in[2];
#define QP_LAUNCH(WK, NP, RAW, NF) qdense_planes_kernel<WK, NP, RAW, NF><<<grid, 256, 0, s>>>(wq, sc, zp, wplanes, d.K, d.N, d.scale_layout, block, rows_per_cta)
#define QP_PLANES(WK, NF) do { if (raw) QP_LAUNCH(WK, 1, true, false); else if (wp == 2) QP_LAUNCH(WK, 2, false, NF); else QP_LAUNCH(WK, 3, false, NF); } while (0)
  if (d.scheme == CB_QUANT_NF4) {
    switch (d.w_dtype) {
      case CB_U8: QP_PLANES(QP_U8, true); break;
      case CB_I8: QP_PLANES(QP_I8, true); break;
      case CB_U4: QP_PLANES(QP_U4, true); break;
      default: QP_PLANES(QP_I4, true); break;
    }
  } else {
    switch (d.w_dtype) {
      case CB_U8: QP_PLANES(QP_U8, false); break;
      case CB_I8: QP_PLANES(QP_I8, false); break;
      case CB_U4: QP_PLANES(QP_U4, false); break;
      default: QP_PLANES(QP_I4, false); break;
    }
  }
#undef QP_PLANES
#undef QP_LAUNCH
  CB_CUDA(cudaGetLastError());

  GemmTcProblem g;
  g.a = in[0];
  g.planes_a = 1;
  if (d.x_dtype == CB_F32) {
    CB_TRY(split_f32_planes((const float*)in[0], xplanes, (size_t)d.M * d.K, nullptr, nullptr, 0, prefill_x_planes(d), s));
    g.a = xplanes;
    g.planes_a = prefill_x_planes(d);
  }
  g.b = wplanes;
  g.planes_b = wp;
  g.out = out[0];
  g.status = (unsigned*)ws;
  g.B = 1; g.M = d.M; g.N = d.N; g.K = d.K;
  g.rhs_transposed = 0;
  g.ab_dtype = CB_BF16;
  g.out_dtype = d.x_dtype;
  g.n_pass = gemm_tc_split_passes(g.planes_a, g.planes_b, g.planes_a == 3 ? 2 : 1, g.pass_a, g.pass_b);
  g.col_scale = raw ? (const float*)in[2] : nullptr;
  g.bias = bias;
  g.activation = d.activation;
  return gemm_tc_run(p->dev, p->blocks, g, s);
}

}  // namespace cb
