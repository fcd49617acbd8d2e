// FusedQuantizedDense for prefill-shaped inputs (M > 16) on the tcgen05 GEMM.
//
//   y[M,N] = act( x[M,K] @ dq(W)[K,N] + bias[N] ),   dq(W) = W * scale (+ zero_point)
// (reference semantics: internal/gobackend/fusedops/quantizeddense.go:330-418 of gomlx/compute).
//
// Two launches (three for float32 x):
//   1. qdense_planes_kernel expands the 8-bit weights to bf16 planes in the workspace.
//      Per-channel scales without zero points: one plane holding bf16(W) exactly, the scale is
//      applied to the f32 accumulator in the GEMM epilogue.  Every other layout (K-group scales,
//      the reference's [K, N/block] scales, zero points): dq(W) in f32, split into 2 planes
//      (16 mantissa bits, for bfloat16 x) or 3 planes (24 bits, for float32 x).
//   2. float32 x is split into 3 bf16 planes.
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
// 0x4B0000bb is 2^23 + bb, and signed bytes are biased by 128 first.
template <bool WUNSIGNED, int NPLANES, bool RAW>
__global__ void __launch_bounds__(256)
qdense_planes_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scales, const float* __restrict__ zps,
                     uint16_t* __restrict__ planes, int64_t K, int64_t N, int layout, int64_t block, int rows_per_cta) {
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
    uint2 raw8 = *reinterpret_cast<const uint2*>(w + krow * N + n);
    if (!WUNSIGNED) { raw8.x ^= 0x80808080u; raw8.y ^= 0x80808080u; }
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; e++)
      v[e] = __uint_as_float(__byte_perm(e < 4 ? raw8.x : raw8.y, 0x4B000000u, 0x7650u | (e & 3))) - magic;
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

static bool prefill_raw(const cb_qdense_desc& d) { return d.scale_layout == CB_SCALE_CHANNEL && !d.has_zero_point; }
static int prefill_w_planes(const cb_qdense_desc& d) { return prefill_raw(d) ? 1 : (d.x_dtype == CB_F32 ? 3 : 2); }

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
                       (d.x_dtype == CB_F32 ? align256((size_t)3 * d.M * d.K * 2) : 0);
  p->has_status = true;
  p->name = std::string("qdense_prefill_tcgen05_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") + (d.w_dtype == CB_U8 ? "_u8" : "_i8");
  return CB_OK;
}

int qdense_prefill_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (d.M == 0 || d.N == 0) return CB_OK;
  int idx = 3;
  const float* zp = d.has_zero_point ? (const float*)in[idx++] : nullptr;
  const float* bias = d.has_bias ? (const float*)in[idx++] : nullptr;
  if ((reinterpret_cast<uintptr_t>(in[0]) & 15) || (reinterpret_cast<uintptr_t>(in[1]) & 7))
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense prefill kernel: x must be 16-byte and weights 8-byte aligned");
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
#define QP_LAUNCH(WU, NP, RAW) qdense_planes_kernel<WU, NP, RAW><<<grid, 256, 0, s>>>(wq, sc, zp, wplanes, d.K, d.N, d.scale_layout, block, rows_per_cta)
  if (d.w_dtype == CB_U8) {
    if (raw) QP_LAUNCH(true, 1, true); else if (wp == 2) QP_LAUNCH(true, 2, false); else QP_LAUNCH(true, 3, false);
  } else {
    if (raw) QP_LAUNCH(false, 1, true); else if (wp == 2) QP_LAUNCH(false, 2, false); else QP_LAUNCH(false, 3, false);
  }
#undef QP_LAUNCH
  CB_CUDA(cudaGetLastError());

  GemmTcProblem g;
  g.a = in[0];
  g.planes_a = 1;
  if (d.x_dtype == CB_F32) {
    CB_TRY(split_f32_planes((const float*)in[0], xplanes, (size_t)d.M * d.K, nullptr, nullptr, 0, 3, s));
    g.a = xplanes;
    g.planes_a = 3;
  }
  g.b = wplanes;
  g.planes_b = wp;
  g.out = out[0];
  g.status = (unsigned*)ws;
  g.B = 1; g.M = d.M; g.N = d.N; g.K = d.K;
  g.rhs_transposed = 0;
  g.ab_dtype = CB_BF16;
  g.out_dtype = d.x_dtype;
  g.n_pass = gemm_tc_split_passes(g.planes_a, g.planes_b, 2, g.pass_a, g.pass_b);
  g.col_scale = raw ? (const float*)in[2] : nullptr;
  g.bias = bias;
  g.activation = d.activation;
  return gemm_tc_run(p->dev, p->blocks, g, s);
}

}  // namespace cb
