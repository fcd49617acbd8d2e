// GGML block formats: FusedQuantizedDense with compute.QuantGGML and QuantizedEmbeddingLookup.
//
// Reference: internal/gobackend/fusedops/quantizeddense_ggml.go:53-302 (dequantisers of Q4_0, Q8_0, IQ4_NL, Q4_K, Q6_K
// and the dense loop: per output the weight row is dequantised, dot = sum_k x[k] * w[k], + bias, activation) and
// internal/gobackend/fusedops/quantizeddense.go:250-321, 455-499 (the lookup: out[i, :] = dequantised row indices[i]).
// Weights / table: [N, bytes_per_row] bytes, a row = K / values_per_block blocks with their scales embedded.
//
// Every format is handled in units of 32 consecutive values owned by one lane: a 32-value block, or one of the
// eight sub-blocks of a 256-value K-quant block (which share the block's d / dmin and pick their own 6-bit or 8-bit
// scale).  The dequantised values are bit-identical to the reference's (same float32 products and differences, no
// fused multiply-add in the dequantiser); the dot product is summed per lane and then across lanes, so the dense
// result agrees to rounding, not bit for bit.
//
// Both kernels give every lane one 32-value unit of a staged 1024-value chunk of a row.
#include "common.cuh"
#include "gemm_tc.h"

#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <string>

namespace cb {
namespace {

constexpr int GG_WARPS = 8;
constexpr int GG_CHUNK = 1024;               // lookup: values per staged chunk, 32 lanes x 32
constexpr int GG_WSTAGE = 1152;              // lookup: bytes per warp, the largest chunk (Q8_0: 1088) + lead and tail slack

__host__ __device__ constexpr int gg_values(int t) { return (t == CB_GGML_Q4_0 || t == CB_GGML_Q8_0 || t == CB_GGML_IQ4_NL) ? 32 : 256; }
__host__ __device__ constexpr int gg_bytes(int t) {
  return t == CB_GGML_Q8_0 ? 34 : t == CB_GGML_Q4_K ? 144 : t == CB_GGML_Q6_K ? 210 : 18;
}
// bytes of 1024 consecutive values
__host__ __device__ constexpr int gg_chunk_bytes(int t) { return GG_CHUNK / gg_values(t) * gg_bytes(t); }

// compute.IQ4NLLookupTable (fused_ops.go:127-130)
__constant__ float c_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

__device__ __forceinline__ float gg_f16(const uint8_t* p) {          // little-endian fp16 at an even address
  return __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(p)));
}

// The 32 values of unit `u` of a staged chunk.  `chunk` points at the chunk's first block (even address); `lut` is the
// IQ4_NL table in shared memory (16 entries in 16 banks: lanes reading different entries do not collide).
template <int GGML>
__device__ __forceinline__ void gg_decode32(const uint8_t* chunk, int u, float (&wv)[32], const float* lut) {
  if (GGML == CB_GGML_Q8_0) {
    const uint8_t* blk = chunk + u * 34;
    const float d = gg_f16(blk);
    const uint16_t* q16 = reinterpret_cast<const uint16_t*>(blk + 2);
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t q = q16[i];
      wv[2 * i] = __fmul_rn(d, (float)(int8_t)(q & 0xFF));
      wv[2 * i + 1] = __fmul_rn(d, (float)(int8_t)(q >> 8));
    }
  } else if (GGML == CB_GGML_Q4_0 || GGML == CB_GGML_IQ4_NL) {
    const uint8_t* blk = chunk + u * 18;
    const float d = gg_f16(blk);
    const uint16_t* q16 = reinterpret_cast<const uint16_t*>(blk + 2);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t q = q16[i];
      const int n0 = q & 0xF, n1 = (q >> 4) & 0xF, n2 = (q >> 8) & 0xF, n3 = q >> 12;      // bytes 2i (n0 low, n1 high), 2i + 1
      if (GGML == CB_GGML_Q4_0) {
        wv[2 * i] = __fmul_rn(d, (float)(n0 - 8));      wv[16 + 2 * i] = __fmul_rn(d, (float)(n1 - 8));
        wv[2 * i + 1] = __fmul_rn(d, (float)(n2 - 8));  wv[16 + 2 * i + 1] = __fmul_rn(d, (float)(n3 - 8));
      } else {
        wv[2 * i] = __fmul_rn(d, lut[n0]);          wv[16 + 2 * i] = __fmul_rn(d, lut[n1]);
        wv[2 * i + 1] = __fmul_rn(d, lut[n2]);      wv[16 + 2 * i + 1] = __fmul_rn(d, lut[n3]);
      }
    }
  } else if (GGML == CB_GGML_Q4_K) {
    // sub-block j of block u / 8: chunk j / 2 of the nibble bytes, low nibbles for even j, high for odd
    const uint8_t* blk = chunk + (u >> 3) * 144;
    const int j = u & 7;
    const float d = gg_f16(blk), dmin = gg_f16(blk + 2);
    const uint8_t* sc = blk + 4;
    int scale, mn;                                   // getScaleMinK4 (quantizeddense_ggml.go:219-228)
    if (j < 4) { scale = sc[j] & 63; mn = sc[j + 4] & 63; }
    else { scale = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); mn = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
    const float d1 = __fmul_rn(d, (float)scale), m1 = __fmul_rn(dmin, (float)mn);
    const uint32_t* q32 = reinterpret_cast<const uint32_t*>(blk + 16 + (j >> 1) * 32);      // 4-byte aligned: blocks are 144 bytes, rows even
    const int shift = (j & 1) * 4;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t q = reinterpret_cast<const uint16_t*>(q32)[i];
      wv[2 * i] = __fsub_rn(__fmul_rn(d1, (float)((q >> shift) & 0xF)), m1);
      wv[2 * i + 1] = __fsub_rn(__fmul_rn(d1, (float)((q >> (8 + shift)) & 0xF)), m1);
    }
  } else {  // Q6_K
    // sub-block j of block u / 8: half j / 4 (128 values), quarter j % 4 of that half (q1..q4 of the reference's loop)
    const uint8_t* blk = chunk + (u >> 3) * 210;
    const int j = u & 7, half = j >> 2, qd = j & 3;
    const uint8_t* ql = blk + half * 64 + (qd & 1) * 32;
    const uint8_t* qh = blk + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + half * 8 + 2 * qd);
    const float d = gg_f16(blk + 208);
    const float s0 = __fmul_rn(d, (float)sc[0]), s1 = __fmul_rn(d, (float)sc[1]);
    const int lshift = (qd >> 1) * 4, hshift = 2 * qd;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t l2 = reinterpret_cast<const uint16_t*>(ql)[i], h2 = reinterpret_cast<const uint16_t*>(qh)[i];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int l = 2 * i + e;
        const int lo = (l2 >> (8 * e + lshift)) & 0xF, hi = (h2 >> (8 * e + hshift)) & 3;
        const int q = (int)(int8_t)(lo | (hi << 4)) - 32;
        wv[l] = __fmul_rn(l < 16 ? s0 : s1, (float)q);
      }
    }
  }
}

// Copies `len` bytes starting at g (anywhere) into the warp's stage with 16-byte loads from the boundary below g and
// returns the staged address of g's first byte.  Vectors that would cross `end` (the end of the whole buffer) are read
// byte by byte.  The caller's __syncwarp separates the copy from the reads.
__device__ __forceinline__ uint4 gg_load16(const uint8_t* s, const uint8_t* end) {
  if (s + 16 <= end) return __ldg(reinterpret_cast<const uint4*>(s));
  uint32_t w[4] = {0, 0, 0, 0};
  for (int b = 0; b < 16; b++) if (s + b < end) w[b >> 2] |= (uint32_t)s[b] << (8 * (b & 3));
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ const uint8_t* gg_stage(uint8_t* stage, const uint8_t* g, int len, const uint8_t* end, int lane) {
  const int lead = (int)(reinterpret_cast<uintptr_t>(g) & 15);
  const uint8_t* src = g - lead;
  const int nvec = (lead + len + 15) >> 4;
  for (int v = lane; v < nvec; v += 32) reinterpret_cast<uint4*>(stage)[v] = gg_load16(src + 16 * v, end);
  return stage + lead;
}
// The same in two halves, so that a row's bytes travel while the previous row is decoded: the loads into registers
// (at most GG_PRE vectors per lane: 1103 bytes are 69 vectors), and later the stores into the stage.
constexpr int GG_PRE = 3;
struct GgPrefetch { uint4 v[GG_PRE]; int lead, nvec; };
__device__ __forceinline__ void gg_prefetch(GgPrefetch& pf, const uint8_t* g, int len, const uint8_t* end, int lane) {
  pf.lead = (int)(reinterpret_cast<uintptr_t>(g) & 15);
  pf.nvec = g ? (pf.lead + len + 15) >> 4 : 0;
  const uint8_t* src = g - pf.lead;
#pragma unroll
  for (int j = 0; j < GG_PRE; j++) {
    const int v = lane + 32 * j;
    if (v < pf.nvec) pf.v[j] = gg_load16(src + 16 * v, end);
  }
}
__device__ __forceinline__ const uint8_t* gg_commit(uint8_t* stage, const GgPrefetch& pf, int lane) {
#pragma unroll
  for (int j = 0; j < GG_PRE; j++) {
    const int v = lane + 32 * j;
    if (v < pf.nvec) reinterpret_cast<uint4*>(stage)[v] = pf.v[j];
  }
  return stage + pf.lead;
}

template <typename XT> __device__ __forceinline__ float gg_x(const XT* p, int64_t i);
template <> __device__ __forceinline__ float gg_x<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <> __device__ __forceinline__ float gg_x<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// Dense kernel.  A CTA of 8 warps stages a [rows, 1024] slice of x in shared memory once (float32, every lane's
// 32-value segment padded to 36 floats so that the lanes' 16-byte reads fall in different banks) and reuses it for 32
// weight rows, four per warp; a warp stages the bytes of its row's 1024-value chunk with coalesced 16-byte loads (requested
// one row ahead, so that they travel while the previous row is decoded) and every lane decodes one 32-value unit from
// there and multiplies it with the rows of x; a butterfly adds the lanes at the end.  MR = rows of x per CTA pass (1, 4 or 16).  (Giving every lane an output column instead — x read as
// broadcasts, no final reduction — measured 1.3-1.7x slower: the decode, not the reduction, is what costs.)
constexpr int GG_RPW = 4;                    // weight rows per warp
constexpr int GG_XPITCH = 36;

template <typename XT, int GGML, int MR>
__global__ void __launch_bounds__(GG_WARPS * 32)
qdense_ggml_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ w, const float* __restrict__ bias, XT* __restrict__ out,
                   int64_t M, int64_t K, int64_t N, int act) {
  extern __shared__ __align__(16) unsigned char gg_smem[];
  __shared__ float s_lut[16];
  if (threadIdx.x < 16) s_lut[threadIdx.x] = c_iq4nl[threadIdx.x];
  float* xs = reinterpret_cast<float*>(gg_smem);                                   // [MR][32][GG_XPITCH]
  uint8_t* wstage = gg_smem + (size_t)MR * 32 * GG_XPITCH * sizeof(float) + (threadIdx.x >> 5) * (2 * GG_WSTAGE);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t n0 = ((int64_t)blockIdx.x * GG_WARPS + warp) * GG_RPW;
  const int64_t m0 = (int64_t)blockIdx.y * MR;
  const int rows = (int)min((int64_t)MR, M - m0);
  constexpr int VPB = gg_values(GGML), BB = gg_bytes(GGML);
  const int64_t bytes_per_row = K / VPB * BB;
  const uint8_t* w_end = w + N * bytes_per_row;
  float acc[GG_RPW][MR];
#pragma unroll
  for (int r = 0; r < GG_RPW; r++)
#pragma unroll
    for (int i = 0; i < MR; i++) acc[r][i] = 0.0f;
  // the bytes of (row r, chunk at kc), or nothing for a row past N or a chunk past K
  auto chunk_ptr = [&](int r, int64_t kc) -> const uint8_t* {
    return (n0 + r < N && kc < K) ? w + (n0 + r) * bytes_per_row + kc / VPB * BB : nullptr;
  };
  auto chunk_len = [&](int64_t kc) { return (int)min((int64_t)gg_chunk_bytes(GGML), bytes_per_row - kc / VPB * BB); };

  // With few rows of x the accumulators leave room for the next row's bytes in registers; with 16 rows (64 accumulators)
  // holding them costs more than the latency they hide (measured 266 against 210 us on 4096 x 14336), so there a row is
  // staged when its turn comes.
  constexpr bool PIPE = MR <= 4;
  GgPrefetch pf;
  pf.nvec = 0; pf.lead = 0;
  if (PIPE) gg_prefetch(pf, chunk_ptr(0, 0), chunk_len(0), w_end, lane);
  for (int64_t kc = 0; kc < K; kc += GG_CHUNK) {
    __syncthreads();                       // the previous slice of x has been used by every warp (and the table is written)
    for (int idx = threadIdx.x; idx < MR * GG_CHUNK; idx += GG_WARPS * 32) {
      const int i = idx / GG_CHUNK, k = idx % GG_CHUNK;
      xs[(i * 32 + (k >> 5)) * GG_XPITCH + (k & 31)] = (i < rows && kc + k < K) ? gg_x<XT>(x, (m0 + i) * K + kc + k) : 0.0f;
    }
    __syncthreads();
    const bool active = kc + 32 * lane < K;
#pragma unroll
    for (int r = 0; r < GG_RPW; r++) {     // unrolled: the accumulators stay in registers
      // Two stage buffers alternate: the bytes of this row were requested one row ago and are written now, and the next
      // row's (or the next chunk's first row's) are requested before this one is decoded.  A buffer is rewritten two rows
      // later, after a __syncwarp that every lane reaches only when it has decoded this row.
      bool have;                           // uniform across the warp
      const uint8_t* chunk;
      if (PIPE) {
        have = pf.nvec > 0;
        chunk = gg_commit(wstage + (r & 1) * GG_WSTAGE, pf, lane);
        __syncwarp();
        if (r + 1 < GG_RPW) gg_prefetch(pf, chunk_ptr(r + 1, kc), chunk_len(kc), w_end, lane);
        else gg_prefetch(pf, chunk_ptr(0, kc + GG_CHUNK), kc + GG_CHUNK < K ? chunk_len(kc + GG_CHUNK) : 0, w_end, lane);
      } else {
        const uint8_t* g = chunk_ptr(r, kc);
        have = g != nullptr;
        __syncwarp();                      // the previous row's bytes have been decoded
        chunk = have ? gg_stage(wstage, g, chunk_len(kc), w_end, lane) : wstage;
        __syncwarp();
      }
      if (have && active) {
        float wv[32];
        gg_decode32<GGML>(chunk, lane, wv, s_lut);
#pragma unroll
        for (int i = 0; i < MR; i++) {
          if (i < rows) {
            const float4* xv = reinterpret_cast<const float4*>(xs + (i * 32 + lane) * GG_XPITCH);
            float s = acc[r][i];
#pragma unroll
            for (int q = 0; q < 8; q++) {
              const float4 t = xv[q];
              s = fmaf(t.x, wv[4 * q], s); s = fmaf(t.y, wv[4 * q + 1], s); s = fmaf(t.z, wv[4 * q + 2], s); s = fmaf(t.w, wv[4 * q + 3], s);
            }
            acc[r][i] = s;
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < GG_RPW; r++) {
    const int64_t n = n0 + r;
#pragma unroll
    for (int i = 0; i < MR; i++) {
      float a = acc[r][i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
      if (lane == 0 && n < N && i < rows) {
        const float v = bias ? __fadd_rn(a, bias[n]) : a;
        Scalar<XT>::store(out, (m0 + i) * N + n, apply_activation(v, act));
      }
    }
  }
}

// ---- QuantizedEmbeddingLookup: one CTA per index, a warp per 1024-value chunk of the row.
template <typename IT, int GGML>
__global__ void __launch_bounds__(GG_WARPS * 32)
embedding_lookup_kernel(const uint8_t* __restrict__ table, const IT* __restrict__ indices, float* __restrict__ out,
                        int64_t vocab, int64_t K, unsigned* __restrict__ status) {
  __shared__ __align__(16) uint8_t stage[GG_WARPS][GG_WSTAGE];
  __shared__ float s_lut[16];
  if (threadIdx.x < 16) s_lut[threadIdx.x] = c_iq4nl[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t i = blockIdx.x;
  const long long row = (long long)indices[i];
  constexpr int VPB = gg_values(GGML), BB = gg_bytes(GGML);
  const int64_t bytes_per_row = K / VPB * BB;
  float* o = out + i * K;
  if (row < 0 || row >= vocab) {
    // the reference returns an error (quantizeddense.go:487-489): flag the position of the first bad index, write zeros
    if (threadIdx.x == 0) { atomicMax(status + 1, 0xFFFFFFFFu - (unsigned)min(i, (int64_t)0x7FFFFFFF)); atomicExch(status, 1u); }
    for (int64_t k = threadIdx.x; k < K; k += GG_WARPS * 32) o[k] = 0.0f;
    return;
  }
  const uint8_t* src = table + row * bytes_per_row;
  const uint8_t* end = table + vocab * bytes_per_row;
  for (int64_t kc = (int64_t)warp * GG_CHUNK; kc < K; kc += (int64_t)GG_WARPS * GG_CHUNK) {
    const int len = (int)min((int64_t)gg_chunk_bytes(GGML), bytes_per_row - kc / VPB * BB);
    __syncwarp();
    const uint8_t* chunk = gg_stage(stage[warp], src + kc / VPB * BB, len, end, lane);
    __syncwarp();
    if (kc + 32 * lane < K) {
      float wv[32];
      gg_decode32<GGML>(chunk, lane, wv, s_lut);
      float4* dst = reinterpret_cast<float4*>(o + kc + 32 * lane);       // out is 16-byte aligned and K a multiple of 32
#pragma unroll
      for (int q = 0; q < 8; q++) dst[q] = make_float4(wv[4 * q], wv[4 * q + 1], wv[4 * q + 2], wv[4 * q + 3]);
    }
  }
}

// ---- prefill: every weight row dequantised once into bf16 planes [plane][N][K] for the tensor-core GEMM
// (w = p0 + p1 (+ p2), p0 = bf16(w), p1 = bf16(w - p0), ...).  One CTA per weight row, a warp per 1024-value chunk.
template <int GGML, int NPLANES>
__global__ void __launch_bounds__(GG_WARPS * 32)
ggml_planes_kernel(const uint8_t* __restrict__ w, uint16_t* __restrict__ planes, int64_t N, int64_t K) {
  // the GEMM that consumes the planes may set itself up meanwhile; it waits for this grid before it loads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ __align__(16) uint8_t stage[GG_WARPS][GG_WSTAGE];
  __shared__ float s_lut[16];
  if (threadIdx.x < 16) s_lut[threadIdx.x] = c_iq4nl[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x;
  constexpr int VPB = gg_values(GGML), BB = gg_bytes(GGML);
  const int64_t bytes_per_row = K / VPB * BB;
  const uint8_t* src = w + row * bytes_per_row;
  const uint8_t* end = w + N * bytes_per_row;
  const size_t plane_elems = (size_t)N * K;
  for (int64_t kc = (int64_t)warp * GG_CHUNK; kc < K; kc += (int64_t)GG_WARPS * GG_CHUNK) {
    const int len = (int)min((int64_t)gg_chunk_bytes(GGML), bytes_per_row - kc / VPB * BB);
    __syncwarp();
    const uint8_t* chunk = gg_stage(stage[warp], src + kc / VPB * BB, len, end, lane);
    __syncwarp();
    if (kc + 32 * lane < K) {
      float wv[32];
      gg_decode32<GGML>(chunk, lane, wv, s_lut);
#pragma unroll
      for (int q = 0; q < NPLANES; q++) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; e++) {
          pk[e] = (uint32_t)f32_to_bf16_bits(wv[2 * e]) | ((uint32_t)f32_to_bf16_bits(wv[2 * e + 1]) << 16);
          // what the planes so far leave over (nothing for non-finite values)
          const float h0 = __uint_as_float(pk[e] << 16), h1 = __uint_as_float(pk[e] & 0xFFFF0000u);
          wv[2 * e] = isfinite(wv[2 * e]) ? wv[2 * e] - h0 : 0.0f;
          wv[2 * e + 1] = isfinite(wv[2 * e + 1]) ? wv[2 * e + 1] - h1 : 0.0f;
        }
        uint4* dst = reinterpret_cast<uint4*>(planes + (size_t)q * plane_elems + (size_t)row * K + kc + 32 * lane);
#pragma unroll
        for (int v = 0; v < 4; v++) dst[v] = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
      }
    }
  }
}

size_t gg_align256(size_t v) { return (v + 255) & ~(size_t)255; }
// More than 16 rows of x and enough work to pay for expanding the weights (the same rule as for 8-bit weights).
bool gg_prefill_supports(const cb_qdense_desc& d) {
  if (d.variant != CB_QDENSE_AUTO && d.variant != CB_QDENSE_PREFILL) return false;
  if (d.K % 32 != 0 || d.N % 8 != 0 || d.K < 32 || d.N < 8 || d.M < 1) return false;
  if (d.M > (1 << 30) || d.K > (1 << 30) || d.N > (1 << 30)) return false;
  return d.variant == CB_QDENSE_PREFILL || (d.M > 16 && (double)d.M * d.K * d.N >= 64.0 * 1024 * 1024);
}
int gg_prefill_w_planes(const cb_qdense_desc& d) { return 2; }    // 16 mantissa bits of d * q
int gg_prefill_x_planes(const cb_qdense_desc& d) { return d.x_dtype == CB_F32 ? 2 : 1; }

template <int GGML>
int gg_planes_launch(const cb_qdense_desc& d, const uint8_t* w, uint16_t* planes, cudaStream_t s) {
  ggml_planes_kernel<GGML, 2><<<(unsigned)d.N, GG_WARPS * 32, 0, s>>>(w, planes, d.N, d.K);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

const char* gg_name(int t) {
  switch (t) {
    case CB_GGML_Q4_0: return "q4_0";
    case CB_GGML_Q8_0: return "q8_0";
    case CB_GGML_IQ4_NL: return "iq4_nl";
    case CB_GGML_Q4_K: return "q4_k";
    case CB_GGML_Q6_K: return "q6_k";
    default: return "?";
  }
}

bool gg_supported(int t) {
  return t == CB_GGML_Q4_0 || t == CB_GGML_Q8_0 || t == CB_GGML_IQ4_NL || t == CB_GGML_Q4_K || t == CB_GGML_Q6_K;
}

int gg_mr(int64_t M) { return M <= 1 ? 1 : M <= 4 ? 4 : 16; }
size_t gg_smem_bytes(int mr) { return (size_t)mr * 32 * GG_XPITCH * sizeof(float) + (size_t)GG_WARPS * 2 * GG_WSTAGE; }

template <typename XT, int GGML, int MR>
int gg_launch_k(const cb_qdense_desc& d, const void* const* in, void* const* out, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  int dev = 0;
  CB_CUDA(cudaGetDevice(&dev));
  const size_t smem = gg_smem_bytes(MR);
  if (smem > 48 * 1024 && (dev >= 64 || !configured[dev].load(std::memory_order_acquire))) {
    CB_CUDA(cudaFuncSetAttribute(qdense_ggml_kernel<XT, GGML, MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  const float* bias = d.has_bias ? (const float*)in[2] : nullptr;
  dim3 grid((unsigned)((d.N + GG_WARPS * GG_RPW - 1) / (GG_WARPS * GG_RPW)), (unsigned)((d.M + MR - 1) / MR));
  qdense_ggml_kernel<XT, GGML, MR><<<grid, GG_WARPS * 32, smem, s>>>((const XT*)in[0], (const uint8_t*)in[1], bias, (XT*)out[0], d.M, d.K, d.N, d.activation);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

template <typename XT, int GGML>
int gg_launch_m(const cb_qdense_desc& d, const void* const* in, void* const* out, cudaStream_t s) {
  switch (gg_mr(d.M)) {
    case 1: return gg_launch_k<XT, GGML, 1>(d, in, out, s);
    case 4: return gg_launch_k<XT, GGML, 4>(d, in, out, s);
    default: return gg_launch_k<XT, GGML, 16>(d, in, out, s);
  }
}

template <typename XT>
int gg_launch_t(const cb_qdense_desc& d, const void* const* in, void* const* out, cudaStream_t s) {
  switch (d.ggml_type) {
    case CB_GGML_Q4_0: return gg_launch_m<XT, CB_GGML_Q4_0>(d, in, out, s);
    case CB_GGML_Q8_0: return gg_launch_m<XT, CB_GGML_Q8_0>(d, in, out, s);
    case CB_GGML_IQ4_NL: return gg_launch_m<XT, CB_GGML_IQ4_NL>(d, in, out, s);
    case CB_GGML_Q4_K: return gg_launch_m<XT, CB_GGML_Q4_K>(d, in, out, s);
    default: return gg_launch_m<XT, CB_GGML_Q6_K>(d, in, out, s);
  }
}

template <typename IT>
int el_launch_t(const HelperDesc& h, const void* const* in, void* const* out, unsigned* status, cudaStream_t s) {
  const int64_t vocab = h.dims[0], K = h.dims[2], n = h.n;
#define CB_EL(G) embedding_lookup_kernel<IT, G><<<(unsigned)n, GG_WARPS * 32, 0, s>>>((const uint8_t*)in[0], (const IT*)in[1], (float*)out[0], vocab, K, status)
  switch (h.axis) {
    case CB_GGML_Q4_0: CB_EL(CB_GGML_Q4_0); break;
    case CB_GGML_Q8_0: CB_EL(CB_GGML_Q8_0); break;
    case CB_GGML_IQ4_NL: CB_EL(CB_GGML_IQ4_NL); break;
    case CB_GGML_Q4_K: CB_EL(CB_GGML_Q4_K); break;
    default: CB_EL(CB_GGML_Q6_K); break;
  }
#undef CB_EL
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

}  // namespace

// quantizeddense.go:181-248: weights [N, bytesPerRow] Uint8, K derived from the row bytes, no zero points
int qdense_ggml_plan(cb_plan* p) {
  cb_qdense_desc& d = p->qd;
  const char* op = "FusedQuantizedDense(GGML)";
  if (!gg_supported(d.ggml_type)) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: GGML type %d not supported in fused path", op, d.ggml_type);
  if (d.w_dtype != CB_U8) return fail(CB_ERR_INVALID_ARG, "%s: weights must be [N, bytesPerRow] Uint8, got %s", op, dtype_name(d.w_dtype));
  if (d.K % gg_values(d.ggml_type) != 0)
    return fail(CB_ERR_INVALID_ARG, "%s: K=%lld is not a whole number of %d-value blocks", op, (long long)d.K, gg_values(d.ggml_type));
  if (d.has_zero_point) return fail(CB_ERR_INVALID_ARG, "%s: ZeroPoint must be nil for GGML scheme", op);
  if (d.activation < CB_ACT_NONE || d.activation > CB_ACT_TANH) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown activation %d", d.activation);
  if (d.gather_ranks > 1) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: a gathered plan needs the tensor-core decode kernel", op);
  const int mr = gg_mr(d.M);
  const int64_t gx = (d.N + GG_WARPS * GG_RPW - 1) / (GG_WARPS * GG_RPW), gy = (d.M + mr - 1) / mr;
  if (gx > 0x7FFFFFFFLL || gy > 65535) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: shape too large for one launch", op);
  p->n_inputs = 2 + (d.has_bias ? 1 : 0);
  p->n_outputs = 1;
  p->variant = CB_QDENSE_GENERIC;
  p->blocks = (int)(gx * gy);
  p->threads = GG_WARPS * 32;
  p->dyn_smem = (int)gg_smem_bytes(mr);
  p->name = std::string("qdense_ggml_") + (d.x_dtype == CB_BF16 ? "bf16_" : "f32_") + gg_name(d.ggml_type);
  // decode shapes of the formats whose blocks feed the integer tensor cores directly (CB_QDENSE_GENERIC keeps this kernel)
  if (qdense_ggml_mma_supports(d)) qdense_ggml_mma_plan(p, gg_name(d.ggml_type));
  else if (gg_prefill_supports(d)) {
    // prefill shapes: the rows of W dequantised to bf16 planes once, then the tensor-core GEMM (W as the transposed operand)
    p->variant = CB_QDENSE_PREFILL;
    p->blocks = gemm_tc_blocks(p->n_sm, 1, d.M, d.N);
    p->threads = gemm_tc_threads();
    p->dyn_smem = gemm_tc_smem();
    p->counter_bytes = 256;
    p->workspace_bytes = 256 + gg_align256((size_t)gg_prefill_w_planes(d) * d.N * d.K * 2) +
                         (d.x_dtype == CB_F32 ? gg_align256((size_t)gg_prefill_x_planes(d) * d.M * d.K * 2) : 0);
    p->has_status = true;
    p->name = std::string("qdense_ggml_prefill_tcgen05_") + (d.x_dtype == CB_BF16 ? "bf16_" : "f32_") + gg_name(d.ggml_type);
  } else if (d.variant == CB_QDENSE_PREFILL) {
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s prefill kernel: K must be a multiple of 32 and N of 8", op);
  }
  return CB_OK;
}

static int qdense_ggml_prefill_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (!ws) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense(GGML): the plan needs its workspace (bf16 planes of the weights)");
  uint8_t* w8 = (uint8_t*)ws;
  const int wp = gg_prefill_w_planes(d), xp = gg_prefill_x_planes(d);
  uint16_t* wplanes = (uint16_t*)(w8 + 256);
  uint16_t* xplanes = (uint16_t*)(w8 + 256 + gg_align256((size_t)wp * d.N * d.K * 2));
  const uint8_t* wq = (const uint8_t*)in[1];
  switch (d.ggml_type) {
    case CB_GGML_Q4_0: CB_TRY(gg_planes_launch<CB_GGML_Q4_0>(d, wq, wplanes, s)); break;
    case CB_GGML_Q8_0: CB_TRY(gg_planes_launch<CB_GGML_Q8_0>(d, wq, wplanes, s)); break;
    case CB_GGML_IQ4_NL: CB_TRY(gg_planes_launch<CB_GGML_IQ4_NL>(d, wq, wplanes, s)); break;
    case CB_GGML_Q4_K: CB_TRY(gg_planes_launch<CB_GGML_Q4_K>(d, wq, wplanes, s)); break;
    default: CB_TRY(gg_planes_launch<CB_GGML_Q6_K>(d, wq, wplanes, s)); break;
  }
  GemmTcProblem g;
  g.a = in[0];
  g.planes_a = 1;
  if (d.x_dtype == CB_F32) {
    CB_TRY(split_f32_planes((const float*)in[0], xplanes, (size_t)d.M * d.K, nullptr, nullptr, 0, xp, s));
    g.a = xplanes;
    g.planes_a = xp;
  }
  g.b = wplanes;
  g.planes_b = wp;
  g.out = out[0];
  g.status = (unsigned*)ws;
  g.B = 1; g.M = d.M; g.N = d.N; g.K = d.K;
  g.rhs_transposed = 1;
  g.ab_dtype = CB_BF16;
  g.out_dtype = d.x_dtype;
  g.n_pass = gemm_tc_split_passes(g.planes_a, g.planes_b, 1, g.pass_a, g.pass_b);
  g.col_scale = nullptr;
  g.bias = d.has_bias ? (const float*)in[2] : nullptr;
  g.activation = d.activation;
  return gemm_tc_run(p->dev, p->blocks, g, s);
}

int qdense_ggml_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (d.M == 0 || d.N == 0) return CB_OK;
  if ((reinterpret_cast<uintptr_t>(in[0]) & 15) != 0 || (reinterpret_cast<uintptr_t>(in[1]) & 15) != 0)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense(GGML): x and weights must be 16-byte aligned");
  if (qdense_ggml_mma_supports(d)) {
    if (!ws) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense(GGML): the plan needs its workspace (digit planes of x)");
    return qdense_ggml_mma_launch(p, in, out, ws, s);
  }
  if (p->variant == CB_QDENSE_PREFILL) return qdense_ggml_prefill_launch(p, in, out, ws, s);
  return d.x_dtype == CB_BF16 ? gg_launch_t<__nv_bfloat16>(d, in, out, s) : gg_launch_t<float>(d, in, out, s);
}

// HelperDesc use: dims[0] vocab, dims[1] bytes per row, dims[2] K, n = number of indices, dtype = index dtype, axis = GGML type.
// The workspace holds two words: [0] != 0 when an index was outside the table, [1] = 0xFFFFFFFF - the position of the
// first such index (so that zeroing the words resets them and atomicMax keeps the first).
int embedding_lookup_plan(cb_plan* p) {
  HelperDesc& h = p->helper;
  const char* op = "QuantizedEmbeddingLookup";
  if (!gg_supported(h.axis)) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: GGML type %d not supported in fused path", op, h.axis);
  if (h.dtype != CB_I8 && h.dtype != CB_U8 && h.dtype != CB_I32 && h.dtype != CB_I64)
    return fail(h.dtype == CB_F32 || h.dtype == CB_F64 || h.dtype == CB_BF16 || h.dtype == CB_F16 || h.dtype == CB_BOOL ? CB_ERR_INVALID_ARG : CB_ERR_NOT_IMPLEMENTED,
                "%s: indices must be integer, got %s", op, dtype_name(h.dtype));
  if (h.dims[0] < 0 || h.dims[1] < 0 || h.n < 0) return fail(CB_ERR_INVALID_ARG, "%s: negative dimension", op);
  const int bb = gg_bytes(h.axis);
  if (h.dims[1] % bb != 0)
    return fail(CB_ERR_INVALID_ARG, "%s: bytesPerRow %lld not divisible by bytesPerBlock %d for %s", op, (long long)h.dims[1], bb, gg_name(h.axis));
  h.dims[2] = h.dims[1] / bb * gg_values(h.axis);
  if (h.n > 0x7FFFFFFFLL) return fail(CB_ERR_NOT_IMPLEMENTED, "%s: too many indices for one launch", op);
  p->n_inputs = 2;
  p->n_outputs = 1;
  p->blocks = (int)h.n;
  p->threads = GG_WARPS * 32;
  p->workspace_bytes = 256;
  p->counter_bytes = 0;
  p->name = std::string("embedding_lookup_") + gg_name(h.axis);
  return CB_OK;
}

int embedding_lookup_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const HelperDesc& h = p->helper;
  if (h.n == 0 || h.dims[2] == 0) return CB_OK;
  if (!ws) return fail(CB_ERR_INVALID_ARG, "QuantizedEmbeddingLookup: the plan needs its workspace (status words)");
  if ((reinterpret_cast<uintptr_t>(in[0]) & 15) || (reinterpret_cast<uintptr_t>(out[0]) & 15))
    return fail(CB_ERR_INVALID_ARG, "QuantizedEmbeddingLookup: table and output must be 16-byte aligned");
  unsigned* status = (unsigned*)ws;
  CB_CUDA(cudaMemsetAsync(status, 0, 2 * sizeof(unsigned), s));
  switch (h.dtype) {
    case CB_I8: return el_launch_t<int8_t>(h, in, out, status, s);
    case CB_U8: return el_launch_t<uint8_t>(h, in, out, status, s);
    case CB_I32: return el_launch_t<int32_t>(h, in, out, status, s);
    default: return el_launch_t<int64_t>(h, in, out, status, s);
  }
}

// Reads the status words (a small blocking copy): an index outside the table is the reference's error.
int embedding_lookup_check(const cb_plan* p, const void* ws) {
  unsigned st[2] = {0, 0};
  CB_CUDA(cudaMemcpy(st, ws, sizeof(st), cudaMemcpyDeviceToHost));
  if (st[0]) return fail(CB_ERR_INVALID_ARG, "QuantizedEmbeddingLookup: index at position %u out of range [0, %lld)", 0xFFFFFFFFu - st[1], (long long)p->helper.dims[0]);
  return CB_OK;
}

}  // namespace cb
