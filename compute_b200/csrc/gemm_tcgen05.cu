// DotGeneral in normalised form on the 5th-generation tensor cores:
//   out[B,M,N] = lhs[B,M,K] x rhs[B,K,N]      (rhs_transposed = 0, rhs is the MN-major operand)
//   out[B,M,N] = lhs[B,M,K] x rhs[B,N,K]^T    (rhs_transposed = 1, K-major operand)
// bf16 / f16 inputs, f32 accumulation in tensor memory, output bf16 / f16 / f32
// (half inputs accumulate in f32: internal/gobackend/dot/dot.go:207-210 of the reference).
//
// Persistent kernel, one CTA per SM, 128 x 256 output tiles, K blocks of 64:
//   warp 8  TMA producer: 128B-swizzled tiles of A and B into a 4-stage shared-memory ring
//   warp 9  MMA issuer:   tcgen05.mma (M=128, N=256, K=16) from shared-memory descriptors
//                         into one of two 256-column TMEM accumulators
//   warps 0-7 epilogue:   tcgen05.ld of the finished accumulator (each warp a 32-row x 128-column
//                         quarter, loads software-pipelined), scale / bias / activation, convert,
//                         store — overlapped with the next tile's main loop through the second
//                         accumulator
// All waits are bounded; a timeout sets the status word, and TMEM is always freed.
//
// Operands wider than 16 bits arrive as bf16 planes stacked in the batch dimension and the
// main loop runs a list of (lhs plane, rhs plane) passes into the same accumulator (gemm_tc.h);
// float32 DotGeneral and the prefill-shaped quantized dense are built on that.  The epilogue
// optionally applies a per-column scale, a bias and an activation before the store.
#include "tc_common.cuh"
#include "gemm_tc.h"

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string.h>

namespace cb {

using namespace tc;

constexpr int GT_BM = 128, GT_BN = 256, GT_BK = 64, GT_STAGES = 4;
constexpr int GT_A_BYTES = GT_BM * GT_BK * 2;        // 16 KB
constexpr int GT_B_BYTES = GT_BN * GT_BK * 2;        // 32 KB
constexpr int GT_STAGE_BYTES = GT_A_BYTES + GT_B_BYTES;
constexpr int GT_EPI_WARPS = 8;                      // warp w reads TMEM lanes 32*(w&3).., columns 128*(w>>2)..
constexpr int GT_TMA_WARP = 8, GT_MMA_WARP = 9;
constexpr int GT_THREADS = 320;
constexpr int GT_EPI_BYTES = GT_EPI_WARPS * 256 * 4; // per epilogue warp: 128 column scales + 128 biases
constexpr int GT_SMEM = 1024 + GT_STAGES * GT_STAGE_BYTES + 256 + GT_EPI_BYTES;
constexpr int GT_TMEM_COLS = 512;

struct GtParams {
  void* out;
  unsigned* status;
  int M, N, K, B;
  int tiles_m, tiles_n;
  long long num_tiles;
  int out_dtype;
  int rhs_transposed;
  int ab_format;       // 0 f16, 1 bf16
  int n_pass;
  int pass_a[GEMM_TC_MAX_PASSES], pass_b[GEMM_TC_MAX_PASSES];   // plane of each pass
  const float* col_scale;
  const float* bias;
  int activation;
  int epilogue;        // 1 when any of col_scale / bias / activation applies
};

__device__ __forceinline__ void gt_fail(const GtParams& p, unsigned* s_failed, unsigned code, unsigned detail) {
  atomicExch(&p.status[0], code);
  atomicExch(&p.status[1], detail);
  atomicExch(s_failed, 1u);
}

template <typename OT> struct GtStore;
template <> struct GtStore<float> {
  __device__ static void store8(float* dst, const uint32_t* r) {
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(r[0], r[1], r[2], r[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(r[4], r[5], r[6], r[7]);
  }
  __device__ static void store1(float* dst, uint32_t r) { *dst = __uint_as_float(r); }
};
template <> struct GtStore<__nv_bfloat16> {
  __device__ static void store8(__nv_bfloat16* dst, const uint32_t* r) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++)
      w[i] = (uint32_t)f32_to_bf16_bits(__uint_as_float(r[2 * i])) | ((uint32_t)f32_to_bf16_bits(__uint_as_float(r[2 * i + 1])) << 16);
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static void store1(__nv_bfloat16* dst, uint32_t r) { Scalar<__nv_bfloat16>::store(dst, 0, __uint_as_float(r)); }
};
template <> struct GtStore<__half> {
  __device__ static void store8(__half* dst, const uint32_t* r) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __half2 h = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static void store1(__half* dst, uint32_t r) { *dst = __float2half_rn(__uint_as_float(r)); }
};

// out = act(acc * scale + bias) on 32 accumulator columns; sc / bi point at this warp's staged
// column vectors in shared memory (every lane reads the same words: broadcasts).  FAST picks the
// hardware exp and reciprocal, whose error is far below one unit of a 16-bit output.
template <int ACT, bool FAST>
__device__ __forceinline__ void gt_epilogue32(uint32_t* r, const float* sc, const float* bi) {
#pragma unroll
  for (int q4 = 0; q4 < 8; q4++) {
    const float4 s4 = *reinterpret_cast<const float4*>(sc + 4 * q4);
    const float4 b4 = *reinterpret_cast<const float4*>(bi + 4 * q4);
    const float ss[4] = {s4.x, s4.y, s4.z, s4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
      float v = fmaf(__uint_as_float(r[4 * q4 + e]), ss[e], bb[e]);
      if (ACT == CB_ACT_SILU && FAST) v = __fdividef(v, 1.0f + __expf(-v));
      else v = apply_activation(v, ACT);
      r[4 * q4 + e] = __float_as_uint(v);
    }
  }
}

template <bool FAST>
__device__ __forceinline__ void gt_epilogue32_any(int act, uint32_t* r, const float* sc, const float* bi) {
  switch (act) {
    case CB_ACT_GELU: gt_epilogue32<CB_ACT_GELU, FAST>(r, sc, bi); break;
    case CB_ACT_RELU: gt_epilogue32<CB_ACT_RELU, FAST>(r, sc, bi); break;
    case CB_ACT_SILU: gt_epilogue32<CB_ACT_SILU, FAST>(r, sc, bi); break;
    case CB_ACT_HARDSWISH: gt_epilogue32<CB_ACT_HARDSWISH, FAST>(r, sc, bi); break;
    case CB_ACT_TANH: gt_epilogue32<CB_ACT_TANH, FAST>(r, sc, bi); break;
    default: gt_epilogue32<CB_ACT_NONE, FAST>(r, sc, bi); break;
  }
}

template <typename OT>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GtParams p) {
  extern __shared__ uint8_t gt_smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gt_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + GT_STAGES * GT_STAGE_BYTES);
  uint64_t* full = bars;                         // [GT_STAGES] TMA -> MMA
  uint64_t* empty = bars + GT_STAGES;            // [GT_STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * GT_STAGES;     // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;            // [2] epilogue -> MMA
  __shared__ uint32_t s_tmem;
  __shared__ unsigned s_failed;

  // The next kernel in the stream, if it was launched for programmatic dependent launch, may be
  // scheduled while this grid drains (such kernels wait before they touch global memory).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kblocks = (p.K + GT_BK - 1) / GT_BK;

  if (tid == 0) {
    for (int s = 0; s < GT_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], GT_EPI_WARPS); }
    s_failed = 0;
    fence_barrier_init();
  }
  if (warp == GT_MMA_WARP) tmem_alloc(&s_tmem, GT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;
  // Set-up above overlaps the tail of the kernel before this one; its outputs (possibly this
  // kernel's operands) and the memory it may still read are touched only after it has finished.
  if (warp != GT_MMA_WARP) asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == GT_TMA_WARP) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_a);
      prefetch_tensormap(&tmap_b);
      long long it = 0;
      for (long long tile = blockIdx.x; tile < p.num_tiles && !*(volatile unsigned*)&s_failed; tile += gridDim.x) {
        const int b = (int)(tile / ((long long)p.tiles_m * p.tiles_n));
        const int rem = (int)(tile % ((long long)p.tiles_m * p.tiles_n));
        const int m0 = (rem % p.tiles_m) * GT_BM, n0 = (rem / p.tiles_m) * GT_BN;
        bool ok = true;
        for (int ps = 0; ps < p.n_pass && ok; ps++) {
          const int za = p.pass_a[ps] * p.B + b, zb = p.pass_b[ps] * p.B + b;
          for (int kb = 0; kb < kblocks; kb++, it++) {
            const int s = (int)(it % GT_STAGES);
            if (it >= GT_STAGES && !mbar_wait(&empty[s], (uint32_t)((it / GT_STAGES - 1) & 1))) { gt_fail(p, &s_failed, 1, (unsigned)it); ok = false; break; }
            uint8_t* sa = base + s * GT_STAGE_BYTES;
            uint8_t* sb = sa + GT_A_BYTES;
            mbar_expect_tx(&full[s], GT_STAGE_BYTES);
            tma_load_3d(sa, &tmap_a, kb * GT_BK, m0, za, &full[s]);
            if (p.rhs_transposed) {
              tma_load_3d(sb, &tmap_b, kb * GT_BK, n0, zb, &full[s]);                 // [256 n rows][64 k]
            } else {
#pragma unroll
              for (int j = 0; j < GT_BN / 64; j++)                                      // 4 x [64 k rows][64 n]
                tma_load_3d(sb + j * (GT_BK * 128), &tmap_b, n0 + 64 * j, kb * GT_BK, zb, &full[s]);
            }
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == GT_MMA_WARP) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = idesc_f16(GT_BM, GT_BN, p.ab_format, 0, p.rhs_transposed ? 0 : 1);
      long long it = 0, local = 0;
      for (long long tile = blockIdx.x; tile < p.num_tiles && !*(volatile unsigned*)&s_failed; tile += gridDim.x, local++) {
        const int buf = (int)(local & 1);
        if (local >= 2 && !mbar_wait(&acc_empty[buf], (uint32_t)((local / 2 - 1) & 1))) { gt_fail(p, &s_failed, 2, (unsigned)local); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * GT_BN);
        bool ok = true;
        const int kiters = kblocks * p.n_pass;
        for (int kb = 0; kb < kiters; kb++, it++) {
          const int s = (int)(it % GT_STAGES);
          if (!mbar_wait(&full[s], (uint32_t)((it / GT_STAGES) & 1))) { gt_fail(p, &s_failed, 3, (unsigned)it); ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(base + s * GT_STAGE_BYTES), sb = sa + GT_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GT_BK / 16; kk++) {
            const uint64_t da = smem_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t db = p.rhs_transposed ? smem_desc_sw128(sb + kk * 32, 16, 1024)
                                                 : smem_desc_sw128(sb + kk * 16 * 128, GT_BK * 128, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);          // the stage is free once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);       // accumulator complete
      }
    }
  } else {
    // ------------------------------ epilogue (warps 0-7) ----------------------
    long long local = 0;
    bool failed = false;
    OT* out = reinterpret_cast<OT*>(p.out);
    const int quarter = warp & 3, half = warp >> 2;
    float* s_sc = reinterpret_cast<float*>(base + GT_STAGES * GT_STAGE_BYTES + 256) + warp * 256;
    float* s_bi = s_sc + 128;
    constexpr bool FAST = sizeof(OT) == 2;
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, local++) {
      const int buf = (int)(local & 1);
      const int b = (int)(tile / ((long long)p.tiles_m * p.tiles_n));
      const int rem = (int)(tile % ((long long)p.tiles_m * p.tiles_n));
      const int m0 = (rem % p.tiles_m) * GT_BM, n0 = (rem / p.tiles_m) * GT_BN + half * 128;
      if (p.epilogue) {        // this warp's 128 column scales and biases, staged while the main loop runs
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int cc = min(n0 + j * 32 + lane, p.N - 1);
          s_sc[j * 32 + lane] = p.col_scale ? __ldg(p.col_scale + cc) : 1.0f;
          s_bi[j * 32 + lane] = p.bias ? __ldg(p.bias + cc) : 0.0f;
        }
        __syncwarp();
      }
      if (!failed && !mbar_wait(&acc_full[buf], (uint32_t)((local / 2) & 1))) { failed = true; gt_fail(p, &s_failed, 4, (unsigned)local); }
      if (failed || *(volatile unsigned*)&s_failed) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      OT* orow = out + ((size_t)b * p.M + (size_t)min(row, p.M - 1)) * p.N;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * GT_BN + half * 128);
      auto finish = [&](uint32_t* r, int c) {
        if (p.epilogue) gt_epilogue32_any<FAST>(p.activation, r, s_sc + c * 32, s_bi + c * 32);
        const int col = n0 + c * 32;
        if (row < p.M) {
          if (col + 32 <= p.N) {
#pragma unroll
            for (int q = 0; q < 4; q++) GtStore<OT>::store8(orow + col + 8 * q, r + 8 * q);
          } else {
            for (int q = 0; q < 32; q++)
              if (col + q < p.N) GtStore<OT>::store1(orow + col + q, r[q]);
          }
        }
      };
      // four chunks of 32 columns; the load of the next chunk is in flight while one is finished
      uint32_t ra[32], rb[32];
      tmem_ld32(taddr, ra);
      tmem_ld_wait();
      tmem_ld32(taddr + 32, rb);
      finish(ra, 0);
      tmem_ld_wait();
      tmem_ld32(taddr + 64, ra);
      finish(rb, 1);
      tmem_ld_wait();
      tmem_ld32(taddr + 96, rb);
      finish(ra, 2);
      tmem_ld_wait();
      // the accumulator has been read completely: hand it back before the last chunk is stored
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      finish(rb, 3);
    }
  }
  // every role ends here; TMEM is released by the warp that allocated it
  tc_fence_before();
  __syncthreads();
  if (warp == GT_MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, GT_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// float32 -> bf16 planes
// ---------------------------------------------------------------------------
// One launch splits both operands: elements [0, n_a) come from src_a, the rest from src_b (both counts are rounded up
// to the 4-element vectors a thread handles, so a vector never straddles the two).
__global__ void __launch_bounds__(256)
split_f32_planes_kernel(const float* __restrict__ src_a, uint16_t* __restrict__ planes_a, size_t n_a,
                        const float* __restrict__ src_b, uint16_t* __restrict__ planes_b, size_t n_b, int n_planes) {
  // the GEMM that consumes the planes may set itself up meanwhile; it waits for this grid before it loads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t va = (n_a + 3) / 4, vb = (n_b + 3) / 4;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  constexpr int UNROLL = 4;            // vectors whose loads are in flight together
  for (size_t v0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < va + vb; v0 += stride * UNROLL) {
    float v[UNROLL][4];
    const float* srcs[UNROLL];
    uint16_t* dsts[UNROLL];
    size_t ns[UNROLL], is[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
      const size_t vi = v0 + (size_t)u * stride;
      const bool live = vi < va + vb, second = vi >= va;
      srcs[u] = second ? src_b : src_a;
      dsts[u] = second ? planes_b : planes_a;
      ns[u] = live ? (second ? n_b : n_a) : 0;
      is[u] = (second ? vi - va : vi) * 4;
      if (is[u] + 4 <= ns[u] && (reinterpret_cast<uintptr_t>(srcs[u]) & 15) == 0) {
        const float4 f = *reinterpret_cast<const float4*>(srcs[u] + is[u]);
        v[u][0] = f.x; v[u][1] = f.y; v[u][2] = f.z; v[u][3] = f.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; e++) v[u][e] = (is[u] + e < ns[u]) ? srcs[u][is[u] + e] : 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
      const size_t n = ns[u], i = is[u];
      if (i >= n) continue;
      uint16_t pl[3][4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const uint16_t h = f32_to_bf16_bits(v[u][e]);
        float rest = v[u][e] - bf16_bits_to_f32(h);
        if (!isfinite(v[u][e])) rest = 0.0f;
        const uint16_t m = f32_to_bf16_bits(rest);
        rest -= bf16_bits_to_f32(m);
        pl[0][e] = h; pl[1][e] = m; pl[2][e] = f32_to_bf16_bits(rest);
      }
#pragma unroll
      for (int q = 0; q < 3; q++) {
        if (q >= n_planes) break;
        uint16_t* dst = dsts[u] + (size_t)q * n + i;
        if (i + 4 <= n && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
          *reinterpret_cast<uint2*>(dst) = make_uint2((uint32_t)pl[q][0] | ((uint32_t)pl[q][1] << 16), (uint32_t)pl[q][2] | ((uint32_t)pl[q][3] << 16));
        } else {
          for (int e = 0; e < 4; e++) if (i + e < n) dst[e] = pl[q][e];
        }
      }
    }
  }
}

int split_f32_planes(const float* src_a, uint16_t* planes_a, size_t n_a, const float* src_b, uint16_t* planes_b, size_t n_b,
                     int n_planes, cudaStream_t s) {
  if (n_a + n_b == 0) return CB_OK;
  if (n_planes < 1 || n_planes > 3) return fail(CB_ERR_INVALID_ARG, "split_f32_planes: %d planes", n_planes);
  const size_t want = ((n_a + n_b) / 16 + 255) / 256;         // four vectors of four elements per thread and pass
  const int blocks = (int)std::min<size_t>(std::max<size_t>(want, 1), 148 * 16);
  split_f32_planes_kernel<<<blocks, 256, 0, s>>>(src_a, planes_a, n_a, src_b, planes_b, n_b, n_planes);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

// Plane products a_i * b_j with i + j <= max_sum (what lies beyond is below the planes' own residual).
int gemm_tc_split_passes(int pa, int pb, int max_sum, int* pass_a, int* pass_b) {
  int n = 0;
  for (int sum = max_sum; sum >= 0; sum--)      // smallest products first
    for (int i = pa - 1; i >= 0; i--) {
      const int j = sum - i;
      if (j < 0 || j >= pb) continue;
      pass_a[n] = i; pass_b[n] = j; n++;
    }
  return n;
}

// ---------------------------------------------------------------------------
// launch
// ---------------------------------------------------------------------------
int gemm_tc_blocks(int n_sm, int64_t B, int64_t M, int64_t N) {
  const long long tiles = (long long)B * ((M + GT_BM - 1) / GT_BM) * ((N + GT_BN - 1) / GT_BN);
  return (int)std::max<long long>(1, std::min<long long>(tiles, n_sm));
}
int gemm_tc_threads() { return GT_THREADS; }
int gemm_tc_smem() { return GT_SMEM; }

static int encode_3d(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1) {
  encode_tiled_fn enc = tensor_map_encoder();
  if (!enc) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(CB_ERR_INVALID_ARG, "tcgen05 GEMM: operands must be 16-byte aligned");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return CB_OK;
}

template <typename OT>
static int launch_t(int dev, int blocks, const CUtensorMap& ta, const CUtensorMap& tb, const GtParams& prm, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  if (dev >= 64 || dev < 0 || !configured[dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM));
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(GT_THREADS);
  cfg.dynamicSmemBytes = GT_SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<OT>, ta, tb, prm));
  return CB_OK;
}

int gemm_tc_run(int dev, int blocks, const GemmTcProblem& g, cudaStream_t s) {
  if (g.M == 0 || g.N == 0 || g.B == 0) return CB_OK;
  if (g.K % 8 != 0 || g.N % 8 != 0 || g.K < 8) return fail(CB_ERR_INVALID_ARG, "tcgen05 GEMM: K and N must be multiples of 8");
  if (g.n_pass < 1 || g.n_pass > GEMM_TC_MAX_PASSES) return fail(CB_ERR_INVALID_ARG, "tcgen05 GEMM: %d passes", g.n_pass);
  CUtensorMap ta, tb;
  CB_TRY(encode_3d(&ta, g.a, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)(g.B * g.planes_a), GT_BK, GT_BM));
  if (g.rhs_transposed) CB_TRY(encode_3d(&tb, g.b, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)(g.B * g.planes_b), GT_BK, GT_BN));
  else CB_TRY(encode_3d(&tb, g.b, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)(g.B * g.planes_b), 64, GT_BK));
  GtParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.out = g.out;
  prm.status = g.status;
  prm.M = (int)g.M; prm.N = (int)g.N; prm.K = (int)g.K; prm.B = (int)g.B;
  prm.tiles_m = (int)((g.M + GT_BM - 1) / GT_BM);
  prm.tiles_n = (int)((g.N + GT_BN - 1) / GT_BN);
  prm.num_tiles = (long long)g.B * prm.tiles_m * prm.tiles_n;
  prm.out_dtype = g.out_dtype;
  prm.rhs_transposed = g.rhs_transposed;
  prm.ab_format = g.ab_dtype == CB_BF16 ? 1 : 0;
  prm.n_pass = g.n_pass;
  for (int i = 0; i < g.n_pass; i++) {
    if (g.pass_a[i] < 0 || g.pass_a[i] >= g.planes_a || g.pass_b[i] < 0 || g.pass_b[i] >= g.planes_b)
      return fail(CB_ERR_INVALID_ARG, "tcgen05 GEMM: pass %d names a plane that does not exist", i);
    prm.pass_a[i] = g.pass_a[i]; prm.pass_b[i] = g.pass_b[i];
  }
  prm.col_scale = g.col_scale;
  prm.bias = g.bias;
  prm.activation = g.activation;
  prm.epilogue = (g.col_scale || g.bias || g.activation != CB_ACT_NONE) ? 1 : 0;
  if (reinterpret_cast<uintptr_t>(g.out) & 15) return fail(CB_ERR_INVALID_ARG, "tcgen05 GEMM: output must be 16-byte aligned");
  switch (g.out_dtype) {
    case CB_F32: return launch_t<float>(dev, blocks, ta, tb, prm, s);
    case CB_BF16: return launch_t<__nv_bfloat16>(dev, blocks, ta, tb, prm, s);
    case CB_F16: return launch_t<__half>(dev, blocks, ta, tb, prm, s);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "tcgen05 GEMM: output dtype %s", dtype_name(g.out_dtype));
  }
}

// ---------------------------------------------------------------------------
// DotGeneral planning
// ---------------------------------------------------------------------------
bool dot_tc_supports(const cb_dot_desc& d, std::string* why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  const int od = d.out_dtype ? d.out_dtype : d.in_dtype;
  if (d.in_dtype != CB_BF16 && d.in_dtype != CB_F16 && d.in_dtype != CB_F32) return no("inputs must be bfloat16, float16 or float32");
  if (od != d.in_dtype && od != CB_F32) return no("output must be the input dtype or float32");
  if (d.B < 1 || d.M < 1 || d.N < 1 || d.K < 1) return no("empty operand");
  if (d.K % 8 != 0) return no("K must be a multiple of 8 (16-byte rows for TMA)");
  if (d.N % 8 != 0) return no("N must be a multiple of 8");
  if (d.M > (1 << 30) || d.N > (1 << 30) || d.K > (1 << 30) || d.B > (1 << 18)) return no("dimension too large");
  // small problems are launch bound: unless asked for explicitly, the generic kernel serves them
  // (float32 pays a split launch on top, so its threshold is higher)
  const double macs = (double)d.B * d.M * d.N * d.K;
  if (d.variant != CB_DOT_TCGEN05 && d.variant != CB_DOT_TCGEN05_EXACT && macs < (d.in_dtype == CB_F32 ? 256.0 * 256 * 256 : 128.0 * 256 * 256))
    return no("problem too small for the tensor-core tile");
  return true;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// FusedDense on half types: the epilogue reads an f32 bias, so a 16-bit bias is widened into the
// workspace first (N elements).
template <typename T>
__global__ void bias_to_f32_kernel(const T* __restrict__ src, float* __restrict__ dst, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = Scalar<T>::load(src, i);
}

static int dot_tc_planes(const cb_dot_desc& d) { return d.variant == CB_DOT_TCGEN05_EXACT ? 3 : 2; }
static size_t dot_tc_planes_bytes(const cb_dot_desc& d) {
  const size_t np = (size_t)dot_tc_planes(d);
  return d.in_dtype == CB_F32 ? align256(np * d.B * d.M * d.K * 2) + align256(np * d.B * d.K * d.N * 2) : 0;
}

int dot_tc_plan(cb_plan* p) {
  const cb_dot_desc& d = p->dot;
  p->blocks = gemm_tc_blocks(p->n_sm, d.B, d.M, d.N);
  p->threads = GT_THREADS;
  p->dyn_smem = GT_SMEM;
  p->counter_bytes = 256;
  p->workspace_bytes = 256;
  p->workspace_bytes += dot_tc_planes_bytes(d);      // float32: two (or, exact, three) bf16 planes of each operand
  if (d.has_bias && d.in_dtype != CB_F32) p->workspace_bytes += align256((size_t)d.N * 4);
  p->has_status = true;
  const int od = d.out_dtype ? d.out_dtype : d.in_dtype;
  const bool dense = d.has_bias || d.activation != CB_ACT_NONE;
  p->name = std::string("gemm_tcgen05_") + dtype_name(d.in_dtype) + "_" + dtype_name(od) + (d.rhs_transposed ? "_nt" : "_nn") + (dense ? "_dense" : "") +
            (d.in_dtype == CB_F32 && d.variant == CB_DOT_TCGEN05_EXACT ? "_6pass" : "");
  return CB_OK;
}

int dot_tc_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_dot_desc& d = p->dot;
  GemmTcProblem g;
  g.a = in[0]; g.b = in[1]; g.out = out[0];
  g.status = (unsigned*)ws;
  g.B = d.B; g.M = d.M; g.N = d.N; g.K = d.K;
  g.rhs_transposed = d.rhs_transposed;
  g.ab_dtype = d.in_dtype;
  g.out_dtype = d.out_dtype ? d.out_dtype : d.in_dtype;
  g.activation = d.activation;
  if (d.has_bias) {
    if (d.in_dtype == CB_F32) {
      g.bias = (const float*)in[2];
    } else {
      float* b32 = (float*)((uint8_t*)ws + 256 + dot_tc_planes_bytes(d));
      const unsigned blocks = (unsigned)((d.N + 255) / 256);
      if (d.in_dtype == CB_BF16) bias_to_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)in[2], b32, d.N);
      else bias_to_f32_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)in[2], b32, d.N);
      CB_CUDA(cudaGetLastError());
      g.bias = b32;
    }
  }
  if (d.in_dtype == CB_F32) {
    uint8_t* w8 = (uint8_t*)ws;
    uint16_t* pa = (uint16_t*)(w8 + 256);
    const int np = dot_tc_planes(d);
    uint16_t* pb = (uint16_t*)(w8 + 256 + align256((size_t)np * d.B * d.M * d.K * 2));
    CB_TRY(split_f32_planes((const float*)in[0], pa, (size_t)d.B * d.M * d.K, (const float*)in[1], pb, (size_t)d.B * d.K * d.N, np, s));
    g.a = pa; g.b = pb;
    g.planes_a = g.planes_b = np;
    g.ab_dtype = CB_BF16;
    g.n_pass = gemm_tc_split_passes(np, np, np == 3 ? 2 : 1, g.pass_a, g.pass_b);
  }
  return gemm_tc_run(p->dev, p->blocks, g, s);
}

}  // namespace cb
