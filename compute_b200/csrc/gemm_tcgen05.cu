// DotGeneral in normalised form on the 5th-generation tensor cores:
//   out[B,M,N] = lhs[B,M,K] x rhs[B,K,N]      (rhs_transposed = 0, rhs is the MN-major operand)
//   out[B,M,N] = lhs[B,M,K] x rhs[B,N,K]^T    (rhs_transposed = 1, K-major operand)
// bf16 / f16 inputs, f32 accumulation in tensor memory, output bf16 / f16 / f32
// (half inputs accumulate in f32: internal/gobackend/dot/dot.go:207-210 of the reference).
//
// Persistent kernel, one CTA per SM, 128 x 256 output tiles, K blocks of 64:
//   warp 4  TMA producer: 128B-swizzled tiles of A and B into a 4-stage shared-memory ring
//   warp 5  MMA issuer:   tcgen05.mma (M=128, N=256, K=16) from shared-memory descriptors
//                         into one of two 256-column TMEM accumulators
//   warps 0-3 epilogue:   tcgen05.ld of the finished accumulator, convert, store — overlapped
//                         with the next tile's main loop through the second accumulator
// All waits are bounded; a timeout sets the status word, and TMEM is always freed.
#include "tc_common.cuh"

#include <atomic>
#include <mutex>
#include <string.h>

namespace cb {

using namespace tc;

constexpr int GT_BM = 128, GT_BN = 256, GT_BK = 64, GT_STAGES = 4;
constexpr int GT_A_BYTES = GT_BM * GT_BK * 2;        // 16 KB
constexpr int GT_B_BYTES = GT_BN * GT_BK * 2;        // 32 KB
constexpr int GT_STAGE_BYTES = GT_A_BYTES + GT_B_BYTES;
constexpr int GT_THREADS = 192;
constexpr int GT_SMEM = 1024 + GT_STAGES * GT_STAGE_BYTES + 256;
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

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kblocks = (p.K + GT_BK - 1) / GT_BK;

  if (tid == 0) {
    for (int s = 0; s < GT_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    s_failed = 0;
    fence_barrier_init();
  }
  if (warp == 5) tmem_alloc(&s_tmem, GT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_a);
      prefetch_tensormap(&tmap_b);
      long long it = 0;
      for (long long tile = blockIdx.x; tile < p.num_tiles && !*(volatile unsigned*)&s_failed; tile += gridDim.x) {
        const int b = (int)(tile / ((long long)p.tiles_m * p.tiles_n));
        const int rem = (int)(tile % ((long long)p.tiles_m * p.tiles_n));
        const int m0 = (rem % p.tiles_m) * GT_BM, n0 = (rem / p.tiles_m) * GT_BN;
        for (int kb = 0; kb < kblocks; kb++, it++) {
          const int s = (int)(it % GT_STAGES);
          if (it >= GT_STAGES && !mbar_wait(&empty[s], (uint32_t)((it / GT_STAGES - 1) & 1))) { gt_fail(p, &s_failed, 1, (unsigned)it); break; }
          uint8_t* sa = base + s * GT_STAGE_BYTES;
          uint8_t* sb = sa + GT_A_BYTES;
          mbar_expect_tx(&full[s], GT_STAGE_BYTES);
          tma_load_3d(sa, &tmap_a, kb * GT_BK, m0, b, &full[s]);
          if (p.rhs_transposed) {
            tma_load_3d(sb, &tmap_b, kb * GT_BK, n0, b, &full[s]);                 // [256 n rows][64 k]
          } else {
#pragma unroll
            for (int j = 0; j < GT_BN / 64; j++)                                      // 4 x [64 k rows][64 n]
              tma_load_3d(sb + j * (GT_BK * 128), &tmap_b, n0 + 64 * j, kb * GT_BK, b, &full[s]);
          }
        }
      }
    }
  } else if (warp == 5) {
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
        for (int kb = 0; kb < kblocks; kb++, it++) {
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
    // ------------------------------ epilogue (warps 0-3) ----------------------
    long long local = 0;
    bool failed = false;
    OT* out = reinterpret_cast<OT*>(p.out);
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, local++) {
      const int buf = (int)(local & 1);
      const int b = (int)(tile / ((long long)p.tiles_m * p.tiles_n));
      const int rem = (int)(tile % ((long long)p.tiles_m * p.tiles_n));
      const int m0 = (rem % p.tiles_m) * GT_BM, n0 = (rem / p.tiles_m) * GT_BN;
      if (!failed && !mbar_wait(&acc_full[buf], (uint32_t)((local / 2) & 1))) { failed = true; gt_fail(p, &s_failed, 4, (unsigned)local); }
      if (failed || *(volatile unsigned*)&s_failed) break;
      tc_fence_after();
      const int row = m0 + warp * 32 + lane;
      OT* orow = out + ((size_t)b * p.M + (size_t)min(row, p.M - 1)) * p.N;
#pragma unroll 1
      for (int c = 0; c < GT_BN / 32; c++) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * GT_BN + c * 32), r);
        tmem_ld_wait();
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  // every role ends here; TMEM is released by the warp that allocated it
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, GT_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// planning and launch
// ---------------------------------------------------------------------------
bool dot_tc_supports(const cb_dot_desc& d, std::string* why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  const int od = d.out_dtype ? d.out_dtype : d.in_dtype;
  if (d.in_dtype != CB_BF16 && d.in_dtype != CB_F16) return no("inputs must be bfloat16 or float16");
  if (od != d.in_dtype && od != CB_F32) return no("output must be the input dtype or float32");
  if (d.B < 1 || d.M < 1 || d.N < 1 || d.K < 1) return no("empty operand");
  if (d.K % 8 != 0) return no("K must be a multiple of 8 (16-byte rows for TMA)");
  if (d.N % 8 != 0) return no("N must be a multiple of 8");
  if (d.M > (1 << 30) || d.N > (1 << 30) || d.K > (1 << 30) || d.B > (1 << 20)) return no("dimension too large");
  // small problems are launch bound: unless asked for explicitly, the generic kernel serves them
  if (d.variant != CB_DOT_TCGEN05 && (double)d.B * d.M * d.N * d.K < 128.0 * 256 * 256)
    return no("problem too small for the tensor-core tile");
  return true;
}

int dot_tc_plan(cb_plan* p) {
  const cb_dot_desc& d = p->dot;
  const long long tiles = (long long)d.B * ((d.M + GT_BM - 1) / GT_BM) * ((d.N + GT_BN - 1) / GT_BN);
  p->blocks = (int)std::min<long long>(tiles, p->n_sm);
  p->threads = GT_THREADS;
  p->dyn_smem = GT_SMEM;
  p->counter_bytes = 64;
  p->workspace_bytes = 64;
  p->has_status = true;
  const int od = d.out_dtype ? d.out_dtype : d.in_dtype;
  p->name = std::string("gemm_tcgen05_") + dtype_name(d.in_dtype) + "_" + dtype_name(od) + (d.rhs_transposed ? "_nt" : "_nn");
  return CB_OK;
}

static int encode_3d(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1) {
  encode_tiled_fn enc = tensor_map_encoder();
  if (!enc) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(CB_ERR_INVALID_ARG, "DotGeneral tcgen05 kernel: operands must be 16-byte aligned");
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
static int launch_t(const cb_plan* p, const CUtensorMap& ta, const CUtensorMap& tb, const GtParams& prm, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  if (p->dev >= 64 || !configured[p->dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM));
    if (p->dev < 64) configured[p->dev].store(true, std::memory_order_release);
  }
  gemm_tcgen05_kernel<OT><<<p->blocks, GT_THREADS, GT_SMEM, s>>>(ta, tb, prm);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

int dot_tc_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_dot_desc& d = p->dot;
  CUtensorMap ta, tb;
  CB_TRY(encode_3d(&ta, in[0], (uint64_t)d.K, (uint64_t)d.M, (uint64_t)d.B, GT_BK, GT_BM));
  if (d.rhs_transposed) CB_TRY(encode_3d(&tb, in[1], (uint64_t)d.K, (uint64_t)d.N, (uint64_t)d.B, GT_BK, GT_BN));
  else CB_TRY(encode_3d(&tb, in[1], (uint64_t)d.N, (uint64_t)d.K, (uint64_t)d.B, 64, GT_BK));
  GtParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.out = out[0];
  prm.status = (unsigned*)ws;
  prm.M = (int)d.M; prm.N = (int)d.N; prm.K = (int)d.K; prm.B = (int)d.B;
  prm.tiles_m = (int)((d.M + GT_BM - 1) / GT_BM);
  prm.tiles_n = (int)((d.N + GT_BN - 1) / GT_BN);
  prm.num_tiles = (long long)d.B * prm.tiles_m * prm.tiles_n;
  prm.out_dtype = d.out_dtype ? d.out_dtype : d.in_dtype;
  prm.rhs_transposed = d.rhs_transposed;
  prm.ab_format = d.in_dtype == CB_BF16 ? 1 : 0;
  if (reinterpret_cast<uintptr_t>(out[0]) & 15) return fail(CB_ERR_INVALID_ARG, "DotGeneral tcgen05 kernel: output must be 16-byte aligned");
  switch (prm.out_dtype) {
    case CB_F32: return launch_t<float>(p, ta, tb, prm, s);
    case CB_BF16: return launch_t<__nv_bfloat16>(p, ta, tb, prm, s);
    case CB_F16: return launch_t<__half>(p, ta, tb, prm, s);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral tcgen05 kernel: output dtype %s", dtype_name(prm.out_dtype));
  }
}

}  // namespace cb
