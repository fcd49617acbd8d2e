// FusedScaledDotProductAttention, flash-style on the 5th-generation tensor cores:
// bf16 / f16, head_dim 128, causal or full, GQA, BHSD and BSHD, no mask / bias / sequence
// lengths (those go to the generic kernel).  Softmax is online, in f32, over the
// reference's definition (internal/gobackend/fusedops/sdpa.go:373-519): row max, exp,
// sum, normalise, P.V — evaluated blockwise, so the [S, Skv] scores never exist in memory.
//
// One CTA owns two 128-row query tiles — consecutive rows of one (batch, query head), or for causal
// attention with an even GQA group the same rows of two heads of one KV group — and walks the key/value
// blocks of 128 rows:
//   warp 8      TMA producer: Q once, K and V blocks into two-stage rings (128B swizzle)
//   warp 9      MMA issuer:  S_t = Q_t K^T (tcgen05.mma, smem x smem -> TMEM) and
//               O_t += P_t V (P_t read from TMEM, V from smem as the MN-major operand)
//   warps 0-3 / 4-7  softmax of tile 0 / tile 1: tcgen05.ld of S, scale, causal mask,
//               running max and sum, exp2, P written back over S as packed 16-bit, announced to the MMA
//               warp in chunks of 32 keys so that P.V starts while the later chunks are still computed
// The two tiles alternate on the tensor core, so one tile's softmax overlaps the other's
// matrix products.  O stays in TMEM and is rescaled only when a row maximum grows by more
// than 2^8 (the stale maximum is used consistently for P and the row sum, so the result is
// exact up to rounding).  Every wait is bounded; TMEM is always released.
#include "tc_common.cuh"

#include <atomic>
#include <math.h>
#include <string.h>

namespace cb {

using namespace tc;

constexpr int FA_BM = 128, FA_BN = 128, FA_D = 128;
constexpr int FA_TILE_BYTES = 128 * FA_D * 2;      // 32 KB: two 64-column halves of 16 KB
constexpr int FA_HALF_BYTES = 128 * 128;           // 16 KB
constexpr int FA_THREADS = 320;
constexpr int FA_SMEM = 1024 + 6 * FA_TILE_BYTES + 256;   // Q0 Q1 K0 K1 V0 V1
constexpr int FA_TMEM_COLS = 512;                  // S0 S1 O0 O1, 128 columns each
constexpr float FA_RESCALE_THRESHOLD = 8.0f;       // log2 units

struct FaParams {
  void* out;
  unsigned* status;
  int B, Hq, Hkv, S, Skv;
  int bshd, causal, ab_format;
  float scale_log2;        // scale * log2(e)
  int q_pairs;             // ceil(S / 256)
  int pair_heads;          // causal with an even GQA group: a CTA's two tiles are the same rows of two neighbouring heads
  // QuerySeqLen / KeyValueSeqLen [B] int32, or null: keys from kv_lens[b] on are not attended (their blocks are not even
  // loaded), query positions from q_lens[b] on give zero rows (sdpa.go:389-411)
  const int* q_lens;
  const int* kv_lens;
};

__device__ __forceinline__ void fa_fail(const FaParams& p, unsigned* s_failed, unsigned code, unsigned detail) {
  atomicExch(&p.status[0], code);
  atomicExch(&p.status[1], detail);
  atomicExch(s_failed, 1u);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The same, kept in program order against the tensor-memory stores and barrier arrivals around it (the compiler may
// otherwise hoist all of a block's exponentials above the first store, which would announce every chunk at the end).
__device__ __forceinline__ float fast_exp2_ordered(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Blackwell's packed-pair f32 arithmetic and three-input max/min: the softmax warps are bound by
// instruction issue, so scaling, the running sum and the row extreme take half the instructions.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (d0, d1) = (a0, a1) * s + m
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float s, float m) {
  asm("{\n\t.reg .b64 ra, rs, rm, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rs, {%4, %4};\n\tmov.b64 rm, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rs, rm;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(s), "f"(m));
}
// (d0, d1) += (a0, a1)
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\tadd.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
// two f32 -> packed bf16x2 (format 1) or f16x2 (format 0), round to nearest even
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi, int ab_format) {
  if (ab_format == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// the same with the format known at compile time (the hot loop of the softmax)
template <typename OT> __device__ __forceinline__ uint32_t pack16x2_t(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack16x2_t<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack16x2_t<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// one [128 rows x 128 columns] tile = two TMA boxes of 64 columns
__device__ __forceinline__ void fa_load_tile(uint8_t* dst, const CUtensorMap* map, int bshd, int row0, int head, int b, uint64_t* bar) {
#pragma unroll
  for (int h = 0; h < 2; h++) {
    if (bshd) tma_load_4d(dst + h * FA_HALF_BYTES, map, 64 * h, head, row0, b, bar);
    else tma_load_4d(dst + h * FA_HALF_BYTES, map, 64 * h, row0, head, b, bar);
  }
}

template <typename OT>
__global__ void __launch_bounds__(FA_THREADS, 1)
sdpa_flash_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const FaParams p) {
  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = base;                              // [2 tiles]
  uint8_t* sK = base + 2 * FA_TILE_BYTES;          // [2 stages]
  uint8_t* sV = base + 4 * FA_TILE_BYTES;          // [2 stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + 6 * FA_TILE_BYTES);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2] per tile: scores ready
  uint64_t* o_done = bars + 11;       // [2] per tile: P.V of a block finished
  uint64_t* p_chunk = bars + 13;      // [2][4] per tile and 32-key chunk of a block: probabilities written
  __shared__ uint32_t s_tmem;
  __shared__ unsigned s_failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Heaviest (late, causal) query tiles first over the whole grid: the last wave then holds only the
  // lightest tiles.  Heads vary fastest, so the query heads of one KV group run side by side.
  // A CTA's two tiles are either two consecutive 128-row tiles of one head, or (causal, even GQA group) the same
  // 128 rows of two neighbouring heads of one KV group: those walk exactly the same key/value blocks, so
  // the two tiles alternate on the tensor core to the last block instead of one of them finishing early.
  int th[2], tq0[2], b;
  if (p.pair_heads) {
    const int n_qt = (p.S + FA_BM - 1) / FA_BM, n_bhp = p.B * (p.Hq / 2);
    const int qi = n_qt - 1 - (int)(blockIdx.x / n_bhp);
    const int bhp = (int)(blockIdx.x % n_bhp);
    b = bhp / (p.Hq / 2);
    th[0] = 2 * (bhp % (p.Hq / 2)); th[1] = th[0] + 1;
    tq0[0] = tq0[1] = qi * FA_BM;
  } else {
    const int n_bh = p.B * p.Hq;
    const int pair = p.q_pairs - 1 - (int)(blockIdx.x / n_bh);
    const int bh = (int)(blockIdx.x % n_bh);
    b = bh / p.Hq;
    th[0] = th[1] = bh % p.Hq;
    tq0[0] = pair * 2 * FA_BM; tq0[1] = tq0[0] + FA_BM;
  }
  const int hk = th[0] / (p.Hq / p.Hkv);
  const int kvl = p.kv_lens ? max(0, min(p.Skv, __ldg(p.kv_lens + b))) : p.Skv;      // keys this sequence attends to
  const int nb_all = (kvl + FA_BN - 1) / FA_BN;
  int nb[2];
#pragma unroll
  for (int t = 0; t < 2; t++) {
    const int qt = tq0[t];
    int n = nb_all;
    if (p.causal) n = min(n, (min(qt + FA_BM, p.S) + FA_BN - 1) / FA_BN);   // blocks with kv <= last row of the tile
    if (qt >= p.S) n = 0;
    nb[t] = n;
  }
  const int nb_max = max(nb[0], nb[1]);

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&o_done[s], 1);
      for (int c = 0; c < 4; c++) mbar_init(&p_chunk[s * 4 + c], 4);
    }
    s_failed = 0;
    fence_barrier_init();
  }
  if (warp == 9) tmem_alloc(&s_tmem, FA_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      mbar_expect_tx(q_full, 2 * FA_TILE_BYTES);
      fa_load_tile(sQ, &tm_q, p.bshd, tq0[0], th[0], b, q_full);
      fa_load_tile(sQ + FA_TILE_BYTES, &tm_q, p.bshd, tq0[1], th[1], b, q_full);
      for (int j = 0; j < nb_max; j++) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(&k_empty[s], (uint32_t)((j / 2 - 1) & 1))) { fa_fail(p, &s_failed, 1, (unsigned)j); break; }
        mbar_expect_tx(&k_full[s], FA_TILE_BYTES);
        fa_load_tile(sK + s * FA_TILE_BYTES, &tm_k, p.bshd, j * FA_BN, hk, b, &k_full[s]);
        if (j >= 2 && !mbar_wait(&v_empty[s], (uint32_t)((j / 2 - 1) & 1))) { fa_fail(p, &s_failed, 2, (unsigned)j); break; }
        mbar_expect_tx(&v_full[s], FA_TILE_BYTES);
        fa_load_tile(sV + s * FA_TILE_BYTES, &tm_v, p.bshd, j * FA_BN, hk, b, &v_full[s]);
        if (*(volatile unsigned*)&s_failed) break;
      }
      // a sequence without keys: nobody else waits for the query tiles, so they are waited for here before the CTA ends
      if (nb_max == 0) mbar_wait(q_full, 0);
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && nb_max > 0) {
      const uint32_t idesc_qk = idesc_f16(FA_BM, FA_BN, p.ab_format, 0, 0);   // A, B K-major
      const uint32_t idesc_pv = idesc_f16(FA_BM, FA_D, p.ab_format, 0, 1);    // B (V) MN-major
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) fa_fail(p, &s_failed, 3, 0);
      // Descriptors of the three tile kinds, built once: the address field sits in the low word in 16-byte units, so a
      // tile, a stage or a k step is an add to the low word (shared-memory addresses stay below 2^18: no carry).
      const uint64_t dq = smem_desc_sw128(q_addr, 16, 1024), dk = smem_desc_sw128(k_addr, 16, 1024);
      const uint64_t dv = smem_desc_sw128(v_addr, FA_HALF_BYTES, 1024);
      const uint32_t q_lo = (uint32_t)dq, q_hi = (uint32_t)(dq >> 32), k_lo = (uint32_t)dk, k_hi = (uint32_t)(dk >> 32);
      const uint32_t v_lo = (uint32_t)dv, v_hi = (uint32_t)(dv >> 32);
      auto issue_qk = [&](int t, int s) {   // S_t = Q_t K_s^T
        const uint32_t d = tmem_base + (uint32_t)(t * 128);
        const uint32_t a_lo = q_lo + (uint32_t)t * (FA_TILE_BYTES >> 4), b_lo = k_lo + (uint32_t)s * (FA_TILE_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < FA_D / 16; kk++) {
          const uint32_t off = (uint32_t)(((kk >> 2) * FA_HALF_BYTES + (kk & 3) * 32) >> 4);
          umma_f16_lh(d, a_lo + off, q_hi, b_lo + off, k_hi, idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      // O_t (+)= P_t V_s, the 32 keys of chunk c: issued as soon as the softmax warps have written that chunk, so the
      // tensor core works on the first chunks while the last ones are still being exponentiated
      auto issue_pv_chunk = [&](int t, int s, int c, bool accumulate) {
        const uint32_t d = tmem_base + (uint32_t)(256 + t * 128);
        const uint32_t a = tmem_base + (uint32_t)(t * 128);
        const uint32_t b_lo = v_lo + (uint32_t)s * (FA_TILE_BYTES >> 4);
#pragma unroll
        for (int kk = 2 * c; kk < 2 * c + 2; kk++)
          umma_f16_ts_lh(d, a + (uint32_t)(kk * 8), b_lo + (uint32_t)((kk * 16 * 128) >> 4), v_hi, idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
        if (c == 3) umma_commit(&o_done[t]);
      };
      if (ok) {
        // block 0 scores
        ok = mbar_wait(&k_full[0], 0);
        if (!ok) fa_fail(p, &s_failed, 4, 0);
        if (ok) {
          tc_fence_after();
          for (int t = 0; t < 2; t++) if (nb[t] > 0) issue_qk(t, 0);
          umma_commit(&k_empty[0]);
        }
      }
      for (int j = 0; j < nb_max && ok; j++) {
        const int s = j & 1, sn = (j + 1) & 1;
        bool k_next_ready = false;
        for (int t = 0; t < 2 && ok; t++) {
          if (j < nb[t]) {
            for (int c = 0; c < 4 && ok; c++) {
              if (!mbar_wait(&p_chunk[t * 4 + c], (uint32_t)(j & 1))) { fa_fail(p, &s_failed, 5, (unsigned)(j * 2 + t)); ok = false; break; }
              if (c == 0 && (t == 0 || j >= nb[0])) {
                if (!mbar_wait(&v_full[s], (uint32_t)((j / 2) & 1))) { fa_fail(p, &s_failed, 6, (unsigned)j); ok = false; break; }
              }
              tc_fence_after();
              issue_pv_chunk(t, s, c, j > 0);
            }
            if (!ok) break;
          }
          if (j + 1 < nb[t]) {
            if (!k_next_ready) {
              if (!mbar_wait(&k_full[sn], (uint32_t)(((j + 1) / 2) & 1))) { fa_fail(p, &s_failed, 7, (unsigned)j); ok = false; break; }
              k_next_ready = true;
              tc_fence_after();
            }
            issue_qk(t, sn);
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[s]);
        if (k_next_ready) umma_commit(&k_empty[sn]);
      }
    }
  } else {
    // ------------------------------ softmax warpgroups ------------------------
    const int t = warp >> 2;                 // tile of this warpgroup
    const int wq = warp & 3;                 // TMEM lane quarter of this warp
    const int row = tq0[t] + wq * 32 + lane;
    const int h = th[t];
    const uint32_t lane_base = tmem_base + ((uint32_t)(wq * 32) << 16);
    const uint32_t s_addr = lane_base + (uint32_t)(t * 128);
    const uint32_t o_addr = lane_base + (uint32_t)(256 + t * 128);
    float m_used = -INFINITY, l = 0.0f;
    bool failed = false;
    const bool pos_scale = p.scale_log2 >= 0.0f;
    // a masked score: the value that scales to -inf-like (never the row extreme, exp2 gives 0)
    const uint32_t neg_biggest = __float_as_uint(pos_scale ? -INFINITY : INFINITY);
    for (int j = 0; j < nb[t]; j++) {
      if (!mbar_wait(&s_full[t], (uint32_t)(j & 1))) { failed = true; fa_fail(p, &s_failed, 8, (unsigned)(j * 2 + t)); break; }
      if (*(volatile unsigned*)&s_failed) { failed = true; break; }
      tc_fence_after();
      const int kv0 = j * FA_BN;
      const bool need_mask = (p.causal && kv0 + FA_BN - 1 > row) || (kv0 + FA_BN > kvl);
      const int kv_limit = p.causal ? min(kvl, row + 1) : kvl;       // first masked kv index
      // the whole score row of this block lives in registers: one TMEM read, one pass for the
      // maximum, one for the probabilities
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; c++) tmem_ld32(s_addr + (uint32_t)(c * 32), sr[c]);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
          for (int i = 0; i < 32; i++)
            if (kv0 + c * 32 + i >= kv_limit) sr[c][i] = neg_biggest;   // -inf after scaling either way
      }
      // max of scale*s = scale*max(s) for a positive scale, scale*min(s) for a negative one
      // (the sign of the scale is decided once per block, not per element; two partial extremes
      // keep the dependency chains short)
      float ea = __uint_as_float(sr[0][0]), eb = __uint_as_float(sr[2][0]);
      if (pos_scale) {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          ea = max3(ea, __uint_as_float(sr[i >> 5][i & 31]), __uint_as_float(sr[i >> 5][(i & 31) + 1]));
          eb = max3(eb, __uint_as_float(sr[2 + (i >> 5)][i & 31]), __uint_as_float(sr[2 + (i >> 5)][(i & 31) + 1]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          ea = min3(ea, __uint_as_float(sr[i >> 5][i & 31]), __uint_as_float(sr[i >> 5][(i & 31) + 1]));
          eb = min3(eb, __uint_as_float(sr[2 + (i >> 5)][i & 31]), __uint_as_float(sr[2 + (i >> 5)][(i & 31) + 1]));
        }
      }
      const float ext = pos_scale ? fmaxf(ea, eb) : fminf(ea, eb);
      const float m_blk = ext * p.scale_log2;
      float m_new = fmaxf(m_used, m_blk);
      if (m_new == -INFINITY) m_new = 0.0f;          // nothing attendable so far
      const bool first = (j == 0);
      const bool grow = !first && (m_new > m_used + FA_RESCALE_THRESHOLD);
      if (first) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        // rescale the running output and sum to the new maximum (whole warp: TMEM access is collective)
        const float alpha = fast_exp2(m_used - m_new);
        l *= alpha;
        m_used = m_new;
#pragma unroll 1
        for (int c = 0; c < 4; c++) {
          uint32_t r[32];
          tmem_ld32(o_addr + (uint32_t)(c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(o_addr + (uint32_t)(c * 32), r);
        }
        tmem_st_wait();
      }
      // probabilities, row sum, P over S as packed 16-bit pairs
      // A chunk of 32 keys is announced one chunk late: its store has had the arithmetic of the next chunk to complete,
      // so the wait for it costs nothing, and the P.V products of the early chunks overlap the rest of this loop.
      float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a0, a1;
          fma2(a0, a1, __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]), p.scale_log2, -m_used);
          const float p0 = fast_exp2_ordered(a0), p1 = fast_exp2_ordered(a1);
          add2(l0, l1, p0, p1);
          pk[i >> 1] = pack16x2_t<OT>(p0, p1);      // P has the dtype of the inputs, which is the output's
        }
        if (c > 0) {
          tmem_st_wait();                            // the store of chunk c - 1
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_chunk[t * 4 + c - 1]);
        }
        tmem_st16(s_addr + (uint32_t)(c * 16), pk);
      }
      l += l0 + l1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_chunk[t * 4 + 3]);
    }
    // epilogue: O / l
    if (!failed && nb[t] > 0) {
      if (!mbar_wait(&o_done[t], (uint32_t)((nb[t] - 1) & 1))) { failed = true; fa_fail(p, &s_failed, 9, (unsigned)t); }
    }
    if (!failed && nb[t] > 0 && !*(volatile unsigned*)&s_failed) {
      tc_fence_after();
      const int ql = p.q_lens ? __ldg(p.q_lens + b) : p.S;           // query positions that are not padding
      const float inv = (l != 0.0f && row < ql) ? 1.0f / l : 0.0f;    // nothing attended, or a padded query position: zeros
      OT* out = reinterpret_cast<OT*>(p.out);
      const int rr = min(row, p.S - 1);
      OT* orow = p.bshd ? out + (((size_t)b * p.S + rr) * p.Hq + h) * FA_D : out + (((size_t)b * p.Hq + h) * p.S + rr) * FA_D;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t r[32];
        tmem_ld32(o_addr + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const float a0 = __uint_as_float(r[8 * q + 2 * i]) * inv, a1 = __uint_as_float(r[8 * q + 2 * i + 1]) * inv;
              w[i] = pack16x2(a0, a1, p.ab_format);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    // a tile of a sequence without keys: its rows are zeros (sdpa.go:471-474)
    if (nb[t] == 0 && row < p.S) {
      OT* out = reinterpret_cast<OT*>(p.out);
      OT* orow = p.bshd ? out + (((size_t)b * p.S + row) * p.Hq + h) * FA_D : out + (((size_t)b * p.Hq + h) * p.S + row) * FA_D;
#pragma unroll
      for (int c = 0; c < FA_D / 8; c++) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// planning and launch
// ---------------------------------------------------------------------------
bool sdpa_flash_supports(const cb_sdpa_desc& d, std::string* why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  if (d.dtype != CB_BF16 && d.dtype != CB_F16) return no("dtype must be bfloat16 or float16");
  if (d.D != FA_D) return no("head_dim must be 128");
  if (d.mask_kind != CB_MASK_NONE || d.bias_rank > 0) return no("mask and bias tensors use the generic kernel");
  if (d.B < 1 || d.S < 1 || d.Skv < 1) return no("empty operand");
  if (d.S < 128 || d.Skv < 128) return no("sequence too short for the tensor-core tile");
  if (d.S > (1 << 24) || d.Skv > (1 << 24) || d.B * d.Hq * ((d.S + 255) / 256) > 0x7fffffffLL) return no("dimension too large");
  return true;
}

int sdpa_flash_plan(cb_plan* p) {
  const cb_sdpa_desc& d = p->sdpa;
  const bool pair_heads = d.causal && d.Hkv > 0 && (d.Hq / d.Hkv) % 2 == 0;
  p->blocks = pair_heads ? (int)(d.B * (d.Hq / 2) * ((d.S + FA_BM - 1) / FA_BM)) : (int)(d.B * d.Hq * ((d.S + 255) / 256));
  p->threads = FA_THREADS;
  p->dyn_smem = FA_SMEM;
  p->counter_bytes = 64;
  p->workspace_bytes = 64;
  p->has_status = true;
  p->name = std::string("sdpa_flash_") + dtype_name(d.dtype) + (d.causal ? "_causal" : "_full") + (d.layout == CB_LAYOUT_BSHD ? "_bshd" : "_bhsd");
  return CB_OK;
}

// [B,H,S,D] (BHSD) or [B,S,H,D] (BSHD) as a 4-D tensor map with boxes of 128 rows x 64 columns
static int encode_qkv(CUtensorMap* m, const void* ptr, int bshd, int64_t B, int64_t H, int64_t S) {
  encode_tiled_fn enc = tensor_map_encoder();
  if (!enc) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(CB_ERR_INVALID_ARG, "flash attention: operands must be 16-byte aligned");
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  dims[0] = FA_D;
  if (bshd) { dims[1] = (cuuint64_t)H; dims[2] = (cuuint64_t)S; box[1] = 1; box[2] = 128; }
  else { dims[1] = (cuuint64_t)S; dims[2] = (cuuint64_t)H; box[1] = 128; box[2] = 1; }
  dims[3] = (cuuint64_t)B;
  box[0] = 64; box[3] = 1;
  strides[0] = FA_D * 2;
  strides[1] = strides[0] * dims[1];
  strides[2] = strides[1] * dims[2];
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return CB_OK;
}

template <typename OT>
static int launch_t(const cb_plan* p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& prm, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  if (p->dev >= 64 || !configured[p->dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(sdpa_flash_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
    if (p->dev < 64) configured[p->dev].store(true, std::memory_order_release);
  }
  sdpa_flash_kernel<OT><<<p->blocks, FA_THREADS, FA_SMEM, s>>>(tq, tk, tv, prm);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

int sdpa_flash_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_sdpa_desc& d = p->sdpa;
  const int bshd = d.layout == CB_LAYOUT_BSHD ? 1 : 0;
  CUtensorMap tq, tk, tv;
  CB_TRY(encode_qkv(&tq, in[0], bshd, d.B, d.Hq, d.S));
  CB_TRY(encode_qkv(&tk, in[1], bshd, d.B, d.Hkv, d.Skv));
  CB_TRY(encode_qkv(&tv, in[2], bshd, d.B, d.Hkv, d.Skv));
  if (reinterpret_cast<uintptr_t>(out[0]) & 15) return fail(CB_ERR_INVALID_ARG, "flash attention: output must be 16-byte aligned");
  FaParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.out = out[0];
  prm.status = (unsigned*)ws;
  prm.B = (int)d.B; prm.Hq = (int)d.Hq; prm.Hkv = (int)d.Hkv; prm.S = (int)d.S; prm.Skv = (int)d.Skv;
  prm.bshd = bshd;
  prm.causal = d.causal;
  prm.ab_format = d.dtype == CB_BF16 ? 1 : 0;
  const double scale = d.scale != 0.0 ? d.scale : 1.0 / sqrt((double)d.D);
  prm.scale_log2 = (float)(scale * 1.4426950408889634);
  prm.q_pairs = (int)((d.S + 255) / 256);
  prm.pair_heads = (d.causal && d.Hkv > 0 && (d.Hq / d.Hkv) % 2 == 0) ? 1 : 0;
  prm.q_lens = d.has_seq_lens ? (const int*)in[3] : nullptr;          // inputs: q, k, v, QuerySeqLen, KeyValueSeqLen
  prm.kv_lens = d.has_seq_lens ? (const int*)in[4] : nullptr;
  return d.dtype == CB_BF16 ? launch_t<__nv_bfloat16>(p, tq, tk, tv, prm, s) : launch_t<__half>(p, tq, tk, tv, prm, s);
}

}  // namespace cb
