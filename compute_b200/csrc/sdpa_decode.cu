// FusedScaledDotProductAttention for decode shapes: a few query tokens per sequence (S * group <= 16 query
// rows per KV head) against a long key / value cache, head_dim 128 or 64, bfloat16 / float16, no mask or bias
// tensors, no sequence lengths.  Reference arithmetic: internal/gobackend/fusedops/sdpa.go:373-636 (scores =
// q.k * scale, row max, exp, sum, P.V; a causal row q sees the keys 0..q); here the softmax is the streaming
// (running max) form in float32, the probabilities are rounded to the operand type for the second product (as
// in the prefill kernel) and the result is rounded once.
//
// The op is bound by reading K and V once: 2 * B * Hkv * Skv * D elements.  The keys of every (batch, KV head)
// pair are split into `splits` ranges, one CTA each; all query heads of the KV head's group ride along as the
// rows of one 16-row tile (the cache is read once per group, not once per query head).  Every warp of a CTA
// streams its own 16-key steps through a private ring of shared-memory stages filled by cp.async (16-byte,
// coalesced, XOR-swizzled so that the fragment reads below are conflict-free), forms Q.K^T and P.V with
// mma.sync m16n8k16 — the tile is far too short for the 128-row tcgen05 shapes — and keeps (max, sum,
// accumulator) per query row in registers.  The warps of a CTA merge through shared memory, the splits
// through a float32 workspace and a second, small kernel.
#include "common.cuh"

#include <algorithm>
#include <atomic>

namespace cb {

constexpr int SD_THREADS = 128;
constexpr int SD_WARPS = SD_THREADS / 32;
constexpr int SD_MAX_ROWS = 16;         // query rows per KV head: one m16 tile
constexpr int SD_STEP = 16;             // keys per warp step (one k16 of the second product)
constexpr int SD_STAGES = 3;            // shared-memory stages per warp: one in use, two in flight

struct SdParams {
  int B, Hq, Hkv, S, Skv, D, group, rows, splits, keys_per_split;
  long long q_b, q_h, q_s, kv_b, kv_h, kv_s;     // element strides (both layouts)
  float scale_log2;                               // scale * log2(e): scores live in the exp2 domain
  int causal;
  float* part_o;        // [B, Hkv, splits, rows, D]
  float* part_ml;       // [B, Hkv, splits, rows, 2]  (max, sum)
  // QuerySeqLen / KeyValueSeqLen [B] int32, or null: keys from kv_lens[b] on are not attended, query positions from
  // q_lens[b] on give zero rows (sdpa.go:389-411)
  const int* q_lens;
  const int* kv_lens;
};

template <typename T> __device__ __forceinline__ void sd_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void sd_mma<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void sd_mma<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t sd_pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t sd_pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t sd_pack2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// 16-byte chunk c of stage row `row` lives at chunk c ^ sd_swz(row) (within each group of 8 chunks): the K fragment
// reads (rows g, g+1; chunks 4*slab + t) and the V fragment reads (rows 2t [+1, +8, +9]; chunks g [+8]) of any
// 8 consecutive lanes then fall into 8 different 16-byte bank groups.
__device__ __forceinline__ int sd_swz(int row) { return ((row & 1) << 2) ^ (row & 6); }

__device__ __forceinline__ void sd_cp16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;      // zero-fills when the key is outside the range
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(n) : "memory");
}

// One CTA = one (split, KV head, batch); one warp = every fourth 16-key step of the split.
// Fragment roles (g = lane / 4, t = lane % 4), with the k indices of the products permuted freely since a dot
// product does not care about the order of its terms:
//   Q.K^T  A = Q: rows g (and g + 8), the 8 head dimensions 32*slab + 8t.. of every slab, straight from global
//          memory; B = K^T: column g of key tile nt is key 8nt + g, the same 8 dimensions — one 16-byte read per
//          slab feeds two mma (dimensions +0..3, +4..7).
//   P.V    A = P: the score fragments of key tiles 0 and 1, exponentiated and packed, are already in A layout;
//          B = V: lane (g, t) reads dimensions 8g.. (and 64 + 8g..) of keys 2t, 2t+1, 8+2t, 9+2t and pairs them
//          by byte permutes; output tile i column c is head dimension 64h + 8c + i.
template <typename T, int D, bool HI>
__global__ void __launch_bounds__(SD_THREADS, 2)
sdpa_decode_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const SdParams p) {
  pdl_enter();
  constexpr int CH = D / 8;                       // 16-byte chunks per row
  constexpr int ROWB = D * 2;                     // bytes per row
  constexpr int STAGE = 2 * SD_STEP * ROWB;       // K rows, then V rows
  constexpr int SL = D / 32;                      // 32-dimension slabs of the first product
  constexpr int NT = D / 8;                       // output tiles of the second product
  extern __shared__ __align__(128) unsigned char sd_smem[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(sd_smem) + warp * SD_STAGES * STAGE;

  const int key0 = split * p.keys_per_split;
  const int kv_limit = p.kv_lens ? min(p.Skv, __ldg(p.kv_lens + b)) : p.Skv;
  const int key1 = min(kv_limit, key0 + p.keys_per_split);
  const T* kb = k + (long long)b * p.kv_b + (long long)kvh * p.kv_h;
  const T* vb = v + (long long)b * p.kv_b + (long long)kvh * p.kv_h;
  const int n_steps = key1 > key0 + warp * SD_STEP ? (key1 - key0 - warp * SD_STEP + SD_WARPS * SD_STEP - 1) / (SD_WARPS * SD_STEP) : 0;

  auto fill = [&](int step) {           // this warp's step -> stage step % SD_STAGES; one commit group per call
    if (step < n_steps) {
      const int jw = key0 + (step * SD_WARPS + warp) * SD_STEP;
      const uint32_t st = ring + (step % SD_STAGES) * STAGE;
#pragma unroll
      for (int it = 0; it < SD_STEP * CH / 32; it++) {
        const int id = it * 32 + lane, row = id / CH, c = id % CH;
        const int key = jw + row;
        const bool valid = key < key1;
        const long long off = (long long)min(key, key1 - 1) * p.kv_s + c * 8;
        const uint32_t dst = st + row * ROWB + ((c ^ sd_swz(row)) << 4);
        sd_cp16(dst, kb + off, valid);
        sd_cp16(dst + SD_STEP * ROWB, vb + off, valid);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int s = 0; s < SD_STAGES - 1; s++) fill(s);

  // query fragments; rows past p.rows are zero
  uint4 qlo[SL], qhi[SL];
  {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const T* ql = nullptr; const T* qh = nullptr;
    if (g < p.rows) { const int hg = g / p.S, s = g - hg * p.S; ql = q + (long long)b * p.q_b + (long long)(kvh * p.group + hg) * p.q_h + (long long)s * p.q_s; }
    if (HI && g + 8 < p.rows) { const int hg = (g + 8) / p.S, s = g + 8 - hg * p.S; qh = q + (long long)b * p.q_b + (long long)(kvh * p.group + hg) * p.q_h + (long long)s * p.q_s; }
#pragma unroll
    for (int sl = 0; sl < SL; sl++) {
      qlo[sl] = ql ? __ldg(reinterpret_cast<const uint4*>(ql + 32 * sl + 8 * t)) : zero;
      qhi[sl] = qh ? __ldg(reinterpret_cast<const uint4*>(qh + 32 * sl + 8 * t)) : zero;
    }
  }
  // a causal row sees the keys 0..(its query position)
  const int spos_lo = p.causal ? (g % p.S) : 0x7FFFFFFF;
  const int spos_hi = p.causal ? ((g + 8) % p.S) : 0x7FFFFFFF;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
  float oacc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f; }

  for (int step = 0; step < n_steps; step++) {
    asm volatile("cp.async.wait_group %0;" :: "n"(SD_STAGES - 2) : "memory");
    __syncwarp();                        // every lane's copies of this stage have landed; the stage of step - 1 is free
    fill(step + SD_STAGES - 1);
    const int jw = key0 + (step * SD_WARPS + warp) * SD_STEP;
    const uint32_t st = ring + (step % SD_STAGES) * STAGE;
    // ---- scores of 2 key tiles x 16 rows
    float sacc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.0f;
      const int row = 8 * nt + g;
#pragma unroll
      for (int sl = 0; sl < SL; sl++) {
        uint4 kf;
        const uint32_t a = st + row * ROWB + (((4 * sl + t) ^ sd_swz(row)) << 4);
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(kf.x), "=r"(kf.y), "=r"(kf.z), "=r"(kf.w) : "r"(a));
        sd_mma<T>(sacc[nt], qlo[sl].x, qhi[sl].x, qlo[sl].y, qhi[sl].y, kf.x, kf.y);
        sd_mma<T>(sacc[nt], qlo[sl].z, qhi[sl].z, qlo[sl].w, qhi[sl].w, kf.z, kf.w);
      }
    }
    // ---- streaming softmax (rows g and g + 8; a row's 16 scores sit in the 4 lanes of a quad)
    float pl[2][2], ph[2][2];
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int key = jw + 8 * nt + 2 * t + e;
        pl[nt][e] = (key < key1 && key <= spos_lo) ? sacc[nt][e] * p.scale_log2 : -INFINITY;
        ph[nt][e] = (HI && key < key1 && key <= spos_hi) ? sacc[nt][2 + e] * p.scale_log2 : -INFINITY;
        mx_lo = fmaxf(mx_lo, pl[nt][e]); mx_hi = fmaxf(mx_hi, ph[nt][e]);
      }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xFFFFFFFFu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xFFFFFFFFu, mx_lo, 2));
    if (HI) { mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xFFFFFFFFu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xFFFFFFFFu, mx_hi, 2)); }
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float c_lo = mn_lo == -INFINITY ? 1.0f : exp2f(m_lo - mn_lo);
    const float c_hi = mn_hi == -INFINITY ? 1.0f : exp2f(m_hi - mn_hi);
    m_lo = mn_lo; m_hi = mn_hi;
    float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        pl[nt][e] = pl[nt][e] == -INFINITY ? 0.0f : exp2f(pl[nt][e] - mn_lo);
        ph[nt][e] = (!HI || ph[nt][e] == -INFINITY) ? 0.0f : exp2f(ph[nt][e] - mn_hi);
        sum_lo += pl[nt][e]; sum_hi += ph[nt][e];
      }
    l_lo = fmaf(l_lo, c_lo, sum_lo); l_hi = fmaf(l_hi, c_hi, sum_hi);
    if (c_lo != 1.0f || c_hi != 1.0f) {
#pragma unroll
      for (int i = 0; i < NT; i++) { oacc[i][0] *= c_lo; oacc[i][1] *= c_lo; oacc[i][2] *= c_hi; oacc[i][3] *= c_hi; }
    }
    const uint32_t a0 = sd_pack2<T>(pl[0][0], pl[0][1]), a2 = sd_pack2<T>(pl[1][0], pl[1][1]);
    const uint32_t a1 = HI ? sd_pack2<T>(ph[0][0], ph[0][1]) : 0u, a3 = HI ? sd_pack2<T>(ph[1][0], ph[1][1]) : 0u;
    // ---- P.V
    const uint32_t vst = st + SD_STEP * ROWB;
#pragma unroll
    for (int h = 0; h < D / 64; h++) {
      uint32_t vr[4][4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int row = 2 * t + (e & 1) + ((e & 2) << 2);          // 2t, 2t+1, 8+2t, 9+2t
        const uint32_t a = vst + row * ROWB + (((g + 8 * h) ^ sd_swz(row)) << 4);
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(vr[e][0]), "=r"(vr[e][1]), "=r"(vr[e][2]), "=r"(vr[e][3]) : "r"(a));
      }
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(vr[0][i >> 1], vr[1][i >> 1], sel);
        const uint32_t b1 = __byte_perm(vr[2][i >> 1], vr[3][i >> 1], sel);
        sd_mma<T>(oacc[8 * h + i], a0, a1, a2, a3, b0, b1);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                       // the stage rings are free: they become the merge buffers
  // ---- merge the quads' sums, then the warps of this CTA
  l_lo += __shfl_xor_sync(0xFFFFFFFFu, l_lo, 1); l_lo += __shfl_xor_sync(0xFFFFFFFFu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xFFFFFFFFu, l_hi, 1); l_hi += __shfl_xor_sync(0xFFFFFFFFu, l_hi, 2);
  float* s_o = reinterpret_cast<float*>(sd_smem);                        // [warp][16][D]
  float* s_m = s_o + SD_WARPS * 16 * D;                                   // [warp][16]
  float* s_l = s_m + SD_WARPS * 16;
  if (t == 0) {
    s_m[warp * 16 + g] = m_lo; s_l[warp * 16 + g] = l_lo;
    s_m[warp * 16 + g + 8] = m_hi; s_l[warp * 16 + g + 8] = l_hi;
  }
#pragma unroll
  for (int i = 0; i < NT; i++) {
    const int h = i >> 3, ii = i & 7;
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int d = 64 * h + 8 * (2 * t + e) + ii;
      s_o[(warp * 16 + g) * D + d] = oacc[i][e];
      s_o[(warp * 16 + g + 8) * D + d] = oacc[i][2 + e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.rows * D; idx += SD_THREADS) {
    const int r = idx / D, d = idx - r * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < SD_WARPS; w++) mm = fmaxf(mm, s_m[w * 16 + r]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < SD_WARPS; w++) {
      const float c = s_m[w * 16 + r] == -INFINITY ? 0.0f : exp2f(s_m[w * 16 + r] - mm);
      ll = fmaf(s_l[w * 16 + r], c, ll);
      oo = fmaf(s_o[(w * 16 + r) * D + d], c, oo);
    }
    const long long pr = (((long long)b * p.Hkv + kvh) * p.splits + split) * p.rows + r;
    p.part_o[pr * D + d] = oo;
    if (d == 0) { p.part_ml[pr * 2] = mm; p.part_ml[pr * 2 + 1] = ll; }
  }
}

// out[b, head, s, :] = sum over splits of partial * exp2(m_split - m) / l; all-masked rows (l == 0) give zeros
// (sdpa.go:471-474).  One block of D threads per query row.
template <typename T>
__global__ void sdpa_decode_merge_kernel(T* __restrict__ out, const SdParams p) {
  pdl_enter();
  const int r = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
  const long long base = (((long long)b * p.Hkv + kvh) * p.splits) * p.rows + r;
  float mm = -INFINITY;
  for (int s = 0; s < p.splits; s++) mm = fmaxf(mm, p.part_ml[(base + (long long)s * p.rows) * 2]);
  float ll = 0.0f, oo = 0.0f;
  for (int s = 0; s < p.splits; s++) {
    const long long pr = base + (long long)s * p.rows;
    const float ms = p.part_ml[pr * 2];
    const float c = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
    ll = fmaf(p.part_ml[pr * 2 + 1], c, ll);
    oo = fmaf(p.part_o[pr * p.D + d], c, oo);
  }
  const int hg = r / p.S, s = r - hg * p.S;
  const bool padded = p.q_lens && s >= __ldg(p.q_lens + b);
  const float res = (ll != 0.0f && !padded) ? oo / ll : 0.0f;
  Scalar<T>::store(out + (long long)b * p.q_b + (long long)(kvh * p.group + hg) * p.q_h + (long long)s * p.q_s, d, res);
}

bool sdpa_decode_supports(const cb_sdpa_desc& d, std::string* why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  if (d.dtype != CB_BF16 && d.dtype != CB_F16) return no("bfloat16 / float16 only");
  if (d.D != 128 && d.D != 64) return no("head_dim must be 64 or 128");
  if (d.mask_kind != CB_MASK_NONE || d.bias_rank > 0) return no("mask and bias tensors go to the generic kernel");
  if (d.Hkv <= 0 || d.Hq % d.Hkv != 0) return no("grouped heads");
  if (d.B < 1 || d.S < 1 || d.Skv < 1) return no("empty");
  if (d.S * (d.Hq / d.Hkv) > SD_MAX_ROWS) return no("more than 16 query rows per KV head");
  if (d.Skv < 256) return no("short caches stay on the generic kernel");
  if (d.B > 65535 || d.Hkv > 65535) return no("too many heads for one grid");
  return true;
}

// Two CTAs per SM are resident.  Among the split lengths (multiples of the CTA's 64-key round) take the one that
// finishes soonest in whole waves of CTAs, charging every CTA a fixed start-and-merge cost of ~96 keys.
static long long sd_keys_per_split(int n_sm, long long pairs, long long Skv) {
  const long long slots = 2LL * n_sm, round = SD_WARPS * SD_STEP;
  long long best_keys = 0, best_cost = 0;
  for (long long keys = 2 * round; ; keys += round) {
    const long long splits = (Skv + keys - 1) / keys;
    if (splits <= 64) {
      const long long waves = (pairs * splits + slots - 1) / slots;
      const long long cost = waves * (keys + 96);
      if (!best_keys || cost < best_cost) { best_keys = keys; best_cost = cost; }
    }
    if (keys >= Skv) break;
  }
  return best_keys;
}

static void sd_fill(const cb_plan* p, SdParams* s) {
  const cb_sdpa_desc& d = p->sdpa;
  s->B = (int)d.B; s->Hq = (int)d.Hq; s->Hkv = (int)d.Hkv; s->S = (int)d.S; s->Skv = (int)d.Skv; s->D = (int)d.D;
  s->group = (int)(d.Hq / d.Hkv);
  s->rows = s->group * s->S;
  if (d.layout == CB_LAYOUT_BSHD) {
    s->q_b = d.S * d.Hq * d.D; s->q_s = d.Hq * d.D; s->q_h = d.D;
    s->kv_b = d.Skv * d.Hkv * d.D; s->kv_s = d.Hkv * d.D; s->kv_h = d.D;
  } else {
    s->q_b = d.Hq * d.S * d.D; s->q_h = d.S * d.D; s->q_s = d.D;
    s->kv_b = d.Hkv * d.Skv * d.D; s->kv_h = d.Skv * d.D; s->kv_s = d.D;
  }
  const double scale = d.scale != 0.0 ? d.scale : 1.0 / sqrt((double)d.D);
  s->scale_log2 = (float)(scale * 1.4426950408889634);
  s->causal = d.causal;
  s->keys_per_split = (int)sd_keys_per_split(p->n_sm, d.B * d.Hkv, d.Skv);
  s->splits = (int)((d.Skv + s->keys_per_split - 1) / s->keys_per_split);
}

static size_t sd_smem_bytes(int D) {
  const size_t ring = (size_t)SD_WARPS * SD_STAGES * 2 * SD_STEP * D * 2;
  const size_t merge = (size_t)SD_WARPS * 16 * (D + 2) * sizeof(float);
  return std::max(ring, merge);
}

int sdpa_decode_plan(cb_plan* p) {
  const cb_sdpa_desc& d = p->sdpa;
  const long long pairs = d.B * d.Hkv;
  const long long keys = sd_keys_per_split(p->n_sm, pairs, d.Skv);
  const long long splits = (d.Skv + keys - 1) / keys;
  p->blocks = (int)splits;           // CTAs per (batch, KV head) pair; the grid is (splits, Hkv, B)
  p->threads = SD_THREADS;
  const long long rows = d.S * (d.Hq / d.Hkv);
  p->workspace_bytes = (size_t)(pairs * splits * rows * (d.D + 2)) * sizeof(float);
  p->counter_bytes = 0;
  p->name = std::string("sdpa_decode_") + dtype_name(d.dtype) + (d.causal ? "_causal" : "") + (d.layout == CB_LAYOUT_BSHD ? "_bshd" : "_bhsd");
  return CB_OK;
}

template <typename T, int D, bool HI>
static int sd_launch_k(const SdParams& s, const T* q, const T* k, const T* v, cudaStream_t st) {
  static std::atomic<bool> configured[64];
  int dev = 0;
  CB_CUDA(cudaGetDevice(&dev));            // the current device: the one this launch goes to
  const size_t smem = sd_smem_bytes(D);
  if (dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(sdpa_decode_kernel<T, D, HI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  dim3 grid((unsigned)s.splits, (unsigned)s.Hkv, (unsigned)s.B);
  CB_CUDA(launch_dependent(sdpa_decode_kernel<T, D, HI>, grid, dim3(SD_THREADS), smem, st, q, k, v, s));
  return CB_OK;
}

template <typename T, int D>
static int sd_launch_t(const SdParams& s, const T* q, const T* k, const T* v, T* out, cudaStream_t st) {
  const int rc = s.rows <= 8 ? sd_launch_k<T, D, false>(s, q, k, v, st) : sd_launch_k<T, D, true>(s, q, k, v, st);
  if (rc != CB_OK) return rc;
  CB_CUDA(launch_dependent(sdpa_decode_merge_kernel<T>, dim3((unsigned)s.rows, (unsigned)s.Hkv, (unsigned)s.B), dim3((unsigned)s.D), 0, st, out, s));
  return CB_OK;
}

int sdpa_decode_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t st) {
  SdParams s;
  sd_fill(p, &s);
  s.part_o = (float*)ws;
  s.part_ml = s.part_o + (size_t)s.B * s.Hkv * s.splits * s.rows * s.D;
  s.q_lens = p->sdpa.has_seq_lens ? (const int*)in[3] : nullptr;      // inputs: q, k, v, QuerySeqLen, KeyValueSeqLen
  s.kv_lens = p->sdpa.has_seq_lens ? (const int*)in[4] : nullptr;
  if ((reinterpret_cast<uintptr_t>(in[0]) & 15) || (reinterpret_cast<uintptr_t>(in[1]) & 15) || (reinterpret_cast<uintptr_t>(in[2]) & 15))
    return fail(CB_ERR_INVALID_ARG, "FusedScaledDotProductAttention: query, key and value must be 16-byte aligned");
  if (p->sdpa.dtype == CB_BF16) {
    typedef __nv_bfloat16 T;
    return s.D == 128 ? sd_launch_t<T, 128>(s, (const T*)in[0], (const T*)in[1], (const T*)in[2], (T*)out[0], st)
                      : sd_launch_t<T, 64>(s, (const T*)in[0], (const T*)in[1], (const T*)in[2], (T*)out[0], st);
  }
  typedef __half T;
  return s.D == 128 ? sd_launch_t<T, 128>(s, (const T*)in[0], (const T*)in[1], (const T*)in[2], (T*)out[0], st)
                    : sd_launch_t<T, 64>(s, (const T*)in[0], (const T*)in[1], (const T*)in[2], (T*)out[0], st);
}

}  // namespace cb
