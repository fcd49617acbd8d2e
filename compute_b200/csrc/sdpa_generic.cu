// FusedScaledDotProductAttention, generic kernel: any head_dim / sequence length,
// f32 / f64 / bf16 / f16, BHSD and BSHD, causal, boolean or additive mask,
// additive bias, per-batch sequence lengths, GQA.  One CTA per (batch, query
// head, query row), following the reference's per-row algorithm
// (internal/gobackend/fusedops/sdpa.go:373-519): scores = q.k*scale (+bias)(+mask),
// row max, exp, sum, normalise (all-masked rows give zeros), then P.V with the kv
// index ascending.  Half types compute in f32 and round once on store.
#include "common.cuh"

namespace cb {

struct SdpaParams {
  int64_t B, Hq, Hkv, S, Skv, D;
  int64_t q_b, q_h, q_s;        // element strides of q/out
  int64_t kv_b, kv_h, kv_s;     // element strides of k/v
  int64_t m_b, m_h, m_s, m_k;   // mask strides (0 = broadcast)
  int64_t b_b, b_h, b_s, b_k;   // bias strides
  double scale;
  int causal, mask_kind, has_bias, has_lens;
};

template <typename T> struct SdpaC { typedef float type; };
template <> struct SdpaC<double> { typedef double type; };

template <typename C> __device__ inline C sdpa_exp(C x);
template <> __device__ inline float sdpa_exp<float>(float x) { return expf(x); }
template <> __device__ inline double sdpa_exp<double>(double x) { return exp(x); }

template <typename C> __device__ inline C sdpa_mul(C a, C b) { return a * b; }
template <> __device__ inline float sdpa_mul<float>(float a, float b) { return __fmul_rn(a, b); }
template <typename C> __device__ inline C sdpa_add(C a, C b) { return a + b; }
template <> __device__ inline float sdpa_add<float>(float a, float b) { return __fadd_rn(a, b); }

template <typename C, bool IS_MAX>
__device__ inline C block_reduce(C v, C* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    C other = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? (other > v ? other : v) : v + other;
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  C r = scratch[0];
  for (int w = 1; w < nw; w++) r = IS_MAX ? (scratch[w] > r ? scratch[w] : r) : r + scratch[w];
  return r;
}

template <typename T>
__global__ void __launch_bounds__(128)
sdpa_generic_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    const void* __restrict__ mask, const T* __restrict__ bias,
                    const int32_t* __restrict__ q_len, const int32_t* __restrict__ kv_len,
                    T* __restrict__ out, const SdpaParams p) {
  typedef typename SdpaC<T>::type C;
  extern __shared__ __align__(16) unsigned char sdpa_smem[];
  C* scores = reinterpret_cast<C*>(sdpa_smem);
  C* qrow = scores + p.Skv;
  C* scratch = qrow + p.D;

  const int64_t row = blockIdx.x;
  const int64_t qi = row % p.S;
  const int64_t h = (row / p.S) % p.Hq;
  const int64_t b = row / (p.S * p.Hq);
  const int64_t hk = h / (p.Hq / p.Hkv);
  const int64_t q_off = b * p.q_b + h * p.q_h + qi * p.q_s;
  const int64_t kv_off = b * p.kv_b + hk * p.kv_h;

  int64_t q_limit = p.S, kv_limit = p.Skv;
  if (p.has_lens) {
    const int64_t ql = q_len[b], kl = kv_len[b];
    q_limit = ql < 0 ? 0 : (ql > p.S ? p.S : ql);
    kv_limit = kl < 0 ? 0 : (kl > p.Skv ? p.Skv : kl);
  }
  if (qi >= q_limit) {   // padded query position: zero row
    for (int64_t d = threadIdx.x; d < p.D; d += blockDim.x) Scalar<T>::store(out, q_off + d, (C)0);
    return;
  }
  int64_t live = kv_limit < p.Skv ? kv_limit : p.Skv;
  if (p.causal && qi + 1 < live) live = qi + 1;

  for (int64_t d = threadIdx.x; d < p.D; d += blockDim.x) qrow[d] = (C)Scalar<T>::load(q, q_off + d);
  __syncthreads();

  const uint8_t* bmask = p.mask_kind == CB_MASK_BOOL ? reinterpret_cast<const uint8_t*>(mask) : nullptr;
  const T* amask = p.mask_kind == CB_MASK_ADDITIVE ? reinterpret_cast<const T*>(mask) : nullptr;
  const int64_t m_row = b * p.m_b + h * p.m_h + qi * p.m_s;
  const int64_t b_row = b * p.b_b + h * p.b_h + qi * p.b_s;
  const C scale = (C)p.scale;
  const C neg_inf = -(C)INFINITY;

  C local_max = neg_inf;
  for (int64_t j = threadIdx.x; j < live; j += blockDim.x) {
    if (bmask && !bmask[m_row + j * p.m_k]) { scores[j] = neg_inf; continue; }
    const T* kr = k + kv_off + j * p.kv_s;
    C dot = (C)0;
    for (int64_t d = 0; d < p.D; d++) dot = sdpa_add<C>(dot, sdpa_mul<C>(qrow[d], (C)Scalar<T>::load(kr, d)));
    C s = sdpa_mul<C>(dot, scale);
    if (p.has_bias) s = sdpa_add<C>(s, (C)Scalar<T>::load(bias, b_row + j * p.b_k));
    if (amask) s = sdpa_add<C>(s, (C)Scalar<T>::load(amask, m_row + j * p.m_k));
    scores[j] = s;
    if (s > local_max) local_max = s;
  }
  const C row_max = block_reduce<C, true>(local_max, scratch);

  C local_sum = (C)0;
  for (int64_t j = threadIdx.x; j < live; j += blockDim.x) {
    const bool masked = bmask && !bmask[m_row + j * p.m_k];
    const C e = masked ? (C)0 : sdpa_exp<C>(scores[j] - row_max);
    scores[j] = e;
    local_sum += e;
  }
  const C sum = block_reduce<C, false>(local_sum, scratch);
  const C inv = (sum != (C)0) ? (C)1 / sum : (C)0;
  for (int64_t j = threadIdx.x; j < live; j += blockDim.x) scores[j] = sdpa_mul<C>(scores[j], inv);
  __syncthreads();

  for (int64_t d = threadIdx.x; d < p.D; d += blockDim.x) {
    C acc = (C)0;
    const T* vc = v + kv_off + d;
    for (int64_t j = 0; j < live; j++) {
      if (bmask && !bmask[m_row + j * p.m_k]) continue;
      acc = sdpa_add<C>(acc, sdpa_mul<C>(scores[j], (C)Scalar<T>::load(vc, j * p.kv_s)));
    }
    Scalar<T>::store(out, q_off + d, acc);
  }
}

// Strides (batch, head, seq, kv) of a mask/bias operand broadcast to [B,H,S,Skv].
// `dims` are the caller's dims: rank 2 [S,Skv]; rank 3 [B,S,Skv]; rank 4 [B,H,S,Skv]
// for BHSD or [B,S,H,Skv] for BSHD (the reference transposes those to BHSD first,
// sdpa.go:259-274 — here the strides do it).
static int operand_strides(const char* what, int rank, const int64_t* dims, const cb_sdpa_desc& d,
                           int64_t* sb, int64_t* sh, int64_t* ss, int64_t* sk) {
  if (rank < 2 || rank > 4) return fail(CB_ERR_INVALID_ARG, "FusedScaledDotProductAttention: %s must have rank 2, 3, or 4, got rank %d", what, rank);
  int64_t full[4] = {1, 1, 1, 1};     // as [B,H,S,Skv] extents in caller order
  const bool bshd4 = (rank == 4 && d.layout == CB_LAYOUT_BSHD);
  // rank 3 is [batch, seq, kv] — the executor's reading (sdpaComputeMaskStrides,
  // sdpa.go:309-329), not a right-aligned [heads, seq, kv].
  if (rank == 3) { full[0] = dims[0]; full[2] = dims[1]; full[3] = dims[2]; }
  else for (int i = 0; i < rank; i++) full[4 - rank + i] = dims[i];
  int64_t eb, eh, es, ek;
  if (bshd4) { eb = full[0]; es = full[1]; eh = full[2]; ek = full[3]; }
  else { eb = full[0]; eh = full[1]; es = full[2]; ek = full[3]; }
  const int64_t want[4] = {d.B, d.Hq, d.S, d.Skv};
  const int64_t got[4] = {eb, eh, es, ek};
  for (int i = 0; i < 4; i++)
    if (got[i] != 1 && got[i] != want[i])
      return fail(CB_ERR_INVALID_ARG,
                  "FusedScaledDotProductAttention: %s dim %lld is not broadcastable to score dim %lld (score shape [%lld,%lld,%lld,%lld])",
                  what, (long long)got[i], (long long)want[i], (long long)d.B, (long long)d.Hq, (long long)d.S, (long long)d.Skv);
  // row-major strides in caller order, zeroed for broadcast axes
  int64_t st[4], mul = 1;
  for (int i = 3; i >= 0; i--) { st[i] = mul; mul *= full[i]; }
  if (bshd4) { *sb = st[0]; *ss = st[1]; *sh = st[2]; *sk = st[3]; }
  else { *sb = st[0]; *sh = st[1]; *ss = st[2]; *sk = st[3]; }
  if (eb == 1) *sb = 0;
  if (eh == 1) *sh = 0;
  if (es == 1) *ss = 0;
  if (ek == 1) *sk = 0;
  return CB_OK;
}

int sdpa_fill_params(const cb_sdpa_desc& d, SdpaParams* p) {
  p->B = d.B; p->Hq = d.Hq; p->Hkv = d.Hkv; p->S = d.S; p->Skv = d.Skv; p->D = d.D;
  if (d.layout == CB_LAYOUT_BSHD) {
    p->q_s = d.Hq * d.D; p->q_h = d.D; p->q_b = d.S * d.Hq * d.D;
    p->kv_s = d.Hkv * d.D; p->kv_h = d.D; p->kv_b = d.Skv * d.Hkv * d.D;
  } else {
    p->q_s = d.D; p->q_h = d.S * d.D; p->q_b = d.Hq * d.S * d.D;
    p->kv_s = d.D; p->kv_h = d.Skv * d.D; p->kv_b = d.Hkv * d.Skv * d.D;
  }
  p->scale = d.scale != 0.0 ? d.scale : 1.0 / sqrt((double)d.D);
  p->causal = d.causal;
  p->mask_kind = d.mask_kind;
  p->has_bias = d.bias_rank > 0;
  p->has_lens = d.has_seq_lens;
  p->m_b = p->m_h = p->m_s = p->m_k = 0;
  p->b_b = p->b_h = p->b_s = p->b_k = 0;
  if (d.mask_kind != CB_MASK_NONE)
    CB_TRY(operand_strides("mask", d.mask_rank, d.mask_dims, d, &p->m_b, &p->m_h, &p->m_s, &p->m_k));
  if (d.bias_rank > 0)
    CB_TRY(operand_strides("bias", d.bias_rank, d.bias_dims, d, &p->b_b, &p->b_h, &p->b_s, &p->b_k));
  return CB_OK;
}

int sdpa_validate_operands(const cb_sdpa_desc& d) {
  SdpaParams tmp;
  return sdpa_fill_params(d, &tmp);
}

// ---------------------------------------------------------------------------
// Tiled kernel: the same operands and options as the row kernel above (any mask, bias, sequence lengths, GQA, both
// layouts; float32 / bfloat16 / float16 with head_dim 32, 64 or 128) for query tiles of 32 rows — what a model built
// on float32 attention with head_dim 64 and padding masks runs on, shapes the tensor-core kernels do not take.
// A CTA of 128 threads owns 32 query rows of one head and walks the keys in blocks of 64: K and V blocks are staged in
// shared memory as float32 (coalesced loads), thread (ty, tx) forms the scores of rows ty + 8 i and keys tx + 16 j
// with 16-byte shared-memory reads along the head dimension, the streaming softmax state of a row is replicated in
// the 16 threads that share it (reductions by shuffles), probabilities go through shared memory, and the same thread
// accumulates rows ty + 8 i x dimensions tx + 16 c of the output.  All arithmetic is float32 FMA; the sums are not in
// the reference's order, so results agree with it to rounding, not bit for bit (the row kernel keeps its order).
constexpr int ST_BQ = 32, ST_BK = 64, ST_THREADS = 128, ST_PP = ST_BK + 4;

template <typename T, int D>
__global__ void __launch_bounds__(ST_THREADS)
sdpa_tile_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                 const void* __restrict__ mask, const T* __restrict__ bias,
                 const int32_t* __restrict__ q_len, const int32_t* __restrict__ kv_len,
                 T* __restrict__ out, const SdpaParams p) {
  pdl_enter();
  constexpr int PD = D + 4, NC = D / 16;
  extern __shared__ __align__(16) unsigned char sdpa_smem[];
  float* Qs = reinterpret_cast<float*>(sdpa_smem);      // [ST_BQ][PD]
  float* Ks = Qs + ST_BQ * PD;                           // [ST_BK][PD]
  float* Vs = Ks + ST_BK * PD;                           // [ST_BK][PD]
  float* Ps = Vs + ST_BK * PD;                           // [ST_BQ][ST_PP]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t nqt = (p.S + ST_BQ - 1) / ST_BQ;
  const int64_t qt = blockIdx.x % nqt, h = (blockIdx.x / nqt) % p.Hq, b = blockIdx.x / (nqt * p.Hq);
  const int64_t hk = h / (p.Hq / p.Hkv);
  const int64_t q0 = qt * ST_BQ;
  int64_t q_limit = p.S, kv_limit = p.Skv;
  if (p.has_lens) {
    const int64_t ql = q_len[b], kl = kv_len[b];
    q_limit = ql < 0 ? 0 : (ql > p.S ? p.S : ql);
    kv_limit = kl < 0 ? 0 : (kl > p.Skv ? p.Skv : kl);
  }
  const int64_t kv_end = p.causal ? min(kv_limit, q0 + ST_BQ) : kv_limit;        // no row of the tile sees keys from here on
  const T* qb = q + b * p.q_b + h * p.q_h;
  const T* kb_ = k + b * p.kv_b + hk * p.kv_h;
  const T* vb = v + b * p.kv_b + hk * p.kv_h;
  for (int idx = tid; idx < ST_BQ * D; idx += ST_THREADS) {
    const int r = idx / D, d = idx - r * D;
    Qs[r * PD + d] = q0 + r < p.S ? (float)Scalar<T>::load(qb, (q0 + r) * p.q_s + d) : 0.0f;
  }
  const uint8_t* bmask = p.mask_kind == CB_MASK_BOOL ? reinterpret_cast<const uint8_t*>(mask) : nullptr;
  const T* amask = p.mask_kind == CB_MASK_ADDITIVE ? reinterpret_cast<const T*>(mask) : nullptr;
  const float scale = (float)p.scale;
  float m[4], l[4], o[4][NC];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    m[i] = -INFINITY; l[i] = 0.0f;
#pragma unroll
    for (int c = 0; c < NC; c++) o[i][c] = 0.0f;
  }
  for (int64_t kb = 0; kb < kv_end; kb += ST_BK) {
    __syncthreads();                                     // the previous block's K, V and P have been read (and Q is written)
    for (int idx = tid; idx < ST_BK * D; idx += ST_THREADS) {
      const int r = idx / D, d = idx - r * D;
      const bool in = kb + r < kv_end;
      Ks[r * PD + d] = in ? (float)Scalar<T>::load(kb_, (kb + r) * p.kv_s + d) : 0.0f;
      Vs[r * PD + d] = in ? (float)Scalar<T>::load(vb, (kb + r) * p.kv_s + d) : 0.0f;
    }
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) s[i][j] = 0.0f;
#pragma unroll 4
    for (int d4 = 0; d4 < D / 4; d4++) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty + 8 * i) * PD + 4 * d4);
#pragma unroll
      for (int j = 0; j < 4; j++) kv[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * PD + 4 * d4);
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
          s[i][j] = fmaf(qv[i].x, kv[j].x, fmaf(qv[i].y, kv[j].y, fmaf(qv[i].z, kv[j].z, fmaf(qv[i].w, kv[j].w, s[i][j]))));
    }
    // scale, bias, masks; the block's row maxima and sums across the 16 threads of a row
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int64_t qi = q0 + ty + 8 * i;
      const int64_t m_row = b * p.m_b + h * p.m_h + qi * p.m_s, b_row = b * p.b_b + h * p.b_h + qi * p.b_s;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int64_t key = kb + tx + 16 * j;
        bool live = qi < p.S && key < kv_limit && (!p.causal || key <= qi);
        if (live && bmask && !bmask[m_row + key * p.m_k]) live = false;
        float sv = s[i][j] * scale;
        if (live && p.has_bias) sv += (float)Scalar<T>::load(bias, b_row + key * p.b_k);
        if (live && amask) sv += (float)Scalar<T>::load(amask, m_row + key * p.m_k);
        s[i][j] = live ? sv : -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int w = 1; w < 16; w <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, w));
      const float m_new = fmaxf(m[i], mx);
      const float corr = m_new == -INFINITY ? 1.0f : expf(m[i] - m_new);
      float sum = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float e = s[i][j] == -INFINITY ? 0.0f : expf(s[i][j] - m_new);
        Ps[(ty + 8 * i) * ST_PP + tx + 16 * j] = e;
        sum += e;
      }
#pragma unroll
      for (int w = 1; w < 16; w <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, w);
      l[i] = fmaf(l[i], corr, sum);
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < NC; c++) o[i][c] *= corr;
    }
    __syncthreads();
#pragma unroll 2
    for (int k4 = 0; k4 < ST_BK / 4; k4++) {
      float4 pv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) pv[i] = *reinterpret_cast<const float4*>(Ps + (ty + 8 * i) * ST_PP + 4 * k4);
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float vv[NC];
#pragma unroll
        for (int c = 0; c < NC; c++) vv[c] = Vs[(4 * k4 + e) * PD + tx + 16 * c];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float pe = e == 0 ? pv[i].x : e == 1 ? pv[i].y : e == 2 ? pv[i].z : pv[i].w;
#pragma unroll
          for (int c = 0; c < NC; c++) o[i][c] = fmaf(pe, vv[c], o[i][c]);
        }
      }
    }
  }
  // rows without a live key and padded query positions are zeros (sdpa.go:389-398, 471-474)
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t qi = q0 + ty + 8 * i;
    if (qi >= p.S) continue;
    const float inv = (l[i] != 0.0f && qi < q_limit) ? 1.0f / l[i] : 0.0f;
    T* orow = out + b * p.q_b + h * p.q_h + qi * p.q_s;
#pragma unroll
    for (int c = 0; c < NC; c++) Scalar<T>::store(orow, tx + 16 * c, o[i][c] * inv);
  }
}

static size_t tile_smem(int64_t D) { return ((size_t)(ST_BQ + 2 * ST_BK) * (D + 4) + (size_t)ST_BQ * ST_PP) * sizeof(float); }

// Shapes worth a tile: enough query rows to fill one, head_dim 32 / 64 / 128, a float type other than float64.  Tiny
// problems (and anything asked for by name) stay on the row kernel, which sums in the reference's order.
bool sdpa_tile_supports(const cb_sdpa_desc& d) {
  if (d.dtype != CB_F32 && d.dtype != CB_BF16 && d.dtype != CB_F16) return false;
  if (d.D != 32 && d.D != 64 && d.D != 128) return false;
  if (d.S < 16 || d.S * d.Skv < 4096) return false;
  return d.B * d.Hq * ((d.S + ST_BQ - 1) / ST_BQ) <= 0x7fffffffLL;
}

int sdpa_tile_plan(cb_plan* p) {
  const cb_sdpa_desc& d = p->sdpa;
  p->blocks = (int)(d.B * d.Hq * ((d.S + ST_BQ - 1) / ST_BQ));
  p->threads = ST_THREADS;
  p->dyn_smem = (int)tile_smem(d.D);
  p->name = std::string("sdpa_tile_") + dtype_name(d.dtype);
  return CB_OK;
}

template <typename T, int D>
static int tile_launch_d(const cb_plan* p, const SdpaParams& prm, const void* const* in, void* const* out, cudaStream_t s) {
  const cb_sdpa_desc& d = p->sdpa;
  int idx = 3;
  const void* mask = d.mask_kind != CB_MASK_NONE ? in[idx++] : nullptr;
  const int32_t* ql = d.has_seq_lens ? (const int32_t*)in[idx++] : nullptr;
  const int32_t* kl = d.has_seq_lens ? (const int32_t*)in[idx++] : nullptr;
  const T* bias = d.bias_rank > 0 ? (const T*)in[idx++] : nullptr;
  if (p->dyn_smem > 48 * 1024)
    CB_CUDA(cudaFuncSetAttribute(sdpa_tile_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, p->dyn_smem));
  CB_CUDA(launch_dependent(sdpa_tile_kernel<T, D>, dim3((unsigned)p->blocks), dim3(ST_THREADS), (size_t)p->dyn_smem, s, (const T*)in[0], (const T*)in[1],
                           (const T*)in[2], mask, bias, ql, kl, (T*)out[0], prm));
  return CB_OK;
}
template <typename T>
static int tile_launch_t(const cb_plan* p, const SdpaParams& prm, const void* const* in, void* const* out, cudaStream_t s) {
  switch (p->sdpa.D) {
    case 32: return tile_launch_d<T, 32>(p, prm, in, out, s);
    case 64: return tile_launch_d<T, 64>(p, prm, in, out, s);
    default: return tile_launch_d<T, 128>(p, prm, in, out, s);
  }
}

int sdpa_tile_launch(const cb_plan* p, const void* const* in, void* const* out, cudaStream_t s) {
  const cb_sdpa_desc& d = p->sdpa;
  if (p->blocks == 0) return CB_OK;
  SdpaParams prm;
  CB_TRY(sdpa_fill_params(d, &prm));
  switch (d.dtype) {
    case CB_F32: return tile_launch_t<float>(p, prm, in, out, s);
    case CB_BF16: return tile_launch_t<__nv_bfloat16>(p, prm, in, out, s);
    default: return tile_launch_t<__half>(p, prm, in, out, s);
  }
}

static size_t generic_smem(const cb_sdpa_desc& d) {
  const size_t c = d.dtype == CB_F64 ? 8 : 4;
  return (size_t)(d.Skv + d.D + 8) * c;
}

int sdpa_generic_plan(cb_plan* p) {
  const cb_sdpa_desc& d = p->sdpa;
  if (generic_smem(d) > 200 * 1024)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedScaledDotProductAttention generic kernel: kv length %lld too long", (long long)d.Skv);
  if (d.B * d.Hq * d.S > 0x7fffffffLL)
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedScaledDotProductAttention generic kernel: too many query rows");
  p->blocks = (int)(d.B * d.Hq * d.S);
  p->threads = 128;
  p->dyn_smem = (int)generic_smem(d);
  p->name = std::string("sdpa_generic_") + dtype_name(d.dtype);
  return CB_OK;
}

template <typename T>
static int launch_t(const cb_plan* p, const SdpaParams& prm, const void* const* in, void* const* out, cudaStream_t s) {
  const cb_sdpa_desc& d = p->sdpa;
  int idx = 3;
  const void* mask = d.mask_kind != CB_MASK_NONE ? in[idx++] : nullptr;
  const int32_t* ql = d.has_seq_lens ? (const int32_t*)in[idx++] : nullptr;
  const int32_t* kl = d.has_seq_lens ? (const int32_t*)in[idx++] : nullptr;
  const T* bias = d.bias_rank > 0 ? (const T*)in[idx++] : nullptr;
  if (p->dyn_smem > 48 * 1024)
    CB_CUDA(cudaFuncSetAttribute(sdpa_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, p->dyn_smem));
  sdpa_generic_kernel<T><<<p->blocks, 128, p->dyn_smem, s>>>((const T*)in[0], (const T*)in[1], (const T*)in[2], mask, bias,
                                                            ql, kl, (T*)out[0], prm);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

int sdpa_generic_launch(const cb_plan* p, const void* const* in, void* const* out, cudaStream_t s) {
  const cb_sdpa_desc& d = p->sdpa;
  if (p->blocks == 0 || d.D == 0) return CB_OK;
  SdpaParams prm;
  CB_TRY(sdpa_fill_params(d, &prm));
  switch (d.dtype) {
    case CB_F32: return launch_t<float>(p, prm, in, out, s);
    case CB_F64: return launch_t<double>(p, prm, in, out, s);
    case CB_BF16: return launch_t<__nv_bfloat16>(p, prm, in, out, s);
    case CB_F16: return launch_t<__half>(p, prm, in, out, s);
    default: return fail(CB_ERR_NOT_IMPLEMENTED, "FusedScaledDotProductAttention: dtype %s is not implemented", dtype_name(d.dtype));
  }
}

}  // namespace cb
