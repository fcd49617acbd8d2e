// Weights with the reference's scale layout [K, N / block] for decode shapes: packed 4-bit (Int4 / Uint4 Linear, NF4)
// and 8-bit (Int8 / Uint8 Linear, NF4 indices one per byte).  The 8-bit formats with compact scales have their own
// tensor-core kernel; this one is what a caller of the reference's interface gets when the scales are per row of W.
// Reference arithmetic: internal/gobackend/fusedops/quantizeddense.go:586-650 (per output column, k ascending:
// x * w * scale, or x * (w * scale + zero point)); nibble order internal/gobackend/ops/convertdtype.go:199-226.
//
// The weights are read once, as they lie: element (k, n) is nibble n & 1 of byte (k N + n) / 2, so a row of W is N / 2
// contiguous bytes and a lane that reads one 32-bit word holds eight neighbouring columns of one k.  The scale of a
// row belongs to (k, n / block): with block a multiple of 8 it is one float for the lane's word, multiplied into x
// instead of into eight weights.  Every lane keeps the sums of its eight columns for up to eight rows of x in
// registers; the rows of W go round the eight warps of a CTA, and the K range is cut over gridDim.z CTAs, so that
// three to four CTAs fill every SM.  Partial sums meet in shared memory (fixed order), then in a workspace
// [cut][M][N]; a second small kernel adds the cuts in order, the bias and the activation.
//
// With 8-bit weights a lane's eight columns are two words (one 64-bit read); everything else is the same.
//
// A nibble becomes a float without a conversion: its four bits go to the top of the mantissa of 1.0, which is
// 1 + n / 16 (for Int4 the nibble's top bit is flipped first: n ^ 8 = n + 8).  The sums run over those floats and the
// sum of the scaled x is kept beside them: sum x s n = 16 (sum x s f - sum x s), and - 8 sum x s for Int4.
#include "tc_common.cuh"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <string>

namespace cb {
namespace {

constexpr int W4_WARPS = 8;
constexpr int W4_COLS = 256;               // columns per CTA: 32 lanes x 8
constexpr size_t W4_HEADER = 256;          // status words at the start of the workspace
// Up to this many rows of x the kernel runs once per 16 rows: two runs of 94 us beat expanding the weights to bf16
// planes for the GEMM (about 265 us whatever M on the 4096 x 14336 projection).
constexpr int W4_MAX_M = 32;
__host__ __device__ constexpr int w4_unroll(int mr) { return mr >= 8 ? 4 : 8; }   // rows of W a lane has in flight
enum { W4_U4 = 0, W4_I4 = 1, W4_NF4 = 2, W8_U8 = 3, W8_I8 = 4, W8_NF4 = 5 };
__host__ __device__ constexpr int w4_wpl(int mode) { return mode >= W8_U8 ? 2 : 1; }         // 32-bit words a lane's eight columns take
__host__ __device__ constexpr int w4_stages(int wpl) { return wpl == 2 ? 4 : 6; }           // TMA form: groups of rows in flight or in use per CTA

// NormalFloat4 (fused_ops.go:114-121)
__constant__ float kW4Nf4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

// shared memory before the barriers: x of the cut, then the reduction buffer with, in the TMA form, the ring under it
__host__ __device__ constexpr size_t w4_data_bytes(int mr, int rows_max, bool tma, int wpl) {
  const size_t xs = (size_t)mr * rows_max * 4, red = (size_t)W4_WARPS * mr * W4_COLS * 4,
               ring = (size_t)w4_stages(wpl) * W4_WARPS * w4_unroll(mr) * 128 * wpl;
  return xs + (tma && ring > red ? ring : red);
}

template <int MODE>
__device__ __forceinline__ float w4_value(uint2 words, int i, const float* lut) {   // column i of the lane's eight
  if (MODE >= W8_U8) {
    const uint32_t wb = i < 4 ? words.x : words.y;
    const int b = i & 3;
    if (MODE == W8_NF4) return lut[(wb >> (8 * b)) & 0xFu];
    // a byte under the exponent of 2^23 is 2^23 + b; signed bytes are biased by 128 first
    if (MODE == W8_U8) return __uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7650u | b)) - 8388608.0f;
    return __uint_as_float(__byte_perm(wb ^ 0x80808080u, 0x4B000000u, 0x7650u | b)) - 8388736.0f;
  }
  const uint32_t word = words.x;
  if (MODE == W4_NF4) return lut[(word >> (4 * i)) & 0xFu];
  const uint32_t at19 = 4 * i <= 19 ? word << (19 - 4 * i) : word >> (4 * i - 19);
  return __uint_as_float((at19 & 0x00780000u) ^ (MODE == W4_I4 ? 0x3FC00000u : 0x3F800000u));
}

// grid (row tiles of x, column tiles, cuts of K); partial [gridDim.z][M][N].  K is counted in groups of 8 warps x
// W4_UNROLL rows; cut z takes groups [z G / cuts, (z + 1) G / cuts).  TAIL: K is not a whole number of groups, so the
// rows of the last group are checked one by one.  TMA: every group of rows arrives as one tile (GROUP rows x 128
// bytes of the CTA's 256 columns) in a ring of W4_STAGES stages, asked for by thread 0; the warps read their rows'
// words from it.  Every wait is bounded; one that gives up ends the kernel with the status word set.  Without TMA (N / 2 not a
// multiple of 16 bytes) every lane loads its words itself, the next group requested before the current one is consumed.
template <typename XT, int MODE, int MR, bool ZP, bool TAIL, bool TMA>
__global__ void __launch_bounds__(W4_WARPS * 32, MR >= 2 ? 2 : 3)
qdense_w4_kernel(const __grid_constant__ CUtensorMap tmap_w, const XT* __restrict__ x, const uint32_t* __restrict__ w,
                 const float* __restrict__ scales, const float* __restrict__ zps, float* __restrict__ partial, unsigned* __restrict__ status,
                 int M, int64_t K, int64_t N, int64_t block, int64_t nblk, int rows_max) {
  constexpr int WPL = w4_wpl(MODE), W4_STAGES = w4_stages(WPL);
  constexpr int W4_UNROLL = w4_unroll(MR), GROUP = W4_WARPS * W4_UNROLL, STAGE = GROUP * 128 * WPL;
  constexpr int VPW = 8, COLS = W4_COLS;
  constexpr bool TABLE = MODE == W4_NF4 || MODE == W8_NF4, DIRECT = MODE >= W4_NF4;          // DIRECT: w4_value is the weight itself
  // the kernel that adds the cuts may be scheduled now; it waits for this grid before it reads the partial sums
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ __align__(1024) unsigned char w4_smem[];
  float* xs = reinterpret_cast<float*>(w4_smem);                               // [MR][rows_max]
  float* red = xs + (size_t)MR * rows_max;                                     // [W4_WARPS][MR][COLS]; the ring lies under it
  const uint32_t* ring = reinterpret_cast<const uint32_t*>(red);               // [W4_STAGES][GROUP][32 WPL words]
  uint64_t* full = reinterpret_cast<uint64_t*>(w4_smem + w4_data_bytes(MR, rows_max, TMA, WPL));
  uint64_t* empty = full + W4_STAGES;
  __shared__ float lut[16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (TMA && threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < W4_STAGES; k++) { tc::mbar_init(&full[k], 1); tc::mbar_init(&empty[k], W4_WARPS); }
    tc::fence_barrier_init();
  }
  const int m0 = blockIdx.x * MR;
  const int64_t G = (K + GROUP - 1) / GROUP;
  const int64_t g0 = (int64_t)blockIdx.z * G / gridDim.z, g1 = ((int64_t)blockIdx.z + 1) * G / gridDim.z;
  const int64_t k0 = g0 * GROUP;
  const int kc = (int)(min(K, g1 * GROUP) - k0);                               // rows of this cut
  const int n_groups = (int)(g1 - g0);
  const int64_t n0 = (int64_t)blockIdx.y * COLS + lane * VPW;
  const bool active = n0 < N;
  if (TABLE && threadIdx.x < 16) lut[threadIdx.x] = kW4Nf4[threadIdx.x];
  for (int idx = threadIdx.x; idx < MR * rows_max; idx += blockDim.x) {
    const int m = idx / rows_max, kk = idx % rows_max;
    xs[idx] = (m0 + m < M && kk < kc) ? (float)Scalar<XT>::load(x, (int64_t)(m0 + m) * K + k0 + kk) : 0.0f;
  }
  __syncthreads();

  float acc[MR][VPW], sx[MR], zacc[MR];
#pragma unroll
  for (int m = 0; m < MR; m++) {
    sx[m] = 0.0f; zacc[m] = 0.0f;
#pragma unroll
    for (int i = 0; i < VPW; i++) acc[m][i] = 0.0f;
  }
  bool failed = false;
  int issued = 0;                                                              // tiles asked for (thread 0 only)
  // TMA form: thread 0 asks for group g + W4_STAGES - 1 when it starts on group g; the stage that tile goes to held
  // group g - 1, which every warp has copied to registers (and said so on the stage's `empty` barrier) by then or soon.
  auto ask = [&](int g) {                                                      // thread 0 only; false if the stage never came free
    const int slot = g % W4_STAGES, round = g / W4_STAGES;
    if (round > 0 && !tc::mbar_wait(&empty[slot], (uint32_t)((round - 1) & 1))) return false;
    tc::mbar_expect_tx(&full[slot], STAGE);
    tc::tma_load_2d(const_cast<uint32_t*>(ring) + (size_t)slot * (STAGE / 4), &tmap_w, (int)(blockIdx.y * 32 * WPL), (int)(k0 + (int64_t)g * GROUP),
                    &full[slot]);
    issued = g + 1;
    return true;
  };
  if (TMA && threadIdx.x == 0)
    for (int g = 0; g < min(n_groups, W4_STAGES - 1); g++) ask(g);
  if ((TMA || active) && n_groups > 0) {
    const int64_t wrow = N / VPW * WPL;                                        // words per row of W
    const int64_t n0s = active ? n0 : 0;                                       // lanes past N (TMA form) work on zeros of column 0's scales
    // this warp's rows of a group: warp, warp + 8, ...; the next group is requested before this one is consumed
    const uint32_t* wq = w + (k0 + warp) * wrow + n0s / VPW * WPL;
    const float* sq = scales + (k0 + warp) * nblk + n0s / block;
    const float* zq = ZP ? zps + (k0 + warp) * nblk + n0s / block : nullptr;
    const int64_t w8 = W4_WARPS * wrow, s8 = W4_WARPS * nblk;
    uint2 wn[W4_UNROLL];
    float sn[W4_UNROLL], zn[W4_UNROLL];
    auto load_words = [&](const uint32_t* q) {                                 // the lane's one or two words of a row
      if (WPL == 2) return __ldg(reinterpret_cast<const uint2*>(q));
      return make_uint2(__ldg(q), 0u);
    };
    auto request = [&](int g) {
#pragma unroll
      for (int u = 0; u < W4_UNROLL; u++) {
        const bool in = !TAIL || g * GROUP + warp + u * W4_WARPS < kc;
        if (!TMA) wn[u] = in ? load_words(wq + u * w8) : make_uint2(0u, 0u);
        sn[u] = in ? __ldg(sq + u * s8) : 0.0f;
        zn[u] = (ZP && in) ? __ldg(zq + u * s8) : 0.0f;
      }
      if (!TMA) wq += GROUP * wrow;
      sq += GROUP * nblk;
      if (ZP) zq += GROUP * nblk;
    };
    request(0);
    const float* xr = xs + warp;
    int slot = 0;
    uint32_t phase = 0;
    for (int g = 0; g < n_groups; g++) {
      uint2 wv[W4_UNROLL];
      float sv[W4_UNROLL], zv[W4_UNROLL];
      if (TMA) {
        bool ok = true;
        if (threadIdx.x == 0 && g + W4_STAGES - 1 < n_groups) ok = ask(g + W4_STAGES - 1);
        ok = ok && tc::mbar_wait(&full[slot], phase);
        if (!__all_sync(0xFFFFFFFFu, ok)) { failed = true; break; }
        const uint32_t* st = ring + (size_t)slot * (STAGE / 4) + (warp * 32 + lane) * WPL;
#pragma unroll
        for (int u = 0; u < W4_UNROLL; u++) {
          if (WPL == 2) wv[u] = *reinterpret_cast<const uint2*>(st + u * W4_WARPS * 32 * WPL);
          else wv[u] = make_uint2(st[u * W4_WARPS * 32], 0u);
        }
        __syncwarp();                                                          // every lane holds its words: the stage may be refilled
        if (lane == 0) tc::mbar_arrive(&empty[slot]);
        if (++slot == W4_STAGES) { slot = 0; phase ^= 1u; }
      }
#pragma unroll
      for (int u = 0; u < W4_UNROLL; u++) { if (!TMA) wv[u] = wn[u]; sv[u] = sn[u]; zv[u] = zn[u]; }
      if (g + 1 < n_groups) request(g + 1);
#pragma unroll
      for (int u = 0; u < W4_UNROLL; u++) {
        float f[VPW];
#pragma unroll
        for (int i = 0; i < VPW; i++) f[i] = w4_value<MODE>(wv[u], i, lut);
#pragma unroll
        for (int m = 0; m < MR; m++) {
          const float xv = xr[m * rows_max + u * W4_WARPS];                    // rows past K hold 0 here and scale 0
          const float xsv = xv * sv[u];
          if (!DIRECT) sx[m] += xsv;
          if (ZP) zacc[m] = fmaf(xv, zv[u], zacc[m]);
#pragma unroll
          for (int i = 0; i < VPW; i++) acc[m][i] = fmaf(xsv, f[i], acc[m][i]);
        }
      }
      xr += GROUP;
    }
  }
  if (TMA) {
    // the ring becomes the reduction buffer once every warp has read its last stage; a wait that gave up ends the CTA
    if (__syncthreads_or(failed ? 1 : 0)) {
      // tiles that were asked for may still land: one more bounded wait for each before the shared memory is given up
      for (int g = max(0, issued - W4_STAGES); g < issued; g++) tc::mbar_wait(&full[g % W4_STAGES], (uint32_t)((g / W4_STAGES) & 1));
      if (threadIdx.x == 0 && atomicCAS(&status[0], 0u, 1u) == 0u) atomicExch(&status[1], blockIdx.y | (blockIdx.z << 16));
      return;
    }
  }
  // ---- the eight warps' sums, added in warp order
#pragma unroll
  for (int m = 0; m < MR; m++) {
    float v[VPW];
#pragma unroll
    for (int i = 0; i < VPW; i++) {
      // Uint4: n = 16 (f - 1); Int4: n = 16 (f - 1) - 8, f built from the nibble with its top bit flipped
      v[i] = DIRECT ? acc[m][i] : MODE == W4_U4 ? 16.0f * (acc[m][i] - sx[m]) : fmaf(16.0f, acc[m][i], -24.0f * sx[m]);
      v[i] += zacc[m];
    }
    float4* dst = reinterpret_cast<float4*>(red + ((size_t)warp * MR + m) * COLS + lane * VPW);
#pragma unroll
    for (int q = 0; q < VPW / 4; q++) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
  __syncthreads();
  const int64_t n = (int64_t)blockIdx.y * COLS + threadIdx.x;
  if (n < N && threadIdx.x < COLS) {
#pragma unroll
    for (int m = 0; m < MR; m++) {
      if (m0 + m >= M) break;
      float v = 0.0f;
#pragma unroll
      for (int wq = 0; wq < W4_WARPS; wq++) v += red[((size_t)wq * MR + m) * COLS + threadIdx.x];
      partial[((int64_t)blockIdx.z * M + m0 + m) * N + n] = v;
    }
  }
}

template <typename XT>
__global__ void __launch_bounds__(256)
qdense_w4_finish_kernel(const float* __restrict__ partial, const float* __restrict__ bias, XT* __restrict__ out, int64_t MN, int64_t N, int cuts, int act) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= MN) return;
  float v = 0.0f;
  for (int c = 0; c < cuts; c++) v += __ldcg(partial + (int64_t)c * MN + i);
  if (bias) v = __fadd_rn(v, bias[i % N]);
  Scalar<XT>::store(out, i, apply_activation(v, act));
}

int w4_rows(const cb_qdense_desc& d) { return d.M <= 1 ? 1 : d.M <= 2 ? 2 : d.M <= 4 ? 4 : 8; }
bool w4_packed(const cb_qdense_desc& d) { return d.w_dtype == CB_I4 || d.w_dtype == CB_U4; }
int w4_desc_wpl(const cb_qdense_desc& d) { return w4_packed(d) ? 1 : 2; }

// How K is cut.  A CTA costs a fixed set-up and a reduction, so few long CTAs beat many short ones, but the CTAs must
// fill whole waves: with `slots` CTAs resident on the GPU at once, the cut count that fills one wave best is taken when
// it reaches 0.8 of the wave, otherwise the best of two waves.  Cuts are whole groups of rows, at least two per cut.
void w4_cuts(const cb_qdense_desc& d, int n_sm, int* cuts, int* rows_max) {
  const int mr = w4_rows(d);
  const int group = W4_WARPS * w4_unroll(mr);
  const long long G = (d.K + group - 1) / group;
  const long long tiles = ((d.M + mr - 1) / mr) * ((d.N + W4_COLS - 1) / W4_COLS);
  const long long slots = (long long)std::max(n_sm, 1) * (mr >= 2 ? 2 : 3);
  const long long max_cuts = std::max(1LL, G / 2);
  long long best = 1;
  double best_fill = 0.0;
  for (int waves = 1; waves <= 2 && best_fill < 0.8; waves++) {
    for (long long c = 1; c <= max_cuts && tiles * c <= waves * slots; c++) {
      const double fill = (double)(tiles * c) / (double)(waves * slots);
      if (fill > best_fill) { best_fill = fill; best = c; }
    }
  }
  *cuts = (int)best;
  *rows_max = (int)(((G + best - 1) / best) * group);
}

size_t w4_smem_bytes(int mr, int rows_max, bool tma, int wpl) {
  return w4_data_bytes(mr, rows_max, tma, wpl) + (tma ? 2 * w4_stages(wpl) * sizeof(uint64_t) : 0);
}
// the rows of W as 32-bit words [K][words per row], in boxes of one group of rows by the 32 words of a column tile;
// a row must be a whole number of 16-byte units
bool w4_tma(const cb_qdense_desc& d) { return (d.N / 8 * w4_desc_wpl(d)) % 4 == 0; }
int w4_encode(CUtensorMap* m, const void* ptr, uint64_t K, uint64_t N, uint32_t group, uint32_t wpl) {   // N: words per row
  struct Entry { const void* ptr; uint64_t K, N; uint32_t group, wpl; bool valid; CUtensorMap map; };
  constexpr int SLOTS = 64;
  static thread_local Entry cache[SLOTS];
  const uintptr_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull;
  Entry& e = cache[(h >> 40) % SLOTS];
  if (e.valid && e.ptr == ptr && e.K == K && e.N == N && e.group == group && e.wpl == wpl) { *m = e.map; return CB_OK; }
  encode_tiled_fn enc = tensor_map_encoder();
  if (!enc) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {N, K};
  cuuint64_t strides[1] = {N * 4};
  cuuint32_t box[2] = {32 * wpl, group};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  e.ptr = ptr; e.K = K; e.N = N; e.group = group; e.wpl = wpl; e.map = *m; e.valid = true;
  return CB_OK;
}

template <typename XT, int MODE, int MR, bool ZP, bool TAIL, bool TMA>
int w4_launch_k(const cb_qdense_desc& d, int n_sm, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  int cuts = 0, rows = 0;
  w4_cuts(d, n_sm, &cuts, &rows);
  constexpr int COLS = W4_COLS, WPL = w4_wpl(MODE);
  const size_t smem = w4_smem_bytes(MR, rows, TMA, WPL);
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  if (TMA) CB_TRY(w4_encode(&tmap, in[1], (uint64_t)d.K, (uint64_t)(d.N / 8 * WPL), (uint32_t)(W4_WARPS * w4_unroll(MR)), (uint32_t)WPL));
  float* partial = (float*)((uint8_t*)ws + W4_HEADER);
  static std::atomic<bool> configured[64];
  int dev = 0;
  CB_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(qdense_w4_kernel<XT, MODE, MR, ZP, TAIL, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    if (dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  int idx = 3;
  const float* zp = d.has_zero_point ? (const float*)in[idx++] : nullptr;
  const float* bias = d.has_bias ? (const float*)in[idx++] : nullptr;
  const int64_t nblk = (d.N + d.block_size - 1) / d.block_size;
  dim3 grid((unsigned)((d.M + MR - 1) / MR), (unsigned)((d.N + COLS - 1) / COLS), (unsigned)cuts);
  qdense_w4_kernel<XT, MODE, MR, ZP, TAIL, TMA><<<grid, W4_WARPS * 32, smem, s>>>(
      tmap, (const XT*)in[0], (const uint32_t*)in[1], (const float*)in[2], zp, partial, (unsigned*)ws, (int)d.M, d.K, d.N, d.block_size, nblk, rows);
  CB_CUDA(cudaGetLastError());
  const int64_t mn = d.M * d.N;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)((mn + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB_CUDA(cudaLaunchKernelEx(&cfg, qdense_w4_finish_kernel<XT>, (const float*)partial, bias, (XT*)out[0], mn, (int64_t)d.N, cuts, (int)d.activation));
  return CB_OK;
}

template <typename XT, int MODE, bool ZP>
int w4_launch_m(const cb_qdense_desc& d, int n_sm, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const int mr = w4_rows(d);
  const bool tail = d.K % (W4_WARPS * w4_unroll(mr)) != 0;
  const bool tma = w4_tma(d) && (reinterpret_cast<uintptr_t>(in[1]) & 15) == 0;
#define W4_GO(MR_) (tma ? (tail ? w4_launch_k<XT, MODE, MR_, ZP, true, true>(d, n_sm, in, out, ws, s) : w4_launch_k<XT, MODE, MR_, ZP, false, true>(d, n_sm, in, out, ws, s)) \
                        : (tail ? w4_launch_k<XT, MODE, MR_, ZP, true, false>(d, n_sm, in, out, ws, s) : w4_launch_k<XT, MODE, MR_, ZP, false, false>(d, n_sm, in, out, ws, s)))
  switch (mr) {
    case 1: return W4_GO(1);
    case 2: return W4_GO(2);
    case 4: return W4_GO(4);
    default: return W4_GO(8);
  }
#undef W4_GO
}

template <typename XT>
int w4_launch_t(const cb_qdense_desc& d, int n_sm, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  if (!w4_packed(d)) {
    if (d.scheme == CB_QUANT_NF4) return w4_launch_m<XT, W8_NF4, false>(d, n_sm, in, out, ws, s);
    if (d.w_dtype == CB_I8) return d.has_zero_point ? w4_launch_m<XT, W8_I8, true>(d, n_sm, in, out, ws, s) : w4_launch_m<XT, W8_I8, false>(d, n_sm, in, out, ws, s);
    return d.has_zero_point ? w4_launch_m<XT, W8_U8, true>(d, n_sm, in, out, ws, s) : w4_launch_m<XT, W8_U8, false>(d, n_sm, in, out, ws, s);
  }
  if (d.scheme == CB_QUANT_NF4) return w4_launch_m<XT, W4_NF4, false>(d, n_sm, in, out, ws, s);
  if (d.w_dtype == CB_I4) return d.has_zero_point ? w4_launch_m<XT, W4_I4, true>(d, n_sm, in, out, ws, s) : w4_launch_m<XT, W4_I4, false>(d, n_sm, in, out, ws, s);
  return d.has_zero_point ? w4_launch_m<XT, W4_U4, true>(d, n_sm, in, out, ws, s) : w4_launch_m<XT, W4_U4, false>(d, n_sm, in, out, ws, s);
}

}  // namespace

// Decode shapes of the 4-bit and 8-bit formats with the reference's scale layout (a column group must be a multiple of
// the eight columns a lane owns).  The generic kernel keeps everything else, and
// these too when the plan asks for it by name (it sums in the reference's order).
bool qdense_w4_supports(const cb_qdense_desc& d) {
  if (d.variant != CB_QDENSE_AUTO) return false;
  if (d.w_dtype != CB_I4 && d.w_dtype != CB_U4 && d.w_dtype != CB_I8 && d.w_dtype != CB_U8) return false;
  if (d.scheme != CB_QUANT_LINEAR && d.scheme != CB_QUANT_NF4) return false;
  const int vpw = 8;                       // a lane's eight columns share one scale
  if (d.scale_layout != CB_SCALE_REF || d.block_size < vpw || d.block_size % vpw != 0) return false;
  if (d.gather_ranks > 1) return false;
  // below a few hundred thousand weights the launch of a second kernel costs more than the generic kernel's loop
  return d.M >= 1 && d.M <= W4_MAX_M && d.N >= vpw && d.N % vpw == 0 && d.K >= 64 && d.K * d.N >= (1 << 18) && d.K < (1LL << 31) && d.N < (1LL << 31);
}

void qdense_w4_plan(cb_plan* p) {
  cb_qdense_desc d = p->qd;
  d.M = std::min<int64_t>(d.M, 16);                                            // one run of the kernel: the workspace is shared by the runs
  int cuts = 0, rows = 0;
  w4_cuts(d, p->n_sm, &cuts, &rows);
  const int mr = w4_rows(d);
  p->blocks = (int)(((d.M + mr - 1) / mr) * ((d.N + W4_COLS - 1) / W4_COLS) * cuts);
  p->threads = W4_WARPS * 32;
  p->dyn_smem = (int)w4_smem_bytes(mr, rows, w4_tma(d), w4_desc_wpl(d));
  p->workspace_bytes = W4_HEADER + (size_t)cuts * (size_t)d.M * (size_t)d.N * sizeof(float);
  p->counter_bytes = W4_HEADER;
  p->has_status = true;
  p->name = std::string(w4_packed(d) ? "qdense_w4_" : "qdense_w8_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") +
            (d.w_dtype == CB_U4 ? "_u4" : d.w_dtype == CB_I4 ? "_i4" : d.w_dtype == CB_U8 ? "_u8" : "_i8") + (d.scheme == CB_QUANT_NF4 ? "_nf4" : "");
}

int qdense_w4_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  const cb_qdense_desc& d = p->qd;
  if (d.M == 0 || d.N == 0) return CB_OK;
  if (!ws) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense (reference scales, decode): the plan needs its workspace (partial sums of the cuts of K)");
  if ((reinterpret_cast<uintptr_t>(in[1]) & (w4_packed(d) ? 3 : 7)) || (reinterpret_cast<uintptr_t>(in[2]) & 3))
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense (reference scales, decode): weights must be 4-byte (bytes: 8-byte) and scales 4-byte aligned");
  // 16 rows of x per run; the runs follow each other on the stream and share the workspace
  const size_t esz = d.x_dtype == CB_BF16 ? 2 : 4;
  const int n_in = 3 + (d.has_zero_point ? 1 : 0) + (d.has_bias ? 1 : 0);
  for (int64_t m0 = 0; m0 < d.M; m0 += 16) {
    cb_qdense_desc c = d;
    c.M = std::min<int64_t>(16, d.M - m0);
    const void* cin[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    for (int i = 0; i < n_in; i++) cin[i] = in[i];
    cin[0] = (const uint8_t*)in[0] + (size_t)m0 * d.K * esz;
    void* cout[1] = {(uint8_t*)out[0] + (size_t)m0 * d.N * esz};
    CB_TRY(c.x_dtype == CB_BF16 ? w4_launch_t<__nv_bfloat16>(c, p->n_sm, cin, cout, ws, s) : w4_launch_t<float>(c, p->n_sm, cin, cout, ws, s));
  }
  return CB_OK;
}

}  // namespace cb
