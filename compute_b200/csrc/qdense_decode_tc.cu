// FusedQuantizedDense for decode shapes (M <= 16) on the integer tensor cores:
//   y[M,N] = act( x[M,K] @ (W[K,N] * scale) + bias[N] ),  W int8/uint8, compact scales
// (reference semantics: internal/gobackend/fusedops/quantizeddense.go:330-418 of gomlx/compute).
//
// The op is bound by reading W once from HBM, so the kernel spends no instruction on the
// weights: TMA lands [128 k x 128 n] byte tiles of W in shared memory and tcgen05.mma kind::i8
// consumes them in place as the MN-major operand.  The activations become the other operand in
// block fixed point: for every row m and every 128-wide k unit u,
//     x[m,k] = unit[m,u] * (d0 + 128 d1 (+ 16384 d2)),   signed base-128 digits,
// with unit[m,u] a power of two taken from the largest |x| of that row inside the unit.
//   float32 x   three digit planes: 20 bits below the unit's maximum (error <= 2^-21 of it)
//   bfloat16 x  two digit planes: 13 bits below the maximum.  A bfloat16 has 8 significant bits, so
//               every element within 2^-6 of the unit's maximum is exact and smaller ones are
//               rounded at 2^-14 of the maximum (1.2e-4 relative to the largest element of the
//               unit; the output is rounded to bfloat16, 3.9e-3, and compared at 2e-2).
// The digits of all rows form a [PLANES*MB x K] int8 matrix (MB rows per plane), so one MMA of
// shape (128 n) x (PLANES*MB) x (32 k) yields the digit sums of 128 output columns, exactly, in
// s32 tensor memory.  Epilogue threads (one per output column) turn a finished 128-k unit into
// f32, recombine the digits, multiply by unit[m,u] and by the scale of that K group, and add it
// to their running totals.
//
// One launch serves a GROUP of independent problems that share M and K (one problem is the
// ordinary case): the work list is the column tiles of all problems in order, so the pipeline is
// filled and drained once per group instead of once per projection.  Each problem has its own
// weights, scales, bias, activation and result buffer(s) in a table of QtProblem records that
// travels in kernel parameter space (the TMA unit reads the tensor maps from there).
//
//   qdense_xdigits_kernel   x -> digits + unit[m,u] (one warp per x, row and k unit, all at once)
//   qdense_decode_tc_kernel persistent over a contiguous range of (column tile, k unit) pairs.
//     Two rings decouple the memory stream from the arithmetic:
//       stages        [weights 128 x 128 B | digit tile NB x 128 B] in shared memory, filled by TMA,
//                     consumed by the MMA and handed back to the producers by the MMA's own
//                     completion (tcgen05.commit), so the bytes in flight do not wait for the epilogue;
//       accumulators  up to 16 TMEM accumulators of NB columns, each with a slot for the unit's 128
//                     scales and 16 unit[m,u], released by the epilogue.
//       warps 8, 12   TMA producers of the weight tiles into the stage ring; the first ones are
//                     requested before the digit kernel has finished
//       warps 10, 13  TMA producers of the digit tiles
//       warps 14, 15  producers of the scale / unit slots
//       warps 9, 11   MMA issuers: 4 MMAs (K = 32) per unit from a stage into an accumulator
//       warps 0-7     epilogue as above, two groups of four warps; a tile whose units are split
//                     between CTAs is finished by the CTA that arrives last, summing the parked
//                     partial tiles in CTA order (deterministic: the result does not depend on
//                     which CTA finishes).  A launch of few column tiles instead gives every tile to a
//                     thread-block cluster of two to four CTAs, each with an equal run of the tile's
//                     units: the partial tiles stay in shared memory and the cluster's first CTA sums
//                     them through distributed shared memory after one cluster barrier (no global
//                     round trips: 17 -> 10.6 us per launch on a 4096 x 4096 projection)
//     Every role comes in a pair, one thread (or group) for the even units and one for the odd ones,
//     and both ring sizes are even: a stage, an accumulator and their barriers therefore always
//     belong to the same member of each pair, which waits for every phase of those barriers in
//     turn.  (A parity wait tells two consecutive phases apart, not three: with an odd ring a
//     barrier alternated between the two members, each saw every other phase, and a thread ahead
//     of a late tile took the previous phase for the one it was waiting for.)
// All mbarrier waits are bounded; a timeout sets the status word and TMEM is always freed.
// Building with -DCB_QT_STAMPS adds per-CTA time stamps (timing diagnosis; off in the shipped build).
#include "tc_common.cuh"

#include <algorithm>
#include <atomic>
#include <memory>
#include <stdlib.h>
#include <string.h>

namespace cb {

using namespace tc;

constexpr int QT_TILE_N = 128;
constexpr int QT_UNIT_K = 128;
constexpr int QT_W_BYTES = QT_TILE_N * QT_UNIT_K;     // 16 KB
constexpr int QT_THREADS = 512;                       // warps 0-7 epilogue, 9 and 11 MMA, six producers
constexpr int QT_TMA_WARP = 8, QT_MMA_WARP = 9, QT_SIDE_WARP = 10, QT_MMA2_WARP = 11;   // weights (even units), MMA, digits (even), MMA
constexpr int QT_TMA2_WARP = 12, QT_SIDE2_WARP = 13;                                      // weights, digits of the odd units
constexpr int QT_SCALE_WARP = 14, QT_SCALE2_WARP = 15;                                    // scale / unit slots of the even / odd units
constexpr int QT_TMEM_COLS = 512;
constexpr int QT_SC_BYTES = QT_TILE_N * 4;             // a unit's 128 scales
constexpr int QT_UN_BYTES = 64;                         // a unit's 16 unit[m,u]
constexpr int QT_SLOT_BYTES = 640;                      // scales, then unit[m,u]; slots stay 128-byte aligned
constexpr int QT_BAR_BYTES = 1024;
constexpr int QT_HEADER = 256;                          // status words, then arrival counters
// Accumulators (even, at most 16) and stages (even: what shared memory holds) by MMA N extent and digit planes.
__host__ __device__ constexpr int qt_accs(int nb) { return nb == 48 ? 10 : 16; }
__host__ __device__ constexpr int qt_tail_bytes(int nb, int planes) {   // barriers, slots, merge tile, staging tile (16-bit results only with two planes)
  return QT_BAR_BYTES + qt_accs(nb) * QT_SLOT_BYTES + (nb / planes) * QT_TILE_N * 4 + (nb / planes) * QT_TILE_N * (planes == 2 ? 2 : 4);
}
__host__ __device__ constexpr int qt_stages(int nb, int planes) {
  return ((232448 - 1024 - qt_tail_bytes(nb, planes)) / (QT_W_BYTES + nb * QT_UNIT_K)) / 2 * 2 > 10 ? 10
       : ((232448 - 1024 - qt_tail_bytes(nb, planes)) / (QT_W_BYTES + nb * QT_UNIT_K)) / 2 * 2;
}

constexpr int QT_MAX_RANKS = 8;
constexpr int QT_MAX_PROBLEMS = CB_QDENSE_GROUP_MAX;

// One problem of a launch.  The tensor maps are read by the TMA unit straight from this record,
// which is part of the kernel parameters.
struct alignas(64) QtProblem {
  CUtensorMap tmap_w;                  // W [K rows][N bytes], 128 x 128 boxes, 128-byte swizzle
  CUtensorMap tmap_s;                  // scales [rows][N] f32, 128 x 1 boxes
  const float* bias;
  void* outs[QT_MAX_RANKS];            // result buffers this problem is stored into (one, or one per rank of a gathered plan)
  int N;
  int out_ld, out_col0;                // row stride (elements) and first column of this kernel's slice
  int activation;
  int pad[10];
};
static_assert(sizeof(QtProblem) == 384, "QtProblem layout");
// The problems of a launch: kernels are instantiated for tables of 1, 4 and 16 records (0.4, 1.5 and 6 KB of parameters).
template <int MAXP> struct QtTable { QtProblem p[MAXP]; };

struct QtParams {
  unsigned* status;
  unsigned* counters;       // one per column tile of the launch, zero between launches
  float* partials;          // [grid][2][MB][128]
  int M, K;
  int n_problems;
  int n_outs;               // 1, or the number of ranks
  int tile_start[QT_MAX_PROBLEMS + 1];     // first column tile of every problem in the launch's list
  int digit_row0[QT_MAX_PROBLEMS];         // first row of the problem's block in the digit matrix
  const float* unit_rows[QT_MAX_PROBLEMS]; // the problem's unit[m,u]: 16 floats per k unit
  int units_per_tile;
  int tiles_total;
  int whole_tiles;          // 1: CTAs take whole tiles; 0: an equal share of the units, shared tiles fixed up
  int cluster;              // > 1: every tile is shared by this many consecutive CTAs, launched as one thread-block cluster,
                            // each with one run of the tile's units; the partial tiles are summed through shared memory
  long long total_units;
  int scale_group;          // 0: one scale per column; else rows of the K group
  int out_bf16;
  uint32_t idesc;
#ifdef CB_QT_STAMPS
  unsigned long long* dbg;  // 8 time stamps per CTA
#endif
};

// The distinct activation matrices of a launch (problems given the same x share one digit block).
struct QtXList {
  const void* x[QT_MAX_PROBLEMS];
  int n;
};

// ---------------------------------------------------------------------------
// x -> digits
// ---------------------------------------------------------------------------
constexpr int QX_THREADS = 256;       // 8 warps, one (x, row, k unit) task each

// Four consecutive elements x[m, k .. k+3] as floats; zeros beyond column K.
__device__ __forceinline__ void qx_load4(const __nv_bfloat16* x, size_t m, int K, int k, float (&v)[4]) {
  const uint2 r = k < K ? __ldg(reinterpret_cast<const uint2*>(x + m * K + k)) : make_uint2(0, 0);
  v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
  v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
}
__device__ __forceinline__ void qx_load4(const float* x, size_t m, int K, int k, float (&v)[4]) {
  const float4 r = k < K ? __ldg(reinterpret_cast<const float4*>(x + m * K + k)) : make_float4(0, 0, 0, 0);
  v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}

// One warp per (activation matrix, row m, 128-wide k unit u): the unit's largest finite |x| fixes
// unit[m,u] = 2^-shift (7*PLANES - 1 bits below it), every element becomes PLANES signed base-128
// digits in the matrix's block of NB rows, and unit[m,u] goes to the unit array, 16 floats per k unit
// (NaN when the unit holds inf or NaN).  No pass over the whole row is needed, so all tasks run at once.
template <typename XT, int PLANES>
__global__ void __launch_bounds__(QX_THREADS)
qdense_xdigits_kernel(const QtXList xl, int M, int K, int NB, int G, int8_t* __restrict__ digits, float* __restrict__ unit_rows
#ifdef CB_QT_STAMPS
                      , unsigned long long* dbg
#endif
                      ) {
  constexpr int QBITS = 7 * PLANES - 1;
  const int MB = NB / PLANES;                      // rows per digit plane (NB = 16 with three planes leaves one row unused)
  // The kernel that consumes the digits may start its own set-up now; it waits for this grid to
  // finish before it reads them.  This grid in turn may have been scheduled while the kernel
  // before it in the stream (which may produce x, and may still read the digit buffer) was
  // running: it waits for that kernel to finish before it touches either.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#ifdef CB_QT_STAMPS
  if (dbg && blockIdx.x == 0 && threadIdx.x == 0) dbg[0] = global_ns();
#endif
  asm volatile("griddepcontrol.wait;" ::: "memory");
#ifdef CB_QT_STAMPS
  if (dbg && blockIdx.x == 0 && threadIdx.x == 0) dbg[1] = global_ns();
#endif
  const int lane = threadIdx.x & 31;
  const int task = blockIdx.x * (QX_THREADS / 32) + (threadIdx.x >> 5);
  if (task >= xl.n * M * G) return;
  const int xi = task / (M * G);
  const int rem = task - xi * (M * G);
  const int u = rem / M, m = rem - u * M;
  const int k = u * QT_UNIT_K + 4 * lane;
  float v[4];
  qx_load4(reinterpret_cast<const XT*>(xl.x[xi]), (size_t)m, K, k, v);
  uint32_t mx = 0;          // bits of the largest finite |x| (non-negative floats order like integers)
  bool bad = false;
#pragma unroll
  for (int e = 0; e < 4; e++) {
    const uint32_t a = __float_as_uint(v[e]) & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) { bad = true; v[e] = 0.0f; } else mx = max(mx, a);
  }
  mx = __reduce_max_sync(0xFFFFFFFFu, mx);
  bad = __any_sync(0xFFFFFFFFu, bad);
  // amax < 2^ex: exponent field - 126 for a normal maximum, the position of the leading bit for a subnormal one
  const int ef = (int)(mx >> 23);
  const int ex = ef > 0 ? ef - 126 : (32 - __clz(mx)) - 149;
  const int shift = min(QBITS - ex, 149);          // |x| * 2^shift <= 2^QBITS; unit = 2^-shift stays a float
  const int sh1 = shift / 2, sh2 = shift - sh1;    // two factors that are always normal floats
  const float p1 = __int_as_float((127 + sh1) << 23), p2 = __int_as_float((127 + sh2) << 23);
  uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
  for (int e = 0; e < 4; e++) {
    // round to nearest through the 1.5 * 2^23 offset (|q| <= 2^20)
    const int q = (int)(__float_as_uint(fmaf(v[e] * p1, p2, 12582912.0f)) - 0x4B400000u);
    const int a = ((q + 64) & 127) - 64;
    const int q1 = (q - a) >> 7;
    w0 |= (uint32_t)(a & 0xFF) << (8 * e);
    if (PLANES == 2) {
      w1 |= (uint32_t)(q1 & 0xFF) << (8 * e);      // |q1| <= 64: the top digit needs no further split
    } else {
      const int b = ((q1 + 64) & 127) - 64;
      const int c = (q1 - b) >> 7;
      w1 |= (uint32_t)(b & 0xFF) << (8 * e);
      w2 |= (uint32_t)(c & 0xFF) << (8 * e);
    }
  }
  const size_t Kp = (size_t)G * QT_UNIT_K;     // row stride of the digit matrix (whole units)
  int8_t* block = digits + (size_t)xi * NB * Kp;
  if (k < K) {               // K is a multiple of 16: a group of four lies inside or outside
    *reinterpret_cast<uint32_t*>(block + (size_t)(0 * MB + m) * Kp + k) = w0;
    *reinterpret_cast<uint32_t*>(block + (size_t)(1 * MB + m) * Kp + k) = w1;
    if (PLANES == 3) *reinterpret_cast<uint32_t*>(block + (size_t)(2 * MB + m) * Kp + k) = w2;
  }
  if (lane == 0) {
    // 2^-shift, possibly a subnormal float (exact); NaN marks a unit holding inf or NaN
    float unit = shift <= 126 ? __int_as_float((127 - shift) << 23) : __int_as_float(1 << (149 - shift));
    if (bad) unit = __int_as_float(0x7FC00000);
    unit_rows[((size_t)xi * G + u) * 16 + m] = unit;
  }
#ifdef CB_QT_STAMPS
  if (dbg && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) dbg[2] = global_ns();
#endif
}

// ---------------------------------------------------------------------------
// schedule helpers (the same arithmetic on every CTA)
// ---------------------------------------------------------------------------
// split schedule: every CTA takes an equal share of the units; tiles shared between CTAs are fixed up at the end
__device__ __forceinline__ long long qt_first_unit(long long total, int grid, int cta) {
  return (total * cta) / grid;
}
// the CTA whose range [first(c), first(c+1)) holds unit u
__device__ __forceinline__ int qt_cta_of(long long total, int grid, long long u) {
  int c = (int)(((u + 1) * grid - 1) / total);
  if (c >= grid) c = grid - 1;
  while (c > 0 && qt_first_unit(total, grid, c) > u) c--;
  while (c + 1 < grid && qt_first_unit(total, grid, c + 1) <= u) c++;
  return c;
}
// Whole-tile schedule: CTA c takes the column tiles c, c + grid, c + 2 grid, ...  At any moment neighbouring
// CTAs therefore stream neighbouring column tiles of the same weight rows, as the CTAs of a single-wave
// launch do: the 256-byte requests the tensor copies are promoted to in L2 are used by both neighbours
// while they are still cached (with a run of consecutive tiles per CTA the second half was evicted before
// its turn: 1.29 x the weight bytes came from DRAM), and the DRAM pages of a weight row are read together.
__device__ __forceinline__ int qt_whole_tiles_of(const QtParams& p, int grid, int cta) {
  return cta < p.tiles_total ? (p.tiles_total - cta + grid - 1) / grid : 0;
}

// The first failure is the one reported (later ones are its consequences): code, then the unit it happened at.
__device__ __forceinline__ void qt_fail(const QtParams& p, unsigned code, unsigned detail) {
  if (atomicCAS(&p.status[0], 0u, code) == 0u) atomicExch(&p.status[1], detail | (blockIdx.x << 16));
}

// Position of a role thread in its CTA's sequence of (column tile, k unit) pairs: the tile counts over
// the whole launch, `pi` is the problem the tile belongs to, `step` the distance to the CTA's next tile
// (1 in the split schedule, the grid size in the whole-tile schedule).
struct QtWalk {
  int tile, g, pi, tile_end, step;
};
__device__ __forceinline__ void qt_walk_init(QtWalk& w, const QtParams& p, int tile0, int g0, int step) {
  w.tile = tile0; w.g = g0; w.pi = 0; w.step = step;
  while (w.pi + 1 < p.n_problems && tile0 >= p.tile_start[w.pi + 1]) w.pi++;
  w.tile_end = p.tile_start[w.pi + 1];
}
// one unit further; true when the walk entered another problem
__device__ __forceinline__ bool qt_walk_next(QtWalk& w, const QtParams& p, int G) {
  if (++w.g < G) return false;
  w.g = 0;
  w.tile += w.step;
  if (w.tile < w.tile_end || w.tile >= p.tiles_total) return false;
  while (w.pi + 1 < p.n_problems && w.tile >= p.tile_start[w.pi + 1]) w.pi++;
  w.tile_end = p.tile_start[w.pi + 1];
  return true;
}
// act(v[m]) -> out[m, n] for the rows that exist, called by the 128 threads of the first epilogue
// group together.  The activation is chosen once, outside the row loop, so the MB rows are
// independent instruction streams; for 16-bit outputs SiLU uses the hardware exp and reciprocal
// (error far below one unit of the output).  The tile is staged in shared memory and leaves in
// 16-byte pieces (256 contiguous bytes per row), to the result buffer of every rank of a gathered plan.
template <int MB, int ACT, bool BF16>
__device__ __forceinline__ void qt_store_rows_act(const float* v, const QtParams& p, const QtProblem* pp, int tile_n0, int nl, uint8_t* stage) {
#pragma unroll
  for (int m = 0; m < MB; m++) {
    float y;
    if (ACT == CB_ACT_SILU && BF16) y = __fdividef(v[m], 1.0f + __expf(-v[m]));
    else y = apply_activation(v[m], ACT);
    if (BF16) reinterpret_cast<uint16_t*>(stage)[m * QT_TILE_N + nl] = f32_to_bf16_bits(y);
    else reinterpret_cast<float*>(stage)[m * QT_TILE_N + nl] = y;
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  constexpr int ESIZE = BF16 ? 2 : 4;
  constexpr int EPC = 16 / ESIZE;              // elements per 16-byte piece
  constexpr int CPR = QT_TILE_N / EPC;         // pieces per row
  const int N = pp->N, out_ld = pp->out_ld, out_col0 = pp->out_col0;
  for (int idx = nl; idx < MB * CPR; idx += 128) {
    const int m = idx / CPR, c = idx - m * CPR;
    const int col = tile_n0 + c * EPC;
    if (m < p.M && col < N) {                  // N is a multiple of 16: a piece lies inside or outside
      const uint4 val = *reinterpret_cast<const uint4*>(stage + ((size_t)m * QT_TILE_N + c * EPC) * ESIZE);
      const size_t off = ((size_t)m * out_ld + out_col0 + col) * ESIZE;
      for (int r = 0; r < p.n_outs; r++)       // own buffer, and the peers' over NVLink for a gathered plan
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pp->outs[r]) + off) = val;
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");   // the staging tile may be rewritten
}
template <int MB, bool BF16>
__device__ __forceinline__ void qt_store_rows(const float* v, const QtParams& p, const QtProblem* pp, int tile_n0, int nl, uint8_t* stage) {
  switch (pp->activation) {
    case CB_ACT_GELU: qt_store_rows_act<MB, CB_ACT_GELU, BF16>(v, p, pp, tile_n0, nl, stage); break;
    case CB_ACT_RELU: qt_store_rows_act<MB, CB_ACT_RELU, BF16>(v, p, pp, tile_n0, nl, stage); break;
    case CB_ACT_SILU: qt_store_rows_act<MB, CB_ACT_SILU, BF16>(v, p, pp, tile_n0, nl, stage); break;
    case CB_ACT_HARDSWISH: qt_store_rows_act<MB, CB_ACT_HARDSWISH, BF16>(v, p, pp, tile_n0, nl, stage); break;
    case CB_ACT_TANH: qt_store_rows_act<MB, CB_ACT_TANH, BF16>(v, p, pp, tile_n0, nl, stage); break;
    default: qt_store_rows_act<MB, CB_ACT_NONE, BF16>(v, p, pp, tile_n0, nl, stage); break;
  }
}

// ---------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------
// global -> shared copy of `bytes` (a multiple of 16, both addresses 16-byte aligned), counted on an mbarrier
__device__ __forceinline__ void qt_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// NB: MMA N extent = PLANES digit planes of MB = NB / PLANES rows
//     (three planes: 16 -> 5 rows, 32 -> 10, 48 -> 16; two planes: 16 -> 8, 32 -> 16).
template <int NB, int PLANES, int MAXP>
__global__ void __launch_bounds__(QT_THREADS, 1)
qdense_decode_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ QtTable<MAXP> table, const QtParams p) {
  constexpr int MB = NB / PLANES;
  constexpr int X_BYTES = NB * QT_UNIT_K;
  constexpr int STAGE_BYTES = QT_W_BYTES + X_BYTES;
  constexpr int STAGES = qt_stages(NB, PLANES);
  constexpr int NACC = qt_accs(NB);
  static_assert(NACC * NB <= QT_TMEM_COLS, "accumulators exceed tensor memory");
  static_assert(STAGES % 2 == 0 && NACC % 2 == 0, "both rings must be even (see the note on parity waits)");
  static_assert((2 * STAGES + 3 * NACC) * 8 <= QT_BAR_BYTES, "barrier area");
  extern __shared__ uint8_t qt_smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(qt_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                         // [STAGES] TMA -> MMA: weights and digits of a unit have landed
  uint64_t* stage_empty = full + STAGES;         // [STAGES] MMA done -> producers: the stage may be refilled
  uint64_t* acc_full = stage_empty + STAGES;     // [NACC]  MMA done -> epilogue
  uint64_t* acc_empty = acc_full + NACC;         // [NACC]  epilogue -> MMA issuers and slot producers
  uint64_t* sc_full = acc_empty + NACC;          // [NACC]  scales and unit[m,u] of a unit have landed
  uint8_t* slots = base + STAGES * STAGE_BYTES + QT_BAR_BYTES;                             // [NACC][640]
  float* s_merge = reinterpret_cast<float*>(slots + NACC * QT_SLOT_BYTES);                 // [MB][128]
  uint8_t* s_stage = reinterpret_cast<uint8_t*>(s_merge + MB * QT_TILE_N);                 // [MB][128] output elements
  __shared__ uint32_t s_tmem;
  __shared__ unsigned s_failed;
  __shared__ unsigned s_last;

  // Lets a following digit kernel of this library be scheduled early (it waits for this grid to
  // finish before it reads or writes anything); kernels launched the ordinary way are unaffected.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef CB_QT_STAMPS
#define QT_STAMP(i) do { if (p.dbg) p.dbg[(size_t)blockIdx.x * 8 + (i)] = global_ns(); } while (0)
#else
#define QT_STAMP(i) do { } while (0)
#endif
  if (tid == 0) QT_STAMP(0);
  const int G = p.units_per_tile;
  int n_units, tile0, g0, tile_step;
  if (p.whole_tiles) {
    n_units = qt_whole_tiles_of(p, gridDim.x, blockIdx.x) * G;
    tile0 = blockIdx.x; g0 = 0; tile_step = gridDim.x;
  } else {
    const long long u0 = qt_first_unit(p.total_units, gridDim.x, blockIdx.x);
    n_units = (int)(qt_first_unit(p.total_units, gridDim.x, blockIdx.x + 1) - u0);
    tile0 = (int)(u0 / G); g0 = (int)(u0 - (long long)tile0 * G); tile_step = 1;
  }
  const QtProblem* const problems = table.p;

  if (warp == QT_TMA_WARP && lane == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&stage_empty[s], 1); }
    fence_barrier_init();
    prefetch_tensormap(&tmap_x);
  }
  if (tid == 0) {
    for (int a = 0; a < NACC; a++) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); mbar_init(&sc_full[a], 1); }
    s_failed = 0;
    fence_barrier_init();
  }
  if (warp == QT_MMA_WARP) tmem_alloc(&s_tmem, QT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;
  // Everything above overlaps the kernels before this one in the stream.  The threads that read what
  // those kernels produce (digits, unit[m,u]) or write what they may still use (output, workspace)
  // wait for them here; the weight producers and the MMA issuers, which touch only weights, shared
  // memory and tensor memory, do not: with a programmatic dependent launch the first STAGES weight
  // tiles are requested while the digit kernel still runs.
  // (Requesting them before the barrier above, by one thread, held the whole CTA back and was slower.)
  if (warp < QT_TMA_WARP || warp == QT_SIDE_WARP || warp == QT_SIDE2_WARP || warp == QT_SCALE_WARP || warp == QT_SCALE2_WARP)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid == 0) QT_STAMP(1);

  if (warp == QT_TMA_WARP || warp == QT_TMA2_WARP || warp == QT_SIDE_WARP || warp == QT_SIDE2_WARP) {
    // ------------------------------ TMA producers: weights, digits ----------------------
    // Issuing one tensor copy keeps a thread busy for several hundred cycles, more than half of what
    // a unit's bytes take to arrive, so every kind of load has two issuing threads in different
    // warps, one for the even units and one for the odd ones.  The weight producer announces the
    // stage's bytes; the digit tile counts towards the same barrier.
    if (lane == 0) {
      const int mine = (warp == QT_TMA_WARP || warp == QT_SIDE_WARP) ? 0 : 1;
      const bool digits = warp == QT_SIDE_WARP || warp == QT_SIDE2_WARP;
      QtWalk w;
      qt_walk_init(w, p, tile0, g0, tile_step);
      const CUtensorMap* map = &problems[w.pi].tmap_w;
      if (!digits) prefetch_tensormap(map);
      for (int it = 0; it < n_units; it++) {
        if ((it & 1) == mine) {
          const int s = it % STAGES;
          if (it >= STAGES) {
            if (!mbar_wait(&stage_empty[s], (uint32_t)((it / STAGES - 1) & 1))) { qt_fail(p, digits ? 5 : 1, (unsigned)it); atomicExch(&s_failed, 1u); break; }
          }
          if (digits) {
            tma_load_2d(base + s * STAGE_BYTES + QT_W_BYTES, &tmap_x, w.g * QT_UNIT_K, p.digit_row0[w.pi], &full[s]);        // [NB rows][128 k]
          } else {
            mbar_expect_tx(&full[s], STAGE_BYTES);
            tma_load_2d(base + s * STAGE_BYTES, map, (w.tile - p.tile_start[w.pi]) * QT_TILE_N, w.g * QT_UNIT_K, &full[s]);
          }
        }
        if (qt_walk_next(w, p, G)) map = &problems[w.pi].tmap_w;
      }
    }
  } else if (warp == QT_SCALE_WARP || warp == QT_SCALE2_WARP) {
    // ------------------------------ producers: scales and unit[m,u] ---------------------
    // A unit's 128 scales and 16 unit[m,u] sit in the slot of the unit's accumulator, which the
    // epilogue releases together with the accumulator.
    if (lane == 0) {
      const int mine = warp == QT_SCALE_WARP ? 0 : 1;
      const int gpr = p.scale_group ? p.scale_group / QT_UNIT_K : 0;    // units per scale row
      QtWalk w;
      qt_walk_init(w, p, tile0, g0, tile_step);
      const CUtensorMap* map = &problems[w.pi].tmap_s;
      prefetch_tensormap(map);
      int srow = gpr ? g0 / gpr : 0, sub = gpr ? g0 - srow * gpr : 0;
      for (int it = 0; it < n_units; it++) {
        if ((it & 1) == mine) {
          const int a = it % NACC;
          if (it >= NACC) {
            if (!mbar_wait(&acc_empty[a], (uint32_t)((it / NACC - 1) & 1))) { qt_fail(p, 6, (unsigned)it); atomicExch(&s_failed, 1u); break; }
          }
          uint8_t* slot = slots + a * QT_SLOT_BYTES;
          mbar_expect_tx(&sc_full[a], QT_SC_BYTES + QT_UN_BYTES);
          tma_load_2d(slot, map, (w.tile - p.tile_start[w.pi]) * QT_TILE_N, srow, &sc_full[a]);
          qt_bulk_load(slot + QT_SC_BYTES, p.unit_rows[w.pi] + (size_t)w.g * 16, QT_UN_BYTES, &sc_full[a]);
        }
        if (gpr && ++sub == gpr) { sub = 0; srow++; }
        if (w.g == G - 1) { srow = 0; sub = 0; }
        if (qt_walk_next(w, p, G)) map = &problems[w.pi].tmap_s;
      }
    }
  } else if (warp == QT_MMA_WARP || warp == QT_MMA2_WARP) {
    // ------------------------------ MMA issuers -------------------------------
    // Issuing a unit (two waits, four MMAs, two commits) costs a single thread several hundred
    // cycles, about what the unit's bytes take to arrive: two threads take the even and the odd units.
    if (lane == 0) {
      const int mine = warp == QT_MMA_WARP ? 0 : 1;
      // W: MN-major, 128 n bytes per k row, 8-row groups 1024 bytes apart, 32 k rows (4096 bytes) per MMA.
      // digits: K-major, 128 k bytes per row, 8-row groups 1024 bytes apart, 32 bytes per MMA.
      // The address field of a descriptor counts 16-byte units, so stepping is an add.
      const uint64_t da0 = smem_desc_sw128(smem_u32(base), QT_W_BYTES, 1024);
      const uint64_t db0 = smem_desc_sw128(smem_u32(base) + QT_W_BYTES, 16, 1024);
      const uint32_t idesc = p.idesc;
      for (int it = mine; it < n_units; it += 2) {
        const int s = it % STAGES, a = it % NACC;
        if (!mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1))) { qt_fail(p, 3, (unsigned)it); atomicExch(&s_failed, 1u); break; }
        if (it >= NACC) {
          if (!mbar_wait(&acc_empty[a], (uint32_t)((it / NACC - 1) & 1))) { qt_fail(p, 7, (unsigned)it); atomicExch(&s_failed, 1u); break; }
        }
        tc_fence_after();
        const uint64_t da = da0 + (uint64_t)((s * STAGE_BYTES) >> 4), db = db0 + (uint64_t)((s * STAGE_BYTES) >> 4);
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * NB);
#pragma unroll
        for (int j = 0; j < QT_UNIT_K / 32; j++)
          umma_i8(d_tmem, da + (uint64_t)((j * 32 * 128) >> 4), db + (uint64_t)((j * 32) >> 4), idesc, j > 0 ? 1u : 0u);
        umma_commit(&stage_empty[s]);      // the stage goes back to the producers as soon as the MMAs have read it
        umma_commit(&acc_full[a]);
      }
    }
  } else {
    // ------------------------------ epilogue (warps 0-7) ----------------------
    // Two groups of four warps take the even and the odd units, so that one group's TMEM load and
    // barrier round trips hide behind the other's arithmetic.  Each thread owns one output column of
    // the tile (TMEM lane) and keeps MB running totals; at the end of the CTA's share of a tile the
    // second group hands its totals to the first through shared memory.
    const int grp = warp >> 2, quarter = warp & 3;
    const int nl = quarter * 32 + lane;             // column within the tile = TMEM lane
    const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float tot[MB];
#pragma unroll
    for (int m = 0; m < MB; m++) tot[m] = 0.0f;
    bool failed = false;
    QtWalk w;
    qt_walk_init(w, p, tile0, g0, tile_step);
    for (int it = 0; it < n_units; it++) {
      // After a timeout this group stops touching the pipeline but keeps walking the units, so that
      // the barriers below still see every thread (the status word reports the failure).
      const bool own = (it & 1) == grp;
      if (own && !failed) {
        const int a = it % NACC;
        const uint32_t parity = (uint32_t)((it / NACC) & 1);
        if (!mbar_wait(&sc_full[a], parity) || !mbar_wait(&acc_full[a], parity)) failed = true;
      }
      if (own && !failed) {
        const int a = it % NACC;
        tc_fence_after();
        uint32_t acc[NB];
#pragma unroll
        for (int c = 0; c < NB / 16; c++) tmem_ld16(tlane + (uint32_t)(a * NB + c * 16), *reinterpret_cast<uint32_t(*)[16]>(&acc[c * 16]));
        const float* slot = reinterpret_cast<const float*>(slots + a * QT_SLOT_BYTES);
        const float sc = slot[nl];                                        // zero beyond column N (TMA fill)
        float un[MB];
#pragma unroll
        for (int m = 0; m < MB; m++) un[m] = slot[QT_TILE_N + m];
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[a]);
        // s32 -> f32 through the 1.5 * 2^23 offset (|sum| < 2^22), digits recombined, unit and group scale applied
#pragma unroll
        for (int m = 0; m < MB; m++) {
          const float f0 = __uint_as_float(acc[m] + 0x4B400000u) - 12582912.0f;
          const float f1 = __uint_as_float(acc[MB + m] + 0x4B400000u) - 12582912.0f;
          float q = fmaf(f1, 128.0f, f0);
          if (PLANES == 3) {
            const float f2 = __uint_as_float(acc[(PLANES - 1) * MB + m] + 0x4B400000u) - 12582912.0f;
            q = fmaf(f2, 16384.0f, q);
          }
          tot[m] = fmaf(q * un[m], sc, tot[m]);
        }
      }
      const int tile = w.tile, g = w.g;
      const bool tile_ends = (g == G - 1);
      const bool final_seg = it + 1 == n_units;
      if (tile_ends || final_seg) {
        // ---- end of this CTA's share of the tile ----
        if (tid == 0 && final_seg) QT_STAMP(2);
        if (grp == 1) {
#pragma unroll
          for (int m = 0; m < MB; m++) s_merge[m * QT_TILE_N + nl] = tot[m];
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (grp == 0) {
#pragma unroll
          for (int m = 0; m < MB; m++) tot[m] += s_merge[m * QT_TILE_N + nl];
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");      // s_merge may be rewritten
        if (grp == 0) {
          const QtProblem* pp = &problems[w.pi];
          const int tile_n0 = (tile - p.tile_start[w.pi]) * QT_TILE_N;
          const int n = tile_n0 + nl;
          const bool whole = tile_ends && (it >= g);          // the tile's first unit is ours too
          bool write = true;
          if (!whole && p.cluster > 1) {
            // the tile's CTAs are one cluster: the partial tile stays in this CTA's shared memory (s_merge is free again
            // after the barrier above) and the cluster's first CTA sums all of them after the cluster barrier at the end
#pragma unroll
            for (int m = 0; m < MB; m++) s_merge[m * QT_TILE_N + nl] = tot[m];
            write = false;
          } else if (!whole) {
            // park the partial tile, count the arrival; the last CTA to arrive sums all of them in CTA order
            const int slot = (tile == tile0) ? 0 : 1;         // first or last share of this CTA's range
            float* mine = p.partials + ((size_t)(blockIdx.x * 2 + slot) * MB) * QT_TILE_N;
#pragma unroll
            for (int m = 0; m < MB; m++) mine[m * QT_TILE_N + nl] = tot[m];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tid == 0 && final_seg) QT_STAMP(5);
            const long long tile_first = (long long)tile * G;
            const int c_first = qt_cta_of(p.total_units, gridDim.x, tile_first);
            const int c_last = qt_cta_of(p.total_units, gridDim.x, tile_first + G - 1);
            if (tid == 0) {
              __threadfence();      // after the barrier: cumulative over the partial tile the group just wrote
              const unsigned old = atomicAdd(&p.counters[tile], 1u);
              s_last = (old == (unsigned)(c_last - c_first)) ? 1u : 0u;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            write = s_last != 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");      // s_last is rewritten at the next shared tile
            if (tid == 0 && final_seg) QT_STAMP(6);
            if (write) {
              __threadfence();
#pragma unroll
              for (int m = 0; m < MB; m++) tot[m] = 0.0f;
              // two contributors per round, their loads in flight together; summed in CTA order
              for (int c = c_first; c <= c_last; c += 2) {
                const bool two = c + 1 <= c_last;
                const int slot_a = (qt_first_unit(p.total_units, gridDim.x, c) / G == tile) ? 0 : 1;
                const int slot_b = (two && qt_first_unit(p.total_units, gridDim.x, c + 1) / G == tile) ? 0 : 1;
                const float* pa = p.partials + ((size_t)(c * 2 + slot_a) * MB) * QT_TILE_N + nl;
                const float* pb = p.partials + ((size_t)((two ? c + 1 : c) * 2 + slot_b) * MB) * QT_TILE_N + nl;
                float va[MB], vb[MB];
#pragma unroll
                for (int m = 0; m < MB; m++) { va[m] = __ldcg(pa + m * QT_TILE_N); vb[m] = __ldcg(pb + m * QT_TILE_N); }
#pragma unroll
                for (int m = 0; m < MB; m++) { tot[m] += va[m]; if (two) tot[m] += vb[m]; }
              }
              if (tid == 0) p.counters[tile] = 0;     // the workspace stays ready for the next launch
              if (tid == 0 && final_seg) QT_STAMP(7);
            }
          }
          if (write) {
            const float* bias_p = pp->bias;
            const float bias = (bias_p && n < pp->N) ? __ldg(bias_p + n) : 0.0f;
#pragma unroll
            for (int m = 0; m < MB; m++) tot[m] += bias;
            if (p.out_bf16) qt_store_rows<MB, true>(tot, p, pp, tile_n0, nl, s_stage);
            else qt_store_rows<MB, false>(tot, p, pp, tile_n0, nl, s_stage);
          }
        }
#pragma unroll
        for (int m = 0; m < MB; m++) tot[m] = 0.0f;
      }
      qt_walk_next(w, p, G);
    }
    if (tid == 0) QT_STAMP(3);
    if (failed) { qt_fail(p, 4, (unsigned)(warp)); atomicExch(&s_failed, 1u); }
  }
  // every role ends here; TMEM is released by the warp that allocated it
  tc_fence_before();
  __syncthreads();
  if (s_failed) {
    // A wait gave up: tensor copies this CTA requested may still be in flight towards its shared
    // memory.  They complete within microseconds of their request; leave them a bounded 200 us.
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (p.cluster > 1) {
    // ---- the tile's partial sums, through distributed shared memory ----
    // Every thread of every CTA of the cluster passes both barriers (no role returns early, and every wait above is
    // bounded).  First barrier: all partial tiles are in place.  The first CTA's first epilogue group then reads them
    // in CTA order (the sum does not depend on timing) and arrives at the second barrier, which keeps the other
    // CTAs' shared memory alive until it has been read; the result is stored while the others leave.
    cluster_arrive();
    cluster_wait();
    const bool leader = (blockIdx.x % (unsigned)p.cluster) == 0 && warp < 4;
    float tot[MB];
    if (leader) {
      const uint32_t local = smem_u32(s_merge) + (uint32_t)tid * 4;
#pragma unroll
      for (int m = 0; m < MB; m++) tot[m] = s_merge[m * QT_TILE_N + tid];
      for (int r = 1; r < p.cluster; r++) {
        const uint32_t remote = cluster_map(local, (uint32_t)r);
        float v[MB];
#pragma unroll
        for (int m = 0; m < MB; m++) v[m] = ld_cluster_f32(remote + (uint32_t)(m * QT_TILE_N * 4));
#pragma unroll
        for (int m = 0; m < MB; m++) tot[m] += v[m];
      }
    }
    cluster_arrive();
    if (leader) {
      QtWalk w;
      qt_walk_init(w, p, tile0, g0, tile_step);
      const QtProblem* pp = &problems[w.pi];
      const int tile_n0 = (tile0 - p.tile_start[w.pi]) * QT_TILE_N;
      const int n = tile_n0 + tid;
      const float bias = (pp->bias && n < pp->N) ? __ldg(pp->bias + n) : 0.0f;
#pragma unroll
      for (int m = 0; m < MB; m++) tot[m] += bias;
      if (p.out_bf16) qt_store_rows<MB, true>(tot, p, pp, tile_n0, tid, s_stage);
      else qt_store_rows<MB, false>(tot, p, pp, tile_n0, tid, s_stage);
    }
    cluster_wait();
  }
  if (warp == QT_MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, QT_TMEM_COLS);
  }
  if (tid == 0) QT_STAMP(4);
#undef QT_STAMP
}

// ---------------------------------------------------------------------------
// waiting for the slices of the other ranks
// ---------------------------------------------------------------------------
// One thread per flag polls it (system scope) until it has reached `target` (compared modulo 2^32) or
// about two seconds have passed; a timeout leaves 1 + flag index in the status word.  The flags are
// written by kernels running on other GPUs, never by kernels of this GPU that might be queued behind
// this one.
__global__ void peer_wait_kernel(const unsigned* flags, int n_flags, unsigned target, unsigned* status_word) {
  const int i = threadIdx.x;
  if (i >= n_flags) return;
  const volatile unsigned* f = flags + i;
  const unsigned long long t0 = global_ns();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int)(v - target) >= 0) break;
    if (global_ns() - t0 > WAIT_NS) { atomicExch(status_word, 1u + (unsigned)i); break; }
    __nanosleep(200);
  }
}

// Runs after the kernels whose peer stores it announces (same stream): when it starts, those
// kernels have completed and their stores have been performed; it adds 1 to word `slot` of the flag
// array of every rank.
struct PeerFlags { unsigned* f[QT_MAX_RANKS]; };
__global__ void peer_signal_kernel(PeerFlags flags, int n_ranks, int slot) {
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < n_ranks; r++) atomicAdd_system(flags.f[r] + slot, 1u);
  }
}

// Both steps in one launch, chained to the kernels before and after it by programmatic dependent launch (its
// launch latency overlaps the tail of the kernel whose stores it announces, and the next kernel of the stream is
// scheduled while it polls): signals once the preceding kernels have completed, then waits for every rank.
__global__ void peer_signal_wait_kernel(PeerFlags flags, int n_ranks, int slot, const unsigned* local, unsigned target, unsigned* status_word) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < n_ranks; r++) atomicAdd_system(flags.f[r] + slot, 1u);
  }
  const int i = threadIdx.x;
  if (i >= n_ranks) return;
  const unsigned long long t0 = global_ns();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local + i) : "memory");
    if ((int)(v - target) >= 0) break;
    if (global_ns() - t0 > WAIT_NS) { atomicExch(status_word, 1u + (unsigned)i); break; }
    __nanosleep(100);
  }
}

int peer_signal_wait_launch(void* const* flags, int n_ranks, int slot, const unsigned* local, uint32_t target, unsigned* status_word, cudaStream_t s) {
  if (n_ranks < 1 || n_ranks > QT_MAX_RANKS) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal_wait: %d ranks", n_ranks);
  PeerFlags pf;
  for (int r = 0; r < QT_MAX_RANKS; r++) pf.f[r] = r < n_ranks ? (unsigned*)flags[r] : nullptr;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB_CUDA(cudaLaunchKernelEx(&cfg, peer_signal_wait_kernel, pf, n_ranks, slot, local, (unsigned)target, status_word));
  return CB_OK;
}

int peer_signal_launch(void* const* flags, int n_ranks, int slot, cudaStream_t s) {
  if (n_ranks < 1 || n_ranks > QT_MAX_RANKS) return fail(CB_ERR_INVALID_ARG, "cb_peer_signal: %d ranks", n_ranks);
  PeerFlags pf;
  for (int r = 0; r < QT_MAX_RANKS; r++) pf.f[r] = r < n_ranks ? (unsigned*)flags[r] : nullptr;
  peer_signal_kernel<<<1, 32, 0, s>>>(pf, n_ranks, slot);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

int peer_wait_launch(const unsigned* flags, int n_flags, uint32_t target, unsigned* status_word, cudaStream_t s) {
  peer_wait_kernel<<<1, 32, 0, s>>>(flags, n_flags, target, status_word);
  CB_CUDA(cudaGetLastError());
  return CB_OK;
}

// ---------------------------------------------------------------------------
// planning and launch
// ---------------------------------------------------------------------------
// Digit planes and MMA N extent by activation type and batch.  Up to five rows three planes fit the
// narrowest MMA (16) for either type; beyond that bfloat16 needs only two planes (8 rows in 16, 16 in 32).
static int qt_planes(const cb_qdense_desc& d) { return (d.x_dtype == CB_BF16 && d.M > 5) ? 2 : 3; }
static int qt_nb(const cb_qdense_desc& d) {
  if (qt_planes(d) == 2) return d.M <= 8 ? 16 : 32;
  return d.M <= 5 ? 16 : (d.M <= 10 ? 32 : 48);
}
static size_t qt_align(size_t v) { return (v + 255) & ~(size_t)255; }
static int qt_smem(int nb, int planes) {
  return 1024 + qt_stages(nb, planes) * (QT_W_BYTES + nb * QT_UNIT_K) + qt_tail_bytes(nb, planes);
}

bool qdense_decode_tc_eligible(const cb_qdense_desc& d, std::string* why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  if (d.M < 1 || d.M > 16) return no("M must be in [1,16]");
  if (d.has_zero_point) return no("zero points are handled by the generic kernel");
  if (d.scale_layout == CB_SCALE_REF) return no("reference [K, N/block] scales are handled by the generic kernel");
  if (d.K < 16 || d.K % 16 != 0) return no("K must be a positive multiple of 16");
  if (d.N < 16 || d.N % 16 != 0) return no("N must be a positive multiple of 16");
  if (d.scale_layout == CB_SCALE_KGROUP && (d.block_size <= 0 || d.block_size % QT_UNIT_K != 0))
    return no("K-group size must be a multiple of 128");
  if (d.K > (1 << 30) || d.N > (1 << 30)) return no("dimension too large");
  if (d.gather_ranks > QT_MAX_RANKS) return no("a gathered plan spans at most 8 ranks");
  if (d.gather_ranks > 1 && (d.gather_rank < 0 || d.gather_rank >= d.gather_ranks)) return no("gather_rank out of range");
  return true;
}

struct QtLayout {
  int nb, mb, planes, n_problems, tiles_total, units_per_tile;
  int tile_start[QT_MAX_PROBLEMS + 1];
  long long total_units;
  size_t off_counters, off_digits, off_units, zero_bytes, off_partials, off_stamps, total;
};

static QtLayout qt_layout(const cb_plan* p, int blocks) {
  const cb_qdense_desc& d = p->qd;
  QtLayout l;
  l.planes = qt_planes(d);
  l.nb = qt_nb(d);
  l.mb = l.nb / l.planes;
  l.n_problems = (int)p->group.size();
  l.tiles_total = 0;
  for (int i = 0; i < l.n_problems; i++) {
    l.tile_start[i] = l.tiles_total;
    l.tiles_total += (int)((p->group[i].N + QT_TILE_N - 1) / QT_TILE_N);
  }
  for (int i = l.n_problems; i <= QT_MAX_PROBLEMS; i++) l.tile_start[i] = l.tiles_total;
  l.units_per_tile = (int)((d.K + QT_UNIT_K - 1) / QT_UNIT_K);
  l.total_units = (long long)l.tiles_total * l.units_per_tile;
  l.off_counters = QT_HEADER;
  l.off_digits = qt_align(l.off_counters + (size_t)l.tiles_total * 4);
  // one block of [NB digit rows][128 * units] per problem, then 16 unit[m,u] per problem and unit.
  // Counters, digits and unit[m,u] start as zeros (rows beyond M are never written).
  l.off_units = qt_align(l.off_digits + (size_t)l.n_problems * l.nb * l.units_per_tile * QT_UNIT_K);
  l.zero_bytes = qt_align(l.off_units + (size_t)l.n_problems * l.units_per_tile * QT_UN_BYTES);
  l.off_partials = l.zero_bytes;
  l.off_stamps = qt_align(l.off_partials + (size_t)blocks * 2 * l.mb * QT_TILE_N * 4);
  l.total = l.off_stamps;
#ifdef CB_QT_STAMPS
  l.total += (size_t)blocks * 8 * 8 + 64;
#endif
  return l;
}

// How many clusters of r CTAs of the main kernel the device holds at once: the CTAs of a cluster need r free SMs of one
// GPC, so this is less than n_sm / r in general.  0 when it cannot be asked (a plan made without a device).  All
// instances of the kernel have the same footprint (512 threads, all of an SM's shared memory), so one is asked.
static int qt_resident_clusters(int dev, int r) {
  static std::atomic<int> cache[64][5];
  if (dev < 0 || r < 2 || r > 4 || sm_count(dev) <= 0) return 0;
  if (dev < 64) { const int c = cache[dev][r].load(std::memory_order_acquire); if (c > 0) return c; }
  int cur = 0, n = 0;
  if (cudaGetDevice(&cur) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); return 0; }
  auto kernel = qdense_decode_tc_kernel<32, 2, 1>;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(r * 64));
  cfg.blockDim = dim3(QT_THREADS);
  cfg.dynamicSmemBytes = (size_t)qt_smem(32, 2);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)r; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, qt_smem(32, 2)) != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  cudaSetDevice(cur);
  if (n > 0 && dev < 64) cache[dev][r].store(n, std::memory_order_release);
  return n;
}

static int qt_finish_plan(cb_plan* p) {
  const cb_qdense_desc& d = p->qd;
  long long tiles = 0;
  for (const cb_qdense_member& m : p->group) tiles += (m.N + QT_TILE_N - 1) / QT_TILE_N;
  if (tiles >= (1ll << 30)) return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense: too many column tiles for one launch");
  const long long units = tiles * ((d.K + QT_UNIT_K - 1) / QT_UNIT_K);
  p->blocks = (int)std::min<long long>(p->n_sm, units);
  p->whole_tiles = false;
  // Whole tiles per CTA when that keeps enough of the machine streaming: every CTA takes an equal
  // share of the column tiles (give or take one), so no tile is split and nothing is parked, counted
  // or gathered at the end.  With one wave three eighths of the SMs are enough (measured: 56 tiles on
  // 148 SMs are still faster whole, 28 are not — the fewer, longer streams still saturate HBM); with
  // several waves the grid must cover three quarters of the SMs, else the units are split evenly
  // over all SMs.
  const long long waves = (tiles + p->n_sm - 1) / p->n_sm;
  const long long whole_grid = (tiles + waves - 1) / waves;
  if ((waves == 1 && tiles * 8 >= (long long)p->n_sm * 3) || (waves > 1 && whole_grid * 4 >= (long long)p->n_sm * 3)) {
    p->blocks = (int)whole_grid;
    p->whole_tiles = true;
  }
  // A launch of few column tiles (one projection of a few thousand columns) is bound by its fixed costs, and the
  // largest of them is the end of a split tile: partial tiles parked, counted, gathered by the last CTA.  It is
  // shortest when every tile is shared by the same small number of CTAs, each with an equal run of the tile's k
  // units, all arriving together: with tiles * r CTAs the even deal of units falls on tile boundaries by itself.
  // Measured at K = 4096, 16 rows, microseconds per launch in a chain of launches, r = 1 (whole) / 2 / 4 / more:
  // 8 tiles 14.4 / 13.0 / 11.7 / 12.0 (r = 8), 32 tiles 15.2 / 14.1 / 12.2 / 17.1 (148 CTAs), 56 tiles 15.4 / 13.9;
  // K = 14336, 32 tiles: 39.7 / 26.0 / 20.6 / 23.9 (148 CTAs).
  const long long units_per_tile = (d.K + QT_UNIT_K - 1) / QT_UNIT_K;
  if (waves == 1) {
    // the most CTAs per tile (four at most: more did not pay) that still leave every CTA four units and let all
    // clusters run at once (asked of the device; seven eighths of n_sm / r when there is none to ask)
    long long r = 0;
    for (long long c = 4; c >= 2 && r == 0; c--) {
      const int resident = qt_resident_clusters(p->dev, (int)c);
      const bool fits = resident > 0 ? tiles <= resident : tiles * c * 8 <= (long long)p->n_sm * 7;
      if (fits && units_per_tile >= 4 * c) r = c;
    }
    if (r) { p->blocks = (int)(tiles * r); p->whole_tiles = false; p->tile_cluster = (int)r; }
  }
  const QtLayout l = qt_layout(p, p->blocks);
  p->threads = QT_THREADS;
  p->dyn_smem = qt_smem(l.nb, l.planes);
  p->counter_bytes = l.zero_bytes;
  p->workspace_bytes = l.total;
  p->has_status = true;
  const int g = d.gather_ranks > 1 ? d.gather_ranks : 1;
  p->n_outputs = (int)p->group.size() * g;
  p->name = std::string("qdense_decode_tc_") + (d.x_dtype == CB_BF16 ? "bf16" : "f32") + "_n" + std::to_string(l.nb) +
            (l.planes == 2 ? "p2" : "") + (d.w_dtype == CB_U8 ? "_u8" : "_i8") +
            (p->group.size() > 1 ? "_x" + std::to_string(p->group.size()) : "");
  return CB_OK;
}

int qdense_decode_tc_plan(cb_plan* p) {
  cb_qdense_member m;
  m.N = p->qd.N; m.has_bias = p->qd.has_bias; m.activation = p->qd.activation;
  p->group.assign(1, m);
  return qt_finish_plan(p);
}

int qdense_group_plan(cb_plan* p) {
  cb_qdense_desc& d = p->qd;
  const int n = (int)p->group.size();
  if (n < 1 || n > QT_MAX_PROBLEMS)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense group: %d members (1 to %d allowed)", n, QT_MAX_PROBLEMS);
  if (d.x_dtype != CB_F32 && d.x_dtype != CB_BF16)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: x must be float32 (or bfloat16), got %s", dtype_name(d.x_dtype));
  if (d.scheme != CB_QUANT_LINEAR || (d.w_dtype != CB_I8 && d.w_dtype != CB_U8))
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense group: Linear int8 / uint8 weights only");
  if (d.scale_layout < CB_SCALE_REF || d.scale_layout > CB_SCALE_KGROUP)
    return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown scale layout %d", d.scale_layout);
  int inputs = 0;
  for (int i = 0; i < n; i++) {
    const cb_qdense_member& m = p->group[i];
    if (m.activation < CB_ACT_NONE || m.activation > CB_ACT_TANH)
      return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: unknown activation %d", m.activation);
    cb_qdense_desc one = d;
    one.N = m.N; one.has_bias = m.has_bias; one.activation = m.activation;
    std::string why;
    if (!qdense_decode_tc_eligible(one, &why))
      return fail(CB_ERR_NOT_IMPLEMENTED, "FusedQuantizedDense group, member %d: %s", i, why.c_str());
    inputs += 3 + (m.has_bias ? 1 : 0);
  }
  d.N = p->group[0].N; d.has_bias = p->group[0].has_bias; d.activation = p->group[0].activation;
  d.variant = CB_QDENSE_DECODE_TC;
  p->variant = CB_QDENSE_DECODE_TC;
  p->n_inputs = inputs;
  return qt_finish_plan(p);
}

// cuTensorMapEncodeTiled of a 2-D row-major matrix, remembered per thread: the encoding is a pure
// function of its arguments, and a decode loop asks for the same few maps on every launch.
// bytes == 1: a byte matrix in 128-byte swizzled tiles; bytes == 4: rows of floats, not swizzled
static int qt_encode_2d(CUtensorMap* m, const void* ptr, int bytes, uint64_t d0, uint64_t d1, uint32_t b0, uint32_t b1) {
  struct Entry { const void* ptr; int bytes; uint64_t d0, d1; uint32_t b0, b1; bool valid; CUtensorMap map; };
  constexpr int SLOTS = 64;
  static thread_local Entry cache[SLOTS];
  const uintptr_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull;
  Entry& e = cache[(h >> 40) % SLOTS];
  if (e.valid && e.ptr == ptr && e.bytes == bytes && e.d0 == d0 && e.d1 == d1 && e.b0 == b0 && e.b1 == b1) {
    *m = e.map;
    return CB_OK;
  }
  encode_tiled_fn enc = tensor_map_encoder();
  if (!enc) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {d0 * (uint64_t)bytes};
  cuuint32_t box[2] = {b0, b1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   bytes == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  e.ptr = ptr; e.bytes = bytes; e.d0 = d0; e.d1 = d1; e.b0 = b0; e.b1 = b1; e.map = *m; e.valid = true;
  return CB_OK;
}

// Everything the two launches of a decode call need.
struct QtArgs {
  CUtensorMap tmap_x;
  QtTable<QT_MAX_PROBLEMS> table;          // the first 1, 4 or 16 records travel as kernel parameters
  QtParams prm;
  QtXList xl;
  int8_t* digits;
  float* unit_rows;
  int nb, planes, mb, n_problems, units_per_tile;
  bool bf16;
  unsigned long long* xdbg;                // time stamps of the digit kernel (diagnostic builds only)
};

static int qt_fill_args(const cb_plan* p, const void* const* in, void* const* out, void* ws, QtArgs* a) {
  const cb_qdense_desc& d = p->qd;
  const QtLayout l = qt_layout(p, p->blocks);
  const int g = d.gather_ranks > 1 ? d.gather_ranks : 1;
  uint8_t* w8 = (uint8_t*)ws;
  memset(&a->prm, 0, sizeof(a->prm));
  memset(&a->xl, 0, sizeof(a->xl));
  a->nb = l.nb; a->planes = l.planes; a->mb = l.mb; a->n_problems = l.n_problems; a->units_per_tile = l.units_per_tile;
  a->bf16 = d.x_dtype == CB_BF16;
  a->digits = (int8_t*)(w8 + l.off_digits);
  a->unit_rows = (float*)(w8 + l.off_units);
  const uint64_t scale_rows = d.scale_layout == CB_SCALE_KGROUP ? (uint64_t)((d.K + d.block_size - 1) / d.block_size) : 1;
  const int block_rows = l.nb;
  int ii = 0;
  for (int i = 0; i < l.n_problems; i++) {
    const cb_qdense_member& m = p->group[i];
    const void* x = in[ii], *w = in[ii + 1], *sc = in[ii + 2];
    const void* bias = m.has_bias ? in[ii + 3] : nullptr;
    ii += 3 + (m.has_bias ? 1 : 0);
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(sc) & 15))
      return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: x, weights and scales must be 16-byte aligned");
    QtProblem& q = a->table.p[i];
    memset(&q, 0, sizeof(q));
    CB_TRY(qt_encode_2d(&q.tmap_w, w, 1, (uint64_t)m.N, (uint64_t)d.K, QT_TILE_N, QT_UNIT_K));
    CB_TRY(qt_encode_2d(&q.tmap_s, sc, 4, (uint64_t)m.N, scale_rows, QT_TILE_N, 1));
    q.bias = (const float*)bias;
    for (int r = 0; r < g; r++) {
      void* o = out[i * g + r];
      if (reinterpret_cast<uintptr_t>(o) & 15) return fail(CB_ERR_INVALID_ARG, "FusedQuantizedDense: outputs must be 16-byte aligned");
      q.outs[r] = o;
    }
    q.N = (int)m.N;
    q.out_ld = (int)(m.N * g);
    q.out_col0 = (int)(m.N * (g > 1 ? d.gather_rank : 0));
    q.activation = m.activation;
    // problems given the same x share one block of digits
    int xi = 0;
    while (xi < a->xl.n && a->xl.x[xi] != x) xi++;
    if (xi == a->xl.n) a->xl.x[a->xl.n++] = x;
    a->prm.digit_row0[i] = xi * block_rows;
    a->prm.unit_rows[i] = reinterpret_cast<const float*>(w8 + l.off_units) + (size_t)xi * l.units_per_tile * 16;
  }
  CB_TRY(qt_encode_2d(&a->tmap_x, a->digits, 1, (uint64_t)l.units_per_tile * QT_UNIT_K, (uint64_t)l.n_problems * block_rows,
                      QT_UNIT_K, (uint32_t)block_rows));
  QtParams& prm = a->prm;
  prm.status = (unsigned*)w8;
  prm.counters = (unsigned*)(w8 + l.off_counters);
  prm.partials = (float*)(w8 + l.off_partials);
  prm.M = (int)d.M; prm.K = (int)d.K;
  prm.n_problems = l.n_problems;
  prm.n_outs = g;
  for (int i = 0; i <= QT_MAX_PROBLEMS; i++) prm.tile_start[i] = l.tile_start[i];
  prm.units_per_tile = l.units_per_tile;
  prm.tiles_total = l.tiles_total;
  prm.whole_tiles = p->whole_tiles ? 1 : 0;
  prm.cluster = p->tile_cluster;
  prm.total_units = l.total_units;
  prm.scale_group = d.scale_layout == CB_SCALE_KGROUP ? (int)d.block_size : 0;
  prm.out_bf16 = a->bf16 ? 1 : 0;
  prm.idesc = idesc_i8(QT_TILE_N, l.nb, d.w_dtype == CB_U8 ? 0 : 1, 1, 1, 0);
  a->xdbg = nullptr;
#ifdef CB_QT_STAMPS
  prm.dbg = (unsigned long long*)(w8 + l.off_stamps);
  a->xdbg = prm.dbg + (size_t)p->blocks * 8;
#endif
  return CB_OK;
}

template <int NB, int PLANES, int MAXP>
static int qt_launch_main_t(const cb_plan* p, const QtArgs& a, cudaStream_t s) {
  static std::atomic<bool> configured[64];
  int dev = 0;
  CB_CUDA(cudaGetDevice(&dev));            // the current device: the one this launch goes to
  if (dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    CB_CUDA(cudaFuncSetAttribute(qdense_decode_tc_kernel<NB, PLANES, MAXP>, cudaFuncAttributeMaxDynamicSharedMemorySize, qt_smem(NB, PLANES)));
    if (dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  // programmatic dependent launch: this grid may be scheduled while the digit kernel still runs
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)p->blocks);
  cfg.blockDim = dim3(QT_THREADS);
  cfg.dynamicSmemBytes = (size_t)qt_smem(NB, PLANES);
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p->tile_cluster > 1) {               // the CTAs of a column tile are co-scheduled and see each other's shared memory
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)p->tile_cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  // the first MAXP records of the table (QtTable<MAXP> is a prefix of QtTable<QT_MAX_PROBLEMS>)
  CB_CUDA(cudaLaunchKernelEx(&cfg, qdense_decode_tc_kernel<NB, PLANES, MAXP>, a.tmap_x, *reinterpret_cast<const QtTable<MAXP>*>(&a.table), a.prm));
  return CB_OK;
}
template <int NB, int PLANES>
static int qt_launch_main(const cb_plan* p, const QtArgs& a, cudaStream_t s) {
  if (a.n_problems == 1) return qt_launch_main_t<NB, PLANES, 1>(p, a, s);
  if (a.n_problems <= 4) return qt_launch_main_t<NB, PLANES, 4>(p, a, s);
  return qt_launch_main_t<NB, PLANES, QT_MAX_PROBLEMS>(p, a, s);
}

template <typename XT, int PLANES>
static int qt_launch_digits(const QtArgs& a, int M, int K, cudaStream_t s) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  const int tasks = a.xl.n * M * a.units_per_tile;
  cfg.gridDim = dim3((unsigned)((tasks + QX_THREADS / 32 - 1) / (QX_THREADS / 32)));
  cfg.blockDim = dim3(QX_THREADS);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#ifdef CB_QT_STAMPS
  CB_CUDA(cudaLaunchKernelEx(&cfg, qdense_xdigits_kernel<XT, PLANES>, a.xl, M, K, a.nb, a.units_per_tile, a.digits, a.unit_rows, a.xdbg));
#else
  CB_CUDA(cudaLaunchKernelEx(&cfg, qdense_xdigits_kernel<XT, PLANES>, a.xl, M, K, a.nb, a.units_per_tile, a.digits, a.unit_rows));
#endif
  return CB_OK;
}

static int qt_issue(const cb_plan* p, const QtArgs& a, cudaStream_t s) {
  const int M = (int)p->qd.M, K = (int)p->qd.K;
  if (a.bf16 && a.planes == 2) CB_TRY((qt_launch_digits<__nv_bfloat16, 2>(a, M, K, s)));
  else if (a.bf16) CB_TRY((qt_launch_digits<__nv_bfloat16, 3>(a, M, K, s)));
  else CB_TRY((qt_launch_digits<float, 3>(a, M, K, s)));
  if (a.planes == 2) return a.nb == 16 ? qt_launch_main<16, 2>(p, a, s) : qt_launch_main<32, 2>(p, a, s);
  switch (a.nb) {
    case 16: return qt_launch_main<16, 3>(p, a, s);
    case 32: return qt_launch_main<32, 3>(p, a, s);
    default: return qt_launch_main<48, 3>(p, a, s);
  }
}

int qdense_decode_tc_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  // A heap object: QtArgs carries 16 problem records and would be a large stack frame.
  std::unique_ptr<QtArgs> a(new QtArgs);
  CB_TRY(qt_fill_args(p, in, out, ws, a.get()));
  return qt_issue(p, *a, s);
}

int qdense_decode_tc_bind(const cb_plan* p, const void* const* in, void* const* out, void* ws, void** impl) {
  std::unique_ptr<QtArgs> a(new QtArgs);
  CB_TRY(qt_fill_args(p, in, out, ws, a.get()));
  *impl = a.release();
  return CB_OK;
}

int qdense_decode_tc_launch_bound(const cb_plan* p, const void* impl, cudaStream_t s) {
  return qt_issue(p, *static_cast<const QtArgs*>(impl), s);
}

void qdense_decode_tc_unbind(void* impl) { delete static_cast<QtArgs*>(impl); }

}  // namespace cb
