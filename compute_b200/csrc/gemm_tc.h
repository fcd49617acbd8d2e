// Internal interface of the tcgen05 GEMM (gemm_tcgen05.cu) for the other translation
// units that lower onto it: DotGeneral on float32 operands and the prefill-shaped
// quantized dense.
//
// The kernel multiplies 16-bit operands.  Wider operands are handed over as "planes":
// a float32 tensor v is split into v = p0 + p1 + p2 with p0 = bf16(v), p1 = bf16(v - p0),
// p2 = bf16(v - p0 - p1) (8 mantissa bits each, so three planes carry all 24), the planes of
// an operand are stacked in its batch dimension ([planes * B, rows, cols]) and the kernel
// accumulates a list of (lhs plane, rhs plane) passes into one f32 accumulator in tensor
// memory.  The products it leaves out (p1*p2, p2*p1, p2*p2) are below 2^-24 of |lhs||rhs|.
#pragma once

#include "common.cuh"

namespace cb {

constexpr int GEMM_TC_MAX_PASSES = 6;

struct GemmTcProblem {
  const void* a = nullptr;     // [planes_a * B, M, K] 16-bit
  const void* b = nullptr;     // [planes_b * B, K, N] (rhs_transposed = 0) or [planes_b * B, N, K]
  void* out = nullptr;         // [B, M, N]
  unsigned* status = nullptr;  // two words, zero before the launch; set on a bounded-wait timeout
  int64_t B = 1, M = 0, N = 0, K = 0;
  int planes_a = 1, planes_b = 1;
  int rhs_transposed = 0;
  int ab_dtype = CB_BF16;      // CB_BF16 or CB_F16
  int out_dtype = CB_BF16;     // CB_BF16, CB_F16 or CB_F32
  int n_pass = 1;
  int pass_a[GEMM_TC_MAX_PASSES] = {0};
  int pass_b[GEMM_TC_MAX_PASSES] = {0};
  // optional epilogue: out = act(acc * col_scale[n] + bias[n])
  const float* col_scale = nullptr;
  const float* bias = nullptr;
  int activation = CB_ACT_NONE;
};

// Persistent grid for the problem on a device with n_sm multiprocessors.
int gemm_tc_blocks(int n_sm, int64_t B, int64_t M, int64_t N);
int gemm_tc_threads();
int gemm_tc_smem();
int gemm_tc_run(int dev, int blocks, const GemmTcProblem& g, cudaStream_t s);

// The passes of a product of an operand with `pa` planes and one with `pb`, smallest terms first; returns their
// number.  Plane index sums above max_sum are left out (2 for three-plane operands, 1 for two-plane ones: what is
// dropped is no larger than what the planes themselves leave out).
int gemm_tc_split_passes(int pa, int pb, int max_sum, int* pass_a, int* pass_b);

// planes_x[i][e] for i < n_planes (2 or 3), e < n_x: the bf16 split of src_x, for two operands in one launch (n_b may
// be 0).  Non-finite values go to plane 0 alone.
int split_f32_planes(const float* src_a, uint16_t* planes_a, size_t n_a, const float* src_b, uint16_t* planes_b, size_t n_b,
                     int n_planes, cudaStream_t s);

}  // namespace cb
