/*
 * CPU oracle for the cudabackend hot path — TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic gomlx/compute's pure-Go `gobackend`
 * performs for the three operators on the accelerated path (fused quantized
 * dense, DotGeneral, fused scaled-dot-product attention).  It is the checker
 * the GPU kernels are compared against and the timed CPU baseline of the
 * benchmark; nothing in the shipped library links, loads or calls it.
 *
 * Parity pins:
 *   - DotGeneral and SDPA are pinned by the reference's own known-answer tests
 *     (support/backendtest/dotgeneral.go, support/backendtest/fusedops.go,
 *     internal/gobackend/fusedops/sdpa_direct_test.go), replayed from
 *     tests/golden/.
 *   - FusedQuantizedDense: PARITY UNPINNED.  The reference holds no test that
 *     asserts a FusedQuantizedDense result (it appears only in an unseeded
 *     benchmark, support/backendtest/benchmarks.go:435-562), and no Go
 *     toolchain exists here to run the reference.  The restatement is checked
 *     against hand-computed cases and against the reference's own "decomposed"
 *     formulation (ConvertDType -> Mul(scales) -> DotGeneral -> +bias).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * `-ffp-contract=off` keeps `(x*w)*s + acc` un-fused, as Go does on amd64.
 */
#ifndef CUDABACKEND_ORACLE_H
#define CUDABACKEND_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* DType codes = gomlx/compute dtypes/dtype_enum.go:18-120. */
enum {
  ORC_BOOL = 1, ORC_I8 = 2, ORC_I16 = 3, ORC_I32 = 4, ORC_I64 = 5,
  ORC_U8 = 6, ORC_U16 = 7, ORC_U32 = 8, ORC_U64 = 9,
  ORC_F16 = 10, ORC_F32 = 11, ORC_F64 = 12, ORC_BF16 = 13
};

/* compute.ActivationType, fused_ops.go:280-289. */
enum { ORC_ACT_NONE = 0, ORC_ACT_GELU = 1, ORC_ACT_RELU = 2, ORC_ACT_SILU = 3,
       ORC_ACT_HARDSWISH = 4, ORC_ACT_TANH = 5 };

/* dtypes/bfloat16/bfloat16.go:25-39 (round-to-nearest-even, NaN/Inf truncated). */
uint16_t orc_bf16_from_f32(float x);
float    orc_bf16_to_f32(uint16_t b);
/* dtypes/float16/float16.go:17-56, :103-165 (IEEE binary16, RNE). */
uint16_t orc_f16_from_f32(float x);
float    orc_f16_to_f32(uint16_t h);
void orc_bf16_from_f32_n(const float* in, uint16_t* out, size_t n);
void orc_bf16_to_f32_n(const uint16_t* in, float* out, size_t n);

/*
 * quantizedDenseLinearInt + fusedDenseApplyActivation
 * (internal/gobackend/fusedops/quantizeddense.go:616-650, dense.go:176-205).
 *   x [M,K] f32; w [K,N] int8 (w_unsigned=0) or uint8 (w_unsigned=1);
 *   scales [K, ceil(N/block_size)] f32; zero_points same shape or NULL;
 *   bias [N] f32 or NULL; out [M,N] f32.
 * threads <= 1 runs the reference's sequential order; threads > 1 uses the
 * reference's parallel split (one task per row if M > 1, N tiles of
 * max(4096/K,1) columns if M == 1; quantizeddense.go:542-579) on OpenMP.
 * The per-element arithmetic and its order do not depend on `threads`.
 */
void orc_qdense_linear(const float* x, const void* w, int w_unsigned,
                       const float* scales, const float* zero_points,
                       const float* bias, float* out,
                       int64_t M, int64_t K, int64_t N, int64_t block_size,
                       int activation, int threads);

/* fusedDenseApplyActivation[float32] (dense.go:176-205; GELU = gelu.go:113-118). */
void orc_activation_f32(float* data, size_t n, int activation);

/*
 * DotGeneral (standard_ops.go:338-363; shapeinference/dotgeneral.go:16-152;
 * internal/gobackend/dot/dot.go:165-285).  Output axes: batch..., lhs cross...,
 * rhs cross...  Half inputs accumulate in f32; an accumulator dtype different
 * from the input converts the inputs first (dot.go:340-372); the result is
 * converted to out_dtype at the end.  acc_f64 != 0 accumulates in double
 * instead (an order-independent truth for tolerance tests).
 * Returns 0, or a negative code on an invalid request.
 */
int orc_dot_general(int in_dtype, const void* lhs, int lhs_rank, const int64_t* lhs_dims,
                    const int* lhs_contract, const int* lhs_batch,
                    const void* rhs, int rhs_rank, const int64_t* rhs_dims,
                    const int* rhs_contract, const int* rhs_batch,
                    int n_contract, int n_batch,
                    int acc_dtype, int out_dtype, void* out, int acc_f64);

/*
 * sdpaMultiHeadGeneric + sdpaGeneric (internal/gobackend/fusedops/sdpa.go:373-636).
 * q [B,Hq,S,D] / k,v [B,Hkv,Skv,D] when bshd == 0, else [B,S,H,D]; all f32.
 * mask: NULL, or boolean bytes (mask_is_bool) / f32 additive, rank 2..4 with
 * dims mask_dims (BHSD convention; rank-4 masks are [B,H,S,Skv]).
 * bias: NULL or f32 additive, same conventions.  q_len / kv_len: NULL or
 * int32 [B], clamped to [0, dim] (sdpa.go:583-590).  out has q's layout.
 */
void orc_sdpa_f32(const float* q, const float* k, const float* v,
                  const void* mask, int mask_is_bool, int mask_rank, const int64_t* mask_dims,
                  const float* bias, int bias_rank, const int64_t* bias_dims,
                  const int32_t* q_len, const int32_t* kv_len,
                  float* out,
                  int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t Skv, int64_t D,
                  int bshd, double scale, int causal);

/* Same loops restricted to batches [b0,b1) and kv heads [h0,h1): lets the
 * benchmark time a bounded slice of a large configuration. */
void orc_sdpa_f32_slice(const float* q, const float* k, const float* v, float* out,
                        int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t Skv, int64_t D,
                        int bshd, double scale, int causal,
                        int64_t b0, int64_t b1, int64_t h0, int64_t h1);

/* Blocked f32 GEMM C[M,N] = A[M,K] * B[K,N] with the reference's large-matmul
 * structure (Nc/Kc/Mc panels, packed operands, register micro-kernel;
 * dot/matmul/avx512_large.go:163-232, params avx512.go:31-37), used as the
 * timed CPU baseline for DotGeneral.  The compiler vectorises the micro-kernel
 * for the host ISA. */
void orc_gemm_f32_blocked(const float* A, const float* B, float* C,
                          int64_t M, int64_t K, int64_t N, int threads);

int orc_max_threads(void);

/* Packed 4-bit weights and the NF4 scheme (convertdtype.go:199-226; quantizeddense.go:586-609). */
void orc_unpack_int4(const uint8_t* packed, int8_t* dst, size_t n_bytes);
void orc_unpack_uint4(const uint8_t* packed, uint8_t* dst, size_t n_bytes);
const float* orc_nf4_values(void);
void orc_qdense_nf4(const float* x, const void* w, const float* scales, const float* bias, float* out,
                    int64_t M, int64_t K, int64_t N, int64_t block_size, int activation, int threads);

/* GGML Q4_0 (type 0) and Q8_0 (type 1) blocks (quantizeddense_ggml.go:98-196). */
void orc_ggml_dequant_row(const uint8_t* data, float* out, int64_t K, int ggml_type);
void orc_qdense_ggml(const float* x, const uint8_t* w, const float* bias, float* out,
                     int64_t M, int64_t K, int64_t N, int ggml_type, int activation);

/* FusedSoftmax over [outer, L, inner], FusedGelu, FusedLayerNorm over trailing rows
 * (softmax.go:83-118, gelu.go:113-126, layernorm.go:129-168). */
void orc_softmax_f32(const float* x, float* y, int64_t outer, int64_t L, int64_t inner);
void orc_softmax_f64(const double* x, double* y, int64_t outer, int64_t L, int64_t inner);
void orc_gelu_f32(const float* x, float* y, size_t n, int exact);
void orc_gelu_f64(const double* x, double* y, size_t n, int exact);
void orc_layernorm_f32(const float* x, const float* gamma, const float* beta, float* y, int64_t rows, int64_t L, double eps);
void orc_layernorm_f64(const double* x, const double* gamma, const double* beta, double* y, int64_t rows, int64_t L, double eps);

#ifdef __cplusplus
}
#endif
#endif
