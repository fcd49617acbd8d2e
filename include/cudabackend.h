/*
 * libcudabackend — C ABI of the B200 (sm_100a) backend for gomlx/compute's
 * inference hot path: FusedQuantizedDense, DotGeneral, FusedScaledDotProductAttention.
 *
 * This is the boundary a cgo shim binds (one C call per Backend / Executable
 * step).  Plain pointers and sizes only; every function returns CB_OK (0) or a
 * cb_status code and leaves a message for cb_last_error() (thread-local).  No
 * C++ exception crosses the boundary and the library never calls back into the
 * host language.  All `void*` data arguments are DEVICE pointers on `dev`
 * unless the parameter name starts with `host_`.
 *
 * Each group below cites the interface of the reference it replaces
 * (paths relative to the gomlx/compute repository).
 */
#ifndef CUDABACKEND_H
#define CUDABACKEND_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  CB_OK = 0,
  CB_ERR_INVALID_ARG = 1,     /* ordinary Go `error` at build/execute time            */
  CB_ERR_NOT_IMPLEMENTED = 2, /* maps to compute.ErrNotImplemented (compute.go:104-115) */
  CB_ERR_OOM = 3,
  CB_ERR_CUDA = 4,
  CB_ERR_TIMEOUT = 5,         /* a bounded device-side wait gave up                    */
  CB_ERR_NO_DEVICE = 6
} cb_status;

/* Element types: numeric codes of dtypes/dtype_enum.go:18-120. */
typedef enum {
  CB_INVALID = 0, CB_BOOL = 1, CB_I8 = 2, CB_I16 = 3, CB_I32 = 4, CB_I64 = 5,
  CB_U8 = 6, CB_U16 = 7, CB_U32 = 8, CB_U64 = 9, CB_F16 = 10, CB_F32 = 11,
  CB_F64 = 12, CB_BF16 = 13, CB_F8E5M2 = 19, CB_F8E4M3FN = 20,
  CB_I4 = 21, CB_U4 = 22     /* two elements per byte, low nibble first (quantized dense weights only) */
} cb_dtype;

/* compute.ActivationType (fused_ops.go:280-289). */
typedef enum { CB_ACT_NONE = 0, CB_ACT_GELU = 1, CB_ACT_RELU = 2, CB_ACT_SILU = 3,
               CB_ACT_HARDSWISH = 4, CB_ACT_TANH = 5 } cb_activation;

typedef void* cb_stream;          /* a cudaStream_t; NULL = the device's default stream */
typedef struct cb_plan cb_plan;   /* immutable after creation; safe to launch from many threads */

/* ---- process / device (Backend: compute.go:68-102; gobackend.New, internal/gobackend/gobackend.go:58-104) */
int cb_init(int* n_devices);                            /* Backend.NumDevices                   */
int cb_device_desc(int dev, char* buf, size_t buf_len); /* Backend.DeviceDescription            */
int cb_device_sm_count(int dev, int* n_sm);
const char* cb_last_error(void);
const char* cb_status_name(int status);

/* ---- buffers (DataInterface.BufferFromFlatData / Buffer.ToFlatData / Finalize / CopyToDevice:
 *      buffer.go:12-61; gobackend buffers.go:117-180, :387-417).  Copies with a NULL stream are
 *      synchronous; with a stream they are ordered on it (host memory should then be pinned). */
int cb_alloc(int dev, size_t bytes, void** dptr);
int cb_free(int dev, void* dptr);
int cb_memset(int dev, void* dptr, int value, size_t bytes, cb_stream stream);
int cb_h2d(int dev, void* dst, const void* host_src, size_t bytes, cb_stream stream);
int cb_d2h(int dev, void* host_dst, const void* src, size_t bytes, cb_stream stream);
int cb_d2d(int dst_dev, void* dst, int src_dev, const void* src, size_t bytes, cb_stream stream);
int cb_host_alloc(size_t bytes, void** host_ptr);       /* pinned host memory */
int cb_host_free(void* host_ptr);

/* ---- streams / events (replace the goroutine pool of internal/gobackend/workerspool) */
int cb_stream_create(int dev, cb_stream* stream);
int cb_stream_sync(int dev, cb_stream stream);
int cb_stream_destroy(int dev, cb_stream stream);
typedef void* cb_event;
int cb_event_create(int dev, cb_event* ev);
int cb_event_record(int dev, cb_event ev, cb_stream stream);
int cb_stream_wait_event(int dev, cb_stream stream, cb_event ev);  /* later work on `stream` waits for `ev`: copies and launches of
                                                                       different Execute calls overlap across streams */
int cb_event_elapsed_ms(cb_event start, cb_event stop, float* ms);  /* syncs on stop */
int cb_event_destroy(int dev, cb_event ev);

/* ---- FusedQuantizedDense, Linear and NF4 schemes, 8-bit and packed 4-bit weights
 *      (FusedOps.FusedQuantizedDense fused_ops.go:413-435; builder/executor
 *       internal/gobackend/fusedops/quantizeddense.go:58-142, :330-418, :616-650;
 *       activation epilogue fusedops/dense.go:176-205).
 * y[M,N] = act( x[M,K] @ dequant(W[K,N]) + bias[N] ),  dequant = w*scale (+ zero_point), or for
 * NF4 table[w & 15]*scale (compute.NF4LookupTable, fused_ops.go:114-121; quantizeddense.go:586-609).
 * Int4 / Uint4 weights are packed two per byte over the flat [K*N] element order, low nibble first,
 * as the reference stores them (internal/gobackend/ops/convertdtype.go:199-226).
 * Launch inputs, in the reference's node-input order: x, weights, scales, zero_points?, bias?. */
typedef enum {
  CB_SCALE_REF = 0,     /* the reference layout: scales [K, ceil(N/block_size)], block along N  */
  CB_SCALE_CHANNEL = 1, /* compact extension: scales [N], one per output channel               */
  CB_SCALE_KGROUP = 2   /* compact extension: scales [ceil(K/block_size), N], groups along K   */
} cb_scale_layout;

/* compute.QuantizationScheme (fused_ops.go:80-98) and compute.GGMLQuantType (:132-145).  GGML weights are
 * [N, bytes_per_row] Uint8 in the native block layout with the scales inside the blocks: launch inputs x, weights,
 * bias? (no scales, no zero points); scale_layout and block_size are ignored.  Built: Q4_0 (18-byte blocks of 32
 * values: fp16 scale, 16 bytes of nibbles, value = (nibble - 8) * scale, low nibbles first half) and Q8_0 (34-byte
 * blocks: fp16 scale, 32 int8); the other block formats return CB_ERR_NOT_IMPLEMENTED. */
typedef enum { CB_QUANT_LINEAR = 0, CB_QUANT_NF4 = 1, CB_QUANT_GGML = 2 } cb_quant_scheme;
typedef enum { CB_GGML_Q4_0 = 0, CB_GGML_Q8_0 = 1, CB_GGML_IQ4_NL = 2, CB_GGML_Q4_K = 5, CB_GGML_Q6_K = 7 } cb_ggml_type;

typedef enum {
  CB_QDENSE_AUTO = 0,
  CB_QDENSE_GENERIC = 1,    /* CUDA-core kernel in the reference's (m,k,n) summation order       */
  CB_QDENSE_DECODE_MMA = 2, /* M <= 16 stream-K kernel: cp.async-staged int8 tiles, f16 mma, f32 acc */
  CB_QDENSE_PREFILL = 3,    /* M > 16: weights expanded to bf16 planes, tcgen05 GEMM, fused epilogue */
  CB_QDENSE_DECODE_TC = 4   /* M <= 16: TMA-fed tcgen05 kind::i8 on the raw weight bytes, x as int8 digits */
} cb_qdense_variant;

typedef struct {
  int64_t M, K, N;
  int32_t x_dtype;        /* CB_F32 (the reference's only type) or CB_BF16 (extension); out has the same type */
  int32_t w_dtype;        /* CB_I8, CB_U8, or packed CB_I4 / CB_U4 (generic kernel) */
  int32_t scale_layout;   /* cb_scale_layout */
  int64_t block_size;     /* REF: columns per scale; KGROUP: rows per scale; CHANNEL: ignored */
  int32_t has_zero_point; /* zero points share the scale layout (f32) */
  int32_t has_bias;       /* bias [N] f32 */
  int32_t activation;     /* cb_activation */
  int32_t variant;        /* cb_qdense_variant; AUTO selects by shape and dtype */
  /* Column-sharded decode with the all-gather fused into the kernel (0 or 1 = off): this rank holds
   * columns [gather_rank * N, (gather_rank + 1) * N) of a [K, N * gather_ranks] projection.  The plan
   * then takes gather_ranks outputs: the [M, N * gather_ranks] result buffer of every rank (own
   * buffer included; peers' buffers opened with cb_ipc_open), and the kernel stores its column slice
   * into all of them as its tiles finish.  cb_peer_signal, enqueued after one or several such
   * launches, tells the other ranks that the slices have landed; cb_peer_wait makes a stream wait
   * for the slices of all ranks.  Decode tensor-core kernel only. */
  int32_t gather_ranks;
  int32_t gather_rank;
  int32_t scheme;         /* cb_quant_scheme; NF4 takes no zero points and runs on the generic kernel */
  int32_t ggml_type;      /* cb_ggml_type when scheme is CB_QUANT_GGML */
} cb_qdense_desc;

int cb_plan_qdense(int dev, const cb_qdense_desc* desc, cb_plan** plan);

/* Several independent decode-shaped projections as ONE launch of the tensor-core decode kernel: the members
 * share M, K, the dtypes and the scale layout of `shared` (its N, has_bias and activation are ignored) and each
 * has its own width, bias and activation — gate / up of a SwiGLU block, q / k / v of an attention block
 * (fused_ops.go:413-461 describes them as separate FusedQuantizedDense calls on one x), or the same projection
 * of several requests.  The fixed cost of a launch (pipeline fill and drain, 5-6 us against 9 us of streaming for a
 * 4096 x 14336 layer) is paid once for the group, and members that are given the same x pointer share one
 * conversion of x.  Launch inputs: x, weights, scales, bias? of member 0, then of member 1, ...; outputs: one per
 * member (gather_ranks of them per member for a gathered plan, own buffer included).  At most 16 members; the
 * decode tensor-core kernel's conditions apply (M <= 16, compact scales, K groups of a multiple of 128). */
typedef struct {
  int64_t N;
  int32_t has_bias;
  int32_t activation;     /* cb_activation */
} cb_qdense_member;
#define CB_QDENSE_GROUP_MAX 16
int cb_plan_qdense_group(int dev, const cb_qdense_desc* shared, const cb_qdense_member* members, int n_members,
                         cb_plan** plan);

/* No counterpart in the reference: a decode-shaped (M <= 16, compact scales) quantized dense
 * for callers that cannot allocate device memory when they launch — a server that gave all of
 * HBM to its own arena, a plugin inside another framework's callback, a process whose allocator
 * is frozen after start-up.  It runs the same kernel as the CB_QDENSE_DECODE_MMA plan, with the
 * stream-K scratch in a 2 MiB array that is part of the library image (every GPU that loads the
 * library holds it until exit).  It allocates nothing; shapes whose scratch would exceed the
 * array are rejected with CB_ERR_INVALID_ARG — use a plan with a caller-owned workspace then.
 * The first call on a device looks up the array's device address; make that call before any
 * stream capture.  All calls share the one array per device: calls that overlap on the GPU
 * (different streams, threads or processes sharing a context) race and give wrong results. */
int cb_qdense_decode_static(int dev, const cb_qdense_desc* desc, const void* x, const void* weights,
                            const void* scales, const void* bias /* or NULL */, void* out, cb_stream stream);

/* ---- DotGeneral in normalised form (StandardOps.DotGeneral standard_ops.go:338-363;
 *      normalisation and dtype rules internal/gobackend/dot/dot.go:165-285; kernels dot/matmul/*).
 * out[B,M,N] = lhs[B,M,K] x rhs, rhs = [B,K,N] (rhs_transposed = 0) or [B,N,K] (= 1).
 * Half inputs accumulate in f32.  Launch inputs: lhs, rhs, bias?.
 * With has_bias / activation the plan is FusedOps.FusedDense (fused_ops.go:336-347; builder and
 * executor internal/gobackend/fusedops/dense.go:34-163): out = act(dot + bias[n]), bias [N] of the
 * input dtype, float dtypes only (the reference executes f32 and f64; bf16 / f16 are this
 * backend's extension, computed in f32 and rounded once). */
typedef enum {
  CB_DOT_AUTO = 0,
  CB_DOT_GENERIC = 1,   /* CUDA-core tiled kernel, every supported dtype                       */
  CB_DOT_TCGEN05 = 2,   /* tcgen05 / TMEM / TMA kernel: bf16, f16; f32 as two bf16 planes per operand and three
                           plane products (a0b0 + a0b1 + a1b0: about 2^-17 relative per term, inside the 1e-4 bar) */
  CB_DOT_TCGEN05_EXACT = 3  /* the same kernel with three planes per operand and six products (about 2e-6)         */
} cb_dot_variant;

typedef struct {
  int64_t B, M, N, K;
  int32_t rhs_transposed;
  int32_t in_dtype;      /* f32, f64, bf16, f16, i32, i64 */
  int32_t out_dtype;     /* dtype stored; CB_INVALID = in_dtype */
  int32_t variant;       /* cb_dot_variant */
  int32_t has_bias;      /* FusedDense: bias [N] follows rhs in the launch inputs */
  int32_t activation;    /* FusedDense: cb_activation applied after the bias */
} cb_dot_desc;

int cb_plan_dot(int dev, const cb_dot_desc* desc, cb_plan** plan);

/* ---- FusedScaledDotProductAttention (fused_ops.go:349-378, :245-277;
 *      internal/gobackend/fusedops/sdpa.go:98-210, :221-329, :373-636).
 * Launch inputs, in the reference's node-input order: q, k, v, mask?, q_len?, kv_len?, bias?. */
typedef enum { CB_LAYOUT_BHSD = 0, CB_LAYOUT_BSHD = 1 } cb_attn_layout;
typedef enum { CB_MASK_NONE = 0, CB_MASK_BOOL = 1, CB_MASK_ADDITIVE = 2 } cb_mask_kind;
typedef enum { CB_SDPA_AUTO = 0, CB_SDPA_GENERIC = 1, CB_SDPA_FLASH = 2,
               CB_SDPA_DECODE = 3,  /* a few query tokens over a long key / value cache: split-KV streaming kernel */
               CB_SDPA_TILE = 4     /* 32-row query tiles on CUDA cores: float32, head_dim 32 / 64, masks, bias */ } cb_sdpa_variant;

typedef struct {
  int64_t B, Hq, Hkv, S, Skv, D;
  int32_t layout;          /* cb_attn_layout */
  int32_t dtype;           /* f32, f64, bf16, f16 (mask/bias additive values share it) */
  double  scale;           /* 0 = 1/sqrt(D) */
  int32_t causal;
  int32_t mask_kind;       /* cb_mask_kind */
  int32_t mask_rank;       /* 2..4 */
  int64_t mask_dims[4];    /* as given by the caller (BSHD rank-4 masks are [B,S,H,Skv]) */
  int32_t has_seq_lens;    /* q_len, kv_len: int32 [B] */
  int32_t bias_rank;       /* 0 = none, else 2..4 */
  int64_t bias_dims[4];
  int32_t variant;         /* cb_sdpa_variant */
} cb_sdpa_desc;

int cb_plan_sdpa(int dev, const cb_sdpa_desc* desc, cb_plan** plan);

/* ---- helper ops the DotGeneral path and its compliance tests need
 *      (internal/gobackend/ops: reshape.go, slice.go, iota.go, convertdtype.go, transpose.go). */
int cb_plan_copy(int dev, int32_t dtype, int64_t n_elements, cb_plan** plan);          /* Reshape */
int cb_plan_convert(int dev, int32_t from, int32_t to, int64_t n_elements, cb_plan** plan);
int cb_plan_iota(int dev, int32_t dtype, int32_t rank, const int64_t* dims, int32_t axis, cb_plan** plan);
int cb_plan_slice(int dev, int32_t dtype, int32_t rank, const int64_t* dims, const int64_t* starts,
                  const int64_t* limits, const int64_t* strides, cb_plan** plan);
int cb_plan_transpose(int dev, int32_t dtype, int32_t rank, const int64_t* dims,
                      const int32_t* permutation, cb_plan** plan);

/* ---- element-wise and reduction ops around the projections of a decoder block (StandardOps, standard_ops.go:131-700;
 *      executors internal/gobackend/ops).  Binary ops follow shapeinference.BinaryOp
 *      (shapeinference/shapeinference.go:219-300): both operands are given with the same rank (a scalar as all
 *      ones) and every dimension pair is equal or has a 1, which is broadcast.  Float dtypes (halves computed in
 *      f32); binary ops also Int32 / Int64.  The reduce plan keeps the axes whose flag is 0 and reduces the others
 *      (cb_reduce_op).  BroadcastInDim: standard_ops.go:232-254. */
/* compute.ReduceOpType minus one (standard_ops.go:65-84) */
typedef enum { CB_REDUCE_SUM = 0, CB_REDUCE_PRODUCT = 1, CB_REDUCE_MAX = 2, CB_REDUCE_MIN = 3 } cb_reduce_op;
typedef enum { CB_BIN_ADD = 0, CB_BIN_SUB = 1, CB_BIN_MUL = 2, CB_BIN_DIV = 3, CB_BIN_MAX = 4, CB_BIN_MIN = 5 } cb_binary_op;
typedef enum { CB_UN_NEG = 0, CB_UN_RSQRT = 1, CB_UN_SQRT = 2, CB_UN_EXP = 3, CB_UN_LOGISTIC = 4, CB_UN_TANH = 5 } cb_unary_op;
int cb_plan_binary(int dev, int32_t op, int32_t dtype, int32_t rank, const int64_t* lhs_dims, const int64_t* rhs_dims, cb_plan** plan);
int cb_plan_unary(int dev, int32_t op, int32_t dtype, int64_t n_elements, cb_plan** plan);
int cb_plan_reduce(int dev, int32_t reduce_op, int32_t dtype, int32_t rank, const int64_t* dims, const int32_t* reduced_axis_flags,
                   cb_plan** plan);
int cb_plan_broadcast_in_dim(int dev, int32_t dtype, int32_t rank, const int64_t* dims, int32_t out_rank, const int64_t* out_dims,
                             const int32_t* broadcast_axes, cb_plan** plan);
/* y = x * rsqrt(mean(x^2 over the row) + epsilon) * gamma?  over rows of row_size trailing elements (launch inputs x,
 * gamma?).  The interface has no fused RMS norm (FusedLayerNorm is mean-centred, internal/gobackend/fusedops/
 * layernorm.go:102-137): Builder.Compile substitutes this plan for the decomposed Mul / ReduceSum / Rsqrt form. */
int cb_plan_rms_norm(int dev, int32_t dtype, int64_t rows, int64_t row_size, double epsilon, int32_t has_gamma, cb_plan** plan);

/* ---- QuantizedEmbeddingLookup (fused_ops.go:394-411; internal/gobackend/fusedops/quantizeddense.go:250-321, 455-499):
 * out[i, 0..K) float32 = the dequantised row indices[i] of a GGML block table [vocab, bytes_per_row] bytes; K follows from
 * bytes_per_row and the block format (deriveGGMLK, quantizeddense.go:165-176; bytes_per_row must be whole blocks).
 * Launch inputs: table, indices (n_indices integers of index_dtype: int8 / uint8 / int32 / int64); output: [n_indices, K].
 * The plan needs its workspace.  An index outside [0, vocab) is an error in the reference; here its row is written as
 * zeros and cb_plan_check_status(plan, workspace) — after the stream has been synchronised — returns CB_ERR_INVALID_ARG
 * naming the first such position. */
int cb_plan_embedding_lookup(int dev, int64_t vocab, int64_t bytes_per_row, int64_t n_indices, int32_t index_dtype, int32_t ggml_type, cb_plan** plan);

/* ---- FusedGelu, FusedSoftmax, FusedLayerNorm (FusedOps, fused_ops.go:318-334; internal/gobackend/fusedops/gelu.go,
 *      softmax.go, layernorm.go).  Float32 / Float64 as the reference, BFloat16 / Float16 computed in f32.
 *      softmax: x viewed as [outer, axis_size, inner].  layer norm: rows of norm_size trailing elements;
 *      launch inputs x, gamma?, beta? (gamma / beta [norm_size], dtype of x). */
int cb_plan_gelu(int dev, int32_t dtype, int64_t n_elements, int32_t exact, cb_plan** plan);
int cb_plan_softmax(int dev, int32_t dtype, int64_t outer, int64_t axis_size, int64_t inner, cb_plan** plan);
int cb_plan_layernorm(int dev, int32_t dtype, int64_t rows, int64_t norm_size, double epsilon, int32_t has_gamma,
                      int32_t has_beta, cb_plan** plan);
/* out[rows, n_cols] = src[rows, total_cols][:, first_col : first_col + n_cols] + bias[n_cols]?  (launch inputs src, bias?):
 * the scatter half of FusedAttentionQKVProjection (fused_ops.go:437-461; fusedops/attentionqkv.go:140-199). */
int cb_plan_cols_bias(int dev, int32_t dtype, int64_t rows, int64_t total_cols, int64_t first_col, int64_t n_cols,
                      int32_t has_bias, cb_plan** plan);

/* ---- plans ("compile-time kernel selection by shape and dtype": created in Builder.Compile,
 *      builder.go:29-82; launched from Executable.Execute, executable.go:10-37) */
int cb_plan_workspace_bytes(const cb_plan* plan, size_t* bytes);
/* Scratch memory is caller-owned.  A freshly allocated workspace must be prepared once
 * (this zeroes the arrival counters and status words some kernels keep in it); launches leave it prepared.
 * Which plans need one is the plan's business (cb_plan_workspace_bytes): the decode kernels of the quantized dense
 * op do - int8 on the tensor cores, GGML blocks on the integer tensor cores, packed 4-bit weights. */
int cb_plan_prepare_workspace(const cb_plan* plan, void* workspace, cb_stream stream);
const char* cb_plan_kernel_name(const cb_plan* plan);
int cb_plan_grid(const cb_plan* plan, int* blocks, int* threads, int* dyn_smem_bytes);
int cb_launch(const cb_plan* plan, const void* const* inputs, int n_inputs,
              void* const* outputs, int n_outputs, void* workspace, cb_stream stream);
/* After a stream sync: reads the status word a kernel with bounded waits keeps in its
 * workspace; CB_ERR_TIMEOUT if a wait gave up.  CB_OK for plans without such waits. */
int cb_plan_check_status(const cb_plan* plan, const void* workspace);
int cb_plan_destroy(cb_plan* plan);

/* ---- bound launches: a plan with its buffers fixed (an Executable whose parameters stay resident between
 *      Execute calls, executable.go:10-37: weights, activations and results of a decode loop live at fixed
 *      addresses).  Binding does once what cb_launch does on every call — argument checks, tensor-map encoding,
 *      the problem table of a grouped plan — so that a launch is only the kernel launches, and
 *      cb_bound_launch_many issues a whole step's launches from one call.  The plan, the buffers and the
 *      workspace must outlive the bound object; one workspace serves one bound object at a time. */
typedef struct cb_bound cb_bound;
int cb_plan_bind(const cb_plan* plan, const void* const* inputs, int n_inputs, void* const* outputs, int n_outputs,
                 void* workspace, cb_bound** bound);
int cb_bound_launch(const cb_bound* bound, cb_stream stream);
int cb_bound_launch_many(const cb_bound* const* bounds, int n_bounds, cb_stream stream);
int cb_bound_destroy(cb_bound* bound);

/* ---- peer memory between the processes of one machine (one process per GPU, NVLink)
 * No counterpart in the reference.  cb_ipc_export names an allocation made by cb_alloc (pass its base
 * pointer); another process maps it with cb_ipc_open and may hand the mapped pointer to kernels as an
 * output of a gathered plan.  Arrival flags are arrays of uint32 (zeroed once) that every rank exports
 * like any buffer: cb_peer_signal enqueues a kernel that, once all earlier work of the stream has
 * completed, adds 1 to word `slot` (the caller's rank) of the flag array of every rank; cb_peer_wait
 * enqueues a kernel that waits (at most ~2 s, then it sets *status_word to a non-zero code and
 * returns) until each of flags[0..n_flags) of the local array has reached `target`. */
#define CB_IPC_HANDLE_BYTES 64
int cb_ipc_export(int dev, const void* dptr, unsigned char* handle /* CB_IPC_HANDLE_BYTES */);
int cb_ipc_open(int dev, const unsigned char* handle, void** dptr);
int cb_ipc_close(int dev, void* dptr);
int cb_peer_signal(int dev, void* const* flags /* one array per rank */, int n_ranks, int slot, cb_stream stream);
int cb_peer_wait(int dev, const void* flags, int n_flags, uint32_t target, void* status_word, cb_stream stream);
/* Both in one kernel (one launch fewer per step, chained to its neighbours in the stream by programmatic dependent
 * launch): adds 1 to word `slot` of every rank's flag array once the earlier work of the stream has completed, then
 * waits (bounded, as cb_peer_wait) until local_flags[0..n_ranks) have all reached `target`. */
int cb_peer_signal_wait(int dev, void* const* flags /* one array per rank */, int n_ranks, int slot, const void* local_flags,
                        uint32_t target, void* status_word, cb_stream stream);

/* ---- collectives: one communicator rank per process and GPU (NCCL, loaded at run time)
 * Replace CollectiveOps.AllReduce (collectiveops.go:10-39) and provide the all-gather at a
 * column-shard boundary that the interface sketches (collectiveops.go:31-32; the reference has
 * no implementation of either).  The 128-byte id is made on one rank and handed to the others by
 * the host program (any channel); every rank then calls cb_comm_init_rank.  Without NCCL on the
 * machine these return CB_ERR_NOT_IMPLEMENTED. */
#define CB_COMM_ID_BYTES 128
typedef struct cb_comm cb_comm;
int cb_comm_unique_id(unsigned char* id /* CB_COMM_ID_BYTES */);
int cb_comm_init_rank(int dev, int nranks, int rank, const unsigned char* id, cb_comm** comm);
/* Failure handling; no counterpart in the reference, which is one process on one device (errors there are returned
 * values, compute.go:39-48).  With timeout_s > 0 the communicator is non-blocking: initialisation and every enqueue poll
 * the asynchronous state under that limit.  When it passes — a rank that never joined, a peer that left — or NCCL
 * reports an error, the communicator is aborted, the call returns CB_ERR_TIMEOUT / CB_ERR_CUDA, and every later call on
 * the handle fails at once (cb_comm_destroy still frees it).  Non-blocking enqueues cost tens of microseconds each, so
 * timeout_s = 0 (and cb_comm_init_rank) makes the blocking kind, whose watchdog is cb_comm_sync alone.
 * dev < 0 = the calling thread's current device.
 *   cb_comm_check  one poll: CB_OK while healthy, the error (and an abort) once NCCL has reported one
 *   cb_comm_sync   waits for `stream` like cb_stream_sync while polling the communicator; past timeout_s (0 = the
 *                  communicator's own limit, else CUDABACKEND_COMM_TIMEOUT_S, else 600 s) it aborts the communicator,
 *                  which ends the collective's kernel, and returns CB_ERR_TIMEOUT */
int cb_comm_init_rank_timeout(int dev, int nranks, int rank, const unsigned char* id, double timeout_s, cb_comm** comm);
int cb_comm_check(cb_comm* comm);
int cb_comm_sync(cb_comm* comm, cb_stream stream, double timeout_s);
int cb_comm_size(const cb_comm* comm, int* nranks, int* rank);
/* recv[r * bytes_per_rank ...] = rank r's send, for every r; in place when send == recv + rank * bytes_per_rank */
int cb_comm_allgather(cb_comm* comm, const void* send, void* recv, size_t bytes_per_rank, cb_stream stream);
int cb_comm_allreduce(cb_comm* comm, const void* send, void* recv, size_t count, int32_t dtype, int32_t op, cb_stream stream);
int cb_comm_destroy(cb_comm* comm);

#ifdef __cplusplus
}
#endif
#endif
