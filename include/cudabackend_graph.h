/*
 * libcudabackend — host-side graph layer: a C-handle rendering of gomlx/compute's
 * Backend / Builder / Function / Executable / Buffer interfaces for the accelerated
 * path (FusedQuantizedDense, DotGeneral, FusedScaledDotProductAttention and the
 * helper ops around them).  It is written in C++ inside the library (no Go toolchain
 * exists where this was built) and keeps the reference's method names, argument
 * meaning and error behaviour; every other op of the interface is not implemented
 * and reports CB_ERR_NOT_IMPLEMENTED, the equivalent of embedding
 * notimplemented.Function (notimplemented/function.go:13).
 *
 * Conventions: as in cudabackend.h (status codes, cb_last_error()).  `host_*`
 * pointers are host memory; handles are opaque and owned by the caller until the
 * matching *_finalize / *_free call.  A Builder/Function is single-threaded; an
 * Executable may be executed from several threads at once (executable.go:10-37).
 */
#ifndef CUDABACKEND_GRAPH_H
#define CUDABACKEND_GRAPH_H

#include "cudabackend.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cbg_backend cbg_backend;   /* compute.Backend   (compute.go:68-102)     */
typedef struct cbg_builder cbg_builder;   /* compute.Builder   (builder.go:29-82)      */
typedef struct cbg_function cbg_function; /* compute.Function  (function.go:23-134)    */
typedef struct cbg_value cbg_value;       /* compute.Value     (builder.go:12)         */
typedef struct cbg_exec cbg_exec;         /* compute.Executable(executable.go:10-37)   */
typedef struct cbg_buffer cbg_buffer;     /* compute.Buffer    (buffer.go:12-42)       */

/* ---- Backend.  config: "" or comma-separated keys, e.g. "devices=0,fallback_only"
 *      (the role of gobackend.New's config string, internal/gobackend/gobackend.go:58-104).
 *      fallback_only forces the generic kernels (like ForceSmallVariant in the reference's tests). */
int cbg_backend_new(const char* config, cbg_backend** backend);          /* compute.NewWithConfig("cuda:<config>") */
const char* cbg_backend_name(const cbg_backend* b);                       /* Backend.Name        */
const char* cbg_backend_description(const cbg_backend* b);                /* Backend.Description */
int cbg_backend_num_devices(const cbg_backend* b);                        /* Backend.NumDevices  */
int cbg_backend_device_description(const cbg_backend* b, int dev, char* buf, size_t n);
/* Backend.Capabilities (capabilities.go:12-39): op codes are optype.go values, dtypes cb_dtype. */
int cbg_backend_capabilities(const cbg_backend* b, int32_t* ops, int* n_ops, int32_t* dtypes, int* n_dtypes);
int cbg_backend_finalize(cbg_backend* b);                                 /* Backend.Finalize    */
int cbg_backend_is_finalized(const cbg_backend* b);
int cbg_backend_free(cbg_backend* b);                                     /* drops the handle itself */

/* ---- DataInterface / Buffer (buffer.go:12-61).  BufferFromFlatData copies host data. */
int cbg_buffer_from_flat(cbg_backend* b, int dev, const void* host_flat, int32_t dtype, int rank,
                         const int64_t* dims, cbg_buffer** buffer);
int cbg_buffer_shape(const cbg_buffer* buf, int32_t* dtype, int* rank, int64_t* dims /* up to 8 */);
int cbg_buffer_device_num(const cbg_buffer* buf, int* dev);
int cbg_buffer_to_flat(const cbg_buffer* buf, void* host_flat, size_t n_bytes);   /* Buffer.ToFlatData */
int cbg_buffer_copy_to_device(const cbg_buffer* buf, int dev, cbg_buffer** out);  /* Buffer.CopyToDevice */
int cbg_buffer_device_ptr(const cbg_buffer* buf, void** dptr);            /* extension: raw device pointer */
int cbg_buffer_finalize(cbg_buffer* buf);                                  /* Buffer.Finalize; frees the handle */

/* ---- Builder */
int cbg_builder_new(cbg_backend* b, const char* name, cbg_builder** builder);   /* Backend.Builder */
int cbg_builder_main(cbg_builder* bld, cbg_function** fn);                       /* Builder.Main    */
int cbg_builder_distributed_spmd(cbg_builder* bld, int num_devices);             /* Builder.DistributedSPMD */
int cbg_builder_device_assignment(cbg_builder* bld, const int* devices, int n);  /* Builder.DeviceAssignment */
int cbg_builder_compile(cbg_builder* bld, cbg_exec** exec);                      /* Builder.Compile */
int cbg_builder_free(cbg_builder* bld);   /* values and functions of the builder die with it */

/* ---- Function: graph building */
int cbg_fn_parameter(cbg_function* f, const char* name, int32_t dtype, int rank, const int64_t* dims, cbg_value** v);
int cbg_fn_constant(cbg_function* f, const void* host_flat, int32_t dtype, int rank, const int64_t* dims, cbg_value** v);
int cbg_fn_shape(const cbg_value* v, int32_t* dtype, int* rank, int64_t* dims /* up to 8 */);   /* Function.Shape */
int cbg_fn_return(cbg_function* f, cbg_value* const* outputs, int n);

/* StandardOps.DotGeneral (standard_ops.go:338-363); acc/out dtype 0 = unset (DotGeneralConfig, :91-111). */
int cbg_fn_dot_general(cbg_function* f, cbg_value* lhs, const int* lhs_contract, int n_contract,
                       const int* lhs_batch, int n_batch, cbg_value* rhs, const int* rhs_contract,
                       const int* rhs_batch, int32_t acc_dtype, int32_t out_dtype, cbg_value** v);
int cbg_fn_reshape(cbg_function* f, cbg_value* x, int rank, const int64_t* dims, cbg_value** v);
int cbg_fn_slice(cbg_function* f, cbg_value* x, const int64_t* starts, const int64_t* limits,
                 const int64_t* strides, cbg_value** v);
int cbg_fn_iota(cbg_function* f, int32_t dtype, int rank, const int64_t* dims, int axis, cbg_value** v);
int cbg_fn_convert_dtype(cbg_function* f, cbg_value* x, int32_t dtype, cbg_value** v);
int cbg_fn_transpose(cbg_function* f, cbg_value* x, const int* permutation, cbg_value** v);

/* FusedOps.FusedSoftmax / FusedGelu / FusedLayerNorm (fused_ops.go:318-334).  Softmax takes one non-negative axis;
 * layer-norm axes may be negative (counted from the end) and need not be trailing; gamma / beta may be NULL. */
int cbg_fn_fused_softmax(cbg_function* f, cbg_value* x, int axis, cbg_value** v);
int cbg_fn_fused_gelu(cbg_function* f, cbg_value* x, int exact, cbg_value** v);
int cbg_fn_fused_layer_norm(cbg_function* f, cbg_value* x, const int* axes, int n_axes, double epsilon,
                            cbg_value* gamma /* or NULL */, cbg_value* beta /* or NULL */, cbg_value** v);

/* FusedOps.FusedAttentionQKVProjection (fused_ops.go:437-461): x [batch..., in] @ wQKV [in, q + 2 kv], split into
 * query [.., q], key [.., kv], value [.., kv], each plus its optional bias. */
int cbg_fn_fused_attention_qkv_projection(cbg_function* f, cbg_value* x, cbg_value* w_qkv, cbg_value* bias_q /* or NULL */,
                                          cbg_value* bias_k /* or NULL */, cbg_value* bias_v /* or NULL */,
                                          int64_t query_dim, int64_t key_value_dim, cbg_value** query, cbg_value** key,
                                          cbg_value** value);

/* FusedOps.FusedDense (fused_ops.go:336-347) with compute.DenseConfig (:72-78): y = act(x @ W + bias).
 * weight_layout: 0 DenseLayoutInputOutputs (weight [in, out...]), 1 DenseLayoutOutputsInput ([out..., in]).
 * Float32 and Float64 as in the reference, BFloat16 / Float16 as an extension. */
int cbg_fn_fused_dense(cbg_function* f, cbg_value* x, cbg_value* weight, cbg_value* bias /* or NULL */,
                       int activation, int weight_layout, cbg_value** v);

/* FusedOps.FusedQuantizedDense (fused_ops.go:413-435) with compute.Quantization (:204-234).
 * scheme: 0 Linear, 1 NF4 (weights as Int8 / Uint8 nibble indices); GGML has its own entry point below.  block_axis 1 is the reference
 * layout scales [K, ceil(N/block_size)]; block_axis 0 is this backend's extension, scales
 * [ceil(K/block_size), N] (block_size = K gives one scale per output channel). */
int cbg_fn_fused_quantized_dense(cbg_function* f, cbg_value* x, cbg_value* weights, cbg_value* bias /* or NULL */,
                                 int scheme, cbg_value* scale, cbg_value* zero_point /* or NULL */,
                                 int block_axis, int64_t block_size, int activation, cbg_value** v);

/* FusedQuantizedDense with compute.QuantGGML (fused_ops.go:92-97, :132-145): weights [N, bytesPerRow] Uint8 in the
 * native GGML block layout, no scales or zero points.  ggml_type is compute.GGMLQuantType: Q4_0 = 0, Q8_0 = 1,
 * IQ4_NL = 2, Q4_K = 5, Q6_K = 7 — the five the reference supports (quantizeddense.go:145-152); the others return
 * CB_ERR_NOT_IMPLEMENTED as there. */
int cbg_fn_fused_quantized_dense_ggml(cbg_function* f, cbg_value* x, cbg_value* weights, cbg_value* bias /* or NULL */,
                                      int ggml_type, int activation, cbg_value** v);
/* FusedOps.QuantizedEmbeddingLookup (fused_ops.go:394-411; internal/gobackend/fusedops/quantizeddense.go:250-321):
 * data [vocabSize, bytesPerRow] Uint8 GGML blocks, indices integer [batch..., 1] -> Float32 [batch..., K].  scheme must be
 * 2 (GGML), else CB_ERR_NOT_IMPLEMENTED.  An index outside the table makes Execute return an error, as the reference's
 * executor does (:487-489). */
int cbg_fn_quantized_embedding_lookup(cbg_function* f, cbg_value* data, cbg_value* indices, int scheme, int ggml_type, cbg_value** v);

/* FusedOps.FusedScaledDotProductAttention (fused_ops.go:349-378) with
 * ScaledDotProductAttentionConfig (:245-277); NULL values = unset. */
typedef struct {
  int quantized_matmuls;          /* optimisation hint; ignored (computed in float) */
  cbg_value* query_seq_len;
  cbg_value* key_value_seq_len;
  cbg_value* bias;
  double scale;                   /* 0 = 1/sqrt(head_dim) */
  int causal;
  cbg_value* mask;
} cbg_sdpa_options;
int cbg_fn_fused_sdpa(cbg_function* f, cbg_value* query, cbg_value* key, cbg_value* value, int axes_layout,
                      const cbg_sdpa_options* options /* or NULL */, cbg_value** output);

/* ---- StandardOps a decoder block needs around its projections (standard_ops.go:131-700): element-wise binary ops
 * with the broadcasting rule of shapeinference.BinaryOp (equal ranks, every dimension pair equal or with a 1; a scalar
 * takes the other side's shape), unary ops, reductions over the listed axes (none = all; negative = from the end;
 * the reduced axes are dropped), BroadcastInDim (:232-254).  Float dtypes; the binary ops also Int32 / Int64.
 * Builder.Compile recognises the decomposed RMS norm  x * Reshape(Rsqrt(ReduceSum(x * x, last) * (1/H) + eps)) [* gamma]
 * and runs it as one row kernel. */
int cbg_fn_add(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v);
int cbg_fn_sub(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v);
int cbg_fn_mul(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v);
int cbg_fn_div(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v);
int cbg_fn_max(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v);
int cbg_fn_min(cbg_function* f, cbg_value* lhs, cbg_value* rhs, cbg_value** v);
int cbg_fn_neg(cbg_function* f, cbg_value* x, cbg_value** v);
int cbg_fn_rsqrt(cbg_function* f, cbg_value* x, cbg_value** v);
int cbg_fn_sqrt(cbg_function* f, cbg_value* x, cbg_value** v);
int cbg_fn_exp(cbg_function* f, cbg_value* x, cbg_value** v);
int cbg_fn_logistic(cbg_function* f, cbg_value* x, cbg_value** v);
int cbg_fn_tanh(cbg_function* f, cbg_value* x, cbg_value** v);
int cbg_fn_reduce_sum(cbg_function* f, cbg_value* x, const int* axes, int n_axes, cbg_value** v);
int cbg_fn_reduce_max(cbg_function* f, cbg_value* x, const int* axes, int n_axes, cbg_value** v);
int cbg_fn_broadcast_in_dim(cbg_function* f, cbg_value* x, int32_t dtype, int rank, const int64_t* dims, const int* broadcast_axes,
                            cbg_value** v);

/* ---- CollectiveOps (collectiveops.go:10-39) under Builder.DistributedSPMD: AllReduce as the interface declares it
 * (reduce_type: compute.ReduceOpType, 1 Sum, 2 Product, 3 Max, 4 Min) and the AllGather it sketches (:31-32; the
 * result's gather axis is the operand's times the group size — call DistributedSPMD first).  replica groups: indices
 * into the device assignment, groups_flat holding group_sizes[0] + group_sizes[1] + ... entries; n_groups = 0 means
 * one group of all replicas; otherwise every replica belongs to exactly one group
 * (distributed/devicemesh.go:224-293 computes them).  One output per operand. */
int cbg_fn_all_reduce(cbg_function* f, cbg_value* const* operands, int n_operands, int reduce_type, const int* groups_flat,
                      const int* group_sizes, int n_groups, cbg_value** outputs);
int cbg_fn_all_gather(cbg_function* f, cbg_value* const* operands, int n_operands, int gather_axis, const int* groups_flat,
                      const int* group_sizes, int n_groups, cbg_value** outputs);

/* Function.Parameter with its ShardingSpec (function.go:57; distributed/shardingspec.go:43-110): the mesh (axis names
 * and sizes) and, per tensor axis, a comma-separated list of mesh axes ("" = replicated; missing axes = replicated).
 * Validated as ShardingSpec.Validate does; under SPMD the declared shape is the shard every replica is given.
 * cbg_exec_input_sharding reads the spec back ("" = declared without one). */
int cbg_fn_parameter_sharded(cbg_function* f, const char* name, int32_t dtype, int rank, const int64_t* dims,
                             const char* const* mesh_axis_names, const int* mesh_axis_sizes, int n_mesh_axes,
                             const char* const* axis_specs, int n_axis_specs, cbg_value** v);

/* Any other op of the interface, by OpType name (e.g. "Neg", "FusedSoftmax", "AllReduce"):
 * returns CB_ERR_NOT_IMPLEMENTED with the reference's wording. */
int cbg_fn_not_implemented(cbg_function* f, const char* op_name);

/* ---- Executable.  inputs: one buffer per parameter (device-major under SPMD,
 * executable.go:33-35); donate may be NULL.  outputs must hold cbg_exec_num_outputs handles per replica and come back
 * device-major too (outputs[replica * num_outputs + i]).  Under SPMD all replicas are launched before any is waited
 * for, so the devices run side by side. */
int cbg_exec_num_inputs(const cbg_exec* e);
int cbg_exec_num_outputs(const cbg_exec* e);
int cbg_exec_input_info(const cbg_exec* e, int i, char* name, size_t name_len, int32_t* dtype, int* rank, int64_t* dims);
int cbg_exec_output_info(const cbg_exec* e, int i, int32_t* dtype, int* rank, int64_t* dims);
int cbg_exec_kernel_names(const cbg_exec* e, char* buf, size_t n);      /* launch plan, one kernel per line */
int cbg_exec_input_sharding(const cbg_exec* e, int i, char* buf, size_t n);
/* Tracing (the reference only logs the chosen implementation at klog -v=1, internal/gobackend/dot/dot.go:176-181; there are
   no timers).  With the backend option "trace" or CUDABACKEND_TRACE=1 in the environment at cbg_backend_new, every Execute
   records an event after each launch and, after its final sync, writes one line per launch to stderr:
     cudabackend trace: exec=<name> device=<d> node=<i> kernel=<plan name> out=<shape> us=<device time>
   The lines of the latest traced Execute can be read back here (empty when tracing is off). */
int cbg_exec_last_trace(cbg_exec* e, char* buf, size_t n);
/* Replay as CUDA graphs (no counterpart in the reference, whose executor walks its nodes on the host every time,
   internal/gobackend/exec.go:176-233).  On one device and without collectives, the second Execute with the same input
   buffers captures one pass over the nodes into a CUDA graph whose intermediate memory and workspaces belong to the
   executable, and that and every later call with those buffers is one graph launch plus the copy of the results into
   fresh buffers.  Calls with other buffers, donated inputs, a traced backend or the backend option "no_graphs" take the
   node-by-node path; up to eight buffer sets are remembered.  Returns how many calls were replays so far. */
int cbg_exec_graph_replays(cbg_exec* e);
int cbg_exec_execute(cbg_exec* e, cbg_buffer* const* inputs, int n_inputs, const uint8_t* donate,
                     int default_device, cbg_buffer** outputs, int n_outputs);
int cbg_exec_finalize(cbg_exec* e);                                        /* Executable.Finalize; frees the handle */

#ifdef __cplusplus
}
#endif
#endif
