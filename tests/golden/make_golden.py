"""Writes the known-answer fixtures in this folder.

The reference (gomlx/compute) is Go and cannot be run on this image, so these
fixtures are the input/expected pairs of the reference's OWN asserting tests,
transcribed case by case (each entry cites the test it comes from).  Expected
values are the ones the reference test asserts — never an output of the code
under test here.  Run:  python tests/golden/make_golden.py
"""
import json
import math
import os

HERE = os.path.dirname(os.path.abspath(__file__))
T = "support/backendtest/dotgeneral.go"
F = "support/backendtest/fusedops.go"
D = "internal/gobackend/fusedops/sdpa_direct_test.go"


def iota(start, n):
    return [float(start + i) for i in range(n)]


dot_cases = [
    dict(name="shuffled-axes", cite=f"{T}:83-115", dtype="f32",
         lhs=dict(shape=[2, 3, 1, 5], data=iota(1, 30)), lhs_contract=[1], lhs_batch=[3, 0],
         rhs=dict(shape=[5, 3, 2, 4], data=iota(1, 120)), rhs_contract=[1], rhs_batch=[0, 2],
         want=dict(shape=[5, 2, 1, 4], data=[
             242, 260, 278, 296, 899, 962, 1025, 1088,
             773, 794, 815, 836, 2522, 2588, 2654, 2720,
             1448, 1472, 1496, 1520, 4289, 4358, 4427, 4496,
             2267, 2294, 2321, 2348, 6200, 6272, 6344, 6416,
             3230, 3260, 3290, 3320, 8255, 8330, 8405, 8480]), cmp="equal"),
    dict(name="AxisTransposition", cite=f"{T}:117-130", dtype="f32",
         lhs=dict(shape=[2, 1, 3], data=[1, 2, 3, 4, 5, 6]), lhs_contract=[1], lhs_batch=[2, 0],
         rhs=dict(shape=[1, 3, 2], data=[1, 1, 1, 1, 1, 1]), rhs_contract=[0], rhs_batch=[1, 2],
         want=dict(shape=[3, 2], data=[1, 4, 2, 5, 3, 6]), cmp="equal"),
    dict(name="bfloat16/DotProduct-with-f32-acc", cite=f"{T}:161-176", dtype="bf16", acc="f32",
         lhs=dict(shape=[1, 3], data=[1, 2, 3]), lhs_contract=[1], lhs_batch=[],
         rhs=dict(shape=[3, 1], data=[10, 11, 12]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[1, 1], data=[68]), cmp="equal"),
    dict(name="float16/DotProduct-with-f32-acc", cite=f"{T}:178-193", dtype="f16", acc="f32",
         lhs=dict(shape=[1, 3], data=[1, 2, 3]), lhs_contract=[1], lhs_batch=[],
         rhs=dict(shape=[3, 1], data=[10, 11, 12]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[1, 1], data=[68]), cmp="equal"),
    dict(name="float16/DotProduct", cite=f"{T}:195-209", dtype="f16",
         lhs=dict(shape=[1, 3], data=[1, 2, 3]), lhs_contract=[1], lhs_batch=[],
         rhs=dict(shape=[3, 1], data=[10, 11, 12]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[1, 1], data=[68]), cmp="equal"),
]

# 2x2 matmuls in four dtypes, both layouts (dotgeneral.go:211-375)
for dt, cite in (("f32", "211-241"), ("bf16", "272-305"), ("f16", "307-340"), ("f64", "342-375")):
    a = dict(shape=[2, 2], data=[1, 2, 3, 4])
    b = dict(shape=[2, 2], data=[10, 11, 12, 13])
    dot_cases.append(dict(name=f"{dt}/small-matmul/LayoutNonTransposed", cite=f"{T}:{cite}", dtype=dt,
                          lhs=a, lhs_contract=[1], lhs_batch=[], rhs=b, rhs_contract=[0], rhs_batch=[],
                          want=dict(shape=[2, 2], data=[1 * 10 + 2 * 12, 1 * 11 + 2 * 13,
                                                        3 * 10 + 4 * 12, 3 * 11 + 4 * 13]), cmp="equal"))
    dot_cases.append(dict(name=f"{dt}/small-matmul/LayoutTransposed", cite=f"{T}:{cite}", dtype=dt,
                          lhs=a, lhs_contract=[1], lhs_batch=[], rhs=b, rhs_contract=[1], rhs_batch=[],
                          want=dict(shape=[2, 2], data=[1 * 10 + 2 * 11, 1 * 12 + 2 * 13,
                                                        3 * 10 + 4 * 11, 3 * 12 + 4 * 13]), cmp="equal"))

dot_cases += [
    dict(name="f32/VectorMatrix_Rank1_x_Rank2", cite=f"{T}:243-255", dtype="f32",
         lhs=dict(shape=[2], data=[1, 2]), lhs_contract=[0], lhs_batch=[],
         rhs=dict(shape=[2, 3], data=[10, 11, 12, 20, 21, 22]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[3], data=[50, 53, 56]), cmp="equal"),
    dict(name="f32/MatrixVector_Rank2_x_Rank1", cite=f"{T}:256-269", dtype="f32",
         lhs=dict(shape=[3, 2], data=[10, 20, 11, 21, 12, 22]), lhs_contract=[1], lhs_batch=[],
         rhs=dict(shape=[2], data=[1, 2]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[3], data=[50, 53, 56]), cmp="equal"),
    dict(name="ConfigDTypes/AccumulatorDType", cite=f"{T}:387-404", dtype="f16", acc="f32", out="f32",
         lhs=dict(shape=[2, 3], data=[1, 2, 3, 4, 5, 6]), lhs_contract=[1], lhs_batch=[],
         rhs=dict(shape=[3, 2], data=[7, 8, 9, 10, 11, 12]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[2, 2], data=[58, 64, 139, 154]), cmp="delta", tol=1e-2),
    dict(name="ConfigDTypes/OutputDType", cite=f"{T}:406-419", dtype="f16", out="f32",
         lhs=dict(shape=[2, 3], data=[1, 2, 3, 4, 5, 6]), lhs_contract=[1], lhs_batch=[],
         rhs=dict(shape=[3, 2], data=[7, 8, 9, 10, 11, 12]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[2, 2], data=[58, 64, 139, 154]), cmp="delta", tol=1e-2),
    dict(name="Dot/vector-vector", cite=f"{T}:423-431", dtype="f32",
         lhs=dict(shape=[3], data=[1, 2, 3]), lhs_contract=[0], lhs_batch=[],
         rhs=dict(shape=[3], data=[10, 11, 12]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[], data=[68]), cmp="equal"),
    dict(name="Dot/matrix-vector", cite=f"{T}:433-441", dtype="f32",
         lhs=dict(shape=[2, 3], data=[1, 2, 3, 2, 4, 6]), lhs_contract=[1], lhs_batch=[],
         rhs=dict(shape=[3], data=[10, 11, 12]), rhs_contract=[0], rhs_batch=[],
         want=dict(shape=[2], data=[68, 136]), cmp="equal"),
    # Shape-only case: zeros in, output dims asserted (dotgeneral.go:25-81)
    dict(name="Shape", cite=f"{T}:25-81", dtype="f32",
         lhs=dict(shape=[2, 3, 4, 5], data=[0.0] * 120), lhs_contract=[1], lhs_batch=[3, 0],
         rhs=dict(shape=[5, 1, 2, 3], data=[0.0] * 30), rhs_contract=[3], rhs_batch=[0, 2],
         want=dict(shape=[5, 2, 4, 1], data=[0.0] * 40), cmp="equal"),
]

sp = 1.0 / (1.0 + math.exp(-20))
bias_want = (1 - sp) * 10 + sp * 20
sq = 1.0 / (1.0 + math.exp(-10))
bias_causal_want = (1 - sq) * 10 + sq * 20

q2 = dict(shape=[1, 1, 2, 1], data=[1, 1])
v2 = dict(shape=[1, 1, 2, 1], data=[10, 20])
ones8 = [1.0] * 8


def x8(*vals):
    out = []
    for v in vals:
        out += [float(v)] * 8
    return out


sdpa_cases = [
    dict(name="BHSD_Causal", cite=f"{F}:216-235", dtype="f32", layout="BHSD", scale=1.0, causal=True,
         q=q2, k=q2, v=v2, want=dict(shape=[1, 1, 2, 1], data=[10, 15]), tol=1e-6),
    dict(name="BHSD_Causal_BF16", cite=f"{F}:237-262", dtype="bf16", layout="BHSD", scale=1.0, causal=True,
         q=dict(shape=[1, 1, 2, 8], data=x8(1, 1)), k=dict(shape=[1, 1, 2, 8], data=x8(1, 1)),
         v=dict(shape=[1, 1, 2, 8], data=x8(10, 20)),
         want=dict(shape=[1, 1, 2, 8], data=x8(10, 15)), tol=1e-6),
    dict(name="BHSD_Causal_F16", cite=f"{F}:264-287", dtype="f16", layout="BHSD", scale=1.0, causal=True,
         q=dict(shape=[1, 1, 2, 8], data=x8(1, 1)), k=dict(shape=[1, 1, 2, 8], data=x8(1, 1)),
         v=dict(shape=[1, 1, 2, 8], data=x8(10, 20)),
         want=dict(shape=[1, 1, 2, 8], data=x8(10, 15)), tol=1e-6),
    dict(name="BSHD_Causal", cite=f"{F}:289-308", dtype="f32", layout="BSHD", scale=1.0, causal=True,
         q=dict(shape=[1, 2, 1, 1], data=[1, 1]), k=dict(shape=[1, 2, 1, 1], data=[1, 1]),
         v=dict(shape=[1, 2, 1, 1], data=[10, 20]),
         want=dict(shape=[1, 2, 1, 1], data=[10, 15]), tol=1e-6),
    dict(name="BSHD_Causal_BF16", cite=f"{F}:310-335", dtype="bf16", layout="BSHD", scale=1.0, causal=True,
         q=dict(shape=[1, 2, 1, 8], data=x8(1, 1)), k=dict(shape=[1, 2, 1, 8], data=x8(1, 1)),
         v=dict(shape=[1, 2, 1, 8], data=x8(10, 20)),
         want=dict(shape=[1, 2, 1, 8], data=x8(10, 15)), tol=1e-6),
    dict(name="BSHD_Causal_F16", cite=f"{F}:337-362", dtype="f16", layout="BSHD", scale=1.0, causal=True,
         q=dict(shape=[1, 2, 1, 8], data=x8(1, 1)), k=dict(shape=[1, 2, 1, 8], data=x8(1, 1)),
         v=dict(shape=[1, 2, 1, 8], data=x8(10, 20)),
         want=dict(shape=[1, 2, 1, 8], data=x8(10, 15)), tol=1e-6),
    dict(name="WithBooleanMask", cite=f"{F}:364-384", dtype="f32", layout="BHSD", scale=1.0, causal=False,
         q=dict(shape=[1, 1, 1, 1], data=[1]), k=q2, v=v2,
         mask=dict(shape=[1, 2], dtype="bool", data=[1, 0]),
         want=dict(shape=[1, 1, 1, 1], data=[10]), tol=1e-6),
    dict(name="QuantizedMatmuls", cite=f"{F}:386-405", dtype="f32", layout="BHSD", scale=1.0, causal=True,
         quantized_matmuls=True, q=q2, k=q2, v=v2,
         want=dict(shape=[1, 1, 2, 1], data=[10, 15]), tol=1e-6),
    dict(name="Bias", cite=f"{F}:407-440", dtype="f32", layout="BHSD", scale=1.0, causal=False,
         q=q2, k=q2, v=v2, bias=dict(shape=[1, 1, 2, 2], data=[-10, 10, -10, 10]),
         want=dict(shape=[1, 1, 2, 1], data=[bias_want, bias_want]), tol=0.01),
    dict(name="BiasWithCausal", cite=f"{F}:442-472", dtype="f32", layout="BHSD", scale=1.0, causal=True,
         q=q2, k=q2, v=v2, bias=dict(shape=[1, 1, 2, 2], data=[0, -100, 0, 10]),
         want=dict(shape=[1, 1, 2, 1], data=[10, bias_causal_want]), tol=0.01),
    dict(name="Bias_BF16", cite=f"{F}:474-495", dtype="bf16", layout="BHSD", scale=1.0, causal=False,
         q=dict(shape=[1, 1, 2, 8], data=x8(1, 1)), k=dict(shape=[1, 1, 2, 8], data=x8(1, 1)),
         v=dict(shape=[1, 1, 2, 8], data=x8(10, 20)),
         bias=dict(shape=[1, 1, 2, 2], data=[-100, 100, -100, 100]),
         want=dict(shape=[1, 1, 2, 8], data=x8(20, 20)), tol=0.05),
    dict(name="Direct/ConfigFieldsCompile", cite=f"{D}:34-60", dtype="f32", layout="BHSD", scale=1.0,
         causal=True, q=q2, k=q2, v=v2, want=dict(shape=[1, 1, 2, 1], data=[10, 15]), tol=1e-5),
    dict(name="Direct/WithSeqLens", cite=f"{D}:62-86", dtype="f32", layout="BHSD", scale=1.0, causal=False,
         q=q2, k=q2, v=v2, q_len=[2], kv_len=[1],
         want=dict(shape=[1, 1, 2, 1], data=[10, 10]), tol=1e-5),
    dict(name="Direct/WithSeqLensCausal", cite=f"{D}:88-109", dtype="f32", layout="BHSD", scale=1.0,
         causal=True, q=q2, k=q2, v=v2, q_len=[2], kv_len=[2],
         want=dict(shape=[1, 1, 2, 1], data=[10, 15]), tol=1e-5),
    dict(name="Direct/SeqLenClamped/negative", cite=f"{D}:164-185", dtype="f32", layout="BHSD", scale=1.0,
         causal=False, q=q2, k=q2, v=v2, q_len=[-5], kv_len=[2],
         want=dict(shape=[1, 1, 2, 1], data=[0, 0]), tol=1e-5),
    dict(name="Direct/SeqLenClamped/too-large", cite=f"{D}:187-203", dtype="f32", layout="BHSD", scale=1.0,
         causal=False, q=q2, k=q2, v=v2, q_len=[999], kv_len=[999],
         want=dict(shape=[1, 1, 2, 1], data=[15, 15]), tol=1e-5),
]

# Requests the reference rejects (sdpa_direct_test.go:139-162, :205-259)
sdpa_error_cases = [
    dict(name="Direct/SeqLenWrongDtype", cite=f"{D}:139-162", q=q2, k=q2, v=v2,
         q_len=[2], kv_len=[2], seq_len_dtype="i64", error="invalid"),
    dict(name="Direct/BiasValidation/rank1", cite=f"{D}:205-237", q=q2, k=q2, v=v2,
         bias=dict(shape=[2], data=[1, 2]), error="invalid"),
    dict(name="Direct/BiasValidation/rank2_bad_kvdim", cite=f"{D}:205-237", q=q2, k=q2, v=v2,
         bias=dict(shape=[2, 3], data=[1, 2, 3, 1, 2, 3]), error="invalid"),
    dict(name="Direct/BiasValidation/rank4_bad_seqdim", cite=f"{D}:205-237", q=q2, k=q2, v=v2,
         bias=dict(shape=[1, 1, 3, 2], data=[1, 2, 1, 2, 1, 2]), error="invalid"),
    dict(name="Direct/FP8NotImplemented", cite=f"{D}:239-259", q=q2, k=q2, v=v2,
         dtype="f8e4m3fn", error="not_implemented"),
]

# FusedDense epilogue semantics (bias then activation; exact) — fusedops.go:178-212.
dense_cases = [
    dict(name="FusedDense/None", cite=f"{F}:184-195", activation="none",
         x=dict(shape=[2, 3], data=[1, 2, 3, 4, 5, 6]),
         w=dict(shape=[3, 4], data=[1, 0, 0, 1, 0, 1, 0, 1, 0, 0, 1, 1]),
         bias=[10, 20, 30, 40], want=dict(shape=[2, 4], data=[11, 22, 33, 46, 14, 25, 36, 55])),
    dict(name="FusedDense/Relu", cite=f"{F}:197-211", activation="relu",
         x=dict(shape=[1, 2], data=[1, -1]), w=dict(shape=[2, 2], data=[1, 1, 0, -1]),
         bias=[-1, -1], want=dict(shape=[1, 2], data=[0, 1])),
]

with open(os.path.join(HERE, "backendtest_dotgeneral.json"), "w") as f:
    json.dump(dict(source="gomlx/compute " + T, cases=dot_cases), f, indent=1)
with open(os.path.join(HERE, "backendtest_sdpa.json"), "w") as f:
    json.dump(dict(source="gomlx/compute " + F + " and " + D, cases=sdpa_cases,
                   error_cases=sdpa_error_cases), f, indent=1)
with open(os.path.join(HERE, "backendtest_dense_epilogue.json"), "w") as f:
    json.dump(dict(source="gomlx/compute " + F, cases=dense_cases), f, indent=1)
print("wrote", len(dot_cases), "dot,", len(sdpa_cases), "+", len(sdpa_error_cases), "sdpa,",
      len(dense_cases), "dense cases")

# compute.NF4LookupTable (fused_ops.go:114-121), the 16 NormalFloat4 values of QLoRA as the
# reference writes them (decimal expansions of float32 values).
nf4 = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
       -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
       0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
       0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0]
with open(os.path.join(HERE, "nf4_table.json"), "w") as f:
    json.dump(dict(source="gomlx/compute fused_ops.go:114-121", values=nf4), f, indent=1)

# FusedSoftmax / FusedGelu / FusedLayerNorm known answers (support/backendtest/fusedops.go:22-177).
small_cases = dict(
    softmax_1d=dict(cite=f"{F}:24-37", x=[1.0, 2.0, 3.0, 4.0], axis=0,
                    want=[0.0320586, 0.0871443, 0.2368828, 0.6439143], tol=1e-3),
    softmax_rows_sum_to_one=dict(cite=f"{F}:39-55", x=[[1, 2, 3], [4, 5, 6]], axis=1, tol=1e-3),
    softmax_stability=dict(cite=f"{F}:67-87", x=[1000, 1001, 1002], axis=0, tol=1e-3),
    gelu_exact=dict(cite=f"{F}:90-103", x=[-2.0, -1.0, -0.5, 0.0, 0.5, 1.0, 2.0],
                    want=[-0.04550028, -0.15865526, -0.15426877, 0.0, 0.34573123, 0.84134474, 1.9544997], tol=1e-3),
    layernorm_simple=dict(cite=f"{F}:128-157", x=[[1, 2, 3, 4], [5, 6, 7, 8]], axes=[1], epsilon=1e-5, mean_tol=1e-5, var_tol=1e-3),
    layernorm_gamma_beta=dict(cite=f"{F}:159-176", x=[1, 2, 3], gamma=[2, 2, 2], beta=[1, 1, 1], axes=[0], epsilon=1e-5,
                              want=[(1.0 - 2.0) / math.sqrt(2.0 / 3.0 + 1e-5) * 2.0 + 1.0, 1.0,
                                    (3.0 - 2.0) / math.sqrt(2.0 / 3.0 + 1e-5) * 2.0 + 1.0], tol=1e-4),
)
with open(os.path.join(HERE, "backendtest_fused_small.json"), "w") as f:
    json.dump(dict(source="gomlx/compute " + F, cases=small_cases), f, indent=1)
