"""GPU parity of FusedQuantizedDense against the CPU oracle, through the C ABI.

Tolerances are the ones the task states: f32 outputs within 1e-4 (max-abs
normalised), bf16 outputs within 2e-2; where the kernel keeps the reference's
summation order the comparison is bit-exact."""
import numpy as np
import pytest

from compute_b200 import BackendError, ErrNotImplemented, device as dv, ops
from oracle import oracle as orc
from tests.helpers import ACT, load_golden, max_abs_normalised, qdense_inputs, tensor

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4
BF16_TOL = 2e-2


def oracle_compact(x, w, s, b, layout, group, act):
    K, N = w.shape
    return orc.qdense_linear(x, w, orc.expand_scales(s, layout, K, N, group), None, b, 1, act,
                             threads=orc.max_threads())


# ------------------------------------------------------------- generic kernel
@pytest.mark.parametrize("act", ["none", "relu", "hard_swish"])
@pytest.mark.parametrize("block", [1, 3, 40])
def test_generic_reference_layout_bit_exact(act, block):
    """Reference scale layout [K, ceil(N/block)]: same summation order as the reference -> identical bits."""
    M, K, N = 5, 96, 40
    x, w, s, b = qdense_inputs(100 + block, M, K, N, scale_layout="ref", block_size=block)
    rng = np.random.default_rng(9)
    zp = rng.uniform(-0.05, 0.05, size=s.shape).astype(np.float32)
    for z in (None, zp):
        got = ops.quantized_dense(x, w, s, z, b, block_size=block, activation=ACT[act], variant=dv.QDENSE_GENERIC)
        want = orc.qdense_linear(x, w, s, z, b, block, ACT[act])
        assert np.array_equal(got, want)


@pytest.mark.parametrize("act", ["silu", "gelu", "tanh"])
def test_generic_transcendental_activations(act):
    x, w, s, b = qdense_inputs(7, 9, 130, 257, scale_layout="ref", block_size=16)
    got = ops.quantized_dense(x, w, s, None, b, block_size=16, activation=ACT[act], variant=dv.QDENSE_GENERIC)
    want = orc.qdense_linear(x, w, s, None, b, 16, ACT[act])
    assert max_abs_normalised(got, want) < 1e-6


def test_generic_uint8_and_batch_dims():
    x, w, s, b = qdense_inputs(8, 6, 64, 48, scale_layout="ref", block_size=48, unsigned=True)
    got = ops.quantized_dense(x.reshape(2, 3, 64), w, s, None, b, block_size=48, variant=dv.QDENSE_GENERIC)
    want = orc.qdense_linear(x, w, s, None, b, 48, orc.ACT_NONE).reshape(2, 3, 48)
    assert got.shape == (2, 3, 48) and np.array_equal(got, want)


@pytest.mark.parametrize("signed", [True, False])
@pytest.mark.parametrize("N", [40, 37])
def test_generic_packed_4bit_linear_bit_exact(signed, N):
    """Int4 / Uint4 weights, two per byte over the flat element order (an odd N makes rows straddle
    bytes): the reference unpacks them and runs the Linear scheme, so the bits are identical."""
    M, K, block = 5, 33, 8
    rng = np.random.default_rng(40 + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    vals = rng.integers(-8, 8, size=(K, N)) if signed else rng.integers(0, 16, size=(K, N))
    packed = orc.pack_nibbles(vals)
    w8 = (orc.unpack_int4(packed, K * N) if signed else orc.unpack_uint4(packed, K * N)).reshape(K, N)
    assert np.array_equal(w8, vals)
    nblk = -(-N // block)
    s = rng.uniform(0.01, 0.2, size=(K, nblk)).astype(np.float32)
    zp = rng.uniform(-0.05, 0.05, size=s.shape).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    for z in (None, zp):
        got, plan = ops.quantized_dense(x, packed, s, z, b, block_size=block, activation=dv.ACT_RELU,
                                        packed=(dv.I4 if signed else dv.U4, N), return_plan=True)
        assert plan.kernel_name == ("qdense_generic_f32_i4" if signed else "qdense_generic_f32_u4")
        assert np.array_equal(got, orc.qdense_linear(x, w8, s, z, b, block, orc.ACT_RELU))


@pytest.mark.parametrize("w_kind", ["i8", "u8", "i4", "u4"])
def test_generic_nf4_bit_exact(w_kind):
    """NF4: the low nibble of each weight indexes the NormalFloat4 table (quantizeddense.go:586-609)."""
    M, K, N, block = 4, 48, 36, 12
    rng = np.random.default_rng(77)
    x = rng.standard_normal((M, K)).astype(np.float32)
    idx = rng.integers(0, 16, size=(K, N))
    s = rng.uniform(0.01, 0.2, size=(K, N // block)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    want = orc.qdense_nf4(x, idx.astype(np.uint8), s, b, block, orc.ACT_SILU)
    # an independent statement of the same arithmetic
    table = orc.nf4_values()
    acc = np.tile(b, (M, 1))
    sx = np.repeat(s, block, axis=1)
    for k in range(K):
        acc = (acc + ((x[:, k:k + 1] * table[idx[k]][None, :]).astype(np.float32) * sx[k][None, :]).astype(np.float32)).astype(np.float32)
    assert max_abs_normalised(want, orc.activation_f64(acc.astype(np.float64), orc.ACT_SILU)) < 1e-6
    if w_kind == "u8":
        got = ops.quantized_dense(x, idx.astype(np.uint8), s, None, b, block_size=block, activation=dv.ACT_SILU, scheme=dv.QUANT_NF4)
    elif w_kind == "i8":      # Int4 values sign-extended to int8, as the reference's unpacking leaves them
        got = ops.quantized_dense(x, np.where(idx >= 8, idx - 16, idx).astype(np.int8), s, None, b, block_size=block,
                                  activation=dv.ACT_SILU, scheme=dv.QUANT_NF4)
    else:
        got = ops.quantized_dense(x, orc.pack_nibbles(idx), s, None, b, block_size=block, activation=dv.ACT_SILU,
                                  scheme=dv.QUANT_NF4, packed=(dv.I4 if w_kind == "i4" else dv.U4, N))
    assert max_abs_normalised(got, want) < 1e-6          # SiLU differs in the last bit between libm and the GPU
    got0 = ops.quantized_dense(x, idx.astype(np.uint8), s, None, b, block_size=block, scheme=dv.QUANT_NF4)
    assert np.array_equal(got0, orc.qdense_nf4(x, idx.astype(np.uint8), s, b, block, orc.ACT_NONE))


@pytest.mark.parametrize("kind", ["i4", "u4", "nf4_u4", "nf4_i4"])
@pytest.mark.parametrize("M,K,N,block,x_dtype", [(1, 4096, 14336, 64, "f32"), (5, 520, 520, 8, "f32"), (16, 1024, 264, 24, "bf16"),
                                                 (2, 300, 1000, 40, "f32"), (9, 2048, 136, 136, "f32"), (21, 1024, 264, 24, "f32"),
                                                 (32, 520, 512, 8, "bf16")])
def test_packed_4bit_decode_shapes(kind, M, K, N, block, x_dtype):
    """Decode shapes of the packed 4-bit formats run on the streaming kernel: one, two, four and eight rows of x per
    thread (and two row tiles), K cut over CTAs with a ragged last cut, ragged column tiles, every block size that is
    a multiple of 8, zero points, bias and activation, float32 and bfloat16 x.  From 17 to 32 rows of x the kernel runs
    once per 16 rows."""
    rng = np.random.default_rng(M * 1000 + N)
    nf4 = kind.startswith("nf4")
    signed = kind.endswith("i4")
    x = rng.standard_normal((M, K)).astype(np.float32)
    if M >= 5:
        x[1] = 0.0
        x[2] *= 100.0
    vals = rng.integers(0, 16, size=(K, N))
    packed = orc.pack_nibbles(vals)
    nblk = -(-N // block)
    s = rng.uniform(0.01, 0.2, size=(K, nblk)).astype(np.float32)
    zp = None if nf4 else rng.uniform(-0.05, 0.05, size=s.shape).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    xw = orc.bf16_to_f32(xin) if x_dtype == "bf16" else x
    tol = BF16_TOL if x_dtype == "bf16" else F32_TOL
    for z in ((None,) if nf4 else (None, zp)):
        if nf4:
            want = orc.qdense_nf4(xw, vals.astype(np.uint8), s, b, block, orc.ACT_GELU)
        else:
            w8 = np.where(vals >= 8, vals - 16, vals) if signed else vals
            want = orc.qdense_linear(xw, w8.astype(np.int8 if signed else np.uint8), s, z, b, block, orc.ACT_GELU)
        got, plan = ops.quantized_dense(xin, packed, s, z, b, x_dtype=code, block_size=block, activation=dv.ACT_GELU,
                                        scheme=dv.QUANT_NF4 if nf4 else dv.QUANT_LINEAR, packed=(dv.I4 if signed else dv.U4, N),
                                        return_plan=True)
        assert plan.kernel_name == f"qdense_w4_{x_dtype}_{'i4' if signed else 'u4'}{'_nf4' if nf4 else ''}" and plan.workspace_bytes > 0
        gotf = orc.bf16_to_f32(got) if x_dtype == "bf16" else got
        for m in range(M):
            assert max_abs_normalised(gotf[m], want[m]) < tol, (m, z is not None)
        # the generic kernel, by name, on the same case
        got_g, plan_g = ops.quantized_dense(xin, packed, s, z, b, x_dtype=code, block_size=block, activation=dv.ACT_GELU,
                                            scheme=dv.QUANT_NF4 if nf4 else dv.QUANT_LINEAR, packed=(dv.I4 if signed else dv.U4, N),
                                            variant=dv.QDENSE_GENERIC, return_plan=True)
        assert plan_g.kernel_name.startswith("qdense_generic_")
        if M * K * N > 2 ** 24:
            break                                  # the generic kernel needs milliseconds per call on the full projection


@pytest.mark.parametrize("kind", ["i8", "u8", "nf4_u8"])
@pytest.mark.parametrize("M,K,N,block,x_dtype", [(1, 4096, 14336, 64, "f32"), (5, 520, 520, 8, "f32"), (16, 1024, 264, 24, "bf16"),
                                                 (2, 300, 1000, 40, "f32"), (21, 2048, 144, 144, "f32")])
def test_reference_scales_8bit_decode_shapes(kind, M, K, N, block, x_dtype):
    """Int8 / Uint8 weights (and NF4 indices one per byte) with the reference's [K, N / block] scales, as a caller of the
    reference's interface passes them, at decode shapes: the streaming kernel with two words per lane, zero points,
    bias and activation; with a TMA ring (N a multiple of 16) and without; 17 to 32 rows run once per 16 rows."""
    rng = np.random.default_rng(M * 1000 + N + 1)
    nf4 = kind.startswith("nf4")
    x = rng.standard_normal((M, K)).astype(np.float32)
    if M >= 5:
        x[1] = 0.0
        x[2] *= 100.0
    if nf4:
        w = rng.integers(0, 16, size=(K, N)).astype(np.uint8)
    elif kind == "i8":
        w = rng.integers(-128, 128, size=(K, N)).astype(np.int8)
    else:
        w = rng.integers(0, 256, size=(K, N)).astype(np.uint8)
    nblk = -(-N // block)
    s = rng.uniform(0.001, 0.02, size=(K, nblk)).astype(np.float32)
    zp = None if nf4 else rng.uniform(-0.05, 0.05, size=s.shape).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    xw = orc.bf16_to_f32(xin) if x_dtype == "bf16" else x
    for z in ((None,) if nf4 else (None, zp)):
        want = orc.qdense_nf4(xw, w, s, b, block, orc.ACT_GELU) if nf4 else orc.qdense_linear(xw, w, s, z, b, block, orc.ACT_GELU, threads=orc.max_threads())
        got, plan = ops.quantized_dense(xin, w, s, z, b, x_dtype=code, block_size=block, activation=dv.ACT_GELU,
                                        scheme=dv.QUANT_NF4 if nf4 else dv.QUANT_LINEAR, return_plan=True)
        assert plan.kernel_name == f"qdense_w8_{x_dtype}_{'i8' if kind == 'i8' else 'u8'}{'_nf4' if nf4 else ''}" and plan.workspace_bytes > 0
        gotf = orc.bf16_to_f32(got) if x_dtype == "bf16" else got
        for m in range(M):
            assert max_abs_normalised(gotf[m], want[m]) < (BF16_TOL if x_dtype == "bf16" else F32_TOL), (m, z is not None)


def test_nf4_and_packed_validation():
    with pytest.raises(BackendError) as e:
        dv.Plan.qdense(2, 8, 8, dv.F32, dv.U8, dv.SCALE_REF, 8, has_zero_point=True, scheme=dv.QUANT_NF4)
    assert "ZeroPoint must be nil for NF4" in str(e.value)
    with pytest.raises(ErrNotImplemented):
        dv.Plan.qdense(2, 8, 8, dv.F32, dv.U8, dv.SCALE_REF, 8, scheme=7)          # no such scheme
    with pytest.raises(ErrNotImplemented):
        dv.Plan.qdense(2, 4096, 4096, dv.BF16, dv.I4, dv.SCALE_KGROUP, 128, variant=dv.QDENSE_DECODE_TC)


@pytest.mark.parametrize("ggml", ["q8_0", "q4_0"])
@pytest.mark.parametrize("x_dtype", ["f32", "bf16"])
@pytest.mark.parametrize("M,K,N", [(1, 4096, 512), (5, 96, 40), (16, 2048, 264), (33, 64, 7)])
def test_ggml_block_formats(M, K, N, x_dtype, ggml):
    """GGML Q8_0 / Q4_0 weights [N, bytesPerRow] (quantizeddense_ggml.go:98-196) against the oracle on the same bytes."""
    gt = orc.GGML_Q8_0 if ggml == "q8_0" else orc.GGML_Q4_0
    rng = np.random.default_rng(M + N)
    wq = orc.ggml_quantize_rows(rng.standard_normal((N, K)).astype(np.float32) * 0.05, gt)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.from_f32(x, orc.BF16) if x_dtype == "bf16" else x
    xw = orc.to_f32(xin, orc.BF16) if x_dtype == "bf16" else x
    want = orc.qdense_ggml(xw, wq, b, gt, orc.ACT_SILU)
    plan = dv.Plan.qdense(M, K, N, code, dv.U8, has_bias=True, activation=dv.ACT_SILU, scheme=dv.QUANT_GGML,
                          ggml_type=dv.GGML_Q8_0 if ggml == "q8_0" else dv.GGML_Q4_0)
    # decode shapes with K in whole 256-value steps run on the integer tensor cores, the rest on the CUDA-core kernel
    assert plan.kernel_name == f"qdense_ggml_{'mma_' if M <= 64 and K % 256 == 0 else ''}{x_dtype}_{ggml}"
    got = ops._run(plan, [xin, wq, b], (M, N), dv.NP_CARRIER[code])
    gotf = orc.to_f32(got, orc.BF16) if x_dtype == "bf16" else got
    assert max_abs_normalised(gotf, want) < (BF16_TOL if x_dtype == "bf16" else F32_TOL)


GGML_TYPES = {"q4_0": dv.GGML_Q4_0, "q8_0": dv.GGML_Q8_0, "iq4_nl": dv.GGML_IQ4_NL, "q4_k": dv.GGML_Q4_K, "q6_k": dv.GGML_Q6_K}


@pytest.mark.parametrize("ggml", list(GGML_TYPES))
@pytest.mark.parametrize("M,K,N,bias,act", [
    (1, 4096, 520, False, "none"),        # one token; N leaves a partly filled CTA and warp
    (3, 256, 33, True, "gelu"),           # one K-quant block per row
    (4, 1280, 64, True, "silu"),          # K is not a multiple of the 1024-value chunk
    (16, 2304, 40, False, "relu"),
    (21, 512, 9, True, "tanh"),           # two passes over the rows of x
])
def test_ggml_every_format_random_blocks(ggml, M, K, N, bias, act):
    """All five block formats of quantizeddense_ggml.go:133-302 on blocks whose quant and packed-scale bytes are random
    (every bit pattern of the 6-bit scale packing and of the high / low quant bits occurs)."""
    gt = GGML_TYPES[ggml]
    rng = np.random.default_rng(1000 * gt + M + N)
    wq = orc.ggml_random_rows(rng, N, K, gt)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32) if bias else None
    if act == "tanh":
        # random block scales give sums in the hundreds: scaled to [-2, 2], so that tanh is compared where it is not
        # saturated (a saturated row would turn an error of 1e-6 of the largest sum into 1e-4 of the largest output)
        top = float(np.max(np.abs(orc.qdense_ggml(x, wq, b, gt, ACT["none"]))))
        x = (x * np.float32(2.0 / top)).astype(np.float32)
        b = None if b is None else (b * np.float32(2.0 / top)).astype(np.float32)
    want = orc.qdense_ggml(x, wq, b, gt, ACT[act])
    plan = dv.Plan.qdense(M, K, N, dv.F32, dv.U8, has_bias=bias, activation=ACT[act], scheme=dv.QUANT_GGML, ggml_type=gt)
    on_tensor_cores = M <= 64 and K % 256 == 0 and ggml != "q6_k"
    assert plan.kernel_name == f"qdense_ggml_{'mma_' if on_tensor_cores else ''}f32_{ggml}"
    got = ops._run(plan, [x, wq] + ([b] if bias else []), (M, N), np.float32)
    assert max_abs_normalised(got, want) < F32_TOL
    # the CUDA-core kernel on the same case
    plan_cc = dv.Plan.qdense(M, K, N, dv.F32, dv.U8, has_bias=bias, activation=ACT[act], scheme=dv.QUANT_GGML, ggml_type=gt,
                             variant=dv.QDENSE_GENERIC)
    assert plan_cc.kernel_name == f"qdense_ggml_f32_{ggml}"
    got_cc = ops._run(plan_cc, [x, wq] + ([b] if bias else []), (M, N), np.float32)
    assert max_abs_normalised(got_cc, want) < F32_TOL


@pytest.mark.parametrize("ggml", ["q4_0", "q8_0", "iq4_nl", "q4_k"])
@pytest.mark.parametrize("M,K,N,x_dtype", [(1, 4096, 14336, "f32"), (2, 256, 64, "f32"), (5, 768, 130, "bf16"), (16, 2048, 1000, "f32"),
                                           (7, 512, 63, "f32"), (40, 512, 136, "f32"), (64, 256, 72, "bf16")])
def test_ggml_on_tensor_cores(ggml, M, K, N, x_dtype):
    """The integer-tensor-core kernel: one, two and six 8-column tiles of (digit plane, row) columns, both halves of K
    with one step or many, ragged N (rows past the end are computed and dropped), a row of x that is all zeros and one
    that is a thousand times larger than the others (its own unit), inf in x -> that row comes back NaN.  From 17 to
    64 rows of x the kernel runs once per 16 rows."""
    gt = GGML_TYPES[ggml]
    rng = np.random.default_rng(77 + gt + M)
    wq = orc.ggml_random_rows(rng, N, K, gt)
    x = rng.standard_normal((M, K)).astype(np.float32)
    if M >= 5:
        x[1] = 0.0
        x[2] *= 1000.0
    b = rng.standard_normal(N).astype(np.float32)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    xw = orc.bf16_to_f32(xin) if x_dtype == "bf16" else x
    want = orc.qdense_ggml(xw, wq, b, gt, orc.ACT_GELU)
    plan = dv.Plan.qdense(M, K, N, code, dv.U8, has_bias=True, activation=dv.ACT_GELU, scheme=dv.QUANT_GGML, ggml_type=gt)
    assert plan.kernel_name == f"qdense_ggml_mma_{x_dtype}_{ggml}" and plan.workspace_bytes > 0
    got = ops._run(plan, [xin, wq, b], (M, N), dv.NP_CARRIER[code])
    gotf = orc.bf16_to_f32(got) if x_dtype == "bf16" else got
    # every row against its own largest value: the huge row must not hide the others
    for m in range(M):
        assert max_abs_normalised(gotf[m], want[m]) < (BF16_TOL if x_dtype == "bf16" else F32_TOL), m
    if M >= 5 and x_dtype == "f32":
        x[3, 17] = np.inf
        got = ops._run(plan, [x, wq, b], (M, N), np.float32)
        assert np.isnan(got[3]).all() and np.isfinite(got[0]).all()
    with pytest.raises(BackendError):            # the digit planes live in the plan's workspace
        plan.launch([0x1000, 0x2000, 0x3000], [0x4000], None)


@pytest.mark.parametrize("ggml", list(GGML_TYPES))
@pytest.mark.parametrize("M,K,N,x_dtype,auto", [(17, 256, 72, "f32", False), (300, 512, 520, "f32", True), (130, 1024, 264, "bf16", False),
                                                (2048, 768, 1000, "bf16", True)])
def test_ggml_prefill_on_the_gemm(ggml, M, K, N, x_dtype, auto):
    """More than 16 rows of x: the weight rows are dequantised once into two bf16 planes and the product runs on the
    tensor-core GEMM with W as the transposed operand; a plan picks this by itself from 2^26 multiply-adds on."""
    gt = GGML_TYPES[ggml]
    rng = np.random.default_rng(5 * M + gt)
    wq = orc.ggml_random_rows(rng, N, K, gt)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    xw = orc.bf16_to_f32(xin) if x_dtype == "bf16" else x
    want = orc.qdense_ggml(xw, wq, b, gt, orc.ACT_SILU)
    plan = dv.Plan.qdense(M, K, N, code, dv.U8, has_bias=True, activation=dv.ACT_SILU, scheme=dv.QUANT_GGML, ggml_type=gt,
                          variant=dv.QDENSE_AUTO if auto else dv.QDENSE_PREFILL)
    assert plan.kernel_name == f"qdense_ggml_prefill_tcgen05_{x_dtype}_{ggml}" and plan.workspace_bytes > 0
    got = ops._run(plan, [xin, wq, b], (M, N), dv.NP_CARRIER[code])
    gotf = orc.bf16_to_f32(got) if x_dtype == "bf16" else got
    assert max_abs_normalised(gotf, want) < (BF16_TOL if x_dtype == "bf16" else 3e-5)


@pytest.mark.parametrize("ggml", list(GGML_TYPES))
def test_ggml_dequantised_values_are_bit_exact(ggml):
    """x = identity rows picks single weights: every dequantised value must carry the reference's bits."""
    gt = GGML_TYPES[ggml]
    K, N = 512, 37
    rng = np.random.default_rng(7 + gt)
    wq = orc.ggml_random_rows(rng, N, K, gt)
    want = orc.ggml_dequant_rows(wq, gt)                  # [N, K]
    for k0 in (0, 256):
        x = np.zeros((16, K), np.float32)
        cols = k0 + rng.choice(256, size=16, replace=False)
        x[np.arange(16), cols] = 1.0
        plan = dv.Plan.qdense(16, K, N, dv.F32, dv.U8, scheme=dv.QUANT_GGML, ggml_type=gt, variant=dv.QDENSE_GENERIC)
        got = ops._run(plan, [x, wq], (16, N), np.float32)
        # every selected weight with the reference's bits (the sum adds +0 to it, so a -0 weight reads back as +0)
        assert np.array_equal(got, want[:, cols].T) and not np.isnan(got).any()


@pytest.mark.parametrize("ggml", list(GGML_TYPES))
@pytest.mark.parametrize("index_dtype", ["i32", "i64", "u8"])
def test_quantized_embedding_lookup(ggml, index_dtype):
    """QuantizedEmbeddingLookup (quantizeddense.go:455-499): rows of a block table, bit for bit."""
    gt = GGML_TYPES[ggml]
    vocab, K = 200, 1280
    rng = np.random.default_rng(31 + gt)
    table = orc.ggml_random_rows(rng, vocab, K, gt)
    npdt, code = {"i32": (np.int32, dv.I32), "i64": (np.int64, dv.I64), "u8": (np.uint8, dv.U8)}[index_dtype]
    idx = rng.integers(0, vocab, size=(3, 5, 1)).astype(npdt)
    idx[0, 0, 0], idx[2, 4, 0] = 0, vocab - 1
    want = orc.embedding_lookup(table, idx, gt)
    plan = dv.Plan.embedding_lookup(vocab, table.shape[1], idx.size, code, gt)
    assert plan.kernel_name == f"embedding_lookup_{ggml}"
    got = ops._run(plan, [table, idx], (3, 5, K), np.float32)         # checks the plan's status words too
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # an index outside the table: zeros for that row and the reference's error from the status check
    bad = idx.copy().astype(np.int64)
    bad[1, 2, 0] = vocab
    plan64 = dv.Plan.embedding_lookup(vocab, table.shape[1], idx.size, dv.I64, gt)
    bufs = [dv.DeviceMem.from_numpy(a) for a in (table, bad)]
    out, ws64 = dv.DeviceMem(15 * K * 4), plan64.new_workspace()
    plan64.launch([b.ptr for b in bufs], [out.ptr], ws64.ptr)
    dv.check(dv._lib.load().cb_stream_sync(0, None))
    got = out.download((3, 5, K), np.float32)
    assert not got[1, 2].any() and np.array_equal(got[0], want[0])
    with pytest.raises(BackendError) as e:
        plan64.check_status(ws64.ptr)
    assert "position 7 out of range [0, 200)" in str(e.value)
    for m in bufs + [out, ws64]:
        m.free()


def test_embedding_lookup_validation():
    with pytest.raises(BackendError):            # bytesPerRow must be whole blocks (quantizeddense.go:171-174)
        dv.Plan.embedding_lookup(10, 100, 4, dv.I32, dv.GGML_Q4_0)
    with pytest.raises(ErrNotImplemented):
        dv.Plan.embedding_lookup(10, 84, 4, dv.I32, 3)              # Q2_K
    with pytest.raises(BackendError) as e:
        dv.Plan.embedding_lookup(10, 36, 4, dv.F32, dv.GGML_Q4_0)
    assert "indices must be integer" in str(e.value)


def test_ggml_validation():
    for unsupported in (3, 4, 6):          # Q2_K, Q3_K, Q5_K: ErrNotImplemented in the reference too (quantizeddense.go:145-152)
        with pytest.raises(ErrNotImplemented):
            dv.Plan.qdense(1, 256, 8, dv.F32, dv.U8, scheme=dv.QUANT_GGML, ggml_type=unsupported)
    with pytest.raises(BackendError):
        dv.Plan.qdense(1, 128, 8, dv.F32, dv.U8, scheme=dv.QUANT_GGML, ggml_type=dv.GGML_Q4_K)  # K-quants: K in whole 256-value blocks
    with pytest.raises(BackendError):
        dv.Plan.qdense(1, 48, 8, dv.F32, dv.U8, scheme=dv.QUANT_GGML, ggml_type=dv.GGML_Q8_0)  # K not whole blocks
    with pytest.raises(BackendError) as e:
        dv.Plan.qdense(1, 64, 8, dv.F32, dv.U8, has_zero_point=True, scheme=dv.QUANT_GGML, ggml_type=dv.GGML_Q8_0)
    assert "ZeroPoint must be nil for GGML" in str(e.value)


def test_dense_epilogue_golden_on_gpu():
    for case in load_golden("backendtest_dense_epilogue.json")["cases"]:
        x = tensor(case["x"], "f32")
        w = tensor(case["w"], "i8")
        K, N = w.shape
        got = ops.quantized_dense(x, w, np.ones((K, N), np.float32), None, np.array(case["bias"], np.float32),
                                  block_size=1, activation=ACT[case["activation"]])
        assert np.array_equal(got.ravel(), np.array(case["want"]["data"], np.float32))


@pytest.mark.parametrize("scale,zp,unsigned", [(0.25, None, False), (0.25, 0.5, False), (0.125, -16.0, True), (1.0, 3.0, False)])
def test_dense_epilogue_golden_with_scales_and_zero_points_on_gpu(scale, zp, unsigned):
    """fusedops.go:178-212 through the generic kernel with q = (w - zero_point) / scale: the reference's expected
    numbers, exactly, with non-unit scales and zero points in the reference's own layout."""
    from tests.test_oracle import requantise
    for case in load_golden("backendtest_dense_epilogue.json")["cases"]:
        x = tensor(case["x"], "f32")
        w_ref = tensor(case["w"], "i8")
        K, N = w_ref.shape
        q = requantise(w_ref, scale, zp or 0.0, unsigned)
        for block in (1, N):
            nblk = (N + block - 1) // block
            got = ops.quantized_dense(x, q, np.full((K, nblk), scale, np.float32), None if zp is None else np.full((K, nblk), zp, np.float32),
                                      np.array(case["bias"], np.float32), block_size=block, activation=ACT[case["activation"]])
            assert np.array_equal(got.ravel(), np.array(case["want"]["data"], np.float32))


@pytest.mark.parametrize("variant,M_pad,x_dtype", [(dv.QDENSE_DECODE_TC, 0, "f32"), (dv.QDENSE_DECODE_TC, 0, "bf16"), (dv.QDENSE_DECODE_TC, 16, "bf16"),
                                                   (dv.QDENSE_DECODE_MMA, 0, "f32"), (dv.QDENSE_PREFILL, 128, "f32")])
def test_dense_epilogue_golden_through_the_tensor_core_kernels(variant, M_pad, x_dtype):
    """The same reference cases embedded in a shape the streaming kernels accept: x padded with zero columns to K = 256
    (the weights under them random), N padded to 256 with random columns, rows padded with zeros; weights q = 4 w with
    scale 1/4 per 128-row group.  Every product and sum is a small dyadic number, so whatever the summation order the
    reference's expected values must come back exactly in the original rows and columns."""
    rng = np.random.default_rng(3)
    for case in load_golden("backendtest_dense_epilogue.json")["cases"]:
        x0 = tensor(case["x"], "f32")
        w0 = tensor(case["w"], "i8")
        (M0, K0), N0 = x0.shape, w0.shape[1]
        K, N, M = 256, 256, max(M0, M_pad)
        x = np.zeros((M, K), np.float32); x[:M0, :K0] = x0
        q = rng.integers(-127, 128, size=(K, N), dtype=np.int64).astype(np.int8)
        q[:K0, :N0] = 4 * w0
        s = np.full((K // 128, N), 0.25, np.float32)
        b = rng.standard_normal(N).astype(np.float32); b[:N0] = np.array(case["bias"], np.float32)
        code = dv.BF16 if x_dtype == "bf16" else dv.F32
        xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x          # the cases' values are exact in bfloat16
        got, plan = ops.quantized_dense(xin, q, s, None, b, x_dtype=code, scale_layout=dv.SCALE_KGROUP, block_size=128,
                                        activation=ACT[case["activation"]], variant=variant, return_plan=True)
        gotf = orc.bf16_to_f32(got) if x_dtype == "bf16" else got
        want = np.array(case["want"]["data"], np.float32).reshape(M0, N0)
        assert np.array_equal(gotf[:M0, :N0], want), (plan.kernel_name, case["name"])


def test_config1_reference_cpu_case():
    """x f32 [64,1024], W int8 [1024,1024], per-output-channel scales, bias, no activation."""
    x, w, s, b = qdense_inputs(0x5EED0001, 64, 1024, 1024, scale_layout="channel")
    got, plan = ops.quantized_dense(x, w, s, None, b, scale_layout=dv.SCALE_CHANNEL, return_plan=True)
    want = oracle_compact(x, w, s, b, "channel", 0, orc.ACT_NONE)
    assert max_abs_normalised(got, want) < F32_TOL
    assert plan.kernel_name.startswith("qdense_prefill_tcgen05_f32")
    # the same numbers through the reference's own scale layout (expanded [K,N], BlockSize=1):
    # identical bits from the kernel that keeps the reference's summation order, and within
    # tolerance from the tensor-core path the planner picks for this size
    sref = orc.expand_scales(s, "channel", 1024, 1024)
    got_ref = ops.quantized_dense(x, w, sref, None, b, block_size=1, variant=dv.QDENSE_GENERIC)
    assert np.array_equal(got_ref, want)
    got_auto = ops.quantized_dense(x, w, sref, None, b, block_size=1)
    assert max_abs_normalised(got_auto, want) < 1e-5


# ------------------------------------------------------------- decode kernel
DECODE_SHAPES = [
    # M, K, N, layout, group
    (1, 16, 16, "channel", 0),
    (3, 80, 144, "channel", 0),        # ragged K chunk and N tile
    (8, 256, 384, "kgroup", 64),
    (9, 512, 1792, "kgroup", 128),
    (16, 1024, 2048, "kgroup", 128),
    (4, 4096, 1792, "kgroup", 128),    # one 8-GPU shard of the 4096x14336 projection
    (2, 192, 100 * 16, "kgroup", 192),
]


DECODE_KERNELS = {dv.QDENSE_DECODE_MMA: "qdense_decode_", dv.QDENSE_DECODE_TC: "qdense_decode_tc_"}


@pytest.mark.parametrize("variant", list(DECODE_KERNELS))
@pytest.mark.parametrize("M,K,N,layout,group", DECODE_SHAPES)
@pytest.mark.parametrize("x_dtype", ["f32", "bf16"])
def test_decode_matches_oracle(M, K, N, layout, group, x_dtype, variant):
    if variant == dv.QDENSE_DECODE_TC and layout == "kgroup" and group % 128:
        with pytest.raises(ErrNotImplemented):     # its K units are 128 rows: finer groups stay on the other kernel
            dv.Plan.qdense(M, K, N, dv.F32, dv.I8, dv.SCALE_KGROUP, group, variant=variant)
        return
    x, w, s, b = qdense_inputs(M * 1000 + K + N, M, K, N, x_dtype=x_dtype, scale_layout=layout, group=group)
    sl = dv.SCALE_CHANNEL if layout == "channel" else dv.SCALE_KGROUP
    want = oracle_compact(x, w, s, b, layout, group, orc.ACT_SILU)
    prefix = DECODE_KERNELS[variant]
    if x_dtype == "bf16":
        got, plan = ops.quantized_dense(orc.bf16_from_f32(x), w, s, None, b, x_dtype=dv.BF16, scale_layout=sl,
                                        block_size=group, activation=dv.ACT_SILU, variant=variant, return_plan=True)
        assert plan.kernel_name.startswith(prefix + "bf16")
        assert max_abs_normalised(orc.bf16_to_f32(got), want) < BF16_TOL
        # tighter: equal to the f32 result rounded to bf16, up to one bf16 ulp of the largest value
        assert max_abs_normalised(orc.bf16_to_f32(got), orc.bf16_to_f32(orc.bf16_from_f32(want))) < 2.0 ** -7
    else:
        got, plan = ops.quantized_dense(x, w, s, None, b, scale_layout=sl, block_size=group,
                                        activation=dv.ACT_SILU, variant=variant, return_plan=True)
        assert plan.kernel_name.startswith(prefix + "f32")
        assert max_abs_normalised(got, want) < F32_TOL
    # and the generic kernel (reference summation order) agrees on the same compact layout
    gen = ops.quantized_dense(x if x_dtype == "f32" else orc.bf16_from_f32(x), w, s, None, b,
                              x_dtype=dv.F32 if x_dtype == "f32" else dv.BF16, scale_layout=sl, block_size=group,
                              activation=dv.ACT_SILU, variant=dv.QDENSE_GENERIC)
    if x_dtype == "f32":
        assert max_abs_normalised(gen, want) < 1e-6


@pytest.mark.parametrize("variant,group", [(dv.QDENSE_DECODE_MMA, 64), (dv.QDENSE_DECODE_TC, 128)])
def test_decode_uint8_no_bias_all_activations(variant, group):
    x, w, s, _ = qdense_inputs(21, 5, 384, 272, scale_layout="kgroup", group=group, bias=False, unsigned=True)
    for act in ACT.values():
        got = ops.quantized_dense(x, w, s, None, None, scale_layout=dv.SCALE_KGROUP, block_size=group, activation=act,
                                  variant=variant)
        want = oracle_compact(x, w, s, None, "kgroup", group, act)
        assert max_abs_normalised(got, want) < F32_TOL


@pytest.mark.parametrize("x_dtype", ["f32", "bf16"])
@pytest.mark.parametrize("M,K,N,ctas_per_tile", [
    (16, 4096, 4096, (4,)),          # an o projection: 32 tiles
    (1, 2048, 1008, (4,)),           # ragged last tile, 16 units per tile: four each
    (7, 4096, 5120, (3, 2)),         # 40 tiles: three CTAs per tile where that many clusters are resident, else two
    (16, 1024, 7168, (2,)),          # 56 tiles, 8 units per tile: two CTAs with four units each
    (5, 1536, 2048, (3, 2)),         # 12 units per tile: three CTAs
    (16, 512, 2048, (1, 9)),         # 4 units per tile are too few to share: no clusters
])
def test_decode_tc_few_tiles_on_cta_clusters(M, K, N, ctas_per_tile, x_dtype):
    """A projection of few column tiles gives every tile to a cluster of CTAs that sum their partial tiles through
    distributed shared memory: the grid is a whole number of CTAs per tile, the result matches the oracle, does not
    change from launch to launch, and agrees with the kernel that keeps the reference's order of summation."""
    x, w, s, b = qdense_inputs(31 * M + K + N, M, K, N, x_dtype=x_dtype, scale_layout="kgroup", group=128)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    want = oracle_compact(x, w, s, b, "kgroup", 128, orc.ACT_GELU)
    runs = []
    for _ in range(3):
        got, plan = ops.quantized_dense(xin, w, s, None, b, x_dtype=code, scale_layout=dv.SCALE_KGROUP, block_size=128,
                                        activation=dv.ACT_GELU, variant=dv.QDENSE_DECODE_TC, return_plan=True)
        runs.append(got)
    tiles = (N + 127) // 128
    assert plan.kernel_name.startswith("qdense_decode_tc_")
    if ctas_per_tile != (1, 9):
        assert plan.blocks % tiles == 0 and plan.blocks // tiles in ctas_per_tile, (plan.blocks, tiles)
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    if x_dtype == "bf16":
        assert max_abs_normalised(orc.bf16_to_f32(runs[0]), want) < BF16_TOL
        assert max_abs_normalised(orc.bf16_to_f32(runs[0]), orc.bf16_to_f32(orc.bf16_from_f32(want))) < 2.0 ** -7
    else:
        assert max_abs_normalised(runs[0], want) < 1e-5
        gen = ops.quantized_dense(x, w, s, None, b, scale_layout=dv.SCALE_KGROUP, block_size=128, activation=dv.ACT_GELU,
                                  variant=dv.QDENSE_GENERIC)
        assert max_abs_normalised(runs[0], gen) < 1e-5


@pytest.mark.parametrize("M", list(range(1, 17)))
def test_decode_tc_every_batch_size(M):
    """M = 1..16 crosses the three digit-tile widths (5, 10 and 16 rows per digit plane)."""
    K, N = 384, 400
    x, w, s, b = qdense_inputs(500 + M, M, K, N, scale_layout="kgroup", group=128)
    got, plan = ops.quantized_dense(x, w, s, None, b, scale_layout=dv.SCALE_KGROUP, block_size=128, activation=dv.ACT_GELU,
                                    variant=dv.QDENSE_DECODE_TC, return_plan=True)
    assert plan.kernel_name == f"qdense_decode_tc_f32_n{16 if M <= 5 else 32 if M <= 10 else 48}_i8"
    want = oracle_compact(x, w, s, b, "kgroup", 128, orc.ACT_GELU)
    assert max_abs_normalised(got, want) < 1e-5


def test_decode_tc_fixed_point_digits_edge_cases():
    """Rows of zeros, rows spanning 30 binades, subnormals and a non-finite value: the int8 digit
    form of x keeps 20 bits below each row's maximum, so small entries beside a large one are
    rounded at 2^-21 of the maximum; a row holding inf or NaN comes back as NaN."""
    M, K, N = 6, 512, 256
    x, w, s, b = qdense_inputs(99, M, K, N, scale_layout="channel")
    x[0] = 0.0
    x[1] *= np.exp2(np.random.default_rng(1).integers(-30, 1, size=K)).astype(np.float32)
    x[2] *= np.float32(1e-41)
    x[3] *= np.float32(1e30)
    x[4, 17] = np.inf
    got = ops.quantized_dense(x, w, s, None, b, scale_layout=dv.SCALE_CHANNEL, variant=dv.QDENSE_DECODE_TC)
    ok = [0, 1, 2, 3, 5]
    want = oracle_compact(np.ascontiguousarray(x[ok]), w, s, b, "channel", 0, orc.ACT_NONE)
    for i, r in enumerate(ok):
        scale = max(np.abs(want[i] - b).max(), 1e-30)
        assert np.abs(got[r] - want[i]).max() / scale < F32_TOL, r
    assert np.isnan(got[4]).all()


@pytest.mark.parametrize("M", list(range(1, 17)))
def test_decode_tc_bf16_two_digit_planes_every_batch_size(M):
    """bfloat16 activations beyond five rows travel as two int8 digit planes (8 rows per plane up to M = 8, 16
    beyond); up to five rows three planes fit the narrowest MMA, as for float32."""
    K, N = 384, 400
    x, w, s, b = qdense_inputs(700 + M, M, K, N, x_dtype="bf16", scale_layout="kgroup", group=128)
    got, plan = ops.quantized_dense(orc.bf16_from_f32(x), w, s, None, b, x_dtype=dv.BF16, scale_layout=dv.SCALE_KGROUP,
                                    block_size=128, activation=dv.ACT_GELU, variant=dv.QDENSE_DECODE_TC, return_plan=True)
    assert plan.kernel_name == "qdense_decode_tc_bf16_" + ("n16" if M <= 5 else "n16p2" if M <= 8 else "n32p2") + "_i8"
    want = oracle_compact(x, w, s, b, "kgroup", 128, orc.ACT_GELU)
    assert max_abs_normalised(orc.bf16_to_f32(got), want) < BF16_TOL
    assert max_abs_normalised(orc.bf16_to_f32(got), orc.bf16_to_f32(orc.bf16_from_f32(want))) < 2.0 ** -7


def test_decode_tc_bf16_two_plane_error_bound():
    """The two-plane fixed point keeps 13 bits below each 128-wide unit's maximum: elements within 2^-6 of it are
    exact, smaller ones are rounded at 2^-14 of it, which is far below the bfloat16 rounding of the result itself
    (2^-8 of its size).  Rows of zeros, a row spanning 30 binades, a huge row and a non-finite value behave as in
    the three-plane form."""
    M, K, N = 6, 512, 256
    x, w, s, b = qdense_inputs(98, M, K, N, x_dtype="bf16", scale_layout="channel")
    x[0] = 0.0
    x[1] = orc.bf16_to_f32(orc.bf16_from_f32(x[1] * np.exp2(np.random.default_rng(1).integers(-30, 1, size=K)).astype(np.float32)))
    x[3] = orc.bf16_to_f32(orc.bf16_from_f32(x[3] * np.float32(1e30)))
    x[4, 17] = np.inf
    got = orc.bf16_to_f32(ops.quantized_dense(orc.bf16_from_f32(x), w, s, None, b, x_dtype=dv.BF16, scale_layout=dv.SCALE_CHANNEL,
                                              variant=dv.QDENSE_DECODE_TC))
    ok = [0, 1, 2, 3, 5]
    want = oracle_compact(np.ascontiguousarray(x[ok]), w, s, b, "channel", 0, orc.ACT_NONE)
    for i, r in enumerate(ok):
        scale = max(np.abs(want[i]).max(), 1e-30)
        # one bfloat16 rounding of the result (2^-9 relative to its own size) plus the digit error
        assert np.abs(got[r] - want[i]).max() / scale < 1.25 * 2.0 ** -8, r
    assert np.isnan(got[4]).all()


# ------------------------------------------------------------- grouped launch, bound launches
def _group_case(x_dtype):
    """Three projections of different widths on two activation matrices (members 0 and 2 share x)."""
    M, K = 7, 512
    widths = [(400, True, "silu"), (1792, False, "none"), (144, True, "gelu")]
    rng = np.random.default_rng(11)
    xs = [rng.standard_normal((M, K), dtype=np.float32) for _ in range(2)]
    if x_dtype == "bf16":
        xs = [orc.bf16_to_f32(orc.bf16_from_f32(x)) for x in xs]
    members = []
    for i, (N, has_b, act) in enumerate(widths):
        _, w, s, b = qdense_inputs(40 + i, M, K, N, scale_layout="kgroup", group=128, bias=has_b)
        members.append(dict(N=N, x=xs[0] if i != 1 else xs[1], xi=0 if i != 1 else 1, w=w, s=s, b=b, act=act))
    return M, K, xs, members


@pytest.mark.parametrize("x_dtype", ["f32", "bf16"])
@pytest.mark.parametrize("bound", [False, True])
def test_decode_group_matches_oracle_and_single_plans(x_dtype, bound):
    """A group of independent projections runs as one launch; every member equals its own single-plan result
    (same arithmetic per column; the order in which k units are summed may differ where tiles are split)."""
    M, K, xs, members = _group_case(x_dtype)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    esize = 2 if x_dtype == "bf16" else 4
    carrier = np.uint16 if x_dtype == "bf16" else np.float32
    up = (lambda a: orc.bf16_from_f32(a)) if x_dtype == "bf16" else (lambda a: a)
    plan = dv.Plan.qdense_group(M, K, [(m["N"], m["b"] is not None, ACT[m["act"]]) for m in members], code, dv.I8,
                                dv.SCALE_KGROUP, 128)
    assert plan.kernel_name.endswith("_x3")
    st = dv.Stream(0)
    xd = [dv.DeviceMem.from_numpy(up(x)) for x in xs]
    ins, outs, keep = [], [], []
    for m in members:
        wd, sd = dv.DeviceMem.from_numpy(m["w"]), dv.DeviceMem.from_numpy(m["s"])
        keep += [wd, sd]
        ins += [xd[m["xi"]].ptr, wd.ptr, sd.ptr]
        if m["b"] is not None:
            bd = dv.DeviceMem.from_numpy(m["b"])
            keep.append(bd)
            ins.append(bd.ptr)
        od = dv.DeviceMem(M * m["N"] * esize)
        od.zero()
        outs.append(od)
    ws = plan.new_workspace()
    if bound:
        b = plan.bind(ins, [o.ptr for o in outs], ws.ptr)
        for _ in range(3):                      # repeated launches leave the workspace ready
            b.launch(st)
        dv.BoundSequence([b, b]).launch(st)
    else:
        for _ in range(2):
            plan.launch(ins, [o.ptr for o in outs], ws.ptr, st)
    st.sync()
    plan.check_status(ws.ptr)
    for m, od in zip(members, outs):
        got = od.download((M, m["N"]), carrier)
        want = oracle_compact(m["x"], m["w"], m["s"], m["b"], "kgroup", 128, ACT[m["act"]])
        single = ops.quantized_dense(up(m["x"]), m["w"], m["s"], None, m["b"], x_dtype=code, scale_layout=dv.SCALE_KGROUP,
                                     block_size=128, activation=ACT[m["act"]], variant=dv.QDENSE_DECODE_TC)
        if x_dtype == "bf16":
            assert max_abs_normalised(orc.bf16_to_f32(got), want) < BF16_TOL
            assert max_abs_normalised(orc.bf16_to_f32(got), orc.bf16_to_f32(single)) < 2.0 ** -7
        else:
            assert max_abs_normalised(got, want) < F32_TOL
            assert max_abs_normalised(got, single) < 1e-6


@pytest.mark.parametrize("L,M,blocks", [(4, 16, 112), (6, 4, 135)])
def test_decode_group_full_size_step(L, M, blocks):
    """The benchmark's step as one launch: L distinct 4096 x 14336 layers (4 x 112 column tiles on 112 CTAs, four
    tiles each; 6 x 112 tiles on 135 CTAs, five tiles each but for three CTAs with four).  CTA c takes the tiles
    c, c + grid, ...  Every layer agrees with its own single launch to one bfloat16 step of the largest value (the two
    epilogue groups share a tile's k units by pipeline stage, so the order of the float32 additions depends on where
    the tile starts in a CTA's run) and the group launch is repeatable bit for bit."""
    K, N = 4096, 14336
    rng = np.random.default_rng(5)
    plan = dv.Plan.qdense_group(M, K, [(N, False, dv.ACT_SILU)] * L, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128)
    assert plan.blocks == blocks
    single = dv.Plan.qdense(M, K, N, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128, False, False, dv.ACT_SILU)
    st = dv.Stream(0)
    ins, outs, ref_outs, keep = [], [], [], []
    for layer in range(L):
        x = orc.bf16_from_f32(rng.standard_normal((M, K), dtype=np.float32))
        w = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
        s = rng.uniform(0.001, 0.02, size=(K // 128, N)).astype(np.float32)
        d = [dv.DeviceMem.from_numpy(a) for a in (x, w, s)]
        keep += d
        ins += [m.ptr for m in d]
        outs.append(dv.DeviceMem(M * N * 2))
        ref_outs.append(dv.DeviceMem(M * N * 2))
        if layer == L - 1:                      # one layer against the oracle; the rest against the single plan's bits
            want = oracle_compact(orc.bf16_to_f32(x), w, s, None, "kgroup", 128, orc.ACT_SILU)
    ws, ws1 = plan.new_workspace(), single.new_workspace()
    bound = plan.bind(ins, [o.ptr for o in outs], ws.ptr)
    bound.launch(st)
    for layer in range(L):
        single.launch(ins[3 * layer:3 * layer + 3], [ref_outs[layer].ptr], ws1.ptr, st)
    st.sync()
    plan.check_status(ws.ptr)
    first = [o.download((M, N), np.uint16) for o in outs]
    for layer in range(L):
        assert max_abs_normalised(orc.bf16_to_f32(first[layer]), orc.bf16_to_f32(ref_outs[layer].download((M, N), np.uint16))) < 2.0 ** -7
    assert max_abs_normalised(orc.bf16_to_f32(first[L - 1]), want) < BF16_TOL
    for o in outs:
        o.zero()
    for _ in range(3):                          # back to back: the next launch's set-up overlaps the previous one's tail
        bound.launch(st)
    st.sync()
    plan.check_status(ws.ptr)
    for layer in range(L):
        assert np.array_equal(outs[layer].download((M, N), np.uint16), first[layer])


@pytest.mark.parametrize("seed", list(range(24)))
def test_decode_group_random_shapes(seed):
    """A seeded sweep over what the grouped launch has to get right together: 1..16 members of unequal, ragged widths (so the
    tile count lands on either side of the whole-tile / split-schedule thresholds), K from one to 24 units (stage and
    accumulator rings wrap many times or never), every batch size (16-, 32- and 48-column MMAs; two or three digit
    planes), shared and private activations, bias and activation per member; each member against the oracle, and the
    launch repeated back to back bit for bit."""
    rng = np.random.default_rng(9000 + seed)
    x_dtype = "bf16" if seed % 3 else "f32"
    M = int(rng.integers(1, 17))
    K = 128 * int(rng.choice([1, 2, 3, 5, 8, 24]))
    n_members = int(rng.choice([1, 2, 3, 5, 8, 16]))
    widths = [int(rng.choice([16, 48, 128, 144, 528, 1792, 3008])) for _ in range(n_members)]
    n_x = int(rng.integers(1, min(3, n_members) + 1))
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    esize, carrier = (2, np.uint16) if x_dtype == "bf16" else (4, np.float32)
    xs = [rng.standard_normal((M, K), dtype=np.float32) * np.float32(10.0 ** rng.integers(-3, 1)) for _ in range(n_x)]
    if x_dtype == "bf16":
        xs = [orc.bf16_to_f32(orc.bf16_from_f32(x)) for x in xs]
    up = (lambda a: orc.bf16_from_f32(a)) if x_dtype == "bf16" else (lambda a: a)
    # Tanh is left to the other tests: here pre-activations reach tens, where its output saturates at 1 while the float32
    # rounding noise of the reference's own k-ascending sum (about 1e-4 absolute at that size) stays, so a bar normalised
    # by the largest output would measure the oracle, not the kernel.
    acts = [v for k_, v in ACT.items() if k_ != "tanh"]
    members = []
    for N in widths:
        members.append({"N": N, "xi": int(rng.integers(0, n_x)), "act": acts[int(rng.integers(0, len(acts)))],
                        "w": rng.integers(-127, 128, size=(K, N), dtype=np.int8),
                        "s": rng.uniform(0.001, 0.02, size=(K // 128, N)).astype(np.float32),
                        "b": (rng.standard_normal(N) * 0.1).astype(np.float32) if rng.integers(0, 2) else None})
    plan = dv.Plan.qdense_group(M, K, [(m["N"], m["b"] is not None, m["act"]) for m in members], code, dv.I8, dv.SCALE_KGROUP, 128)
    st = dv.Stream(0)
    xd = [dv.DeviceMem.from_numpy(up(x)) for x in xs]
    ins, outs, keep = [], [], []
    for m in members:
        wd, sd = dv.DeviceMem.from_numpy(m["w"]), dv.DeviceMem.from_numpy(m["s"])
        keep += [wd, sd]
        ins += [xd[m["xi"]].ptr, wd.ptr, sd.ptr]
        if m["b"] is not None:
            keep.append(dv.DeviceMem.from_numpy(m["b"]))
            ins.append(keep[-1].ptr)
        outs.append(dv.DeviceMem(M * m["N"] * esize))
        outs[-1].zero()
    ws = plan.new_workspace()
    bound = plan.bind(ins, [o.ptr for o in outs], ws.ptr)
    bound.launch(st)
    st.sync()
    plan.check_status(ws.ptr)
    first = [o.download((M, m["N"]), carrier) for o, m in zip(outs, members)]
    for m, got in zip(members, first):
        want = oracle_compact(xs[m["xi"]], m["w"], m["s"], m["b"], "kgroup", 128, m["act"])
        gotf = orc.bf16_to_f32(got) if x_dtype == "bf16" else got
        assert max_abs_normalised(gotf, want) < (BF16_TOL if x_dtype == "bf16" else F32_TOL), (plan.kernel_name, plan.blocks, m["N"])
    for o in outs:
        o.zero()
    dv.BoundSequence([bound, bound, bound]).launch(st)
    st.sync()
    plan.check_status(ws.ptr)
    for o, m, f in zip(outs, members, first):
        assert np.array_equal(o.download((M, m["N"]), carrier), f), (plan.kernel_name, plan.blocks, m["N"])
    for d in xd + keep + outs + [ws]:
        d.free()


def test_bound_launch_of_other_plans():
    """cb_plan_bind works for every plan kind; plans without prepared state go through their ordinary launch."""
    x, w, s, b = qdense_inputs(3, 40, 256, 272, scale_layout="channel")
    plan = dv.Plan.qdense(40, 256, 272, dv.F32, dv.I8, dv.SCALE_CHANNEL, 0, False, True, dv.ACT_RELU, variant=dv.QDENSE_GENERIC)
    d = [dv.DeviceMem.from_numpy(a) for a in (x, w, s, b)]
    out = dv.DeviceMem(40 * 272 * 4)
    bnd = plan.bind([m.ptr for m in d], [out.ptr], None)
    bnd.launch(None)
    dv.check(dv._lib.load().cb_stream_sync(0, None))
    want = oracle_compact(x, w, s, b, "channel", 0, orc.ACT_RELU)
    assert np.array_equal(out.download((40, 272), np.float32), want)
    with pytest.raises(BackendError):
        plan.bind([m.ptr for m in d[:3]], [out.ptr], None)


@pytest.mark.parametrize("M", [1, 4, 16])
def test_config3_full_size(M):
    """Decode-shaped projection 4096 x 14336, bf16 x, group-128 scales along K, SiLU."""
    K, N = 4096, 14336
    x, w, s, _ = qdense_inputs(0x5EED0003 + M, M, K, N, x_dtype="bf16", scale_layout="kgroup", group=128, bias=False)
    xb = orc.bf16_from_f32(x)
    got, plan = ops.quantized_dense(xb, w, s, None, None, x_dtype=dv.BF16, scale_layout=dv.SCALE_KGROUP,
                                    block_size=128, activation=dv.ACT_SILU, return_plan=True)
    assert plan.kernel_name.startswith("qdense_decode_tc_bf16")
    want = oracle_compact(x, w, s, None, "kgroup", 128, orc.ACT_SILU)
    assert max_abs_normalised(orc.bf16_to_f32(got), want) < BF16_TOL
    # size-independent properties: repeatable bit for bit, and column shards agree with the full result
    again = ops.quantized_dense(xb, w, s, None, None, x_dtype=dv.BF16, scale_layout=dv.SCALE_KGROUP,
                                block_size=128, activation=dv.ACT_SILU)
    assert np.array_equal(got, again)
    g = 8
    for r in (0, g - 1):
        cols = slice(r * N // g, (r + 1) * N // g)
        part = ops.quantized_dense(xb, np.ascontiguousarray(w[:, cols]), np.ascontiguousarray(s[:, cols]), None, None,
                                   x_dtype=dv.BF16, scale_layout=dv.SCALE_KGROUP, block_size=128,
                                   activation=dv.ACT_SILU)
        assert max_abs_normalised(orc.bf16_to_f32(part), orc.bf16_to_f32(got[:, cols])) < 2.0 ** -7


def test_decode_linearity_property():
    """(a*x1 + x2) W == a*(x1 W) + x2 W without activation, at full width."""
    K, N = 2048, 14336
    x1, w, s, _ = qdense_inputs(33, 2, K, N, scale_layout="channel", bias=False)
    x2 = np.random.default_rng(34).standard_normal((2, K)).astype(np.float32)
    run = lambda x: ops.quantized_dense(x, w, s, None, None, scale_layout=dv.SCALE_CHANNEL).astype(np.float64)
    lhs = run(2.0 * x1 + x2)
    rhs = 2.0 * run(x1) + run(x2)
    assert max_abs_normalised(lhs, rhs) < 1e-5


# ------------------------------------------------------------- prefill kernel
PREFILL_SHAPES = [
    # M, K, N, layout, block/group, zero points
    (17, 64, 72, "channel", 0, False),       # smallest M beyond the decode kernel, ragged tiles
    (130, 200, 264, "kgroup", 40, False),
    (300, 512, 520, "ref", 16, True),
    (257, 1024, 1024, "kgroup", 128, False),
    (64, 320, 136, "ref", 1, False),
    (40, 200, 272, "channel", 0, False),     # ragged K block and tiles
    (129, 4096, 512, "channel", 0, False),
]


@pytest.mark.parametrize("M,K,N,layout,block,with_zp", PREFILL_SHAPES)
@pytest.mark.parametrize("x_dtype", ["f32", "bf16"])
def test_prefill_matches_oracle(M, K, N, layout, block, with_zp, x_dtype):
    if layout == "ref":
        x, w, s, b = qdense_inputs(M + K + N, M, K, N, x_dtype=x_dtype, scale_layout="ref", block_size=block)
        full, sl = s, dv.SCALE_REF
    else:
        x, w, s, b = qdense_inputs(M + K + N, M, K, N, x_dtype=x_dtype, scale_layout=layout, group=block)
        full, sl = orc.expand_scales(s, layout, K, N, block), (dv.SCALE_CHANNEL if layout == "channel" else dv.SCALE_KGROUP)
    zp = np.random.default_rng(5).uniform(-0.05, 0.05, size=s.shape).astype(np.float32) if with_zp else None
    want = orc.qdense_linear(x, w, full, zp, b, block if layout == "ref" else 1, orc.ACT_GELU, threads=orc.max_threads())
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    got, plan = ops.quantized_dense(xin, w, s, zp, b, x_dtype=dv.BF16 if x_dtype == "bf16" else dv.F32, scale_layout=sl,
                                    block_size=block, activation=dv.ACT_GELU, variant=dv.QDENSE_PREFILL, return_plan=True)
    assert plan.kernel_name.startswith("qdense_prefill_tcgen05_" + x_dtype)
    if x_dtype == "bf16":
        assert max_abs_normalised(orc.bf16_to_f32(got), want) < BF16_TOL
        assert max_abs_normalised(orc.bf16_to_f32(got), orc.bf16_to_f32(orc.bf16_from_f32(want))) < 2.0 ** -7
    else:
        assert max_abs_normalised(got, want) < 1e-5


@pytest.mark.parametrize("kind", ["i4", "u4", "nf4_u4", "nf4_i4", "nf4_u8"])
@pytest.mark.parametrize("M,K,N,block,with_zp,x_dtype", [(17, 64, 72, 8, False, "f32"), (300, 512, 520, 16, True, "f32"),
                                                        (130, 1024, 264, 24, True, "bf16"), (2048, 520, 1000, 40, False, "f32")])
def test_prefill_packed_4bit_and_nf4(kind, M, K, N, block, with_zp, x_dtype):
    """More than 16 rows of x on packed Int4 / Uint4 weights and NF4 indices (packed or one per byte): the weights are
    expanded to bf16 planes and multiplied on the tensor cores; above 2^26 multiply-adds that is what a plan picks by
    itself."""
    rng = np.random.default_rng(M + N)
    nf4, signed = kind.startswith("nf4"), kind.endswith("i4")
    x = rng.standard_normal((M, K)).astype(np.float32)
    vals = rng.integers(0, 16, size=(K, N))
    nblk = -(-N // block)
    s = rng.uniform(0.01, 0.2, size=(K, nblk)).astype(np.float32)
    zp = rng.uniform(-0.05, 0.05, size=s.shape).astype(np.float32) if with_zp and not nf4 else None
    b = rng.standard_normal(N).astype(np.float32)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    xw = orc.bf16_to_f32(xin) if x_dtype == "bf16" else x
    if nf4:
        want = orc.qdense_nf4(xw, vals.astype(np.uint8), s, b, block, orc.ACT_GELU)
    else:
        w8 = np.where(vals >= 8, vals - 16, vals).astype(np.int8) if signed else vals.astype(np.uint8)
        want = orc.qdense_linear(xw, w8, s, zp, b, block, orc.ACT_GELU, threads=orc.max_threads())
    big = M * K * N >= 2 ** 26
    if kind == "nf4_u8":
        got, plan = ops.quantized_dense(xin, vals.astype(np.uint8), s, None, b, x_dtype=code, block_size=block, activation=dv.ACT_GELU,
                                        scheme=dv.QUANT_NF4, variant=dv.QDENSE_AUTO if big else dv.QDENSE_PREFILL, return_plan=True)
    else:
        got, plan = ops.quantized_dense(xin, orc.pack_nibbles(vals), s, zp, b, x_dtype=code, block_size=block, activation=dv.ACT_GELU,
                                        scheme=dv.QUANT_NF4 if nf4 else dv.QUANT_LINEAR, packed=(dv.I4 if signed else dv.U4, N),
                                        variant=dv.QDENSE_AUTO if big else dv.QDENSE_PREFILL, return_plan=True)
    wname = "u8" if kind == "nf4_u8" else ("i4" if signed else "u4")
    assert plan.kernel_name == f"qdense_prefill_tcgen05_{x_dtype}_{wname}{'_nf4' if nf4 else ''}"
    gotf = orc.bf16_to_f32(got) if x_dtype == "bf16" else got
    assert max_abs_normalised(gotf, want) < (BF16_TOL if x_dtype == "bf16" else 2e-5)


@pytest.mark.parametrize("N", [264, 272])
def test_prefill_uint8_all_activations(N):
    x, w, s, b = qdense_inputs(77, 40, 256, N, scale_layout="channel", unsigned=True)
    for act in ACT.values():
        got = ops.quantized_dense(x, w, s, None, b, scale_layout=dv.SCALE_CHANNEL, activation=act, variant=dv.QDENSE_PREFILL)
        want = oracle_compact(x, w, s, b, "channel", 0, act)
        assert max_abs_normalised(got, want) < F32_TOL


@pytest.mark.parametrize("layout,group", [("channel", 0), ("kgroup", 128)])
def test_prefill_llama_projection_full_size(layout, group):
    """Prefill batch 4 x 512 tokens through the 4096 x 14336 projection, bf16 activations; a sample of
    rows against the oracle, and the rows the decode kernel computes agree with it."""
    M, K, N = 2048, 4096, 14336
    x, w, s, _ = qdense_inputs(0x5EED0005, M, K, N, x_dtype="bf16", scale_layout=layout, group=group, bias=False)
    xb = orc.bf16_from_f32(x)
    sl = dv.SCALE_CHANNEL if layout == "channel" else dv.SCALE_KGROUP
    got, plan = ops.quantized_dense(xb, w, s, None, None, x_dtype=dv.BF16, scale_layout=sl, block_size=group,
                                    activation=dv.ACT_SILU, return_plan=True)
    assert plan.kernel_name.startswith("qdense_prefill_tcgen05_bf16")
    rows = [0, 127, 128, 1000, 2047]
    want = oracle_compact(np.ascontiguousarray(x[rows]), w, s, None, layout, group, orc.ACT_SILU)
    assert max_abs_normalised(orc.bf16_to_f32(got[rows]), want) < BF16_TOL
    dec = ops.quantized_dense(np.ascontiguousarray(xb[rows]), w, s, None, None, x_dtype=dv.BF16, scale_layout=sl,
                              block_size=group, activation=dv.ACT_SILU)
    assert max_abs_normalised(orc.bf16_to_f32(dec), orc.bf16_to_f32(got[rows])) < 2.0 ** -7


# ------------------------------------------------------------- fused all-gather of column shards
def test_gathered_decode_two_ranks_on_one_gpu():
    """The kernel of a gathered plan stores its column slice into every rank's result buffer; a signal kernel
    then bumps every rank's arrival flag.  Here both ranks are plans on one GPU, launched one after the other
    (nothing waits on anything that has not finished): both result buffers must hold the full projection, and
    the flags count the signals."""
    M, K, N, g = 7, 512, 768, 2
    n_loc = N // g
    x, w, s, b = qdense_inputs(321, M, K, N, x_dtype="bf16", scale_layout="kgroup", group=128)
    xb = orc.bf16_from_f32(x)
    st = dv.Stream(0)
    xd = dv.DeviceMem.from_numpy(xb)
    bufs = [dv.DeviceMem(M * N * 2) for _ in range(g)]
    flags = [dv.DeviceMem(256) for _ in range(g)]
    for m in bufs + flags:
        m.zero()
    for r in range(g):
        cols = slice(r * n_loc, (r + 1) * n_loc)
        plan = dv.Plan.qdense(M, K, n_loc, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128, False, True, dv.ACT_SILU,
                              gather_ranks=g, gather_rank=r)
        assert plan.kernel_name.startswith("qdense_decode_tc_bf16")
        ws = plan.new_workspace()
        wd = dv.DeviceMem.from_numpy(np.ascontiguousarray(w[:, cols]))
        sd = dv.DeviceMem.from_numpy(np.ascontiguousarray(s[:, cols]))
        bd = dv.DeviceMem.from_numpy(np.ascontiguousarray(b[cols]))
        for rep in range(2):                      # two launches and signals per rank: the flags count signals
            plan.launch([xd.ptr, wd.ptr, sd.ptr, bd.ptr], [m.ptr for m in bufs], ws.ptr, st)
            dv.peer_signal(0, [f.ptr for f in flags], r, st)
        st.sync()
        plan.check_status(ws.ptr)
    for f in flags:
        dv.peer_wait(0, f.ptr, g, 2, f.ptr + 64, st)
    st.sync()
    want = oracle_compact(x, w, s, b, "kgroup", 128, orc.ACT_SILU)
    full = ops.quantized_dense(xb, w, s, None, b, x_dtype=dv.BF16, scale_layout=dv.SCALE_KGROUP, block_size=128,
                               activation=dv.ACT_SILU)
    for r in range(g):
        got = bufs[r].download((M, N), np.uint16)
        assert max_abs_normalised(orc.bf16_to_f32(got), want) < BF16_TOL
        assert np.array_equal(got, full)          # the same bits as the unsharded plan
        fl = flags[r].download((64,), np.uint32)
        assert list(fl[:g]) == [2, 2] and fl[16] == 0
    # a wait for arrivals that never come gives up and reports which flag it was waiting for
    dv.peer_wait(0, flags[0].ptr, g, 3, flags[0].ptr + 64, st)
    st.sync()
    assert flags[0].download((64,), np.uint32)[16] in (1, 2)
    with pytest.raises(ErrNotImplemented):        # only the tensor-core decode kernel has the fused gather
        dv.Plan.qdense(64, K, n_loc, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128, gather_ranks=2, gather_rank=0)


# ------------------------------------------------------------- dequantisation, bit for bit
@pytest.mark.parametrize("variant,rows", [(dv.QDENSE_GENERIC, 16), (dv.QDENSE_DECODE_MMA, 16), (dv.QDENSE_DECODE_TC, 16),
                                          (dv.QDENSE_PREFILL, 64)])
@pytest.mark.parametrize("unsigned", [False, True])
def test_dequantised_weights_are_bit_exact(variant, rows, unsigned):
    """One-hot activations read the dequantised weights back through each kernel: out[m, n] = 1 * W[m, n] * s[n]
    must equal float32(W) * s bit for bit (the integer -> float conversion and the scale product are exact
    operations in every kernel's arithmetic)."""
    K, N = 256, 384
    _, w, s, _ = qdense_inputs(5, rows, K, N, scale_layout="channel", bias=False, unsigned=unsigned)
    x = np.zeros((rows, K), np.float32)
    pick = np.random.default_rng(6).choice(K, size=rows, replace=False)
    x[np.arange(rows), pick] = 1.0
    got = ops.quantized_dense(x, w, s, None, None, scale_layout=dv.SCALE_CHANNEL, variant=variant)
    want = w[pick].astype(np.float32) * s[None, :]
    assert np.array_equal(got, want)


# ------------------------------------------------------------- validation / errors
def test_validation_errors():
    x, w, s, b = qdense_inputs(1, 2, 32, 32, scale_layout="ref", block_size=1)
    with pytest.raises(BackendError):      # weights must be [K, N]
        ops.quantized_dense(x[:, :16], w, s, None, b, block_size=1)
    with pytest.raises(BackendError):      # scales must be [K, numBlocks]
        ops.quantized_dense(x, w, s[:, :7], None, b, block_size=1)
    with pytest.raises(BackendError):      # x dtype
        dv.Plan.qdense(2, 32, 32, dv.F16)
    with pytest.raises(ErrNotImplemented):  # int4 weights: other schemes of the op are not built
        dv.Plan.qdense(2, 32, 32, dv.F32, dv.I16)
    with pytest.raises(ErrNotImplemented):  # decode kernel refuses what it cannot do
        dv.Plan.qdense(64, 32, 32, dv.F32, dv.I8, dv.SCALE_CHANNEL, variant=dv.QDENSE_DECODE_MMA)


def test_empty_inputs():
    w = np.zeros((8, 16), np.int8)
    s = np.ones((8, 16), np.float32)
    got = ops.quantized_dense(np.zeros((0, 8), np.float32), w, s, block_size=1)
    assert got.shape == (0, 16)
