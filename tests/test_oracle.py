"""CPU tests that pin the oracle: the reference's own known-answer vectors
(tests/golden/, transcribed from the reference's asserting tests) and, for the
quantized dense op the reference never asserts, hand-computed cases plus the
reference's decomposed formulation."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import ACT, DT, as_f64, load_golden, max_abs_normalised, qdense_inputs, tensor

DOT = load_golden("backendtest_dotgeneral.json")["cases"]
SDPA = load_golden("backendtest_sdpa.json")["cases"]
DENSE = load_golden("backendtest_dense_epilogue.json")["cases"]


# ---------------------------------------------------------------- bf16 / f16
def test_bf16_known_answers():
    # dtypes/bfloat16/bfloat16_test.go:10-60
    for v in [0, 1, -1, 0.5, 1.5, 100, 1000, np.inf, -np.inf]:
        assert orc.bf16_to_f32(orc.bf16_from_f32(np.float32(v))) == np.float32(v)
    assert orc.bf16_to_f32(orc.bf16_from_f32(np.float32(65504))) == 65536
    assert np.isnan(orc.bf16_to_f32(orc.bf16_from_f32(np.float32(np.nan))))
    assert orc.bf16_from_f32(np.float32(1.0)) == 0x3F80
    # ties to even: 1 + 2^-8 is halfway between 0x3F80 and 0x3F81 -> even (0x3F80)
    assert orc.bf16_from_f32(np.float32(1.0 + 2.0 ** -8)) == 0x3F80
    assert orc.bf16_from_f32(np.float32(1.0 + 3 * 2.0 ** -8)) == 0x3F82


def test_f16_matches_ieee():
    rng = np.random.default_rng(1)
    v = np.concatenate([rng.standard_normal(2000).astype(np.float32) * 100,
                        np.float32([0, -0.0, 65504, 65520, 1e-8, 6.2e-5, np.inf, -np.inf])])
    with np.errstate(over="ignore"):
        want = v.astype(np.float16).view(np.uint16)
    assert np.array_equal(orc.f16_from_f32(v), want)
    assert np.array_equal(orc.f16_to_f32(want), want.view(np.float16).astype(np.float32))
    # The reference's FromFloat32 shifts subnormal results by (14 - exp) bits
    # (dtypes/float16/float16.go:131-143), which flushes them to zero; the
    # restatement keeps that behaviour.  Subnormal *inputs* still widen exactly.
    assert orc.f16_from_f32(np.float32([6.0e-5]))[0] == 0
    sub = np.uint16([0x0001, 0x03FF, 0x8200])
    assert np.array_equal(orc.f16_to_f32(sub), sub.view(np.float16).astype(np.float32))


# ---------------------------------------------------------------- DotGeneral
@pytest.mark.parametrize("case", DOT, ids=[c["name"] for c in DOT])
def test_dot_general_golden(case):
    code = DT[case["dtype"]]
    lhs = tensor(case["lhs"], case["dtype"])
    rhs = tensor(case["rhs"], case["dtype"])
    acc = DT[case["acc"]] if "acc" in case else 0
    out = DT[case["out"]] if "out" in case else 0
    got = orc.dot_general(lhs, case["lhs_contract"], case["lhs_batch"],
                          rhs, case["rhs_contract"], case["rhs_batch"], code, acc, out)
    assert list(got.shape) == case["want"]["shape"]
    g = as_f64(got, out or code).ravel()
    w = np.array(case["want"]["data"], np.float64)
    if case["cmp"] == "equal":
        assert np.array_equal(g, w)
    else:
        assert np.max(np.abs(g - w)) <= case["tol"]


def test_dot_general_f64_very_large():
    # support/backendtest/dotgeneral.go:132-159: out[0,0,0] = sum_{i<384} (i+1)*1e-5 = 0.7392
    lhs = (np.arange(16 * 13 * 384, dtype=np.float64) + 1.0) * 1e-5
    lhs = lhs.reshape(16, 13, 384)
    rhs = np.ones((384, 1536), np.float64)
    got = orc.dot_general(lhs, [2], [], rhs, [0], [], orc.F64)
    assert got.shape == (16, 13, 1536)
    assert abs(got[0, 0, 0] - 0.7392) < 1e-4


def transposed_large_inputs():
    """Inputs and f64 reference of support/backendtest/dotgeneral.go:499-560."""
    g_idx = np.arange(4 * 32 * 8 * 2, dtype=np.float64).reshape(4, 32, 8, 2, 1)
    lhs = np.broadcast_to((g_idx.astype(np.float32) * np.float32(0.0001)), (4, 32, 8, 2, 256))
    lhs = np.ascontiguousarray(lhs, np.float32)
    rhs = (np.arange(4 * 32 * 8 * 256).astype(np.float32) * np.float32(0.0001)).reshape(4, 32, 8, 256)
    want = np.einsum("bqhgd,bkhd->bhqgk", lhs.astype(np.float64), rhs.astype(np.float64)).astype(np.float32)
    return lhs, rhs, want


def check_transposed_large(got, want):
    diff = np.abs(want.astype(np.float64) - got.astype(np.float64))
    ok = (diff <= 0.5) | ((np.abs(want) > 0) & (diff / np.maximum(np.abs(want), 1e-30) < 0.03))
    assert ok.all()


def test_dot_general_transposed_large():
    lhs, rhs, want = transposed_large_inputs()
    got = orc.dot_general(lhs, [4], [0, 2], rhs, [3], [0, 2], orc.F32)
    assert got.shape == (4, 8, 32, 2, 32)
    check_transposed_large(got, want)


def test_dot_general_dtype_sweep():
    # dotgeneral.go:444-497: iota(16) . iota(16) = 1240 for every supported combination
    for name in ("f32", "f64", "bf16", "f16"):
        code = DT[name]
        v = orc.from_f32(np.arange(16, dtype=np.float32), code) if code in (orc.BF16, orc.F16) \
            else np.arange(16).astype({orc.F32: np.float32, orc.F64: np.float64}[code])
        for out in (0, orc.F32, orc.F64):
            got = orc.dot_general(v, [0], [], v, [0], [], code, 0, out)
            assert float(as_f64(got, out or code).ravel()[0]) == 1240.0


# ---------------------------------------------------------------- SDPA
@pytest.mark.parametrize("case", SDPA, ids=[c["name"] for c in SDPA])
def test_sdpa_golden(case):
    code = DT[case["dtype"]]
    up = lambda key: as_f64(tensor(case[key], case["dtype"]), code).astype(np.float32)
    mask = tensor(case["mask"], "bool") if "mask" in case else None
    bias = up("bias") if "bias" in case else None
    got = orc.sdpa(up("q"), up("k"), up("v"), mask=mask, bias=bias,
                   q_len=case.get("q_len"), kv_len=case.get("kv_len"),
                   layout=case["layout"], scale=case["scale"], causal=case["causal"])
    if code in (orc.BF16, orc.F16):      # half inputs: upcast, f32 arithmetic, round to the half type
        got = orc.to_f32(orc.from_f32(got, code), code)
    want = np.array(case["want"]["data"], np.float64).reshape(case["want"]["shape"])
    assert np.max(np.abs(got - want)) <= case["tol"]


def test_sdpa_gqa_matches_numpy():
    rng = np.random.default_rng(7)
    B, Hq, Hkv, S, Skv, D = 2, 4, 2, 5, 7, 8
    q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, Skv, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, Skv, D), dtype=np.float32)
    bias = rng.standard_normal((B, Hq, S, Skv), dtype=np.float32)
    got = orc.sdpa(q, k, v, bias=bias, scale=0.0, causal=False)
    kk = np.repeat(k, Hq // Hkv, axis=1).astype(np.float64)
    vv = np.repeat(v, Hq // Hkv, axis=1).astype(np.float64)
    s = np.einsum("bhsd,bhtd->bhst", q.astype(np.float64), kk) / np.sqrt(D) + bias
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bhst,bhtd->bhsd", p, vv)
    assert max_abs_normalised(got, want) < 1e-5
    # BSHD gives the same numbers in the other layout
    got2 = orc.sdpa(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3),
                    bias=bias.transpose(0, 2, 1, 3), layout="BSHD")
    assert np.array_equal(got2.transpose(0, 2, 1, 3), got)


# ---------------------------------------------------------------- quantized dense
@pytest.mark.parametrize("case", DENSE, ids=[c["name"] for c in DENSE])
def test_dense_epilogue_golden(case):
    """fusedops.go:178-212 pins bias-then-activation; with unit scales the
    quantized op must reproduce those numbers exactly."""
    x = tensor(case["x"], "f32")
    w = tensor(case["w"], "i8")
    K, N = w.shape
    got = orc.qdense_linear(x, w, np.ones((K, N), np.float32), None,
                            np.array(case["bias"], np.float32), 1, ACT[case["activation"]])
    assert np.array_equal(got.ravel(), np.array(case["want"]["data"], np.float32))


def requantise(w_ref, scale, zero_point, unsigned):
    """Integer weights q with q * scale + zero_point == w_ref exactly (power-of-two scale, dyadic zero point)."""
    q = (w_ref.astype(np.float64) - zero_point) / scale
    assert np.array_equal(q, np.rint(q))
    q = q.astype(np.int64)
    assert q.min() >= (0 if unsigned else -128) and q.max() <= (255 if unsigned else 127)
    return q.astype(np.uint8 if unsigned else np.int8)


SCALED = [(0.25, None, False), (0.5, None, False), (0.25, 0.5, False), (0.125, -16.0, True), (1.0, 3.0, False)]


@pytest.mark.parametrize("scale,zp,unsigned", SCALED)
@pytest.mark.parametrize("case", DENSE, ids=[c["name"] for c in DENSE])
def test_dense_epilogue_golden_with_scales_and_zero_points(case, scale, zp, unsigned):
    """The reference's FusedDense numbers (fusedops.go:178-212) replayed through the quantized op with weights
    stored as q = (w - zero_point) / scale: non-unit power-of-two scales and dyadic zero points dequantise to the
    reference's weights exactly (quantizeddense.go:637-647: w * s + zp), so its expected values bind the scale and
    zero-point path too."""
    x = tensor(case["x"], "f32")
    w_ref = tensor(case["w"], "i8")
    K, N = w_ref.shape
    q = requantise(w_ref, scale, zp or 0.0, unsigned)
    for block in (1, 2, N):
        nblk = (N + block - 1) // block
        got = orc.qdense_linear(x, q, np.full((K, nblk), scale, np.float32), None if zp is None else np.full((K, nblk), zp, np.float32),
                                np.array(case["bias"], np.float32), block, ACT[case["activation"]])
        assert np.array_equal(got.ravel(), np.array(case["want"]["data"], np.float32))


@pytest.mark.parametrize("case", DENSE, ids=[c["name"] for c in DENSE])
def test_fused_dense_golden(case):
    """The same reference cases (fusedops.go:178-212) through the oracle's FusedDense restatement."""
    x = tensor(case["x"], "f32")
    w = tensor(case["w"], "i8").astype(np.float32)
    got = orc.fused_dense(x, w, np.array(case["bias"], np.float32), ACT[case["activation"]])
    assert np.array_equal(got.ravel(), np.array(case["want"]["data"], np.float32))
    got_t = orc.fused_dense(x, np.ascontiguousarray(w.T), np.array(case["bias"], np.float32), ACT[case["activation"]], outputs_input=True)
    assert np.array_equal(got_t, got)


def test_qdense_hand_computed():
    # K=2, N=4, BlockSize=2, power-of-two scales: every product is exact.
    x = np.float32([[1, 2], [-3, 0.5]])
    w = np.int8([[1, -2, 3, 4], [5, 6, -7, 8]])
    s = np.float32([[0.5, 2.0], [0.25, 1.0]])          # [K, N/2]
    bias = np.float32([1, 1, -1, 0])
    want = np.float32([[1 + 0.5 + 2.5, 1 - 1 + 3, -1 + 6 - 14, 8 + 16],
                       [1 - 1.5 + 0.625, 1 + 3 + 0.75, -1 - 18 - 3.5, -24 + 4]])
    got = orc.qdense_linear(x, w, s, None, bias, 2, orc.ACT_NONE)
    assert np.array_equal(got, want)
    zp = np.float32([[1, 0], [0, -1]])
    want_zp = want + np.float32([[1, 1, -2, -2], [-3, -3, -0.5, -0.5]])
    assert np.array_equal(orc.qdense_linear(x, w, s, zp, bias, 2, orc.ACT_NONE), want_zp)
    # uint8 weights
    wu = np.uint8([[200, 0, 3, 4], [5, 255, 7, 8]])
    got_u = orc.qdense_linear(x, wu, s, None, None, 2, orc.ACT_RELU)
    want_u = np.maximum(x.astype(np.float64) @ (wu.astype(np.float64) * s[:, [0, 0, 1, 1]]), 0)
    assert np.array_equal(got_u, want_u.astype(np.float32))


@pytest.mark.parametrize("act", list(ACT))
@pytest.mark.parametrize("block", [1, 3, 16, 40])
def test_qdense_matches_decomposed(act, block):
    K, N, M = 96, 40, 5
    x, w, s, b = qdense_inputs(11 + block, M, K, N, scale_layout="ref", block_size=block)
    rng = np.random.default_rng(5)
    zp = rng.uniform(-0.05, 0.05, size=s.shape).astype(np.float32)
    for z in (None, zp):
        got = orc.qdense_linear(x, w, s, z, b, block, ACT[act])
        want = orc.qdense_decomposed(x, w, s, z, b, block, ACT[act])
        assert max_abs_normalised(got, want) < 1e-5


def test_qdense_thread_split_is_bit_identical():
    for M in (1, 3):
        x, w, s, b = qdense_inputs(3, M, 256, 300, scale_layout="ref", block_size=7)
        one = orc.qdense_linear(x, w, s, None, b, 7, orc.ACT_SILU, threads=1)
        many = orc.qdense_linear(x, w, s, None, b, 7, orc.ACT_SILU, threads=4)
        fast = orc.qdense_linear(x, w, s, None, b, 7, orc.ACT_SILU, threads=4, fast=True)
        assert np.array_equal(one, many) and np.array_equal(one, fast)


def test_nibble_unpack_known_answers():
    """The reference's own vectors (internal/gobackend/ops/convertdtype_test.go:13-80): byte 0xF0 is
    (0, -1) as Int4 and (0, 15) as Uint4; byte 0x87 is (7, -8) and (7, 8)."""
    packed = np.array([0xF0, 0x87], np.uint8)
    assert orc.unpack_int4(packed, 4).tolist() == [0, -1, 7, -8]
    assert orc.unpack_uint4(packed, 4).tolist() == [0, 15, 7, 8]
    rng = np.random.default_rng(3)
    v = rng.integers(-8, 8, size=101)
    assert np.array_equal(orc.unpack_int4(orc.pack_nibbles(v), v.size), v)
    u = rng.integers(0, 16, size=100)
    assert np.array_equal(orc.unpack_uint4(orc.pack_nibbles(u), u.size), u)


def test_nf4_table_and_dense():
    """NormalFloat4: 16 increasing values in [-1, 1] with an exact zero at index 7 (fused_ops.go:114-121);
    the dense op is sum_k (x * table[w & 15]) * scale in f32 (quantizeddense.go:586-609)."""
    t = orc.nf4_values()
    assert t.dtype == np.float32 and t[0] == -1.0 and t[7] == 0.0 and t[15] == 1.0 and np.all(np.diff(t) > 0)
    golden = load_golden("nf4_table.json")["values"]
    assert [float(v) for v in t] == golden
    x = np.array([[1.0, 2.0], [0.5, -1.0]], np.float32)
    w = np.array([[0, 15, 7], [15 | 0x30, 0, 8]], np.uint8)          # bits above the nibble are ignored
    s = np.array([[2.0], [0.5]], np.float32)
    got = orc.qdense_nf4(x, w, s, np.array([0.0, 1.0, 0.0], np.float32), 3, orc.ACT_NONE)
    t8 = float(t[8])
    want = np.array([[1 * -1 * 2 + 2 * 1 * 0.5, 1 + 1 * 1 * 2 + 2 * -1 * 0.5, 2 * t8 * 0.5],
                     [0.5 * -1 * 2 - 1 * 0.5, 1 + 0.5 * 2 + 1 * 0.5, -1 * t8 * 0.5]], np.float32)
    assert np.allclose(got, want, rtol=0, atol=1e-7)


SMALL = load_golden("backendtest_fused_small.json")["cases"]


def check_fused_small(softmax, gelu, layer_norm):
    """The reference's assertions for FusedSoftmax / FusedGelu / FusedLayerNorm (fusedops.go:22-177), against any
    implementation of the three ops on float32 arrays."""
    c = SMALL["softmax_1d"]
    assert np.allclose(softmax(np.float32(c["x"]), c["axis"]), np.float32(c["want"]), rtol=0, atol=c["tol"])
    c = SMALL["softmax_rows_sum_to_one"]
    assert np.allclose(softmax(np.float32(c["x"]), c["axis"]).sum(axis=1), 1.0, rtol=0, atol=c["tol"])
    c = SMALL["softmax_stability"]
    y = softmax(np.float32(c["x"]), c["axis"])
    assert np.isfinite(y).all() and abs(float(y.sum()) - 1.0) < c["tol"]
    c = SMALL["gelu_exact"]
    exact = gelu(np.float32(c["x"]), True)
    assert np.allclose(exact, np.float32(c["want"]), rtol=0, atol=c["tol"])
    assert np.abs(gelu(np.float32(c["x"]), False) - exact).max() > 1e-7          # the tanh form differs
    c = SMALL["layernorm_simple"]
    y = layer_norm(np.float32(c["x"]), c["axes"], c["epsilon"], None, None)
    assert np.abs(y.mean(axis=1)).max() < c["mean_tol"] and np.abs(y.var(axis=1) - 1.0).max() < c["var_tol"]
    c = SMALL["layernorm_gamma_beta"]
    y = layer_norm(np.float32(c["x"]), c["axes"], c["epsilon"], np.float32(c["gamma"]), np.float32(c["beta"]))
    assert np.allclose(y, np.float32(c["want"]), rtol=0, atol=c["tol"])


def test_fused_small_ops_golden():
    check_fused_small(orc.softmax, orc.gelu, orc.layer_norm)
    # non-trailing and negative axes: the same numbers as normalising the transposed tensor
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 4, 5)).astype(np.float32)
    g = rng.standard_normal((3, 5)).astype(np.float32)
    y = orc.layer_norm(x, [0, -1], 1e-5, g, None)
    xt = np.transpose(x, (1, 0, 2)).reshape(4, 15)
    want = ((xt - xt.mean(1, keepdims=True)) / np.sqrt(xt.var(1, keepdims=True) + 1e-5) * g.reshape(1, 15)).reshape(4, 3, 5).transpose(1, 0, 2)
    assert np.allclose(y, want, rtol=0, atol=1e-5)
    z = rng.standard_normal((2, 7, 3)).astype(np.float64)
    e = np.exp(z - z.max(1, keepdims=True))
    assert np.allclose(orc.softmax(z, 1), e / e.sum(1, keepdims=True), rtol=0, atol=1e-14)


def check_qkv_projection(fn):
    """support/backendtest/fusedops.go:497-524."""
    x = np.float32([[1, 2, 3]])
    w = np.float32([[1, 0, 0, 1], [0, 1, 0, 1], [0, 0, 1, 1]])
    q, k, v = fn(x, w, np.float32([10, 20]), np.float32([100]), np.float32([1000]), 2, 1)
    assert np.array_equal(q, np.float32([[11, 22]])) and np.array_equal(k, np.float32([[103]])) and np.array_equal(v, np.float32([[1006]]))


def test_qkv_projection_golden():
    check_qkv_projection(orc.qkv_projection)


def test_ggml_blocks_hand_computed():
    """Block layouts of quantizeddense_ggml.go:159-196 on hand-built bytes."""
    q8 = np.zeros((1, 34), np.uint8)
    q8[0, 0:2] = [0x00, 0x38]                                   # fp16 0.5, little endian
    q8[0, 2:] = np.arange(32, dtype=np.int8).view(np.uint8)
    q8[0, 2 + 5] = np.int8(-3).view(np.uint8)
    want = 0.5 * np.arange(32, dtype=np.float32)
    want[5] = -1.5
    assert np.array_equal(orc.ggml_dequant_rows(q8, orc.GGML_Q8_0)[0], want)
    q4 = np.zeros((1, 18), np.uint8)
    q4[0, 0:2] = [0x00, 0x40]                                   # fp16 2.0
    q4[0, 2:] = [i | ((15 - i) << 4) for i in range(16)]
    d = orc.ggml_dequant_rows(q4, orc.GGML_Q4_0)[0]
    assert np.array_equal(d[:16], 2.0 * (np.arange(16) - 8)) and np.array_equal(d[16:], 2.0 * (7 - np.arange(16)))
    # dense: x @ dequant(w)^T + bias, then the activation
    x = np.float32([[1.0] * 32, [0.5] * 32])
    got = orc.qdense_ggml(x, q8, np.float32([1.0]), orc.GGML_Q8_0, orc.ACT_RELU)
    assert np.array_equal(got, np.float32([[want.sum() + 1.0], [0.5 * want.sum() + 1.0]]))
    rng = np.random.default_rng(0)
    w = rng.standard_normal((4, 64)).astype(np.float32)
    for t, tol in ((orc.GGML_Q8_0, 0.02), (orc.GGML_Q4_0, 0.3)):
        assert np.abs(orc.ggml_dequant_rows(orc.ggml_quantize_rows(w, t), t) - w).max() < tol


def test_expand_scales_layouts():
    s = np.arange(6, dtype=np.float32).reshape(2, 3)
    e = orc.expand_scales(s, "kgroup", 4, 3, group=2)
    assert e.shape == (4, 3) and np.array_equal(e[0], e[1]) and np.array_equal(e[2], s[1])
    c = orc.expand_scales(np.float32([1, 2, 3]), "channel", 4, 3)
    assert c.shape == (4, 3) and np.array_equal(c[3], [1, 2, 3])


def test_blocked_gemm_baseline_is_a_gemm():
    rng = np.random.default_rng(2)
    a = rng.standard_normal((70, 300), dtype=np.float32)
    b = rng.standard_normal((300, 530), dtype=np.float32)
    got = orc.gemm_f32_blocked(a, b, threads=2)
    assert max_abs_normalised(got, a.astype(np.float64) @ b.astype(np.float64)) < 1e-5
