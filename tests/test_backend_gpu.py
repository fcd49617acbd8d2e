"""The reference's compliance cases for the accelerated path, replayed through the host-side
mirror of its Backend / Builder / Function / Executable / Buffer interface
(support/backendtest/dotgeneral.go, exec.go, fusedops.go of gomlx/compute)."""
import numpy as np
import pytest

from compute_b200 import BackendError, ErrNotImplemented, backend as be, device as dv
from oracle import oracle as orc
from tests.helpers import ACT, DT, as_f64, load_golden, max_abs_normalised, qdense_inputs, tensor
from tests.test_oracle import check_transposed_large, transposed_large_inputs

pytestmark = pytest.mark.gpu
DOT = load_golden("backendtest_dotgeneral.json")["cases"]
SDPA = load_golden("backendtest_sdpa.json")


@pytest.fixture(scope="module", params=["", "fallback_only"])
def backend(request):
    b = be.New(request.param)
    yield b
    b.Finalize()


def test_backend_identity(backend):
    assert backend.Name() == "cuda" and backend.NumDevices() >= 1
    assert "B200" in backend.Description() or "cuda:0" in backend.Description()
    caps = backend.Capabilities()
    for op in (be.OP_PARAMETER, be.OP_CONSTANT, be.OP_DOT_GENERAL, be.OP_FUSED_QUANTIZED_DENSE, be.OP_FUSED_SDPA,
               be.OP_FUSED_DENSE, be.OP_FUSED_SOFTMAX, be.OP_FUSED_GELU, be.OP_FUSED_LAYER_NORM,
               be.OP_FUSED_ATTENTION_QKV_PROJECTION, be.OP_ALL_REDUCE, be.OP_ALL_GATHER, be.OP_QUANTIZED_EMBEDDING_LOOKUP):
        assert caps.Operations.get(op)
    assert len(caps.Operations) == 13        # element-wise and data-movement helpers exist but are not advertised
    assert caps.DTypes.get(dv.BF16) and caps.DTypes.get(dv.F64) and not caps.Functions
    assert not backend.HasSharedBuffers()


# ---------------------------------------------------------------- DotGeneral (dotgeneral.go)
@pytest.mark.parametrize("case", DOT, ids=[c["name"] for c in DOT])
def test_dot_general_known_answers(backend, case):
    code = DT[case["dtype"]]
    cfg = be.DotGeneralConfig(DT[case["acc"]] if "acc" in case else 0, DT[case["out"]] if "out" in case else 0)
    ins = [(tensor(case["lhs"], case["dtype"]), code), (tensor(case["rhs"], case["dtype"]), code)]
    (got,), (shape,) = be.exec_graph(backend, ins, lambda f, p: f.DotGeneral(
        p[0], case["lhs_contract"], case["lhs_batch"], p[1], case["rhs_contract"], case["rhs_batch"], cfg))
    assert list(shape.dimensions) == case["want"]["shape"]
    assert shape.dtype == (cfg.OutputDType or code)
    g = as_f64(got, shape.dtype).ravel()
    w = np.array(case["want"]["data"], np.float64)
    if case["cmp"] == "equal":
        assert np.array_equal(g, w)
    else:
        assert np.max(np.abs(g - w)) <= case["tol"]


def test_dot_general_shape_inference(backend):
    # dotgeneral.go:25-58: Function.Shape before compiling
    f = backend.Builder("DotGeneral Test").Main()
    lhs = f.Parameter("lhs", be.make_shape(dv.F32, 2, 3, 4, 5))
    rhs = f.Parameter("rhs", be.make_shape(dv.F32, 5, 1, 2, 3))
    out = f.DotGeneral(lhs, [1], [3, 0], rhs, [3], [0, 2])
    assert f.Shape(out) == be.make_shape(dv.F32, 5, 2, 4, 1)


def test_dot_general_f64_very_large_with_constants_and_slice(backend):
    # dotgeneral.go:132-159
    def build(f, _):
        lhs = f.Constant((np.arange(16 * 13 * 384, dtype=np.float64) + 1.0) * 1e-5, 16, 13, 384)
        rhs = f.Constant(np.ones(384 * 1536, np.float64), 384, 1536)
        out = f.DotGeneral(lhs, [2], None, rhs, [0], None)
        return f.Slice(out, [0, 0, 0], [1, 1, 1], [1, 1, 1])
    (got,), (shape,) = be.exec_graph(backend, [], build)
    assert shape == be.make_shape(dv.F64, 1, 1, 1)
    assert abs(got[0, 0, 0] - 0.7392) < 1e-4


def test_dot_general_dtype_sweep(backend):
    # dotgeneral.go:444-497: iota(16) . iota(16); unsupported combinations must say so
    floats = [dv.F16, dv.F32, dv.F64, dv.BF16]
    for in_dt in floats:
        for acc in floats + [0]:
            for out in floats + [0]:
                def build(f, _):
                    a = f.Iota(be.make_shape(in_dt, 16), 0)
                    b = f.Iota(be.make_shape(in_dt, 16), 0)
                    return f.DotGeneral(a, [0], None, b, [0], None, be.DotGeneralConfig(acc, out))
                try:
                    (got,), (shape,) = be.exec_graph(backend, [], build)
                except ErrNotImplemented:
                    continue
                assert shape.dtype == (out or in_dt)
                assert float(as_f64(got, shape.dtype).ravel()[0]) == 1240.0


def test_dot_general_transposed_large(backend):
    # dotgeneral.go:499-599
    lhs, rhs, want = transposed_large_inputs()
    def build(f, p):
        l = f.Reshape(p[0], 4, 32, 8, 2, 256)
        r = f.Reshape(p[1], 4, 32, 8, 256)
        return f.Reshape(f.DotGeneral(l, [4], [0, 2], r, [3], [0, 2]), 65536)
    (got,), _ = be.exec_graph(backend, [(lhs.ravel(), dv.F32), (rhs.ravel(), dv.F32)], build)
    check_transposed_large(got.reshape(want.shape), want)


def test_dot_general_validation(backend):
    f = backend.Builder("bad").Main()
    a = f.Parameter("a", be.make_shape(dv.F32, 2, 3))
    b = f.Parameter("b", be.make_shape(dv.F32, 4, 5))
    c = f.Parameter("c", be.make_shape(dv.F64, 3, 5))
    with pytest.raises(BackendError):   # contracting dimensions do not match
        f.DotGeneral(a, [1], [], b, [0], [])
    with pytest.raises(BackendError):   # same dtype required
        f.DotGeneral(a, [1], [], c, [0], [])
    with pytest.raises(BackendError):   # axis out of bounds
        f.DotGeneral(a, [2], [], b, [0], [])
    with pytest.raises(BackendError):   # axis used twice
        f.DotGeneral(a, [1], [1], b, [0], [0])
    with pytest.raises(ErrNotImplemented):
        f.Abs(a)
    with pytest.raises(ErrNotImplemented):
        f.While(a)
    with pytest.raises(BackendError):   # ReduceOpUndefined
        f.AllReduce([a], 0, [[0]])


# ---------------------------------------------------------------- Exec protocol (exec.go)
def test_exec_protocol(backend):
    builder = backend.Builder("passthrough")
    f = builder.Main()
    x = f.Parameter("x", be.make_shape(dv.F32, 2, 2))
    y = f.Parameter("y", be.make_shape(dv.I32, 3))
    f.Return([x, y, f.Reshape(x, 4)])
    exe = builder.Compile()
    names, shapes = exe.Inputs()
    assert names == ["x", "y"] and shapes[0] == be.make_shape(dv.F32, 2, 2)
    assert exe.Outputs()[2] == be.make_shape(dv.F32, 4)
    bx = backend.BufferFromFlatData(0, np.float32([[1, 2], [3, 4]]), be.make_shape(dv.F32, 2, 2))
    by = backend.BufferFromFlatData(0, np.int32([7, 8, 9]), be.make_shape(dv.I32, 3))
    outs = exe.Execute([bx, by], None, 0)
    assert np.array_equal(outs[0].ToNumpy(), [[1, 2], [3, 4]]) and np.array_equal(outs[1].ToNumpy(), [7, 8, 9])
    assert np.array_equal(outs[2].ToNumpy(), [1, 2, 3, 4])
    assert outs[0].DevicePtr() != bx.DevicePtr()          # outputs are new buffers
    # exec.go:72-111: wrong number of inputs, wrong shape, wrong dtype
    with pytest.raises(BackendError):
        exe.Execute([bx], None, 0)
    wrong_shape = backend.BufferFromFlatData(0, np.zeros(3, np.float32), be.make_shape(dv.F32, 3))
    with pytest.raises(BackendError):
        exe.Execute([wrong_shape, by], None, 0)
    wrong_dtype = backend.BufferFromFlatData(0, np.zeros((2, 2), np.int32), be.make_shape(dv.I32, 2, 2))
    with pytest.raises(BackendError):
        exe.Execute([wrong_dtype, by], None, 0)
    # donation: the donated buffer becomes invalid and a later Finalize must not fail (exec.go:143-147)
    outs2 = exe.Execute([bx, by], [True, False], 0)
    assert np.array_equal(outs2[0].ToNumpy(), [[1, 2], [3, 4]])
    with pytest.raises(BackendError):
        bx.ToNumpy()
    bx.Finalize()
    # exact-size ToFlatData
    with pytest.raises(BackendError):
        outs[1].ToFlatData(np.zeros(2, np.int32))
    for b in outs + outs2 + [by, wrong_shape, wrong_dtype]:
        b.Finalize()
    exe.Finalize()
    with pytest.raises(BackendError):   # a compiled builder cannot be reused
        builder.Compile()


# ---------------------------------------------------------------- FusedDense (fusedops.go:178-212)
@pytest.mark.parametrize("case", load_golden("backendtest_dense_epilogue.json")["cases"], ids=lambda c: c["name"])
@pytest.mark.parametrize("outputs_input", [False, True])
def test_fused_dense_known_answers_through_api(backend, case, outputs_input):
    x = tensor(case["x"], "f32")
    w = tensor(case["w"], "i8").astype(np.float32)
    bias = np.array(case["bias"], np.float32)
    wv = np.ascontiguousarray(w.T) if outputs_input else w
    cfg = be.DenseConfig(Activation=ACT[case["activation"]],
                         WeightLayout=be.DENSE_LAYOUT_OUTPUTS_INPUT if outputs_input else be.DENSE_LAYOUT_INPUT_OUTPUTS)
    (got,), _ = be.exec_graph(backend, [(x, dv.F32), (wv, dv.F32), (bias, dv.F32)], lambda f, p: f.FusedDense(p[0], p[1], p[2], cfg))
    assert np.array_equal(got.ravel(), np.array(case["want"]["data"], np.float32))


def test_fused_dense_shapes_and_validation(backend):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 16)).astype(np.float32)
    w = rng.standard_normal((16, 4, 5)).astype(np.float32)           # out features of rank 2
    b = rng.standard_normal((4, 5)).astype(np.float32)
    cfg = be.DenseConfig(Activation=dv.ACT_TANH)
    (got,), (shape,) = be.exec_graph(backend, [(x, dv.F32), (w, dv.F32), (b, dv.F32)], lambda f, p: f.FusedDense(p[0], p[1], p[2], cfg))
    assert shape == be.make_shape(dv.F32, 2, 3, 4, 5)
    want = orc.fused_dense(x.reshape(6, 16), w.reshape(16, 20), b.reshape(20), orc.ACT_TANH).reshape(2, 3, 4, 5)
    assert max_abs_normalised(got, want) < 1e-6
    (plain,), _ = be.exec_graph(backend, [(x, dv.F32), (w, dv.F32)], lambda f, p: f.FusedDense(p[0], p[1], None))
    assert max_abs_normalised(plain.reshape(6, 20), orc.fused_dense(x.reshape(6, 16), w.reshape(16, 20))) < 1e-6
    f = backend.Builder("fd").Main()
    xp = f.Parameter("x", be.make_shape(dv.F32, 2, 16))
    wp = f.Parameter("w", be.make_shape(dv.F32, 8, 4))
    with pytest.raises(BackendError) as e:        # dense.go:62-65
        f.FusedDense(xp, wp, None)
    assert "must match weight's first dim" in str(e.value)
    with pytest.raises(BackendError):             # dense.go:81-82
        f.FusedDense(xp, wp, None, be.DenseConfig(WeightLayout=7))
    xi = f.Parameter("xi", be.make_shape(dv.I32, 2, 8))
    wi = f.Parameter("wi", be.make_shape(dv.I32, 8, 4))
    with pytest.raises(ErrNotImplemented):        # dense.go:160-162
        f.FusedDense(xi, wi, None)


# ---------------------------------------------------------------- FusedQuantizedDense
@pytest.mark.parametrize("layout", ["ref", "channel", "kgroup"])
def test_fused_quantized_dense_through_api(backend, layout):
    M, K, N, G = 4, 256, 320, 64
    block = {"ref": 16, "channel": K, "kgroup": G}[layout]
    x, w, s, b = qdense_inputs(5, M, K, N, scale_layout=layout if layout != "channel" else "channel", group=G, block_size=block)
    s_api = s.reshape(1, N) if layout == "channel" else s
    def build(f, p):
        q = be.Quantization(be.QUANT_LINEAR, p[2], None, 1 if layout == "ref" else 0, block)
        return f.FusedQuantizedDense(p[0], p[1], p[3], q, dv.ACT_SILU)
    (got,), (shape,) = be.exec_graph(backend, [(x.reshape(2, 2, K), dv.F32), (w, dv.I8), (s_api, dv.F32), (b, dv.F32)], build)
    assert shape == be.make_shape(dv.F32, 2, 2, N)
    se = s if layout == "ref" else orc.expand_scales(s, layout, K, N, G)
    want = orc.qdense_linear(x, w, se, None, b, block if layout == "ref" else 1, orc.ACT_SILU)
    assert max_abs_normalised(got.reshape(M, N), want) < 1e-4


def test_fused_quantized_dense_validation(backend):
    f = backend.Builder("qd").Main()
    x = f.Parameter("x", be.make_shape(dv.F32, 2, 32))
    x16 = f.Parameter("x16", be.make_shape(dv.F16, 2, 32))
    w = f.Parameter("w", be.make_shape(dv.I8, 32, 48))
    w_bad = f.Parameter("wb", be.make_shape(dv.I8, 16, 48))
    s = f.Parameter("s", be.make_shape(dv.F32, 32, 3))
    q = lambda **kw: be.Quantization(**{**dict(Scheme=be.QUANT_LINEAR, Scale=s, BlockAxis=1, BlockSize=16), **kw})
    assert f.Shape(f.FusedQuantizedDense(x, w, None, q())) == be.make_shape(dv.F32, 2, 48)
    with pytest.raises(BackendError) as e:     # quantizeddense.go:93: x must be float32
        f.FusedQuantizedDense(x16, w, None, q())
    assert not isinstance(e.value, ErrNotImplemented)
    with pytest.raises(BackendError):          # :104 weights must be [K, N]
        f.FusedQuantizedDense(x, w_bad, None, q())
    with pytest.raises(BackendError):          # :111 scales must be [K, numBlocks]
        f.FusedQuantizedDense(x, w, None, q(BlockSize=8))
    with pytest.raises(BackendError):          # :123 only Axis=1 (and this backend's Axis=0)
        f.FusedQuantizedDense(x, w, None, q(BlockAxis=2))
    with pytest.raises(BackendError):          # GGML: weights must be [N, bytesPerRow] Uint8 (quantizeddense.go:205-208)
        f.FusedQuantizedDense(x, w, None, q(Scheme=be.QUANT_GGML))
    with pytest.raises(BackendError) as e:     # :126 NF4 takes no zero points
        f.FusedQuantizedDense(x, w, None, q(Scheme=be.QUANT_NF4, ZeroPoint=s))
    assert "ZeroPoint must be nil for NF4" in str(e.value)


def test_fused_quantized_dense_ggml_through_api(backend):
    M, K, N = 3, 128, 24
    rng = np.random.default_rng(13)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    for gt in (orc.GGML_Q8_0, orc.GGML_Q4_0):
        wq = orc.ggml_quantize_rows(rng.standard_normal((N, K)).astype(np.float32), gt)
        def build(f, p):
            return f.FusedQuantizedDense(p[0], p[1], p[2], be.Quantization(be.QUANT_GGML, None, None, 0, 0, GGMLType=gt), dv.ACT_NONE)
        (got,), (shape,) = be.exec_graph(backend, [(x, dv.F32), (wq, dv.U8), (b, dv.F32)], build)
        assert shape == be.make_shape(dv.F32, M, N)
        assert max_abs_normalised(got, orc.qdense_ggml(x, wq, b, gt)) < 1e-5
    f = backend.Builder("ggml").Main()
    xp = f.Parameter("x", be.make_shape(dv.F32, 2, 64))
    wp = f.Parameter("w", be.make_shape(dv.U8, 8, 68))
    with pytest.raises(BackendError) as e:     # quantizeddense.go:222-225: K derived from the row bytes is 64 for Q8_0, 96+ for Q4_0
        f.FusedQuantizedDense(xp, wp, None, be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q4_0))
    assert not isinstance(e.value, ErrNotImplemented)
    f.FusedQuantizedDense(xp, wp, None, be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q8_0))
    with pytest.raises(ErrNotImplemented):      # Q2_K: not supported in the fused path, as in the reference (quantizeddense.go:145-152)
        f.FusedQuantizedDense(xp, wp, None, be.Quantization(be.QUANT_GGML, GGMLType=3))


def test_quantized_embedding_lookup_through_api(backend):
    """A token-embedding table in Q4_K blocks feeding a Q6_K projection: lookup -> FusedQuantizedDense in one Executable."""
    vocab, K, N = 64, 512, 24
    rng = np.random.default_rng(17)
    table = orc.ggml_random_rows(rng, vocab, K, orc.GGML_Q4_K)
    wq = orc.ggml_random_rows(rng, N, K, orc.GGML_Q6_K)
    idx = rng.integers(0, vocab, size=(2, 3, 1)).astype(np.int32)
    def build(f, p):
        emb = f.QuantizedEmbeddingLookup(p[0], p[1], be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q4_K))
        return [emb, f.FusedQuantizedDense(emb, p[2], None, be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q6_K))]
    (emb, y), (s_emb, s_y) = be.exec_graph(backend, [(table, dv.U8), (idx, dv.I32), (wq, dv.U8)], build)
    assert s_emb == be.make_shape(dv.F32, 2, 3, K) and s_y == be.make_shape(dv.F32, 2, 3, N)
    want = orc.embedding_lookup(table, idx, orc.GGML_Q4_K)
    assert np.array_equal(emb.view(np.uint32), want.view(np.uint32))
    assert max_abs_normalised(y, orc.qdense_ggml(want, wq, None, orc.GGML_Q6_K)) < 1e-4
    # an index outside the table is an error of Execute (quantizeddense.go:487-489)
    bad = idx.copy()
    bad[1, 1, 0] = vocab + 3
    with pytest.raises(BackendError) as e:
        be.exec_graph(backend, [(table, dv.U8), (bad, dv.I32), (wq, dv.U8)], build)
    assert "out of range [0, 64)" in str(e.value)
    # builder validation (quantizeddense.go:262-302)
    f = backend.Builder("lookup").Main()
    tp = f.Parameter("t", be.make_shape(dv.U8, vocab, 144 * 2))
    ip = f.Parameter("i", be.make_shape(dv.I32, 4, 1))
    with pytest.raises(ErrNotImplemented):
        f.QuantizedEmbeddingLookup(tp, ip, be.Quantization(be.QUANT_LINEAR))
    with pytest.raises(BackendError) as e:
        f.QuantizedEmbeddingLookup(tp, f.Parameter("i2", be.make_shape(dv.I32, 4)), be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q4_K))
    assert "indices last dim must be 1" in str(e.value)
    with pytest.raises(BackendError) as e:
        f.QuantizedEmbeddingLookup(tp, f.Parameter("i3", be.make_shape(dv.F32, 4, 1)), be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q4_K))
    assert "indices must be integer" in str(e.value)
    with pytest.raises(BackendError):           # 288 bytes are not whole Q6_K blocks
        f.QuantizedEmbeddingLookup(tp, ip, be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q6_K))


def test_fused_quantized_dense_nf4_through_api(backend):
    M, K, N, block = 3, 64, 48, 16
    rng = np.random.default_rng(12)
    x = rng.standard_normal((M, K)).astype(np.float32)
    idx = rng.integers(0, 16, size=(K, N)).astype(np.uint8)
    s = rng.uniform(0.01, 0.2, size=(K, N // block)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    def build(f, p):
        return f.FusedQuantizedDense(p[0], p[1], p[3], be.Quantization(be.QUANT_NF4, p[2], None, 1, block), dv.ACT_NONE)
    (got,), (shape,) = be.exec_graph(backend, [(x, dv.F32), (idx, dv.U8), (s, dv.F32), (b, dv.F32)], build)
    assert shape == be.make_shape(dv.F32, M, N)
    assert np.array_equal(got, orc.qdense_nf4(x, idx, s, b, block, orc.ACT_NONE))


# ---------------------------------------------------------------- SDPA (fusedops.go, sdpa_direct_test.go)
@pytest.mark.parametrize("case", SDPA["cases"], ids=[c["name"] for c in SDPA["cases"]])
def test_sdpa_known_answers_through_api(backend, case):
    code = DT[case["dtype"]]
    ins = [(tensor(case[k], case["dtype"]), code) for k in ("q", "k", "v")]
    names = []
    if "mask" in case:
        ins.append((tensor(case["mask"], "bool"), dv.BOOL)); names.append("mask")
    if "q_len" in case:
        ins.append((np.array(case["q_len"], np.int32), dv.I32)); names.append("q_len")
        ins.append((np.array(case["kv_len"], np.int32), dv.I32)); names.append("kv_len")
    if "bias" in case:
        ins.append((tensor(case["bias"], case["dtype"]), code)); names.append("bias")
    def build(f, p):
        extra = dict(zip(names, p[3:]))
        cfg = be.ScaledDotProductAttentionConfig(
            QuantizedMatmuls=case.get("quantized_matmuls", False), QuerySeqLen=extra.get("q_len"),
            KeyValueSeqLen=extra.get("kv_len"), Bias=extra.get("bias"), Scale=case["scale"], Causal=case["causal"],
            Mask=extra.get("mask"))
        out, states = f.FusedScaledDotProductAttention(p[0], p[1], p[2], {"BHSD": 0, "BSHD": 1}[case["layout"]], cfg)
        assert states == []
        return out
    (got,), _ = be.exec_graph(backend, ins, build)
    want = np.array(case["want"]["data"], np.float64).reshape(case["want"]["shape"])
    assert np.max(np.abs(as_f64(got, code) - want)) <= case["tol"]


@pytest.mark.parametrize("case", SDPA["error_cases"], ids=[c["name"] for c in SDPA["error_cases"]])
def test_sdpa_rejected_through_api(backend, case):
    f = backend.Builder("sdpa-bad").Main()
    q = f.Parameter("q", be.make_shape(dv.F32, 1, 1, 2, 1))
    opts = be.ScaledDotProductAttentionConfig(Scale=1.0)
    if "bias" in case:
        opts.Bias = f.Parameter("bias", be.make_shape(dv.F32, *case["bias"]["shape"]))
    if "q_len" in case:
        dt = dv.I64 if case.get("seq_len_dtype") == "i64" else dv.I32
        opts.QuerySeqLen = f.Parameter("ql", be.make_shape(dt, 1))
        opts.KeyValueSeqLen = f.Parameter("kl", be.make_shape(dt, 1))
    if case["error"] == "not_implemented":
        with pytest.raises(ErrNotImplemented):     # float8 operands cannot even be produced
            q8 = f.ConvertDType(q, dv.F8E4M3FN)
            f.FusedScaledDotProductAttention(q8, q8, q8, 0, be.ScaledDotProductAttentionConfig(Scale=1.0, Causal=True))
    else:
        with pytest.raises(BackendError) as e:
            f.FusedScaledDotProductAttention(q, q, q, 0, opts)
        assert not isinstance(e.value, ErrNotImplemented)
    with pytest.raises(BackendError):              # QuerySeqLen without KeyValueSeqLen
        f.FusedScaledDotProductAttention(q, q, q, 0, be.ScaledDotProductAttentionConfig(QuerySeqLen=q))


def test_decoder_style_graph(backend):
    """Several ops in one Executable: quantized dense -> reshape to heads -> SDPA -> DotGeneral."""
    rng = np.random.default_rng(4)
    B, S, H, D, E = 2, 8, 4, 16, 64
    x = rng.standard_normal((B * S, E), dtype=np.float32)
    w = rng.integers(-127, 128, size=(E, 3 * H * D), dtype=np.int8)
    sc = rng.uniform(0.001, 0.02, size=(1, 3 * H * D)).astype(np.float32)
    wo = rng.standard_normal((H * D, E), dtype=np.float32) * 0.1
    def build(f, p):
        qkv = f.FusedQuantizedDense(p[0], p[1], None, be.Quantization(be.QUANT_LINEAR, p[2], None, 0, E))
        qkv = f.Reshape(qkv, B, S, 3, H, D)
        parts = [f.Reshape(f.Slice(qkv, [0, 0, i, 0, 0], [B, S, i + 1, H, D]), B, S, H, D) for i in range(3)]
        att, _ = f.FusedScaledDotProductAttention(parts[0], parts[1], parts[2], be.LAYOUT_BSHD,
                                                  be.ScaledDotProductAttentionConfig(Causal=True))
        return f.DotGeneral(f.Reshape(att, B * S, H * D), [1], [], p[3], [0], [])
    (got,), _ = be.exec_graph(backend, [(x, dv.F32), (w, dv.I8), (sc, dv.F32), (wo, dv.F32)], build)
    qkv = orc.qdense_linear(x, w, orc.expand_scales(sc[0], "channel", E, 3 * H * D), None, None, 1).reshape(B, S, 3, H, D)
    att = orc.sdpa(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], layout="BSHD", causal=True)
    want = att.reshape(B * S, H * D).astype(np.float64) @ wo.astype(np.float64)
    assert max_abs_normalised(got, want) < 1e-4


def test_trace_option_reports_every_launch(capfd):
    """The "trace" option: one line per launch with its device time, on stderr and through LastTrace."""
    b = be.New("trace")
    try:
        rng = np.random.default_rng(12)
        x = rng.standard_normal((4, 256), dtype=np.float32)
        w = rng.integers(-127, 128, size=(256, 384), dtype=np.int8)
        sc = rng.uniform(0.001, 0.02, size=(1, 384)).astype(np.float32)
        builder = b.Builder("traced")
        fn = builder.Main()
        px = fn.Parameter("x", be.make_shape(dv.F32, 4, 256))
        pw = fn.Parameter("w", be.make_shape(dv.I8, 256, 384))
        ps = fn.Parameter("s", be.make_shape(dv.F32, 1, 384))
        y = fn.FusedQuantizedDense(px, pw, None, be.Quantization(be.QUANT_LINEAR, ps, None, 0, 256))
        fn.Return([fn.FusedSoftmax(y, 1)])
        exe = builder.Compile()
        bufs = [b.BufferFromFlatData(0, a, be.make_shape(d, *a.shape)) for a, d in ((x, dv.F32), (w, dv.I8), (sc, dv.F32))]
        assert exe.LastTrace() == []
        (out,) = exe.Execute(bufs, None, 0)
        rows = exe.LastTrace()
        assert [r["kernel"] for r in rows] == exe.KernelNames() and len(rows) == 2
        assert all(r["device"] == 0 and 0.0 < r["us"] < 1e5 for r in rows)
        err = capfd.readouterr().err
        assert err.count("cudabackend trace: exec=traced") == 2
        out.Finalize()
        for t in bufs:
            t.Finalize()
        exe.Finalize()
    finally:
        b.Finalize()
    with pytest.raises(BackendError):
        be.New("traces")          # unknown options are still rejected
