"""GPU parity of FusedSoftmax, FusedGelu and FusedLayerNorm against the CPU oracle and the reference's own
assertions (support/backendtest/fusedops.go:22-177), through the C ABI and through the Backend interface."""
import numpy as np
import pytest

from compute_b200 import BackendError, ErrNotImplemented, backend as be, device as dv, ops
from oracle import oracle as orc
from tests.helpers import DT, as_f64, max_abs_normalised
from tests.test_oracle import check_fused_small, check_qkv_projection

pytestmark = pytest.mark.gpu
TOL = {"f32": 2e-5, "f64": 1e-12, "bf16": 2e-2, "f16": 2e-2}     # f32: sums of 10^4 terms in another order


@pytest.fixture(scope="module")
def backend():
    b = be.New("")
    yield b
    b.Finalize()


def make(seed, shape, dtype, sigma=1.0):
    a = (np.random.default_rng(seed).standard_normal(shape) * sigma).astype(np.float32)
    code = DT[dtype]
    if code in (orc.BF16, orc.F16):
        return orc.from_f32(a, code)
    return a.astype(np.float64 if code == orc.F64 else np.float32)


def widen(a, dtype):
    code = DT[dtype]
    return orc.to_f32(a, code).astype(np.float64) if code in (orc.BF16, orc.F16) else a


def test_reference_assertions_on_the_gpu():
    check_fused_small(lambda x, axis: ops.softmax(x, axis), lambda x, exact: ops.gelu(x, exact),
                      lambda x, axes, eps, g, b: ops.layer_norm_rows(x.reshape(-1, x.shape[-1]), eps, g, b).reshape(x.shape))


@pytest.mark.parametrize("dtype", ["f32", "f64", "bf16", "f16"])
@pytest.mark.parametrize("shape,axis", [((5, 37), 1), ((3, 11000), 1), ((4, 9, 33), 1), ((7, 5), 0), ((2, 3, 1), 2), ((300, 128), 1)])
def test_softmax_matches_oracle(shape, axis, dtype):
    x = make(1, shape, dtype, 3.0)
    want = orc.softmax(widen(x, dtype), axis)
    got = ops.softmax(x, axis, dtype=DT[dtype])
    assert max_abs_normalised(as_f64(got, DT[dtype]), want.astype(np.float64)) < TOL[dtype]
    assert np.allclose(as_f64(got, DT[dtype]).sum(axis=axis), 1.0, atol=5e-2 if dtype in ("bf16", "f16") else 1e-5)


@pytest.mark.parametrize("dtype", ["f32", "f64", "bf16", "f16"])
@pytest.mark.parametrize("exact", [True, False])
def test_gelu_matches_oracle(dtype, exact):
    x = make(2, (1000003,), dtype, 2.0)
    want = orc.gelu(widen(x, dtype), exact)
    got = ops.gelu(x, exact, dtype=DT[dtype])
    assert max_abs_normalised(as_f64(got, DT[dtype]), want.astype(np.float64)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["f32", "f64", "bf16"])
@pytest.mark.parametrize("rows,L", [(6, 40), (3, 4096), (2, 12001), (1000, 64)])
@pytest.mark.parametrize("affine", [False, True])
def test_layer_norm_matches_oracle(rows, L, affine, dtype):
    x = make(3, (rows, L), dtype, 2.0)
    g = make(4, (L,), dtype) if affine else None
    b = make(5, (L,), dtype) if affine else None
    want = orc.layer_norm(widen(x, dtype), [1], 1e-5, None if g is None else widen(g, dtype), None if b is None else widen(b, dtype))
    got = ops.layer_norm_rows(x, 1e-5, g, b, dtype=DT[dtype])
    assert max_abs_normalised(as_f64(got, DT[dtype]), want.astype(np.float64)) < (1e-5 if dtype == "f32" else TOL[dtype])


def test_through_the_backend_interface(backend):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((3, 4, 5)).astype(np.float32)
    g = rng.standard_normal((3, 5)).astype(np.float32)
    b = rng.standard_normal((3, 5)).astype(np.float32)
    (sm,), (shape,) = be.exec_graph(backend, [(x, dv.F32)], lambda f, p: f.FusedSoftmax(p[0], 1))
    assert shape == be.make_shape(dv.F32, 3, 4, 5) and max_abs_normalised(sm, orc.softmax(x, 1)) < 1e-6
    (ge,), _ = be.exec_graph(backend, [(x, dv.F32)], lambda f, p: f.FusedGelu(p[0], False))
    assert max_abs_normalised(ge, orc.gelu(x, False)) < 1e-6
    # axes that are neither trailing nor in order, one of them negative
    (ln,), (shape,) = be.exec_graph(backend, [(x, dv.F32), (g, dv.F32), (b, dv.F32)],
                                    lambda f, p: f.FusedLayerNorm(p[0], [0, -1], 1e-5, p[1], p[2]))
    assert shape == be.make_shape(dv.F32, 3, 4, 5)
    assert max_abs_normalised(ln, orc.layer_norm(x, [0, -1], 1e-5, g, b)) < 1e-5
    (ln2,), _ = be.exec_graph(backend, [(x, dv.F32)], lambda f, p: f.FusedLayerNorm(p[0], [2], 1e-5))
    assert max_abs_normalised(ln2, orc.layer_norm(x, [2], 1e-5)) < 1e-5
    f = backend.Builder("small").Main()
    xp = f.Parameter("x", be.make_shape(dv.F32, 2, 3))
    xi = f.Parameter("xi", be.make_shape(dv.I32, 2, 3))
    with pytest.raises(BackendError) as e:          # fusedops.go:57-65: negative axes are rejected
        f.FusedSoftmax(xp, -1)
    assert not isinstance(e.value, ErrNotImplemented)
    with pytest.raises(BackendError):               # layernorm.go:59-61
        f.FusedLayerNorm(xp, [2], 1e-5)
    for build in (lambda: f.FusedSoftmax(xi, 1), lambda: f.FusedGelu(xi, True), lambda: f.FusedLayerNorm(xi, [1], 1e-5)):
        with pytest.raises(ErrNotImplemented):
            build()


@pytest.mark.parametrize("dtype", ["f32", "f64", "bf16"])
def test_attention_qkv_projection(backend, dtype):
    code = DT[dtype]
    def run(x, w, bq, bk, bv, qd, kvd, c=dv.F32):
        ins = [(x, c), (w, c)] + [(b, c) for b in (bq, bk, bv) if b is not None]
        def build(f, p):
            it = iter(p[2:])
            return list(f.FusedAttentionQKVProjection(p[0], p[1], next(it) if bq is not None else None,
                                                      next(it) if bk is not None else None, next(it) if bv is not None else None, qd, kvd))
        outs, shapes = be.exec_graph(backend, ins, build)
        return outs, shapes
    if dtype == "f32":
        check_qkv_projection(lambda *a: run(*a)[0])
    x = make(1, (2, 5, 64), dtype)
    w = make(2, (64, 48 + 2 * 16), dtype, 0.2)
    bq, bv = make(3, (48,), dtype), make(4, (16,), dtype)
    (q, k, v), shapes = run(x, w, bq, None, bv, 48, 16, code)
    assert shapes == [be.make_shape(code, 2, 5, 48), be.make_shape(code, 2, 5, 16), be.make_shape(code, 2, 5, 16)]
    wq, wk, wv = orc.qkv_projection(widen(x, dtype), widen(w, dtype), widen(bq, dtype), None, widen(bv, dtype), 48, 16,
                                    in_dtype=orc.F64 if dtype != "f32" else orc.F32)
    tol = {"f32": 1e-5, "f64": 1e-12, "bf16": 2e-2}[dtype]
    for got, want in ((q, wq), (k, wk), (v, wv)):
        assert max_abs_normalised(as_f64(got, code), want.astype(np.float64)) < tol
    f = backend.Builder("qkv").Main()
    xp = f.Parameter("x", be.make_shape(dv.F32, 2, 8))
    wp = f.Parameter("w", be.make_shape(dv.F32, 8, 7))
    with pytest.raises(BackendError):
        f.FusedAttentionQKVProjection(xp, wp, None, None, None, 4, 2)      # 4 + 2 * 2 != 7
