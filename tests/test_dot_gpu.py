"""GPU parity of the normalised DotGeneral kernels ([B,M,K] x [B,K,N] or [B,N,K]) against the
CPU oracle, through the C ABI."""
import numpy as np
import pytest

from compute_b200 import ErrNotImplemented, device as dv, ops
from oracle import oracle as orc
from tests.helpers import DT, as_f64, max_abs_normalised

pytestmark = pytest.mark.gpu
TOL = {"f32": 1e-4, "f64": 1e-12, "bf16": 2e-2, "f16": 2e-2}


def make(seed, shape, dtype, sigma=1.0):
    a = (np.random.default_rng(seed).standard_normal(shape) * sigma).astype(np.float32)
    code = DT[dtype]
    if code in (orc.BF16, orc.F16):
        return orc.from_f32(a, code)
    return a.astype(np.float64 if code == orc.F64 else np.float32)


def oracle_dot(lhs, rhs, code, transposed, out=0):
    rc = [2] if transposed else [1]
    return orc.dot_general(lhs, [2], [0], rhs, rc, [0], code, 0, out, acc_f64=True)


@pytest.mark.parametrize("variant", [dv.DOT_GENERIC, dv.DOT_AUTO])
@pytest.mark.parametrize("dtype", ["f32", "f64", "bf16", "f16"])
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("B,M,N,K", [(1, 1, 1, 1), (3, 5, 7, 9), (2, 65, 130, 33), (1, 128, 256, 192), (4, 200, 72, 264)])
def test_dot_matches_oracle(B, M, N, K, transposed, dtype, variant):
    code = DT[dtype]
    lhs = make(1, (B, M, K), dtype)
    rhs = make(2, (B, N, K) if transposed else (B, K, N), dtype)
    want = as_f64(oracle_dot(lhs, rhs, code, transposed), code)
    got = ops.dot_normalised(lhs, rhs, in_dtype=code, rhs_transposed=transposed, variant=variant)
    assert got.shape == (B, M, N)
    assert max_abs_normalised(as_f64(got, code), want) < TOL[dtype]


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("B,M,N,K", [(1, 128, 256, 192), (4, 200, 72, 264), (2, 65, 136, 40), (1, 300, 520, 1024)])
def test_dot_f32_on_tensor_cores(B, M, N, K, transposed):
    """float32 operands as bf16 planes in one f32 accumulator: two planes each and three plane products by default
    (inside the 1e-4 bar with a margin), three planes and six products as the exact variant."""
    lhs = make(11, (B, M, K), "f32")
    rhs = make(12, (B, N, K) if transposed else (B, K, N), "f32")
    want = oracle_dot(lhs, rhs, orc.F32, transposed).astype(np.float64)
    got, plan = ops.dot_normalised(lhs, rhs, in_dtype=dv.F32, rhs_transposed=transposed, variant=dv.DOT_TCGEN05,
                                   return_plan=True)
    assert plan.kernel_name.startswith("gemm_tcgen05_Float32_Float32") and not plan.kernel_name.endswith("_6pass")
    assert max_abs_normalised(got.astype(np.float64), want) < 2e-5
    got6, plan6 = ops.dot_normalised(lhs, rhs, in_dtype=dv.F32, rhs_transposed=transposed, variant=dv.DOT_TCGEN05_EXACT,
                                     return_plan=True)
    assert plan6.kernel_name.endswith("_6pass")
    assert max_abs_normalised(got6.astype(np.float64), want) < 2e-6
    # non-finite inputs propagate as in IEEE arithmetic
    lhs[0, 3, 5] = np.inf
    got = ops.dot_normalised(lhs, rhs, in_dtype=dv.F32, rhs_transposed=transposed, variant=dv.DOT_TCGEN05)
    assert not np.isfinite(got[0, 3]).all() and np.isfinite(got[0, 4]).all()


def test_dot_output_dtypes_and_ints():
    lhs = make(1, (1, 4, 6), "bf16")
    rhs = make(2, (1, 6, 5), "bf16")
    got = ops.dot_normalised(lhs, rhs, in_dtype=dv.BF16, out_dtype=dv.F32)
    want = oracle_dot(lhs, rhs, orc.BF16, False, orc.F32)
    assert got.dtype == np.float32 and max_abs_normalised(got, want) < 1e-6
    a = np.arange(24, dtype=np.int32).reshape(1, 4, 6)
    b = np.arange(30, dtype=np.int32).reshape(1, 6, 5) - 7
    assert np.array_equal(ops.dot_normalised(a, b, in_dtype=dv.I32)[0], a[0] @ b[0])
    a64, b64 = a.astype(np.int64), b.astype(np.int64)
    assert np.array_equal(ops.dot_normalised(a64, b64, in_dtype=dv.I64)[0], a64[0] @ b64[0])
    with pytest.raises(ErrNotImplemented):
        dv.Plan.dot(1, 2, 2, 2, dv.I32, dv.F32)


def check_rows(got, lhs, rhs, code, rows, tol):
    """Oracle (f64 accumulation) on a sample of output rows of a large product."""
    sub = np.ascontiguousarray(lhs[:, rows, :])
    want = as_f64(oracle_dot(sub, rhs, code, False), code)
    assert max_abs_normalised(as_f64(got[:, rows, :], code), want) < tol


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_config2_gemm_4096(dtype):
    """A[4096,4096] x B[4096,4096], entries ~ N(0, 1/sqrt(K)); sampled rows against the oracle."""
    code = DT[dtype]
    lhs = make(0x5EED0002, (1, 4096, 4096), dtype, 1.0 / 64)
    rhs = make(0x5EED0012, (1, 4096, 4096), dtype, 1.0 / 64)
    got = ops.dot_normalised(lhs, rhs, in_dtype=code)
    check_rows(got, lhs, rhs, code, [0, 1, 127, 128, 2049, 4095], TOL[dtype])
    # linearity in the left operand: (A1 + A2) B == A1 B + A2 B, over the full output
    if dtype == "f32":
        lhs2 = make(7, (1, 4096, 4096), dtype, 1.0 / 64)
        s = ops.dot_normalised(lhs + lhs2, rhs, in_dtype=code).astype(np.float64)
        t = got.astype(np.float64) + ops.dot_normalised(lhs2, rhs, in_dtype=code)
        assert max_abs_normalised(s, t) < 1e-4


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_config2_batched(dtype):
    """[32,512,128] x [32,128,512], batch axis 0."""
    code = DT[dtype]
    lhs = make(3, (32, 512, 128), dtype, 128 ** -0.5)
    rhs = make(4, (32, 128, 512), dtype, 128 ** -0.5)
    got = ops.dot_normalised(lhs, rhs, in_dtype=code)
    want = as_f64(oracle_dot(lhs, rhs, code, False), code)
    assert max_abs_normalised(as_f64(got, code), want) < TOL[dtype]


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("B,M,N,K,dtype", [
    (10, 512, 1024, 192, "bf16"),     # 160 tiles on 148 persistent CTAs: a second, short round
    (10, 512, 1000, 192, "f16"),      # the same with a ragged last column tile
    (5, 512, 2048, 64, "f32"),        # float32 planes: three passes through the ring per tile
    (40, 512, 512, 64, "bf16"),       # one k-block per tile: the ring never fills
    (3, 200, 520, 128, "bf16"),       # ragged tiles, fewer tiles than CTAs
])
def test_dot_tile_schedules(B, M, N, K, dtype, transposed):
    """Shapes that stress the persistent schedule of the tensor-core kernel: more tiles than CTAs by a few, ragged
    edges, very short K, several passes per tile."""
    code = DT[dtype]
    lhs = make(21, (B, M, K), dtype, K ** -0.5)
    rhs = make(22, (B, N, K) if transposed else (B, K, N), dtype, 1.0)
    got, plan = ops.dot_normalised(lhs, rhs, in_dtype=code, rhs_transposed=transposed, variant=dv.DOT_TCGEN05, return_plan=True)
    assert plan.kernel_name.startswith("gemm_tcgen05_")
    want = as_f64(oracle_dot(lhs, rhs, code, transposed), code)
    assert max_abs_normalised(as_f64(got, code), want) < (2e-5 if dtype == "f32" else TOL[dtype])


# ---------------------------------------------------------------- FusedDense (DotGeneral + bias + activation)
@pytest.mark.parametrize("act", ["none", "relu", "gelu", "silu", "hard_swish", "tanh"])
@pytest.mark.parametrize("dtype", ["f32", "f64"])
def test_fused_dense_generic_matches_oracle(dtype, act):
    """The reference's dtypes (fusedops/dense.go:149-163) on the CUDA-core kernel, both weight layouts."""
    from tests.helpers import ACT
    M, K, N = 7, 40, 37
    code = DT[dtype]
    x = make(3, (1, M, K), dtype)
    w = make(4, (1, K, N), dtype, 0.3)
    b = make(5, (N,), dtype)
    want = orc.fused_dense(x[0], w[0], b, ACT[act], in_dtype=code)
    got, plan = ops.dot_normalised(x, w, in_dtype=code, bias=b, activation=ACT[act], variant=dv.DOT_GENERIC, return_plan=True)
    assert plan.kernel_name.endswith("_dense")
    tol = 1e-6 if dtype == "f32" else 1e-13
    assert max_abs_normalised(got[0].astype(np.float64), want.astype(np.float64)) < tol
    got_t = ops.dot_normalised(x, np.ascontiguousarray(w.transpose(0, 2, 1)), in_dtype=code, rhs_transposed=True, bias=b,
                               activation=ACT[act], variant=dv.DOT_GENERIC)
    assert np.array_equal(got_t, got)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("act", ["none", "silu", "gelu"])
def test_fused_dense_on_tensor_cores(dtype, act):
    from tests.helpers import ACT
    M, K, N = 200, 264, 136
    code = DT[dtype]
    x = make(6, (1, M, K), dtype)
    w = make(7, (1, K, N), dtype, 0.1)
    b = make(8, (N,), dtype)
    f = lambda a: orc.to_f32(a, code) if dtype != "f32" else a
    want = orc.fused_dense(f(x)[0].astype(np.float64), f(w)[0].astype(np.float64), f(b).astype(np.float64), ACT[act], in_dtype=orc.F64)
    got, plan = ops.dot_normalised(x, w, in_dtype=code, bias=b, activation=ACT[act], variant=dv.DOT_TCGEN05, return_plan=True)
    assert plan.kernel_name.startswith("gemm_tcgen05_") and plan.kernel_name.endswith("_dense")
    assert max_abs_normalised(as_f64(got[0], code), want) < (1e-4 if dtype == "f32" else 2e-2)
    # bias only, activation only
    got_b = ops.dot_normalised(x, w, in_dtype=code, bias=b, variant=dv.DOT_TCGEN05)
    want_b = orc.fused_dense(f(x)[0].astype(np.float64), f(w)[0].astype(np.float64), f(b).astype(np.float64), orc.ACT_NONE, in_dtype=orc.F64)
    assert max_abs_normalised(as_f64(got_b[0], code), want_b) < (1e-4 if dtype == "f32" else 2e-2)


def test_fused_dense_validation():
    with pytest.raises(ErrNotImplemented):
        dv.Plan.dot(1, 4, 4, 4, dv.I32, has_bias=True)
    from compute_b200 import BackendError
    with pytest.raises(BackendError):
        dv.Plan.dot(1, 4, 4, 4, dv.F32, activation=17)
