"""GPU tests of the graph layer around the projections: element-wise / reduce ops, the fused RMS norm the compiler
substitutes for its decomposed form, grouped FusedQuantizedDense launches, re-entrant Execute, constant scales in
the reference layout, packed 4-bit weights, and SPMD execution with AllReduce / AllGather (two or more GPUs)."""
import threading

import numpy as np
import pytest

from compute_b200 import BackendError, ErrNotImplemented, backend as be, device as dv
from oracle import oracle as orc
from tests.helpers import ACT, max_abs_normalised, qdense_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    b = be.New("")
    yield b
    b.Finalize()


def run(backend, inputs, build, device=0):
    arrays, shapes = be.exec_graph(backend, inputs, build, device)
    return arrays, shapes


# ---------------------------------------------------------------- element-wise, reduce, broadcast
def test_binary_ops_broadcast_like_the_reference(backend):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((3, 1, 5), dtype=np.float32)
    b = rng.standard_normal((3, 4, 1), dtype=np.float32) + 3.0
    sc = np.float32([2.5]).reshape(())
    for name, fn in (("Add", np.add), ("Sub", np.subtract), ("Mul", np.multiply), ("Div", np.divide), ("Max", np.maximum), ("Min", np.minimum)):
        (got,), (shape,) = run(backend, [(a, dv.F32), (b, dv.F32)], lambda f, p, name=name: getattr(f, name)(p[0], p[1]))
        assert shape.dimensions == (3, 4, 5)
        assert np.array_equal(got, fn(a, b)), name
    (got,), _ = run(backend, [(a, dv.F32), (sc, dv.F32)], lambda f, p: f.Mul(p[1], p[0]))      # a scalar takes the other shape
    assert np.array_equal(got, a * sc)
    with pytest.raises(BackendError):        # ranks must match unless one side is a scalar
        run(backend, [(a, dv.F32), (b[0], dv.F32)], lambda f, p: f.Add(p[0], p[1]))
    with pytest.raises(BackendError):        # 5 against 4 cannot be broadcast
        run(backend, [(a, dv.F32), (np.zeros((3, 4, 4), np.float32), dv.F32)], lambda f, p: f.Add(p[0], p[1]))
    i = np.arange(12, dtype=np.int32).reshape(3, 4)
    (got,), _ = run(backend, [(i, dv.I32), (i.T.copy().T, dv.I32)], lambda f, p: f.Mul(p[0], p[1]))
    assert np.array_equal(got, i * i)


def test_unary_reduce_broadcast(backend):
    rng = np.random.default_rng(1)
    x = rng.uniform(0.1, 4.0, size=(6, 7, 33)).astype(np.float32)
    for name, fn, tol in (("Neg", np.negative, 0), ("Rsqrt", lambda v: 1 / np.sqrt(v), 1e-6), ("Sqrt", np.sqrt, 1e-6), ("Exp", np.exp, 1e-6),
                          ("Logistic", lambda v: 1 / (1 + np.exp(-v)), 1e-6), ("Tanh", np.tanh, 1e-6)):
        (got,), _ = run(backend, [(x, dv.F32)], lambda f, p, name=name: getattr(f, name)(p[0]))
        assert max_abs_normalised(got, fn(x.astype(np.float64))) <= tol, name
    (got,), (shape,) = run(backend, [(x, dv.F32)], lambda f, p: f.ReduceSum(p[0], -1))
    assert shape.dimensions == (6, 7) and max_abs_normalised(got, x.astype(np.float64).sum(-1)) < 1e-6
    (got,), (shape,) = run(backend, [(x, dv.F32)], lambda f, p: f.ReduceSum(p[0], 0, 2))
    assert shape.dimensions == (7,) and max_abs_normalised(got, x.astype(np.float64).sum((0, 2))) < 1e-6
    (got,), (shape,) = run(backend, [(x, dv.F32)], lambda f, p: f.ReduceMax(p[0]))
    assert shape.dimensions == () and got == x.max()
    v = rng.standard_normal(7, dtype=np.float32)
    (got,), _ = run(backend, [(v, dv.F32)], lambda f, p: f.BroadcastInDim(p[0], be.make_shape(dv.F32, 6, 7, 2), [1]))
    assert np.array_equal(got, np.broadcast_to(v[None, :, None], (6, 7, 2)))
    xb = orc.bf16_from_f32(x)
    (got,), _ = run(backend, [(xb, dv.BF16)], lambda f, p: f.Exp(p[0]))
    assert max_abs_normalised(orc.bf16_to_f32(got), np.exp(orc.bf16_to_f32(xb).astype(np.float64))) < 2.0 ** -8


def _rms_graph(f, x, gamma, H, eps, dtype, with_gamma=True, div=False):
    """x * Reshape(Rsqrt(ReduceSum(x*x, -1) * (1/H) + eps)) * gamma, as a caller of the interface writes RMS norm."""
    one = lambda v: f.Constant(np.asarray([v], dv.NP_CARRIER[dtype] if dtype != dv.BF16 else np.float32).astype(np.float32)
                               if dtype != dv.BF16 else orc.bf16_from_f32(np.float32([v])), dtype=dtype)
    ss = f.ReduceSum(f.Mul(x, x), -1)
    ms = f.Div(ss, one(float(H))) if div else f.Mul(ss, one(1.0 / H))
    r = f.Rsqrt(f.Add(ms, one(eps)))
    dims = list(f.Shape(x).dimensions)
    xn = f.Mul(x, f.Reshape(r, *(dims[:-1] + [1])))
    if not with_gamma:
        return xn
    return f.Mul(xn, f.Reshape(gamma, *([1] * (len(dims) - 1) + [H])))


@pytest.mark.parametrize("dtype,with_gamma,div", [("f32", True, False), ("f32", False, True), ("bf16", True, False)])
def test_decomposed_rms_norm_runs_as_one_kernel(backend, dtype, with_gamma, div):
    rng = np.random.default_rng(2)
    B, S, H, eps = 3, 5, 4096, 1e-5
    x = rng.standard_normal((B, S, H), dtype=np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    code = dv.BF16 if dtype == "bf16" else dv.F32
    if dtype == "bf16":
        xin, gin = orc.bf16_from_f32(x), orc.bf16_from_f32(g)
        x, g = orc.bf16_to_f32(xin), orc.bf16_to_f32(gin)
    else:
        xin, gin = x, g
    builder = backend.Builder("rms")
    f = builder.Main()
    px = f.Parameter("x", be.make_shape(code, B, S, H))
    pg = f.Parameter("g", be.make_shape(code, H))
    f.Return([_rms_graph(f, px, pg, H, eps, code, with_gamma, div)])
    exe = builder.Compile()
    names = exe.KernelNames()
    assert len(names) == 1 and names[0].startswith("rms_norm_"), names     # the intermediate values are never computed
    bx = backend.BufferFromFlatData(0, xin, be.make_shape(code, B, S, H))
    bg = backend.BufferFromFlatData(0, gin, be.make_shape(code, H))
    out = exe.Execute([bx, bg], None, 0)[0].ToNumpy()
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps) * (g if with_gamma else 1.0)
    if dtype == "bf16":
        assert max_abs_normalised(orc.bf16_to_f32(out), want) < 2.0 ** -7
    else:
        assert max_abs_normalised(out, want) < 1e-6
    exe.Finalize()


def test_rms_pattern_is_not_matched_when_it_is_not_one(backend):
    """A different constant, or a reduction over another axis, stays decomposed and still computes the right thing."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 64), dtype=np.float32)
    def build(f, p):
        ss = f.ReduceSum(f.Mul(p[0], p[0]), -1)
        r = f.Rsqrt(f.Add(f.Mul(ss, f.Constant(np.float32([0.5]), dtype=dv.F32)), f.Constant(np.float32([1e-5]), dtype=dv.F32)))
        return f.Mul(p[0], f.Reshape(r, 4, 1))
    (got,), _ = run(backend, [(x, dv.F32)], build)
    want = x / np.sqrt((x.astype(np.float64) ** 2).sum(-1, keepdims=True) * 0.5 + 1e-5)
    assert max_abs_normalised(got, want) < 1e-6


# ---------------------------------------------------------------- grouped projections through the graph
def test_independent_projections_compile_to_one_grouped_launch(backend):
    """gate / up of a SwiGLU block: two FusedQuantizedDense nodes on one x become one launch (one conversion of x); the
    product and a third, dependent projection follow."""
    M, K, N = 8, 512, 1792
    rng = np.random.default_rng(4)
    x = orc.bf16_to_f32(orc.bf16_from_f32(rng.standard_normal((M, K), dtype=np.float32)))
    _, wg, sg, _ = qdense_inputs(10, M, K, N, scale_layout="channel", bias=False)
    _, wu, su, _ = qdense_inputs(11, M, K, N, scale_layout="channel", bias=False)
    _, wd, sd, _ = qdense_inputs(12, M, N, K, scale_layout="channel", bias=False)
    builder = backend.Builder("swiglu")
    f = builder.Main()
    px = f.Parameter("x", be.make_shape(dv.BF16, M, K))
    consts = {}
    def qd(xv, w, s, act, tag):
        Kd, Nd = w.shape
        cw = f.Constant(w, Kd, Nd, dtype=dv.I8)
        cs = f.Constant(s.reshape(1, Nd), 1, Nd, dtype=dv.F32)
        return f.FusedQuantizedDense(xv, cw, None, be.Quantization(be.QUANT_LINEAR, cs, None, BlockAxis=0, BlockSize=Kd), act)
    gate = qd(px, wg, sg, dv.ACT_SILU, "g")
    up = qd(px, wu, su, dv.ACT_NONE, "u")
    h = f.Mul(gate, up)
    f.Return([qd(h, wd, sd, dv.ACT_NONE, "d"), gate])
    exe = builder.Compile()
    names = exe.KernelNames()
    assert sum(n.startswith("qdense_decode_tc_") for n in names) == 2 and any(n.endswith("_x2") for n in names), names
    bx = backend.BufferFromFlatData(0, orc.bf16_from_f32(x), be.make_shape(dv.BF16, M, K))
    outs = exe.Execute([bx], None, 0)
    y, g_out = orc.bf16_to_f32(outs[0].ToNumpy()), orc.bf16_to_f32(outs[1].ToNumpy())
    ref = lambda xv, w, s, act: orc.qdense_linear(xv, w, orc.expand_scales(s, "channel", *w.shape), None, None, 1, act)
    g_ref = orc.bf16_to_f32(orc.bf16_from_f32(ref(x, wg, sg, orc.ACT_SILU)))
    u_ref = orc.bf16_to_f32(orc.bf16_from_f32(ref(x, wu, su, orc.ACT_NONE)))
    assert max_abs_normalised(g_out, g_ref) < 2.0 ** -7
    h_ref = orc.bf16_to_f32(orc.bf16_from_f32(g_ref * u_ref))
    assert max_abs_normalised(y, ref(h_ref, wd, sd, orc.ACT_NONE)) < 2e-2
    exe.Finalize()


def test_execute_is_reentrant(backend):
    """Executable.Execute from several threads at once (executable.go:17-37): every call gets its own stream and
    workspaces; results are the single-threaded ones."""
    M, K, N = 4, 1024, 2048
    x0, w, s, b = qdense_inputs(20, M, K, N, scale_layout="kgroup", group=128)
    builder = backend.Builder("threads")
    f = builder.Main()
    px = f.Parameter("x", be.make_shape(dv.F32, M, K))
    cw = f.Constant(w, K, N, dtype=dv.I8)
    cs = f.Constant(s, K // 128, N, dtype=dv.F32)
    cb_ = f.Constant(b, N, dtype=dv.F32)
    f.Return([f.FusedQuantizedDense(px, cw, cb_, be.Quantization(be.QUANT_LINEAR, cs, None, BlockAxis=0, BlockSize=128), dv.ACT_GELU)])
    exe = builder.Compile()
    xs = [x0 * np.float32(1 + t) for t in range(4)]
    want = [orc.qdense_linear(x, w, orc.expand_scales(s, "kgroup", K, N, 128), None, b, 1, orc.ACT_GELU) for x in xs]
    errors = []
    def worker(t):
        try:
            for _ in range(25):
                bx = backend.BufferFromFlatData(0, xs[t], be.make_shape(dv.F32, M, K))
                out = exe.Execute([bx], None, 0)[0]
                got = out.ToNumpy()
                out.Finalize(); bx.Finalize()
                if max_abs_normalised(got, want[t]) > 1e-4:
                    errors.append((t, max_abs_normalised(got, want[t])))
        except Exception as e:      # noqa: BLE001
            errors.append((t, repr(e)))
    threads = [threading.Thread(target=worker, args=(t,)) for t in range(4)]
    for th in threads: th.start()
    for th in threads: th.join()
    assert not errors, errors
    exe.Finalize()


def test_constant_scales_in_the_reference_layout_reach_the_decode_kernel(backend):
    """The reference's own Quantization (BlockAxis = 1) expresses per-channel and K-group scales as [K, N] with
    BlockSize 1; when such a scale is a Constant whose rows repeat within K groups the compiler folds it to the
    compact layout and the tensor-core decode kernel runs.  A scale that is a Parameter cannot be inspected and
    stays on the reference-order kernel."""
    M, K, N, G = 4, 512, 768, 128
    x, w, s, b = qdense_inputs(30, M, K, N, scale_layout="kgroup", group=G)
    full = orc.expand_scales(s, "kgroup", K, N, G)          # [K, N], BlockSize 1
    def build_const(f, p):
        return f.FusedQuantizedDense(p[0], f.Constant(w, K, N, dtype=dv.I8), f.Constant(b, N, dtype=dv.F32),
                                     be.Quantization(be.QUANT_LINEAR, f.Constant(full, K, N, dtype=dv.F32), None, BlockAxis=1, BlockSize=1), dv.ACT_RELU)
    builder = backend.Builder("ref-layout")
    f = builder.Main()
    px = f.Parameter("x", be.make_shape(dv.F32, M, K))
    f.Return([build_const(f, [px])])
    exe = builder.Compile()
    assert exe.KernelNames()[0].startswith("qdense_decode_tc_f32"), exe.KernelNames()
    bx = backend.BufferFromFlatData(0, x, be.make_shape(dv.F32, M, K))
    got = exe.Execute([bx], None, 0)[0].ToNumpy()
    want = orc.qdense_linear(x, w, full, None, b, 1, orc.ACT_RELU)
    assert max_abs_normalised(got, want) < 1e-4
    exe.Finalize()
    # the same scales as a parameter: generic kernel, bit-exact with the reference order
    def build_param(f, p):
        return f.FusedQuantizedDense(p[0], f.Constant(w, K, N, dtype=dv.I8), f.Constant(b, N, dtype=dv.F32),
                                     be.Quantization(be.QUANT_LINEAR, p[1], None, BlockAxis=1, BlockSize=1), dv.ACT_RELU)
    (got2,), _ = run(backend, [(x, dv.F32), (full, dv.F32)], build_param)
    assert np.array_equal(got2, want)


def test_packed_4bit_weights_through_the_graph(backend):
    """Int4 weights as the reference stores them: two per byte, low nibble first (internal/gobackend/ops/convertdtype.go:199-226)."""
    M, K, N = 3, 64, 48
    rng = np.random.default_rng(40)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w4 = rng.integers(-8, 8, size=(K, N), dtype=np.int8)
    s = rng.uniform(0.01, 0.1, size=(K, N // 16)).astype(np.float32)
    packed = orc.pack_nibbles(w4.ravel())
    builder = backend.Builder("int4")
    f = builder.Main()
    px = f.Parameter("x", be.make_shape(dv.F32, M, K))
    pw = f.Parameter("w", be.make_shape(dv.I4, K, N))
    ps = f.Parameter("s", be.make_shape(dv.F32, K, N // 16))
    f.Return([f.FusedQuantizedDense(px, pw, None, be.Quantization(be.QUANT_LINEAR, ps, None, BlockAxis=1, BlockSize=16), dv.ACT_NONE)])
    exe = builder.Compile()
    assert exe.KernelNames()[0] == "qdense_generic_f32_i4"
    bufs = [backend.BufferFromFlatData(0, x, be.make_shape(dv.F32, M, K)), backend.BufferFromFlatData(0, packed, be.make_shape(dv.I4, K, N)),
            backend.BufferFromFlatData(0, s, be.make_shape(dv.F32, K, N // 16))]
    got = exe.Execute(bufs, None, 0)[0].ToNumpy()
    want = orc.qdense_linear(x, w4, s, None, None, 16, orc.ACT_NONE)
    assert np.array_equal(got, want)
    exe.Finalize()


# ---------------------------------------------------------------- SPMD and collectives (two or more GPUs)
def _need_gpus(backend, n):
    if backend.NumDevices() < n:
        pytest.skip(f"needs {n} GPUs, {backend.NumDevices()} visible")


def test_execute_on_another_device(backend):
    """One executable run with defaultDevice = 1: plans, streams, workspaces and constants all belong to that device."""
    _need_gpus(backend, 2)
    M, K, N = 4, 512, 1792
    x, w, s, b = qdense_inputs(50, M, K, N, scale_layout="kgroup", group=128)
    def build(f, p):
        return f.FusedQuantizedDense(p[0], f.Constant(w, K, N, dtype=dv.I8), f.Constant(b, N, dtype=dv.F32),
                                     be.Quantization(be.QUANT_LINEAR, f.Constant(s, K // 128, N, dtype=dv.F32), None, BlockAxis=0, BlockSize=128), dv.ACT_SILU)
    (got,), _ = run(backend, [(x, dv.F32)], build, device=1)
    want = orc.qdense_linear(x, w, orc.expand_scales(s, "kgroup", K, N, 128), None, b, 1, orc.ACT_SILU)
    assert max_abs_normalised(got, want) < 1e-4


@pytest.mark.parametrize("g", [2, 4, 8])
def test_column_sharded_projection_as_one_spmd_executable(backend, g):
    """The 4096-wide projection sharded along its output columns over g devices as ONE executable: every replica
    computes its slice, AllGather along the column axis gives every replica the full result (the same bits as the
    unsharded plan: a column's arithmetic does not depend on its neighbours), and an AllReduce(sum) of a row-parallel
    product follows, as after the down projection of a decoder block."""
    _need_gpus(backend, g)
    M, K, N = 8, 1024, 14336 // 4
    x, w, s, _ = qdense_inputs(60, M, K, N, x_dtype="bf16", scale_layout="kgroup", group=128, bias=False)
    xb = orc.bf16_from_f32(x)
    n_loc = N // g
    mesh = be.DeviceMesh(("tp",), (g,))
    builder = backend.Builder("column-parallel")
    builder.DistributedSPMD(g)
    builder.DeviceAssignment(*range(g))
    f = builder.Main()
    px = f.Parameter("x", be.make_shape(dv.BF16, M, K), be.ShardingSpec(mesh, ((), ())))
    pw = f.Parameter("w", be.make_shape(dv.I8, K, n_loc), be.ShardingSpec(mesh, ((), ("tp",))))
    ps = f.Parameter("s", be.make_shape(dv.F32, K // 128, n_loc), be.ShardingSpec(mesh, ((), ("tp",))))
    y_loc = f.FusedQuantizedDense(px, pw, None, be.Quantization(be.QUANT_LINEAR, ps, None, BlockAxis=0, BlockSize=128), dv.ACT_SILU)
    groups = mesh.ComputeReplicaGroups(["tp"])
    (y_all,) = f.AllGather([y_loc], 1, groups)
    (total,) = f.AllReduce([f.ConvertDType(y_loc, dv.F32)], be.REDUCE_OP_SUM, groups)
    f.Return([y_all, total])
    exe = builder.Compile()
    assert exe.InputSharding(1) == ";tp" and exe.InputSharding(0) == "replicated"
    assert "all_gather" in exe.KernelNames() and "all_reduce" in exe.KernelNames()
    inputs = []
    for r in range(g):
        cols = slice(r * n_loc, (r + 1) * n_loc)
        inputs += [backend.BufferFromFlatData(r, xb, be.make_shape(dv.BF16, M, K)),
                   backend.BufferFromFlatData(r, np.ascontiguousarray(w[:, cols]), be.make_shape(dv.I8, K, n_loc)),
                   backend.BufferFromFlatData(r, np.ascontiguousarray(s[:, cols]), be.make_shape(dv.F32, K // 128, n_loc))]
    outs = exe.Execute(inputs, None, 0)
    assert len(outs) == 2 * g
    want = orc.qdense_linear(x, w, orc.expand_scales(s, "kgroup", K, N, 128), None, None, 1, orc.ACT_SILU)
    first = outs[0].ToNumpy()
    assert max_abs_normalised(orc.bf16_to_f32(first), want) < 2e-2
    slices = [orc.bf16_to_f32(first[:, r * n_loc:(r + 1) * n_loc]) for r in range(g)]
    total_want = np.sum(slices, axis=0, dtype=np.float32) if g == 2 else None
    for r in range(g):
        assert outs[2 * r].DeviceNum() == r
        assert np.array_equal(outs[2 * r].ToNumpy(), first)                 # every replica holds the same gathered bits
        tot = outs[2 * r + 1].ToNumpy()
        assert np.array_equal(tot, outs[1].ToNumpy())                       # and the same reduced bits
        ref = slices[0].copy()
        for k in range(1, g):
            ref = ref + slices[k]                                           # float32, in group order
        assert np.array_equal(tot, ref)
    exe.Finalize()


def test_replica_groups_are_validated(backend):
    builder = backend.Builder("groups")
    builder.DistributedSPMD(1)
    f = builder.Main()
    a = f.Parameter("a", be.make_shape(dv.F32, 4))
    (r,) = f.AllReduce([a], be.REDUCE_OP_MAX, [[0]])
    f.Return([r])
    exe = builder.Compile()
    buf = backend.BufferFromFlatData(0, np.float32([1, 5, 2, 4]), be.make_shape(dv.F32, 4))
    assert np.array_equal(exe.Execute([buf], None, 0)[0].ToNumpy(), [1, 5, 2, 4])      # one replica: the identity
    b2 = backend.Builder("bad-groups")
    f2 = b2.Main()
    a2 = f2.Parameter("a", be.make_shape(dv.F32, 4))
    (r2,) = f2.AllReduce([a2], be.REDUCE_OP_SUM, [[0, 1]])
    f2.Return([r2])
    with pytest.raises(BackendError):        # replica 1 does not exist in a one-device computation
        b2.Compile()
    mesh = be.DeviceMesh(("data", "model"), (2, 4))
    assert mesh.ComputeReplicaGroups(["model"]) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert mesh.ComputeReplicaGroups(["data"]) == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert mesh.ComputeReplicaGroups(["data", "model"]) == [list(range(8))]
    with pytest.raises(BackendError):
        f2b = backend.Builder("bad-spec").Main()
        f2b.Parameter("p", be.make_shape(dv.F32, 4, 4), be.ShardingSpec(mesh, (("nope",),)))


def test_repeated_execute_replays_a_cuda_graph():
    """The second and later calls with the same input buffers are one graph launch: same bits as the node-by-node call,
    for a graph with a grouped decode launch, an RMS norm pattern, element-wise ops and attention in it."""
    rng = np.random.default_rng(41)
    H, N = 512, 768
    x = orc.bf16_from_f32(rng.standard_normal((8, H), dtype=np.float32))
    g = orc.bf16_from_f32(rng.uniform(0.5, 1.5, size=(H,)).astype(np.float32))
    w1 = rng.integers(-127, 128, size=(H, N), dtype=np.int8)
    w2 = rng.integers(-127, 128, size=(H, N), dtype=np.int8)
    s1 = rng.uniform(0.001, 0.02, size=(1, N)).astype(np.float32)
    s2 = rng.uniform(0.001, 0.02, size=(1, N)).astype(np.float32)
    results = {}
    for cfg in ("", "no_graphs"):
        b = be.New(cfg)
        builder = b.Builder("replay")
        f = builder.Main()
        px = f.Parameter("x", be.make_shape(dv.BF16, 8, H))
        pg = f.Parameter("g", be.make_shape(dv.BF16, H))
        pw1, pw2 = f.Parameter("w1", be.make_shape(dv.I8, H, N)), f.Parameter("w2", be.make_shape(dv.I8, H, N))
        ps1, ps2 = f.Parameter("s1", be.make_shape(dv.F32, 1, N)), f.Parameter("s2", be.make_shape(dv.F32, 1, N))
        xn = _rms_graph(f, px, pg, H, 1e-5, dv.BF16, True, False)
        a = f.FusedQuantizedDense(xn, pw1, None, be.Quantization(be.QUANT_LINEAR, ps1, None, 0, H), dv.ACT_SILU)
        c = f.FusedQuantizedDense(xn, pw2, None, be.Quantization(be.QUANT_LINEAR, ps2, None, 0, H), dv.ACT_NONE)
        f.Return([f.Mul(a, c), xn])
        exe = builder.Compile()
        bufs = [b.BufferFromFlatData(0, arr, be.make_shape(d, *arr.shape)) for arr, d in
                ((x, dv.BF16), (g, dv.BF16), (w1, dv.I8), (w2, dv.I8), (s1, dv.F32), (s2, dv.F32))]
        outs = []
        for _ in range(5):
            res = exe.Execute(bufs, None, 0)
            outs.append([r.ToNumpy() for r in res])
            for r in res:
                r.Finalize()
        assert exe.GraphReplays() == (4 if cfg == "" else 0)
        for o in outs[1:]:
            assert all(np.array_equal(p, q) for p, q in zip(o, outs[0]))
        results[cfg] = outs[0]
        # other input buffers: the plain path again, then a second instance
        x2 = orc.bf16_from_f32(rng.standard_normal((8, H), dtype=np.float32))
        bx2 = b.BufferFromFlatData(0, x2, be.make_shape(dv.BF16, 8, H))
        r1 = [r.ToNumpy() for r in exe.Execute([bx2] + bufs[1:], None, 0)]
        r2 = [r.ToNumpy() for r in exe.Execute([bx2] + bufs[1:], None, 0)]
        assert all(np.array_equal(p, q) for p, q in zip(r1, r2)) and not np.array_equal(r1[1], outs[0][1])
        assert exe.GraphReplays() == (5 if cfg == "" else 0)
        bx2.Finalize()
        for t in bufs:
            t.Finalize()
        exe.Finalize()
        b.Finalize()
    assert all(np.array_equal(p, q) for p, q in zip(results[""], results["no_graphs"]))


def test_packed_4bit_and_ggml_decode_kernels_in_a_replayed_graph():
    """FusedQuantizedDense at decode shapes through the Backend API: packed Uint4 under NF4 runs on the streaming kernel,
    Q4_K and Q8_0 on the integer tensor cores.  All need workspaces, are dependent launches, and two of them take a tensor
    map in their parameters; from the second Execute on they are replayed from a captured CUDA graph.  Every call gives the
    bits of the first, and the first agrees with the oracle."""
    rng = np.random.default_rng(43)
    M, K, N, block = 3, 512, 640, 64
    x = rng.standard_normal((M, K)).astype(np.float32)
    idx = rng.integers(0, 16, size=(K, N))
    packed = orc.pack_nibbles(idx)
    s = rng.uniform(0.01, 0.2, size=(K, N // block)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    wq4k = orc.ggml_random_rows(rng, N, K, orc.GGML_Q4_K)
    wq80 = orc.ggml_random_rows(rng, N, K, orc.GGML_Q8_0)
    want = [orc.qdense_nf4(x, idx.astype(np.uint8), s, bias, block, orc.ACT_NONE),
            orc.qdense_ggml(x, wq4k, bias, orc.GGML_Q4_K, orc.ACT_NONE),
            orc.qdense_ggml(x, wq80, None, orc.GGML_Q8_0, orc.ACT_NONE)]
    b = be.New("")
    builder = b.Builder("w4_ggml")
    f = builder.Main()
    px = f.Parameter("x", be.make_shape(dv.F32, M, K))
    pw = f.Parameter("w", be.make_shape(dv.U4, K, N))
    ps = f.Parameter("s", be.make_shape(dv.F32, K, N // block))
    pb = f.Parameter("b", be.make_shape(dv.F32, N))
    pk = f.Parameter("wk", be.make_shape(dv.U8, *wq4k.shape))
    p8 = f.Parameter("w8", be.make_shape(dv.U8, *wq80.shape))
    y0 = f.FusedQuantizedDense(px, pw, pb, be.Quantization(be.QUANT_NF4, ps, None, 1, block), dv.ACT_NONE)
    y1 = f.FusedQuantizedDense(px, pk, pb, be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q4_K), dv.ACT_NONE)
    y2 = f.FusedQuantizedDense(px, p8, None, be.Quantization(be.QUANT_GGML, GGMLType=orc.GGML_Q8_0), dv.ACT_NONE)
    f.Return([y0, y1, y2])
    exe = builder.Compile()
    bufs = [b.BufferFromFlatData(0, x, be.make_shape(dv.F32, M, K)), b.BufferFromFlatData(0, packed, be.make_shape(dv.U4, K, N)),
            b.BufferFromFlatData(0, s, be.make_shape(dv.F32, *s.shape)), b.BufferFromFlatData(0, bias, be.make_shape(dv.F32, N)),
            b.BufferFromFlatData(0, wq4k, be.make_shape(dv.U8, *wq4k.shape)), b.BufferFromFlatData(0, wq80, be.make_shape(dv.U8, *wq80.shape))]
    outs = []
    for _ in range(4):
        res = exe.Execute(bufs, None, 0)
        outs.append([r.ToNumpy() for r in res])
        for r in res:
            r.Finalize()
    assert exe.GraphReplays() == 3
    for got, w in zip(outs[0], want):
        assert max_abs_normalised(got, w) < 1e-4
    for o in outs[1:]:
        assert all(np.array_equal(p, q) for p, q in zip(o, outs[0]))
    for t in bufs:
        t.Finalize()
    exe.Finalize()
    b.Finalize()
