"""The allocation-free decode entry point (cb_qdense_decode_static) against the planned,
workspace-based one.  Collected last on purpose: a failure here must not hide other tests.

Who needs it: callers that cannot allocate device memory at launch time (an inference server
whose arena owns all of HBM, a plugin running inside another framework's callback, a process
with a frozen allocator).  Both entry points run the same kernel, so their outputs must be
bit-identical; two calls in a row check that the built-in scratch is left reusable."""
import ctypes as C

import numpy as np
import pytest

from compute_b200 import BackendError, _lib, device as dv, ops
from oracle import oracle as orc
from tests.helpers import max_abs_normalised, qdense_inputs

pytestmark = pytest.mark.gpu


def run_static(x, w, s, b, desc, out_shape, dev=0):
    lib = _lib.load()
    bufs = [dv.DeviceMem.from_numpy(a, dev) for a in (x, w, s)]
    bias = dv.DeviceMem.from_numpy(b, dev) if b is not None else None
    out = dv.DeviceMem(int(np.prod(out_shape)) * x.dtype.itemsize, dev)
    try:
        _lib.check(lib.cb_qdense_decode_static(dev, C.byref(desc), bufs[0].ptr, bufs[1].ptr, bufs[2].ptr,
                                               bias.ptr if bias else None, out.ptr, None))
        _lib.check(lib.cb_stream_sync(dev, None))
        return out.download(out_shape, x.dtype)
    finally:
        for m in bufs + [out] + ([bias] if bias else []):
            m.free()


@pytest.mark.parametrize("M,K,N,x_dtype", [(4, 512, 1792, "bf16"), (16, 1024, 2048, "f32"), (1, 4096, 14336, "bf16")])
def test_static_scratch_matches_planned_kernel_twice(M, K, N, x_dtype):
    G = 128
    x, w, s, b = qdense_inputs(77 + M, M, K, N, x_dtype=x_dtype, scale_layout="kgroup", group=G)
    code = dv.BF16 if x_dtype == "bf16" else dv.F32
    xin = orc.bf16_from_f32(x) if x_dtype == "bf16" else x
    want = ops.quantized_dense(xin, w, s, None, b, x_dtype=code, scale_layout=dv.SCALE_KGROUP, block_size=G,
                               activation=dv.ACT_SILU, variant=dv.QDENSE_DECODE_MMA)
    desc = _lib.QDenseDesc(M, K, N, code, dv.I8, dv.SCALE_KGROUP, G, 0, 1, dv.ACT_SILU, dv.QDENSE_AUTO)
    for _ in range(2):          # the second call reuses whatever the first left in the scratch
        got = run_static(xin, w, s, b, desc, (M, N))
        assert np.array_equal(got, want)


def test_static_scratch_uint8_weights_per_channel_scales_no_bias():
    """The other template arm of the entry point: unsigned weights, one scale per column, no bias, no activation."""
    M, K, N = 8, 768, 1024
    x, wu, s, _ = qdense_inputs(91, M, K, N, x_dtype="f32", scale_layout="channel", bias=False, unsigned=True)
    want = ops.quantized_dense(x, wu, s, None, None, x_dtype=dv.F32, scale_layout=dv.SCALE_CHANNEL, variant=dv.QDENSE_DECODE_MMA)
    ref = orc.qdense_linear(x, wu, orc.expand_scales(s, "channel", K, N, 0), None, None, 1, orc.ACT_NONE, threads=orc.max_threads())
    assert max_abs_normalised(want, ref) < 1e-4
    desc = _lib.QDenseDesc(M, K, N, dv.F32, dv.U8, dv.SCALE_CHANNEL, 0, 0, 0, dv.ACT_NONE, dv.QDENSE_AUTO)
    for _ in range(2):
        got = run_static(x, wu, s, None, desc, (M, N))
        assert np.array_equal(got, want)


def test_static_scratch_rejects_bad_descriptors():
    lib = _lib.load()
    d = dv.DeviceMem(4096)
    bad_act = _lib.QDenseDesc(4, 512, 512, dv.F32, dv.I8, dv.SCALE_CHANNEL, 0, 0, 0, 99, 0)
    assert lib.cb_qdense_decode_static(0, C.byref(bad_act), d.ptr, d.ptr, d.ptr, None, d.ptr, None) == _lib.ERR_INVALID_ARG
    assert b"activation" in lib.cb_last_error()
    gathered = _lib.QDenseDesc(4, 512, 512, dv.F32, dv.I8, dv.SCALE_CHANNEL, 0, 0, 0, 0, 0, 2, 0)
    assert lib.cb_qdense_decode_static(0, C.byref(gathered), d.ptr, d.ptr, d.ptr, None, d.ptr, None) == _lib.ERR_NOT_IMPLEMENTED
    d.free()


def test_static_scratch_rejects_what_it_cannot_hold():
    lib = _lib.load()
    too_wide = _lib.QDenseDesc(1, 64, 64 * 700000, dv.F32, dv.I8, dv.SCALE_CHANNEL, 0, 0, 0, 0, 0)
    d = dv.DeviceMem(256)
    st = lib.cb_qdense_decode_static(0, C.byref(too_wide), d.ptr, d.ptr, d.ptr, None, d.ptr, None)
    assert st == _lib.ERR_INVALID_ARG and b"scratch" in lib.cb_last_error()
    not_decode = _lib.QDenseDesc(64, 64, 64, dv.F32, dv.I8, dv.SCALE_CHANNEL, 0, 0, 0, 0, 0)
    assert lib.cb_qdense_decode_static(0, C.byref(not_decode), d.ptr, d.ptr, d.ptr, None, d.ptr, None) == _lib.ERR_NOT_IMPLEMENTED
    d.free()
