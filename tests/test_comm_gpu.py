"""Collectives of the C ABI on one GPU: a one-rank communicator (all-gather and all-reduce are
copies) and the argument checks.  The multi-rank path runs under `bench.py --gpus N`."""
import numpy as np
import pytest

from compute_b200 import BackendError, ErrNotImplemented, device as dv

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm():
    try:
        uid = dv.Comm.unique_id()
    except ErrNotImplemented:
        pytest.skip("NCCL is not installed on this machine")
    c = dv.Comm(0, 1, 0, uid)
    yield c
    c.close()


def test_single_rank_allgather_and_allreduce(comm):
    st = dv.Stream(0)
    a = np.arange(1000, dtype=np.float32) - 300.0
    src = dv.DeviceMem.from_numpy(a)
    dst = dv.DeviceMem(a.nbytes)
    dst.zero()
    comm.allgather(src.ptr, dst.ptr, a.nbytes, st)
    st.sync()
    assert np.array_equal(dst.download(a.shape, np.float32), a)
    for op in (dv.REDUCE_SUM, dv.REDUCE_MAX, dv.REDUCE_MIN, dv.REDUCE_PRODUCT):
        dst.zero()
        comm.allreduce(src.ptr, dst.ptr, a.size, dv.F32, op, st)
        st.sync()
        assert np.array_equal(dst.download(a.shape, np.float32), a)
    # bf16 payloads travel as their bit patterns
    h = (np.arange(64, dtype=np.uint16) << 7)
    hs, hd = dv.DeviceMem.from_numpy(h), dv.DeviceMem(h.nbytes)
    comm.allreduce(hs.ptr, hd.ptr, h.size, dv.BF16, dv.REDUCE_MAX, st)
    st.sync()
    assert np.array_equal(hd.download(h.shape, np.uint16), h)


def test_argument_checks(comm):
    buf = dv.DeviceMem(64)
    with pytest.raises(ErrNotImplemented):      # boolean reductions are not built
        comm.allreduce(buf.ptr, buf.ptr, 4, dv.BOOL)
    with pytest.raises(BackendError):
        comm.allreduce(buf.ptr, buf.ptr, 4, dv.F32, 9)
    with pytest.raises(BackendError):
        dv.Comm(0, 2, 5, bytes(dv.COMM_ID_BYTES))
    comm.allgather(buf.ptr, buf.ptr, 0)          # empty payloads are fine
