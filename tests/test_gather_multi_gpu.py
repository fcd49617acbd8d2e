"""Fused all-gather of a column-sharded decode projection across two processes and two GPUs:
every rank's kernel stores its slice into both ranks' result buffers over NVLink (buffers shared
with cb_ipc_export / cb_ipc_open), signals, and waits for both arrival flags.  Skipped with
fewer than two GPUs."""
import multiprocessing as mp

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

M, K, N, G = 16, 1024, 2048, 128


def _worker(rank, g, conn):
    try:
        from compute_b200 import device as dv
        from oracle import oracle as orc
        from tests.helpers import qdense_inputs
        dv.init()
        dev = rank
        n_loc = N // g
        x, w, s, _ = qdense_inputs(11, M, K, N, x_dtype="bf16", scale_layout="kgroup", group=G, bias=False)
        cols = slice(rank * n_loc, (rank + 1) * n_loc)
        st = dv.Stream(dev)
        xd = dv.DeviceMem.from_numpy(orc.bf16_from_f32(x), dev)
        wd = dv.DeviceMem.from_numpy(np.ascontiguousarray(w[:, cols]), dev)
        sd = dv.DeviceMem.from_numpy(np.ascontiguousarray(s[:, cols]), dev)
        y = dv.DeviceMem(M * N * 2, dev)
        flags = dv.DeviceMem(256, dev)
        y.zero(); flags.zero()
        conn.send((dv.ipc_export(y), dv.ipc_export(flags)))
        everyone = conn.recv()
        outs = [y.ptr if r == rank else dv.ipc_open(dev, everyone[r][0]) for r in range(g)]
        fls = [flags.ptr if r == rank else dv.ipc_open(dev, everyone[r][1]) for r in range(g)]
        plan = dv.Plan.qdense(M, K, n_loc, dv.BF16, dv.I8, dv.SCALE_KGROUP, G, False, False, dv.ACT_SILU, dev=dev,
                              gather_ranks=g, gather_rank=rank)
        ws = plan.new_workspace()
        for rep in range(3):
            plan.launch([xd.ptr, wd.ptr, sd.ptr], outs, ws.ptr, st)
            dv.peer_signal(dev, fls, rank, st)
            dv.peer_wait(dev, flags.ptr, g, rep + 1, flags.ptr + 64, st)
        # the same step with the signal and the wait as one kernel
        barrier = dv.PeerBarrier(dev, fls, rank, flags.ptr, flags.ptr + 64)
        plan.launch([xd.ptr, wd.ptr, sd.ptr], outs, ws.ptr, st)
        barrier.signal_wait(4, st)
        st.sync()
        plan.check_status(ws.ptr)
        got = y.download((M, N), np.uint16)
        fl = flags.download((64,), np.uint32)
        conn.send(("ok", got, fl[:g].tolist(), int(fl[16])))
        conn.recv()                       # nobody frees memory a peer may still be writing
    except Exception as e:                # reported to the parent, which fails the test
        conn.send(("error", repr(e)))


def test_two_processes_two_gpus():
    from compute_b200 import device as dv
    if dv.init() < 2:
        pytest.skip("needs two GPUs")
    from oracle import oracle as orc
    from tests.helpers import max_abs_normalised, qdense_inputs
    g = 2
    ctx = mp.get_context("spawn")
    pipes = [ctx.Pipe() for _ in range(g)]
    procs = [ctx.Process(target=_worker, args=(r, g, pipes[r][1])) for r in range(g)]
    for p in procs:
        p.start()
    try:
        handles = []
        for r in range(g):
            assert pipes[r][0].poll(120), "worker did not start"
            handles.append(pipes[r][0].recv())
        for r in range(g):
            pipes[r][0].send(handles)
        results = []
        for r in range(g):
            assert pipes[r][0].poll(120), "worker did not finish"
            results.append(pipes[r][0].recv())
        for r in range(g):
            pipes[r][0].send("done")
    finally:
        for p in procs:
            p.join(30)
            if p.is_alive():
                p.kill()
    x, w, s, _ = qdense_inputs(11, M, K, N, x_dtype="bf16", scale_layout="kgroup", group=G, bias=False)
    want = orc.qdense_linear(x, w, orc.expand_scales(s, "kgroup", K, N, G), None, None, 1, orc.ACT_SILU, threads=orc.max_threads())
    for r, res in enumerate(results):
        assert res[0] == "ok", res
        _, got, arrivals, status = res
        assert arrivals == [4, 4] and status == 0
        assert max_abs_normalised(orc.bf16_to_f32(got), want) < 2e-2
    assert np.array_equal(results[0][1], results[1][1])
