"""Failure handling of the NCCL communicator, on the host: a stand-in libnccl (tests/fake/fake_nccl.c, built
here with gcc) scripts what the real library would report — an initialisation that never completes because a
rank never joined, an asynchronous error, an enqueue that stays in progress — and the tests check the status
the C ABI returns, that the communicator was aborted, and that the handle fails cleanly afterwards.  Every
case runs in a child process: the library resolves NCCL once per process."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fake_lib(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libnccl_fake.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), os.path.join(ROOT, "tests", "fake", "fake_nccl.c")], check=True)
    return str(out)


def run_case(fake_lib, body, **env):
    script = textwrap.dedent("""
        import ctypes as C, sys, time
        sys.path.insert(0, %r)
        from compute_b200 import BackendError, _lib, device as dv
        fake = C.CDLL(%r)
        uid = dv.Comm.unique_id()
    """) % (ROOT, fake_lib) + textwrap.dedent(body)
    full_env = dict(os.environ, CUDABACKEND_NCCL_LIB=fake_lib, **{k: str(v) for k, v in env.items()})
    r = subprocess.run([sys.executable, "-c", script], env=full_env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_init_completes_after_a_few_polls(fake_lib):
    out = run_case(fake_lib, """
        c = dv.Comm(-1, 2, 0, uid, timeout_s=5.0)
        c.check()
        c.allgather(1, 1, 16)          # the enqueue is reported in progress, then settles
        c.allreduce(1, 1, 4, dv.F32)
        c.close()
        print("aborts", fake.fake_nccl_aborts(), "destroys", fake.fake_nccl_destroys())
    """, FAKE_NCCL_POLLS=3)
    assert "aborts 0 destroys 1" in out


def test_rank_that_never_joins_times_out_and_aborts(fake_lib):
    out = run_case(fake_lib, """
        t0 = time.time()
        try:
            dv.Comm(-1, 2, 0, uid, timeout_s=0.3)
            print("no error")
        except BackendError as e:
            print("code", e.status, "timeout" if e.status == _lib.ERR_TIMEOUT else "other", "aborted" in str(e))
        print("waited", 0.3 <= time.time() - t0 < 10.0, "aborts", fake.fake_nccl_aborts())
    """, FAKE_NCCL_POLLS=-1)
    assert "timeout True" in out and "waited True aborts 1" in out


def test_async_error_aborts_and_later_calls_fail_at_once(fake_lib):
    out = run_case(fake_lib, """
        import os
        c = dv.Comm(-1, 2, 1, uid, timeout_s=5.0)
        os.environ["FAKE_NCCL_ASYNC_RESULT"] = "3"        # from now on the library reports an internal error
        try:
            c.allreduce(1, 1, 4, dv.F32)
            print("no error")
        except BackendError as e:
            print("first", e.status == _lib.ERR_CUDA, "internal error" in str(e))
        for call in (lambda: c.allgather(1, 1, 16), lambda: c.check(), lambda: c.allreduce(1, 1, 4, dv.F32)):
            try:
                call()
                print("no error")
            except BackendError as e:
                print("later", "aborted" in str(e))
        c.close()
        print("aborts", fake.fake_nccl_aborts(), "destroys", fake.fake_nccl_destroys())
    """, FAKE_NCCL_POLLS=2)
    assert "first True True" in out and out.count("later True") == 3 and "no error" not in out
    assert "aborts 1 destroys 0" in out          # an aborted communicator is not destroyed a second time


def test_enqueue_that_stays_in_progress_times_out(fake_lib):
    out = run_case(fake_lib, """
        import os
        c = dv.Comm(-1, 4, 2, uid, timeout_s=0.2)
        os.environ["FAKE_NCCL_POLLS"] = "-1"              # a peer has left: the enqueue never settles
        try:
            c.allgather(1, 1, 16)
            print("no error")
        except BackendError as e:
            print("timeout", e.status == _lib.ERR_TIMEOUT, "rank 2 of 4" in str(e))
        print("aborts", fake.fake_nccl_aborts())
    """, FAKE_NCCL_POLLS=1)
    assert "timeout True True" in out and "aborts 1" in out


def test_no_time_limit_keeps_the_blocking_kind(fake_lib):
    out = run_case(fake_lib, """
        c = dv.Comm(-1, 2, 0, uid)
        c.allreduce(1, 1, 4, dv.F32)
        c.check()
        c.close()
        print("inits", fake.fake_nccl_inits(), "destroys", fake.fake_nccl_destroys())
    """, FAKE_NCCL_REFUSE_CONFIG=1, FAKE_NCCL_ENQUEUE_RESULT=0, FAKE_NCCL_POLLS=0)
    assert "inits 1 destroys 1" in out         # the configuration record was never offered


def test_library_that_refuses_the_config_record_falls_back_to_blocking(fake_lib):
    out = run_case(fake_lib, """
        c = dv.Comm(-1, 2, 0, uid, timeout_s=1.0)
        c.allreduce(1, 1, 4, dv.F32)
        c.close()
        print("inits", fake.fake_nccl_inits(), "destroys", fake.fake_nccl_destroys())
    """, FAKE_NCCL_REFUSE_CONFIG=1, FAKE_NCCL_ENQUEUE_RESULT=0)
    assert "inits 1 destroys 1" in out         # the refused record did not count; the blocking initialiser ran once


@pytest.mark.gpu
def test_real_nccl_rank_that_never_joins():
    """The real library on one GPU: rank 0 of a two-rank communicator whose other rank never starts.  Nothing is
    launched on the device — the initialisation stays in progress on the host until the limit passes."""
    script = textwrap.dedent("""
        import sys, time
        sys.path.insert(0, %r)
        from compute_b200 import BackendError, _lib, device as dv
        dv.init()
        uid = dv.Comm.unique_id()
        t0 = time.time()
        try:
            dv.Comm(0, 2, 0, uid, timeout_s=3.0)
            print("no error")
        except BackendError as e:
            print("status", e.status, "timeout" if e.status == _lib.ERR_TIMEOUT else "other", str(e))
        print("waited %%.1f" %% (time.time() - t0))
        # the device is still usable afterwards
        a = dv.DeviceMem(1 << 20, 0)
        a.free()
        print("device ok")
    """) % ROOT
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "timeout" in r.stdout and "device ok" in r.stdout, r.stdout + r.stderr
