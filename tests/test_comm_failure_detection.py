"""CPU: failure detection of the data-parallel layer, with every failure made on the host.

Two halves:
  * the communicator of libodl_b200.so (csrc/comm_nccl.cpp) against a stand-in NCCL library that misbehaves on request
    (tests/cpp/fake_nccl.c, loaded through ODL_NCCL_LIBRARY): an asynchronous error is reported by odl_comm_status, the
    host watchdog odl_comm_watch returns ODL_ERR_COMM on an error and ODL_ERR_COMM_TIMEOUT when the watched work never
    completes, aborts the communicator either way, and an aborted communicator refuses later calls;
  * two gloo ranks on the CPU where one rank never joins a gradient all-reduce: the other rank's guarded reduction
    (origindl_b200.dp.guarded) ends with an error status after the short process-group time-out instead of hanging.
No GPU is involved and nothing is made to fault: the reference's counterpart is CUDA_CHECK_ASYNC
(include/origin/mat/origin/cuda/cuda_utils.cuh:14-33), which only covers CUDA errors -- it has no collectives."""
import os
import subprocess
import sys
import textwrap
from datetime import timedelta
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _run_with_fake_nccl(body: str) -> str:
    from origindl_b200 import build

    build.build()
    fake = build.build_fake_nccl()
    prologue = textwrap.dedent(f"""
        import ctypes, sys, time
        sys.path.insert(0, {str(ROOT)!r})
        from origindl_b200 import capi
        L = capi.lib()
        F = ctypes.CDLL({str(fake)!r})
        OK, ERR_COMM, ERR_COMM_TIMEOUT = 0, 8, 9
        DONE = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)
        L.odl_comm_unique_id.argtypes = [ctypes.c_void_p]
        L.odl_comm_create.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]
        L.odl_comm_destroy.argtypes = [ctypes.c_void_p]
        L.odl_comm_status.argtypes = [ctypes.c_void_p]
        L.odl_comm_allreduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        L.odl_comm_watch.argtypes = [ctypes.c_void_p, ctypes.c_int, DONE, ctypes.c_void_p]
        def make(rank=0, world=2):
            token = ctypes.create_string_buffer(128)
            assert L.odl_comm_unique_id(token) == OK
            comm = ctypes.c_void_p()
            status = L.odl_comm_create(token, rank, world, ctypes.byref(comm))
            return status, comm
        def msg():
            return L.odl_last_error().decode()
    """)
    env = dict(os.environ, ODL_NCCL_LIBRARY=str(fake))
    r = subprocess.run([sys.executable, "-c", prologue + textwrap.dedent(body)], env=env, capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_async_error_is_reported_by_the_status_poll():
    out = _run_with_fake_nccl("""
        status, comm = make()
        assert status == OK and comm.value
        assert L.odl_comm_status(comm) == OK
        F.fake_nccl_set_async_error(0, 6)                 # from now on: "remote process exited"
        assert L.odl_comm_status(comm) == ERR_COMM
        assert "asynchronous error" in msg() and "remote process exited" in msg()
        F.fake_nccl_set_async_error(0, 7)                 # "in progress" is not an error
        assert L.odl_comm_status(comm) == OK
        assert L.odl_comm_destroy(comm) == OK and F.fake_nccl_live_comms() == 0
        print("polled")
    """)
    assert "polled" in out


def test_watchdog_times_out_aborts_and_the_communicator_refuses_later_calls():
    out = _run_with_fake_nccl("""
        status, comm = make()
        never = DONE(lambda arg: 0)                       # the watched collective never completes (a peer never joined)
        t0 = time.monotonic()
        assert L.odl_comm_watch(comm, 150, never, None) == ERR_COMM_TIMEOUT
        waited = time.monotonic() - t0
        assert 0.14 <= waited < 5.0, waited
        assert "did not complete within 150 ms" in msg() and "aborted" in msg()
        assert F.fake_nccl_abort_count() == 1 and F.fake_nccl_live_comms() == 0
        # an aborted communicator is not used again: no call reaches NCCL
        assert L.odl_comm_status(comm) == ERR_COMM and "was aborted" in msg()
        assert L.odl_comm_allreduce(comm, ctypes.c_void_p(16), 4, None) == ERR_COMM
        assert F.fake_nccl_allreduce_count() == 0
        assert L.odl_comm_watch(comm, 10, never, None) == ERR_COMM
        assert L.odl_comm_destroy(comm) == OK and F.fake_nccl_abort_count() == 1
        print("timed out")
    """)
    assert "timed out" in out


def test_watchdog_returns_when_done_and_stops_on_an_async_error():
    out = _run_with_fake_nccl("""
        status, comm = make()
        calls = []
        soon = DONE(lambda arg: calls.append(1) or int(len(calls) >= 5))
        assert L.odl_comm_watch(comm, 5000, soon, None) == OK and len(calls) == 5
        assert F.fake_nccl_abort_count() == 0
        F.fake_nccl_set_async_error(3, 2)                 # an error shows up on the fourth poll from now
        status2, comm2 = make()
        never = DONE(lambda arg: 0)
        t0 = time.monotonic()
        assert L.odl_comm_watch(comm2, 60000, never, None) == ERR_COMM      # long before the time-out
        assert time.monotonic() - t0 < 5.0
        assert "asynchronous error" in msg() and "aborted" in msg() and F.fake_nccl_abort_count() == 1
        L.odl_comm_destroy(comm); L.odl_comm_destroy(comm2)
        print("watched")
    """)
    assert "watched" in out


def test_bad_rendezvous_and_failed_initialisation_are_errors():
    out = _run_with_fake_nccl("""
        comm = ctypes.c_void_p()
        token = ctypes.create_string_buffer(128)
        assert L.odl_comm_unique_id(token) == OK
        assert L.odl_comm_create(token, 2, 2, ctypes.byref(comm)) == 1          # rank outside the world
        assert L.odl_comm_create(None, 0, 2, ctypes.byref(comm)) == 1
        garbage = ctypes.create_string_buffer(b"x" * 127)
        assert L.odl_comm_create(garbage, 0, 2, ctypes.byref(comm)) == ERR_COMM  # a token NCCL did not make
        F.fake_nccl_set_init_error(2)
        assert L.odl_comm_create(token, 0, 2, ctypes.byref(comm)) == ERR_COMM and "ncclCommInitRank" in msg()
        print("refused")
    """)
    assert "refused" in out


def test_missing_nccl_library_is_a_clear_error():
    from origindl_b200 import build

    build.build()
    code = textwrap.dedent(f"""
        import ctypes, sys
        sys.path.insert(0, {str(ROOT)!r})
        from origindl_b200 import capi
        L = capi.lib()
        L.odl_comm_unique_id.argtypes = [ctypes.c_void_p]
        token = ctypes.create_string_buffer(128)
        assert L.odl_comm_unique_id(token) == 8
        assert b"ODL_NCCL_LIBRARY" in L.odl_last_error()
    """)
    env = dict(os.environ, ODL_NCCL_LIBRARY="/nonexistent/libnccl.so.2")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr


def test_communicator_host_code_under_address_and_ub_sanitizers(tmp_path):
    """comm_nccl.cpp built with -fsanitize=address,undefined (tests/cpp/comm_sanitized.cpp) and run against the stand-in
    NCCL: create / poll / all-reduce / watchdog time-out + abort / refusal / destroy leave no leak, no use after free
    and no undefined behaviour."""
    from origindl_b200 import build

    fake = build.build_fake_nccl()
    exe = tmp_path / "comm_sanitized"
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    r = None
    for cxx in ("/usr/bin/g++", "g++", os.environ.get("CXX", "c++")):   # the first one that has the sanitizer runtimes
        cmd = [cxx, "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-I",
               str(cuda / "include"), str(ROOT / "tests" / "cpp" / "comm_sanitized.cpp"), "-o", str(exe), "-ldl", "-lpthread"]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True)
        except OSError:
            continue
        if r.returncode == 0:
            break
    if r is None or (r.returncode != 0 and ("-lasan" in r.stderr or "libasan" in r.stderr)):
        pytest.skip("no compiler with the AddressSanitizer runtime on this machine")
    assert r.returncode == 0, r.stdout + r.stderr
    env = dict(os.environ, ODL_NCCL_LIBRARY=str(fake), ASAN_OPTIONS="detect_leaks=1:abort_on_error=0")
    r = subprocess.run([str(exe)], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "sanitized communicator run ok" in r.stdout, r.stdout + r.stderr
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr


# ---- two gloo ranks, one of which never joins the all-reduce of a gradient bucket -------------------------------------
SIZES = [12, 16, 8, 5]


def _worker(rank, world, port, out_dir):
    from origindl_b200 import dp

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    n = sum(a * b + b for a, b in zip(SIZES[:-1], SIZES[1:]))
    grads = torch.full((n,), float(rank + 1))
    # step 1: both ranks reduce -- the guard is transparent
    status, message = dp.guarded(dp.allreduce_gradients, grads, SIZES)
    first_ok = status == dp.COMM_OK and bool((grads == 3.0).all())
    dist.barrier()
    # step 2: rank 1 leaves between steps (never enters the collective); rank 0 must get a status, not a hang
    if rank == 1:
        (Path(out_dir) / "rank1_left").write_text("left before the second reduction")
        os._exit(0)
    import time

    t0 = time.monotonic()
    status, message = dp.guarded(dp.allreduce_gradients, grads, SIZES)
    (Path(out_dir) / "rank0.txt").write_text(f"{int(first_ok)}\n{status}\n{time.monotonic() - t0:.2f}\n{message}")
    os._exit(0)  # the process group is broken by design: skip its teardown


def test_rank_that_never_joins_surfaces_as_a_status_on_the_other_rank(tmp_path):
    from origindl_b200 import dp

    ctx = mp.get_context("spawn")
    port = 29500 + os.getpid() % 1500
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert p.exitcode == 0
    assert (tmp_path / "rank1_left").exists()
    first_ok, status, seconds, message = (tmp_path / "rank0.txt").read_text().split("\n", 3)
    assert first_ok == "1"
    assert int(status) == dp.COMM_FAILED
    assert float(seconds) < 30.0
    assert message.strip()
