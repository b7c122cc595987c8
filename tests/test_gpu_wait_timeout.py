"""GPU: the time-out path of the pipeline waits, executed once in the safe form -- a wait that gives up by itself.

Every mbarrier wait inside the GEMM kernels is bounded (csrc/ptx_sm100.cuh): when it runs out the waiting role raises a
shared abort flag that releases the CTA's other roles, the CTA raises the per-device error flag, odl_device_status
reports ODL_ERR_KERNEL_TIMEOUT and clears it, and GEMM launches issued while the flag is up leave at once.  The
reference's counterpart is CUDA_CHECK_ASYNC (include/origin/mat/origin/cuda/cuda_utils.cuh:14-33): synchronise, then
turn the device's error into an exception.

A GEMM cannot be made to time out without breaking it, so a test-only kernel (tests/cuda/wait_timeout_kernel.cu) calls
the same wait, compiled with a 1 ms limit, on a barrier nobody arrives on.  Nothing faults or hangs: the kernel returns
after about a millisecond and the context stays usable, which the rest of the test relies on."""
import ctypes
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
pytestmark = pytest.mark.gpu
KERNELS = Path(__file__).resolve().parent / "cuda" / "build" / "libodl_test_kernels.so"
ERR_KERNEL_TIMEOUT = 4


@pytest.mark.parametrize("pair", [False, True])
def test_wait_that_runs_out_is_reported_and_later_launches_recover(pair):
    from origindl_b200 import build, capi, ops

    if not KERNELS.exists():
        build.build_test_kernels()
    capi.init(0)
    L = capi.lib()
    T = ctypes.CDLL(str(KERNELS))
    T.odl_test_wait_that_gives_up.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    T.odl_test_wait_that_gives_up.restype = ctypes.c_int
    L.odl_debug_error_flag.restype = ctypes.c_void_p
    L.odl_debug_error_flag.argtypes = []
    flag = L.odl_debug_error_flag()
    assert flag
    capi.device_status()                                   # clean before we start

    report = torch.full((4,), -1, dtype=torch.int64, device="cuda")
    assert T.odl_test_wait_that_gives_up(flag, report.data_ptr(), capi.stream_handle()) == 0
    torch.cuda.synchronize()                               # returns: the kernel ended by itself
    role0, role1, abort_flag, waited_ns = report.tolist()
    assert role0 == 1 and role1 == 1                       # both waits returned false ...
    assert abort_flag == 1                                 # ... the first one to run out released the other
    assert 1_000_000 <= waited_ns < 100_000_000            # after the 1 ms limit, not much later

    # while the flag is up, a GEMM launch does no work (its output buffer keeps the sentinel)
    if pair:
        capi.call("odl_debug_set_pair_mode", 2)
        capi.call("odl_debug_set_tile_n", 256)
    else:
        capi.call("odl_debug_set_split_k", 1)              # one CTA per tile (the CTAs of a K-splitting cluster meet at
                                                           # cluster barriers and therefore never leave early)
    try:
        M, N, K = (512, 512, 256) if pair else (200, 136, 264)
        gen = torch.Generator(device="cuda").manual_seed(5)
        a, b = torch.randn(M, K, device="cuda", generator=gen), torch.randn(K, N, device="cuda", generator=gen)
        d = torch.full((M, N), float("nan"), device="cuda")
        launches = L.odl_launch_count()
        capi.call("odl_gemm_ex", 0, 0, M, N, K, a.data_ptr(), None, K, b.data_ptr(), None, N, d.data_ptr(), None, N, None,
                  None, 0, None, 0, capi.PRECISION_3XTF32, capi.stream_handle())
        assert L.odl_launch_count() > launches             # it was launched ...
        torch.cuda.synchronize()
        assert torch.isnan(d).all()                        # ... and every CTA left before touching D

        # the host learns of it at its next status call, which also clears the flag
        with pytest.raises(capi.OdlError) as err:
            capi.device_status()
        assert err.value.status == ERR_KERNEL_TIMEOUT
        assert "bounded wait" in str(err.value)
        capi.device_status()                               # cleared: no second report

        # and the next launch computes again
        got = ops.gemm(a, b)
        want = a.double() @ b.double()
        assert ((got.double() - want).abs().max() / want.abs().max()).item() <= 1e-5
        capi.device_status()
    finally:
        capi.call("odl_debug_set_pair_mode", 0)
        capi.call("odl_debug_set_tile_n", 0)
        capi.call("odl_debug_set_split_k", 0)
        L.odl_device_status(ctypes.c_void_p(capi.stream_handle()))   # never leave the flag up for the tests that follow
