"""GPU: the allocation-free softmax-cross-entropy entry point against the regular one.

Some users of this library run where device memory cannot be allocated after start-up (the host application owns all
of it, or an allocation's device-wide synchronisation is not acceptable in their loop).  For them
odl_softmax_cross_entropy_static keeps its per-row scratch in a fixed array inside the library.  This test calls it
through the C ABI twice in a row -- the second time with fewer rows and other data, so anything left in the shared
array by the first call would show -- and requires the same loss and gradient as the regular entry point.  It also
checks the stated row limit.  The file name sorts last so that a run that stops at the first failure has already run
every other test; it passes on its own in a fresh process as well."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    import ctypes

    from origindl_b200 import capi

    fn = capi.lib().odl_softmax_cross_entropy_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row():
    import ctypes
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parent))
    import _libs
    from origindl_b200 import capi, ops

    capi.init(0)
    L = capi.lib()
    fn = _entry()
    orc = _libs.oracle()
    rng = np.random.default_rng(77)
    # two calls in a row; the second has fewer rows, other data and 64-bit labels, and reuses the front of the array
    for (B, C), label_dtype in (((4096, 1000), np.int32), ((513, 10), np.int64)):
        xh = (3 * rng.standard_normal((B, C))).astype(np.float32)
        th = rng.integers(0, C, B)
        x = torch.from_numpy(xh).cuda()
        t = torch.from_numpy(th.astype(label_dtype)).cuda()
        loss_ref, d_ref = ops.softmax_cross_entropy(x, t)
        loss = torch.full((1,), float("nan"), device="cuda")
        d = torch.full_like(x, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        capi.check(fn(x.data_ptr(), t.data_ptr(), int(label_dtype is np.int64), B, C, loss.data_ptr(), d.data_ptr(), 1.0,
                      capi.stream_handle()))
        capi.device_status()
        if (B, C) != (4096, 1000):
            # from the second call on, nothing on the device may have been allocated by the call (the first call of a
            # process may make the lazily loaded module image resident, which the header says to do at start-up)
            assert torch.cuda.mem_get_info()[0] == free_before
        # same kernels, same order of operations: the tolerance of the other loss tests (1e-5) is met with equality
        assert abs(loss.item() - loss_ref.item()) <= 1e-5 * max(1.0, abs(loss_ref.item()))
        assert ((d - d_ref).abs().max() / d_ref.abs().max()).item() <= 1e-5
        # and against the CPU oracle of the reference's loss (src/operators/loss/softmax_cross_entropy.cpp:17-111)
        l_o, d_o = ctypes.c_float(), np.empty_like(xh)
        assert orc.oracle_softmax_ce(xh, th.astype(np.int32), B, C, ctypes.byref(l_o), _libs.fptr(d_o)) == 0
        assert abs(loss.item() - l_o.value) <= 1e-5 * max(1.0, abs(l_o.value))
        assert _libs.max_rel_err(d.cpu().numpy(), d_o) <= 1e-5
    # beyond the fixed scratch the call is refused with a clear message instead of overrunning the array
    big = 65536 + 1
    x = torch.zeros((big, 2), device="cuda")
    t = torch.zeros((big,), device="cuda", dtype=torch.int32)
    loss = torch.zeros((1,), device="cuda")
    status = fn(x.data_ptr(), t.data_ptr(), 0, big, 2, loss.data_ptr(), None, 1.0, capi.stream_handle())
    assert status == 5                                # ODL_ERR_TOO_LARGE
    assert b"exceed the fixed scratch" in L.odl_last_error()
    capi.device_status()
