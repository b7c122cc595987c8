"""CPU: the C-ABI library builds for sm_100a, loads without a GPU and exports every function include/odl_b200.h
declares; without a device the entry points fail loudly instead of falling back to anything."""
import ctypes

import pytest


def test_library_exports_every_declared_symbol():
    from origindl_b200 import build, capi

    build.build()
    L = capi.lib()
    names = capi.declared_symbols()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_no_cpu_fallback_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from origindl_b200 import capi

    L = capi.lib()
    assert L.odl_init(0) != 0                                   # no device: refuses to initialise
    status = L.odl_matmul(None, None, None, 4, 4, 4, 1, 0, 0, None)
    assert status != 0 and L.odl_last_error()                   # and nothing computes on the host


def test_oracle_is_not_reachable_from_the_package():
    """The product never imports, links or executes anything under oracle/."""
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent / "origindl_b200"
    for f in list(root.rglob("*.py")) + list(root.rglob("*.cu")) + list(root.rglob("*.h")) + list(root.rglob("*.cuh")):
        text = f.read_text()
        assert "liboracle" not in text and "odl_ref" not in text and "oracle/" not in text, f
