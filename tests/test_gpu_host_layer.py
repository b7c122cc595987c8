"""GPU: runs the C++ test program of the host layer (tests/cpp/test_host_api.cpp), whose cases mirror the reference's
own unit tests for MatMul / Linear / ReLU / softmax-CE / Conv2d / WeightDecay / Adam / linear regression."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def test_cpp_host_layer_program():
    from origindl_b200 import build, capi

    exe = Path(__file__).resolve().parent / "cpp" / "build" / "test_host_api"
    if not capi.LIB_PATH.exists():
        build.build()
    if not exe.exists():
        exe = build.build_host_tests()
    golden = Path(__file__).resolve().parent / "golden"
    r = subprocess.run([str(exe), str(golden)], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "0 failed" in r.stdout
