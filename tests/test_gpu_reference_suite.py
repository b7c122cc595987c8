"""GPU: the reference's OWN unit-test programs for the hot path, run against the reference built with the B200 backend.

shim/Makefile links every object of the unmodified reference except the six translation units the shim replaces
(origin::cuda::matmul / relu / sum_to / im2col / col2im / conv2d / conv2d_backward, functional::LinearOp and
functional::MatMul) together with shim/*.cu|cpp and libodl_b200.so, and builds the reference's gtest sources
(tests/unit_test/{operator,autograd,nn,optim}/test_*.cpp, its googletest, unchanged) against that library.  Each program
instantiates every TEST_P once per device (tests/unit_test/common/device_test_base.h:104-162): the /CUDA instances are the
drop-in proof -- the reference's own expectations, through its own Tensor / Operator / Mat interfaces, on the tcgen05
kernels.  test_linear_backward is this repository's addition in the same idiom (the reference has no test for the
backward rule it does not implement).

The programs are built where the reference tree is mounted (`make -C shim tests`, also run by __graft_entry__.build())
and travel prebuilt; the test is skipped, with the reason, where neither the tree nor the binaries exist."""
import os
import re
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BUILD = ROOT / "shim" / "_build" / "tests"
PROGRAMS = ["test_matmul", "test_matmul_3d", "test_linear", "test_linear_backward", "test_relu", "test_conv2d",
            "test_softmax_cross_entropy", "test_sum_to", "test_add", "test_broadcast_to", "test_linear_regression",
            "test_mlp", "test_conv2d_layer", "test_adam", "test_weight_decay"]


def _ensure_built():
    ref = Path(os.environ.get("ODL_REFERENCE_TREE", ROOT.parent / "reference"))
    if ref.exists():
        subprocess.run(["make", "-C", str(ROOT / "shim"), "tests", "-j8", f"REF={ref}"], check=True, capture_output=True)
    if not BUILD.exists():
        pytest.skip("shim/_build/tests is not built and the reference tree is not mounted here")


@pytest.mark.parametrize("program", PROGRAMS)
def test_reference_program_passes_on_the_b200_backend(program):
    _ensure_built()
    exe = BUILD / program
    assert exe.exists(), f"{exe} missing: run `make -C shim tests` where the reference tree is mounted"
    r = subprocess.run([str(exe), "--gtest_color=no"], capture_output=True, text=True, timeout=600, cwd=str(BUILD))
    out = r.stdout + r.stderr
    ok_cuda = re.findall(r"\[\s+OK \] \S+/CUDA", out)
    failed = re.findall(r"\[\s+FAILED\s+\] (\S+)", out)
    assert r.returncode == 0 and not failed, out[-3000:]
    assert ok_cuda, "no /CUDA instance ran:\n" + out[-1500:]
