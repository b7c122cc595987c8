"""GPU, two ranks (skipped on a one-GPU machine): the data-parallel step driven by a plain C++ host through the C ABI.

tests/cpp/dp_two_ranks.cpp links only libodl_b200.so and the CUDA runtime -- no Python, no torch.  Two such processes
(one per GPU) exchange NCCL's rendezvous token through a file, attach the library's communicator to their MLP and run six
odl_mlp_train_step_dp steps, each followed by the watchdog (odl_mlp_dp_wait) and the status polls.  Checks: both ranks end
with bit-identical parameters, and parameters and the mean of the per-rank losses equal one process training the whole
global batch alone, up to fp32 rounding (1e-5) -- the same statements tests/test_gpu_dp_nccl.py makes for the Python driver."""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_cpp_host_two_ranks_equal_full_batch(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from origindl_b200 import build

    exe = build.build_dp_host()
    nccl = Path(torch.__file__).resolve().parent.parent / "nvidia" / "nccl" / "lib" / "libnccl.so.2"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if nccl.exists():
        env["ODL_NCCL_LIBRARY"] = str(nccl)
    procs = [subprocess.Popen([str(exe), str(r), "2", str(tmp_path)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    r = subprocess.run([str(exe), "full", "2", str(tmp_path)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    p0, p1, pf = (np.fromfile(tmp_path / f"params_{t}.bin", np.float32) for t in ("0", "1", "full"))
    assert np.array_equal(p0, p1)                                     # replicas stay identical
    assert np.abs(p0 - pf).max() / np.abs(pf).max() <= 1e-5           # and equal full-batch training
    l0, l1, lf = (np.fromfile(tmp_path / f"losses_{t}.bin", np.float32) for t in ("0", "1", "full"))
    assert np.abs((l0 + l1) / 2 - lf).max() <= 1e-5                   # the global loss is the mean of the per-rank means
    assert lf[-1] < lf[0]
