"""GPU, two ranks over NCCL (skipped on a one-GPU machine): the data-parallel MLP trainer -- batch rows sharded by rank,
per-layer gradient buckets all-reduced head first on a side stream while earlier layers still run their backward, 1/world
folded into the optimizer -- reproduces single-GPU training on the global batch.  Four drivers of the same step run on
the same inputs: the library's own step behind the C ABI (odl_mlp_train_step_dp: its own NCCL communicator, stream and
events) with layer 0's weight gradient in one piece and in four row panels, and the older Python driver over
torch.distributed with and without overlap.  Checks: replicas stay bit-identical, all four drivers give the same bits,
parameters and the mean of the per-rank losses equal the full-batch run up to fp32 rounding (1e-5), and the watchdog /
status poll of the library's communicator report a healthy step.  The host-side plan and the failure paths are covered
on CPU (test_dp_gloo.py, test_comm_failure_detection.py)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

pytestmark = pytest.mark.gpu
SIZES, GLOBAL_B, STEPS = [256, 384, 256, 10], 256, 6
KW = dict(optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)


def _inputs():
    import _libs

    rng = np.random.default_rng(77)
    params = _libs.mlp_params(rng, SIZES)
    xs = rng.standard_normal((2, GLOBAL_B, SIZES[0])).astype(np.float32)
    ts = rng.integers(0, SIZES[-1], (2, GLOBAL_B)).astype(np.int32)
    return params, xs, ts


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    from origindl_b200 import capi, dp
    from origindl_b200.trainer import MLPTrainer

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    capi.init(rank)
    params, xs, ts = _inputs()
    lo, hi = dp.shard_rows(GLOBAL_B, rank, world)
    xd, td = torch.from_numpy(xs[:, lo:hi].copy()).cuda(), torch.from_numpy(ts[:, lo:hi].copy()).cuda()
    results = {}
    drivers = {"native": dict(native_dp=True, dw0_panels=1), "native_panels": dict(native_dp=True, dw0_panels=4),
               "python_overlap": dict(native_dp=False, overlap=True), "python_serial": dict(native_dp=False, overlap=False)}
    for name, kw in drivers.items():
        tr = MLPTrainer(SIZES, hi - lo, device=rank, process_group=dist.group.WORLD, **kw, **KW)
        tr.set_params(params)
        losses = []
        for s in range(STEPS):
            losses.append(tr.train_step(xd[s % 2], td[s % 2]).clone())
            if kw["native_dp"]:
                tr.wait(20000)       # host watchdog: the step's last all-reduce completed, no asynchronous error
                tr.comm_status()
        losses = torch.stack(losses)
        torch.cuda.synchronize()
        dist.all_reduce(losses)  # the global loss is the mean of the per-rank means
        results[name] = (tr.get_params(), (losses / world).cpu().numpy())
        tr.close()
    capi.device_status()
    np.savez(Path(out_dir) / f"rank_{rank}.npz", loss=results["native"][1], **{"p_" + k: v[0] for k, v in results.items()})
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_nccl_training_equals_full_batch(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from origindl_b200 import capi
    from origindl_b200.trainer import MLPTrainer

    world = 2
    mp.spawn(_worker, args=(world, 29100 + os.getpid() % 800, str(tmp_path)), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "rank_0.npz"), np.load(tmp_path / "rank_1.npz")
    for name in ("native", "native_panels", "python_overlap", "python_serial"):
        assert np.array_equal(r0["p_" + name], r1["p_" + name]), name       # replicas stay identical
        assert np.array_equal(r0["p_" + name], r0["p_native"]), name        # the schedule changes, not the arithmetic
    capi.init(0)
    params, xs, ts = _inputs()
    full = MLPTrainer(SIZES, GLOBAL_B, **KW)
    full.set_params(params)
    xd, td = torch.from_numpy(xs).cuda(), torch.from_numpy(ts).cuda()
    want = np.array([full.train_step(xd[s % 2], td[s % 2]).item() for s in range(STEPS)], np.float32)
    import _libs

    assert np.abs(r0["loss"] - want).max() <= 1e-5
    assert _libs.max_rel_err(r0["p_native"], full.get_params()) <= 1e-5
    full.close()
