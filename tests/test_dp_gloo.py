"""CPU, world_size 2 over gloo: the data-parallel plan (row sharding, per-layer buckets reduced head first, 1/world in
the optimizer) reproduces single-process training on the full batch.  The per-rank arithmetic is the oracle's, so the
only thing under test is the N > 1 host logic the GPU trainer shares (origindl_b200/dp.py)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

SIZES = [12, 16, 8, 5]
GLOBAL_B, STEPS = 16, 4


def _inputs():
    import _libs

    rng = np.random.default_rng(99)
    params = _libs.mlp_params(rng, SIZES)
    xs = rng.standard_normal((2, GLOBAL_B, SIZES[0])).astype(np.float32)
    ts = rng.integers(0, SIZES[-1], (2, GLOBAL_B)).astype(np.int32)
    return params, xs, ts


def _worker(rank, world, port, out_dir):
    import _libs
    from origindl_b200 import dp

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    params, xs, ts = _inputs()
    lo, hi = dp.shard_rows(GLOBAL_B, rank, world)

    def hook(grads):
        t = torch.from_numpy(grads)           # shares memory: reduced in place
        dp.allreduce_gradients(t, SIZES)
        grads *= np.float32(1.0 / world)      # what the fused optimizer does with grad_scale

    losses, final, _ = _libs.oracle_mlp_train(SIZES, params, xs[:, lo:hi], ts[:, lo:hi], STEPS, opt="adam", lr=1e-2,
                                              hook_wd=1e-4, grad_hook=hook)
    # the global loss is the mean of the per-rank means
    lt = torch.from_numpy(losses.copy())
    dist.all_reduce(lt)
    np.save(Path(out_dir) / f"params_{rank}.npy", final)
    np.save(Path(out_dir) / f"loss_{rank}.npy", (lt / world).numpy())
    dist.destroy_process_group()


def test_two_rank_data_parallel_equals_full_batch(tmp_path):
    import _libs

    world = 2
    port = 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    params, xs, ts = _inputs()
    ref_losses, ref_params, _ = _libs.oracle_mlp_train(SIZES, params, xs, ts, STEPS, opt="adam", lr=1e-2, hook_wd=1e-4)
    p0, p1 = np.load(tmp_path / "params_0.npy"), np.load(tmp_path / "params_1.npy")
    assert np.array_equal(p0, p1)                                   # replicas stay identical
    assert _libs.max_rel_err(p0, ref_params) <= 1e-5                # and equal the full-batch run up to fp32 rounding
    assert np.abs(np.load(tmp_path / "loss_0.npy") - ref_losses).max() <= 1e-5


def test_plan_helpers():
    from origindl_b200 import dp

    assert dp.shard_rows(65536, 3, 8) == (24576, 32768)
    with pytest.raises(ValueError):
        dp.shard_rows(10, 0, 4)
    b = dp.layer_buckets_packed([784, 1000, 1000, 10])
    assert b[0] == (0, 785000) and b[-1][0] + b[-1][1] == 784 * 1000 + 1000 + 1000 * 1000 + 1000 + 10010
    assert dp.reduce_order(3) == [2, 1, 0]


def test_epoch_order_shards_cover_the_epoch_once():
    """DataLoader(shard=(rank, world)): all ranks draw the same permutation and take interleaved positions of it."""
    import numpy as np

    from origindl_b200 import dp

    order = np.random.default_rng(3).permutation(103)
    shards = [dp.shard_epoch_order(order, r, 4) for r in range(4)]
    assert all(len(s) == 25 for s in shards)                       # 103 -> 100 kept, equally many per rank
    assert np.array_equal(np.sort(np.concatenate(shards)), np.sort(order[:100]))
    assert np.array_equal(shards[1], order[1:100:4])
    import pytest

    with pytest.raises(ValueError):
        dp.shard_epoch_order(order, 4, 4)
