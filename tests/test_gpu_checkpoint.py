"""GPU: state dict and checkpoint of the device-resident MLP (MLPTrainer.state_dict / save_checkpoint / load_checkpoint).

The reference's checkpoint holds the parameters only (its optimizer.odl is never written), so a resumed reference run
restarts Adam from zero moments; here the moments and the step count travel too and a resumed run continues the SAME
trajectory, which is what these tests pin."""
from pathlib import Path

import numpy as np
import pytest
import torch

import _libs
from golden import make_odl_fixtures as fx

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
SIZES, BATCH = [48, 64, 40, 10], 32


@pytest.fixture(scope="module")
def trainer_cls():
    from origindl_b200 import capi
    from origindl_b200.trainer import MLPTrainer

    capi.init(0)
    yield MLPTrainer
    capi.device_status()


def batches(n):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((n, BATCH, SIZES[0])).astype(np.float32)
    t = rng.integers(0, SIZES[-1], (n, BATCH)).astype(np.int32)
    return torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()


def steps(tr, x, t, lo, hi):
    return np.array([tr.train_step(x[s], t[s]).item() for s in range(lo, hi)], np.float32)


@pytest.mark.parametrize("kw", [dict(optimizer="adam", lr=1e-3, hook_weight_decay=1e-4),
                                dict(optimizer="sgd", lr=5e-2, momentum=0.9)])
def test_resume_continues_the_same_trajectory(trainer_cls, tmp_path, kw):
    x, t = batches(12)
    a = trainer_cls(SIZES, BATCH, **kw)
    a.set_params(_libs.mlp_params(np.random.default_rng(3), SIZES))
    steps(a, x, t, 0, 6)
    path = str(tmp_path / "run_epoch_1.ckpt")
    d = Path(a.save_checkpoint(path, epoch=1, step=6, loss=0.25))
    assert (d / "model.odl").exists() and (d / "optimizer.odl").exists() and (d / "metadata.json").exists()
    tail_a = steps(a, x, t, 6, 12)

    b = trainer_cls(SIZES, BATCH, **kw)
    ck = b.load_checkpoint(path)
    assert (ck.epoch, ck.step, ck.optimizer_type) == (1, 6, {"adam": "Adam", "sgd": "SGD"}[kw["optimizer"]])
    assert ck.optimizer_config["lr"] == pytest.approx(kw["lr"])
    tail_b = steps(b, x, t, 6, 12)
    # same kernels, same inputs, same state: bit-identical continuation
    assert np.array_equal(tail_a, tail_b)
    assert np.array_equal(a.get_params(), b.get_params())

    # what the reference's own checkpoint gives: parameters only -> the optimizer restarts and the run drifts
    c = trainer_cls(SIZES, BATCH, **kw)
    c.load_state_dict(ck.model_state_dict)
    tail_c = steps(c, x, t, 6, 12)
    assert tail_c[0] == tail_a[0]  # the first loss depends on the parameters only
    assert not np.array_equal(tail_c[1:], tail_a[1:])
    for tr in (a, b, c):
        tr.close()


def test_state_dict_names_shapes_and_strictness(trainer_cls):
    tr = trainer_cls(SIZES, BATCH)
    packed = _libs.mlp_params(np.random.default_rng(4), SIZES)
    tr.set_params(packed)
    sd = tr.state_dict()
    assert list(sd) == [f"layer_{i}.{p}" for i in range(3) for p in ("weight", "bias")]
    assert sd["layer_0.weight"].shape == (48, 64) and sd["layer_2.bias"].shape == (1, 10)
    assert np.array_equal(np.concatenate([v.ravel() for v in sd.values()]), packed)
    with pytest.raises(RuntimeError, match="Missing parameter 'layer_1.bias'"):
        tr.load_state_dict({k: v for k, v in sd.items() if k != "layer_1.bias"})
    with pytest.raises(RuntimeError, match="Unexpected parameter 'extra'"):
        tr.load_state_dict({**sd, "extra": np.zeros((1, 1), np.float32)})
    with pytest.raises(RuntimeError, match="Shape mismatch for parameter 'layer_0.weight'"):
        tr.load_state_dict({**sd, "layer_0.weight": np.zeros((64, 48), np.float32)})
    # non-strict: missing names keep their values, the rest is replaced
    tr.load_state_dict({"layer_1.bias": np.full((1, 40), 2.0, np.float32)}, strict=False)
    sd2 = tr.state_dict()
    assert np.all(sd2["layer_1.bias"] == 2.0) and np.array_equal(sd2["layer_0.weight"], sd["layer_0.weight"])
    tr.close()


def test_loads_a_checkpoint_written_by_the_reference(trainer_cls):
    """tests/golden/ref_checkpoint is origin::save(Checkpoint) of an nn::MLP({4, 8, 2}) by the unmodified reference."""
    tr = trainer_cls(fx.CKPT_SIZES, 8)
    ck = tr.load_checkpoint(str(GOLDEN / "ref_checkpoint.ckpt"))
    assert ck.epoch == fx.CKPT_META["epoch"] and ck.optimizer_state_dict == {}
    assert np.array_equal(tr.get_params(), fx.checkpoint_params())
    # and the forward pass uses them: logits of the oracle's Linear chain on the same parameters
    x = np.random.default_rng(1).standard_normal((8, 4)).astype(np.float32)
    t = np.zeros(8, np.int32)
    _libs.oracle()  # builds the checker on demand
    losses, _, _ = _libs.oracle_mlp_train(fx.CKPT_SIZES, fx.checkpoint_params(), x[None], t[None], 1, opt="sgd", lr=0.0)
    got = tr.train_step(torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()).item()
    assert abs(got - losses[0]) <= 1e-5
    tr.close()
