"""GPU: the deep, wide MLP benchmark configuration -- batch 8192, six 4096->4096 ReLU layers and a 4096->1000 head with
softmax cross-entropy, Kaiming-uniform weights, SGD with momentum 0.9, 50 steps with the loss curve recorded.

Two legs, both through the C ABI (odl_mlp_*):
* a width/32 twin of the same depth against the oracle (the reference's CPU arithmetic; nn::MLP + SGD,
  src/nn/models/mlp.cpp:11-61, src/optim/sgd.cpp:18-75), every one of the 50 losses within 1e-3 and the final parameters
  within 1e-4;
* the full-size configuration against a plain fp32 statement of the same step (torch matmuls with TF32 off, the
  reference's loss with its +1e-8 inside the log, the reference's momentum rule), where the scalar CPU oracle would need
  hours: 50 losses within 1e-3.
"""
import numpy as np
import pytest
import torch

import _libs
from _libs import max_rel_err

pytestmark = pytest.mark.gpu
MOMENTUM, STEPS = 0.9, 50
# Learning rates at which the 50-step curve is a property of the configuration and not of rounding: with 1e-2 the twin
# memorises its 256 random-label samples, the loss oscillates, and a 1e-6 relative perturbation of the initial
# parameters moves the ORACLE's own curve by 3.5e-3; with 1e-3 that figure is 2e-4.
LR_TWIN, LR = 1e-3, 1e-2


@pytest.fixture(scope="module")
def trainer_cls():
    from origindl_b200 import capi
    from origindl_b200.trainer import MLPTrainer

    capi.init(0)
    yield MLPTrainer
    capi.device_status()


def test_deep_mlp_twin_tracks_the_oracle_for_50_steps(trainer_cls):
    sizes, batch = [128] * 7 + [40], 64
    rng = np.random.default_rng(3)
    params = _libs.mlp_params(rng, sizes)
    xs = rng.standard_normal((4, batch, sizes[0])).astype(np.float32)
    ts = rng.integers(0, sizes[-1], (4, batch)).astype(np.int32)
    want, want_params, _ = _libs.oracle_mlp_train(sizes, params, xs, ts, STEPS, opt="sgd", lr=LR_TWIN,
                                                  momentum=MOMENTUM)
    tr = trainer_cls(sizes, batch, optimizer="sgd", lr=LR_TWIN, momentum=MOMENTUM)
    tr.set_params(params)
    xd, td = torch.from_numpy(xs).cuda(), torch.from_numpy(ts).cuda()
    got = np.array([tr.train_step(xd[s % 4], td[s % 4]).item() for s in range(STEPS)], np.float32)
    assert np.abs(got - np.asarray(want)).max() <= 1e-3
    assert max_rel_err(tr.get_params(), want_params) <= 1e-4
    assert got[-4:].mean() < got[:4].mean()  # and it trains
    tr.close()


def fp32_step(ws, bs, vws, vbs, x, t):
    """One training step in plain fp32: forward, the reference's loss, hand-written backward, momentum SGD."""
    acts, h = [x], x
    for i, (w, b) in enumerate(zip(ws, bs)):
        h = torch.addmm(b, h, w)
        if i + 1 < len(ws):
            h = torch.relu_(h)
        acts.append(h)
    p = torch.softmax(acts[-1], dim=1)
    rows = torch.arange(x.shape[0], device=x.device)
    loss = -(torch.log(p[rows, t] + 1e-8)).sum() / x.shape[0]   # softmax_cross_entropy.cpp:63-73
    g = p
    g[rows, t] -= 1.0
    g /= x.shape[0]
    for i in range(len(ws) - 1, -1, -1):
        gw, gb = acts[i].t() @ g, g.sum(0)
        if i:
            g = (g @ ws[i].t()) * (acts[i] > 0)
        for prm, grad, vel in ((ws[i], gw, vws[i]), (bs[i], gb, vbs[i])):
            vel.mul_(MOMENTUM).add_(grad)        # sgd.cpp:18-75: buf = momentum*buf + g ; p -= lr*buf
            prm.sub_(vel, alpha=LR)
    return loss.item()


def test_deep_mlp_full_size_50_step_curve_against_plain_fp32(trainer_cls):
    sizes, batch = [4096] * 7 + [1000], 8192
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        gen = torch.Generator(device="cuda").manual_seed(50)
        ws, bs = [], []
        for i in range(len(sizes) - 1):
            bound = (6.0 / sizes[i]) ** 0.5
            ws.append((torch.rand(sizes[i], sizes[i + 1], device="cuda", generator=gen) * 2 - 1) * bound)
            bs.append(torch.zeros(sizes[i + 1], device="cuda"))
        xs = torch.randn(2, batch, sizes[0], device="cuda", generator=gen)
        ts = torch.randint(0, sizes[-1], (2, batch), device="cuda", generator=gen)
        packed = torch.cat([v.reshape(-1) for pair in zip(ws, bs) for v in pair]).cpu().numpy()
        tr = trainer_cls(sizes, batch, optimizer="sgd", lr=LR, momentum=MOMENTUM)
        tr.set_params(packed)
        t32 = ts.to(torch.int32)
        got = np.array([tr.train_step(xs[s % 2], t32[s % 2]).item() for s in range(STEPS)], np.float32)
        vws, vbs = [torch.zeros_like(w) for w in ws], [torch.zeros_like(b) for b in bs]
        want = np.array([fp32_step(ws, bs, vws, vbs, xs[s % 2], ts[s % 2]) for s in range(STEPS)], np.float32)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 1e-3, (got[::7], want[::7])
        assert got[-2:].mean() < got[:2].mean()
        print("deep MLP 50 steps: loss %.4f -> %.4f, max |loss - fp32 loss| = %.2e" % (got[0], got[-1], np.abs(got - want).max()))
        # parameters after 50 steps, on a strided sample of the 105 M values: a loose sanity bound (two fp32 trajectories
        # drift apart; the stated tolerance is on the loss curve)
        mine = torch.from_numpy(tr.get_params()[::997]).cuda()
        theirs = torch.cat([v.reshape(-1) for pair in zip(ws, bs) for v in pair])[::997]
        assert ((mine - theirs).abs().max() / theirs.abs().max()).item() <= 1e-2
        tr.close()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
