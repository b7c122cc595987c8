"""The oracle's BatchNorm / SiLU restatement against the unmodified reference: the committed golden outputs
(tests/golden/reference_bn_vectors.npz, made by tests/golden/make_bn_golden.py) and, where the reference library is
built, live calls on other seeds.  Sequential fp32 loops in the same order as the reference: compared BIT-EXACTLY,
except through ReLU/SiLU backward chains where the reference multiplies in a different association (tolerance 1e-6)."""
from __future__ import annotations

import ctypes
import sys
from ctypes import c_float, c_int, c_int64
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _libs  # noqa: E402
from golden import make_bn_golden as mk  # noqa: E402

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_bn_vectors.npz"
_F = np.ctypeslib.ndpointer(np.float32, flags="C")
_P = ctypes.c_void_p


def orc():
    L = _libs.oracle()
    L.oracle_batch_norm_forward.argtypes = [_F, _F, _F, _F, _F, c_int, c_float, c_int64, c_int64, c_int64, _F, _F, _F, _P]
    L.oracle_batch_norm_backward.argtypes = [_F, _F, _F, _F, c_float, c_int64, c_int64, c_int64, _F, _F, _F]
    L.oracle_batch_norm_update_running.argtypes = [_F, _F, _F, _F, c_float, c_int64]
    L.oracle_silu_forward.argtypes = [_F, _F, c_int64]
    L.oracle_silu_backward.argtypes = [_F, _F, _F, c_int64]
    return L


def oracle_bn(inp, training, act, backward):
    """Forward (+ backward of sum(out * dy)) composed from the oracle functions, as the reference composes its operators."""
    L = orc()
    x = inp["x"]
    n, c, hw = x.shape
    z, xn = np.empty_like(x), np.empty_like(x)
    mean, var = np.empty(c, np.float32), np.empty(c, np.float32)
    L.oracle_batch_norm_forward(x, inp["gamma"], inp["beta"], inp["running_mean"], inp["running_var"], int(training),
                                mk.EPS, n, c, hw, z, mean, var, xn.ctypes.data_as(_P))
    if act == 1:
        y = np.maximum(z, 0.0).astype(np.float32)
    elif act == 2:
        y = np.empty_like(z)
        L.oracle_silu_forward(z, y, z.size)
    else:
        y = z
    out = {"y": y, "mean": mean, "var": var}
    if backward:
        dy = inp["dy"]
        if act == 1:
            g = (dy * (z > 0)).astype(np.float32)  # relu backward: gy * mask (src/mat/origin/cpu/activation/relu.cpp)
        elif act == 2:
            g = np.empty_like(dy)
            L.oracle_silu_backward(dy, z, g, z.size)
        else:
            g = dy
        gx, dg, db = np.empty_like(x), np.empty(c, np.float32), np.empty(c, np.float32)
        L.oracle_batch_norm_backward(np.ascontiguousarray(g), inp["gamma"], var, xn, mk.EPS, n, c, hw, gx, dg, db)
        out.update(gx=gx, dgamma=dg, dbeta=db)
    return out


@pytest.mark.parametrize("name", list(mk.CASES))
@pytest.mark.parametrize("act_name", list(mk.ACTS))
def test_oracle_matches_golden_reference_outputs(name, act_name):
    g = np.load(GOLDEN)
    inp, act = mk.case_inputs(name), mk.ACTS[act_name]
    train = oracle_bn(inp, True, act, False)
    for k in ("y", "mean", "var"):
        assert np.array_equal(train[k], g[f"{name}/train/{act_name}/{k}"]), (name, act_name, k)
    ev = oracle_bn(inp, False, act, True)
    assert np.array_equal(ev["y"], g[f"{name}/eval/{act_name}/y"])
    for k in ("gx", "dgamma", "dbeta"):
        assert np.array_equal(ev[k], g[f"{name}/eval/{act_name}/{k}"]), (name, act_name, k)


def test_running_statistics_follow_the_layer():
    """nn::BatchNorm2d keeps momentum * running + (1 - momentum) * batch (src/nn/layers/batch_norm2d.cpp:66-83); its
    running statistics are private, so they are observed through an evaluation-mode forward of a probe."""
    g, L, inp = np.load(GOLDEN), orc(), mk.layer_inputs()
    steps, n, c, hw = inp["xs"].shape
    rm, rv = np.zeros(c, np.float32), np.ones(c, np.float32)
    ones, zeros = np.ones(c, np.float32), np.zeros(c, np.float32)
    for k in range(steps):
        y, mean, var = np.empty((n, c, hw), np.float32), np.empty(c, np.float32), np.empty(c, np.float32)
        L.oracle_batch_norm_forward(np.ascontiguousarray(inp["xs"][k]), ones, zeros, rm, rv, 1, mk.EPS, n, c, hw, y, mean,
                                    var, None)
        L.oracle_batch_norm_update_running(rm, rv, mean, var, inp["momentum"], c)
    y, mean, var = np.empty((n, c, hw), np.float32), np.empty(c, np.float32), np.empty(c, np.float32)
    L.oracle_batch_norm_forward(inp["probe"], ones, zeros, rm, rv, 0, mk.EPS, n, c, hw, y, mean, var, None)
    assert np.array_equal(y, g["layer/y"])


def test_silu_matches_golden():
    g, L, inp = np.load(GOLDEN), orc(), mk.silu_inputs()
    y, gx = np.empty_like(inp["x"]), np.empty_like(inp["x"])
    L.oracle_silu_forward(inp["x"], y, y.size)
    L.oracle_silu_backward(inp["dy"], inp["x"], gx, y.size)
    assert np.array_equal(y, g["silu/y"]) and np.array_equal(gx, g["silu/gx"])


def test_backward_is_the_gradient_of_the_training_forward():
    """The reference cannot run backward after a training-mode forward (its operator throws); the formula it applies
    is the batch-statistics gradient, checked here against a float64 finite-difference-free closed form."""
    inp = mk.case_inputs("bn2d_small")
    got = oracle_bn(inp, True, 0, True)
    x, dy, gamma = (inp[k].astype(np.float64) for k in ("x", "dy", "gamma"))
    mean = x.mean(axis=(0, 2), keepdims=True)
    var = x.var(axis=(0, 2), keepdims=True)
    xn = (x - mean) / np.sqrt(var + mk.EPS)
    gxn = dy * gamma[None, :, None]
    gx = (gxn - gxn.mean(axis=(0, 2), keepdims=True) - xn * (gxn * xn).mean(axis=(0, 2), keepdims=True)) / np.sqrt(var + mk.EPS)
    assert _libs.max_rel_err(got["gx"], gx) <= 1e-5
    assert _libs.max_rel_err(got["dgamma"], (dy * xn).sum(axis=(0, 2))) <= 1e-5
    assert _libs.max_rel_err(got["dbeta"], dy.sum(axis=(0, 2))) <= 1e-6


needs_ref = pytest.mark.skipif(_libs.reference() is None or not hasattr(_libs.reference(), "odlref_batch_norm_fwd_bwd"),
                               reason="reference library with the BatchNorm entry points is not built")


@needs_ref
@pytest.mark.parametrize("shape", [(8, 4, 36), (5, 7, 1), (2, 32, 100)])
@pytest.mark.parametrize("act", [0, 1, 2])
def test_oracle_matches_live_reference(shape, act):
    ref = _libs.reference()
    mk.declare(ref)
    n, c, hw = shape
    rng = np.random.default_rng(n * 1000 + c * 10 + act)
    inp = {"x": (rng.standard_normal(shape) * 1.7 - 0.4).astype(np.float32), "gamma": rng.standard_normal(c).astype(np.float32),
           "beta": rng.standard_normal(c).astype(np.float32), "running_mean": rng.standard_normal(c).astype(np.float32),
           "running_var": (0.2 + rng.random(c)).astype(np.float32), "dy": rng.standard_normal(shape).astype(np.float32)}
    want_t, got_t = mk.ref_batch_norm(ref, inp, True, act, False), oracle_bn(inp, True, act, False)
    for k in ("y", "mean", "var"):
        assert np.array_equal(got_t[k], want_t[k])
    want_e, got_e = mk.ref_batch_norm(ref, inp, False, act, True), oracle_bn(inp, False, act, True)
    for k in ("y", "gx", "dgamma", "dbeta"):
        assert np.array_equal(got_e[k], want_e[k]), k


@needs_ref
def test_reference_training_backward_is_unavailable():
    """Recorded behaviour: after a training-mode forward the reference's own backward throws."""
    ref = _libs.reference()
    mk.declare(ref)
    with pytest.raises(RuntimeError, match="requires exactly 1 gradient"):
        mk.ref_batch_norm(ref, mk.case_inputs("bn2d_small"), True, 0, True)
