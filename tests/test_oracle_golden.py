"""CPU: the oracle against the committed golden vectors (outputs of the unmodified reference, tests/golden/) and the
known-answer cases transcribed from the reference's unit tests.  Runs anywhere (no reference tree, no GPU)."""
import ctypes
import json
from pathlib import Path

import numpy as np

import _libs
from _libs import fptr

GOLDEN = Path(__file__).resolve().parent / "golden"
orc = _libs.oracle()


def test_known_answers():
    ka = json.loads((GOLDEN / "known_answers.json").read_text())
    for c in ka["matmul"]:
        out = np.empty((c["M"], c["N"]), np.float32)
        orc.oracle_matmul(np.array(c["a"], np.float32), np.array(c["b"], np.float32), out, c["M"], c["N"], c["K"])
        assert np.allclose(out.ravel(), c["c"], atol=1e-3), c["source"]
    for c in ka["matmul_backward_ones"]:
        M, N, K = c["M"], c["N"], c["K"]
        a, b = np.array(c["a"], np.float32).reshape(M, K), np.array(c["b"], np.float32).reshape(K, N)
        gy, ga, gb = np.ones((M, N), np.float32), np.empty((M, K), np.float32), np.empty((K, N), np.float32)
        # y = a . b with nn::Linear-style weight b {K,N}: dx = gy . b^T, dw = a^T . gy
        orc.oracle_linear_backward(a, b, None, gy, fptr(ga), fptr(gb), None, M, N, K, 1, 0)
        assert np.allclose(ga.ravel(), c["ga"], atol=1e-3) and np.allclose(gb.ravel(), c["gb"], atol=1e-3)
    for c in ka["custom_linear"]:
        y = np.empty((c["M"], c["N"]), np.float32)
        b = None if c["b"] is None else np.array(c["b"], np.float32)
        orc.oracle_linear_forward(np.array(c["x"], np.float32), np.array(c["w"], np.float32), fptr(b), y, c["M"], c["N"],
                                  c["K"], 0, 0)
        assert np.allclose(y.ravel(), c["y"], atol=1e-3), c["source"]
    for c in ka["softmax_ce"]:
        loss = ctypes.c_float()
        assert orc.oracle_softmax_ce(np.array(c["x"], np.float32), np.array(c["t"], np.int32), c["B"], c["C"],
                                     ctypes.byref(loss), None) == 0
        assert abs(loss.value - c["loss"]) < c["tol"]
    for c in ka["conv2d_forward"]:
        OH = (c["H"] - c["KH"] + 2 * c["pad"]) // c["stride"] + 1
        OW = (c["W"] - c["KW"] + 2 * c["pad"]) // c["stride"] + 1
        y = np.empty((c["N"], c["OC"], OH, OW), np.float32)
        b = None if c["b"] is None else np.array(c["b"], np.float32)
        orc.oracle_conv2d_forward(np.array(c["x"], np.float32), np.array(c["w"], np.float32), fptr(b), y, c["N"], c["C"],
                                  c["H"], c["W"], c["OC"], c["KH"], c["KW"], c["stride"], c["pad"])
        assert np.allclose(y.ravel(), c["y"], atol=1e-3), c["source"]
    for c in ka["weight_decay_hook"]:
        p, g = np.array(c["p"], np.float32), np.array(c["g"], np.float32)
        orc.oracle_sgd_step(p, g, None, 1, 0.01, 0.0, 0.0, 0, c["rate"])
        assert np.allclose(g, c["g_after"], atol=1e-5)


def test_golden_linear_and_loss_bit_exact():
    g = np.load(GOLDEN / "reference_vectors.npz")
    for tag in ("lin_a", "lin_b"):
        for wl in (0, 1):
            k = f"{tag}_l{wl}_"
            x, w, b, dy = g[k + "x"], g[k + "w"], g[k + "b"], g[k + "dy"]
            M, K = x.shape
            N = dy.shape[1]
            y, dx, dw, db = np.empty((M, N), np.float32), np.empty_like(x), np.empty_like(w), np.empty(N, np.float32)
            orc.oracle_linear_forward(x, w, fptr(b), y, M, N, K, wl, 1)
            orc.oracle_linear_backward(x, w, fptr(y), dy, fptr(dx), fptr(dw), fptr(db), M, N, K, wl, 1)
            assert np.array_equal(y, g[k + "y"]) and np.array_equal(dx, g[k + "dx"])
            assert np.array_equal(dw, g[k + "dw"]) and np.array_equal(db, g[k + "db"].ravel())
    loss, d = ctypes.c_float(), np.empty_like(g["ce_x"])
    orc.oracle_softmax_ce(g["ce_x"], g["ce_t"], 64, 1000, ctypes.byref(loss), fptr(d))
    assert loss.value == float(g["ce_loss"]) and np.array_equal(d, g["ce_dx"])


def test_golden_mlp_training_bit_exact():
    g = np.load(GOLDEN / "reference_vectors.npz")
    for tag, kw in {"adam": dict(opt="adam", lr=1e-3, hook_wd=1e-4), "sgd": dict(opt="sgd", lr=5e-2, momentum=0.9)}.items():
        losses, params, grads = _libs.oracle_mlp_train(g["mlp_sizes"], g["mlp_params0"], g["mlp_x"], g["mlp_t"], 12, **kw)
        assert np.array_equal(losses, g[f"mlp_{tag}_losses"]), tag
        assert np.array_equal(params, g[f"mlp_{tag}_params"]), tag


def test_golden_c1_curve_prefix():
    """First steps of the MNIST-shaped 200-step reference curve (the full curve is the GPU test's target)."""
    from golden.make_golden import c1_inputs

    g = np.load(GOLDEN / "reference_vectors.npz")
    params, x, t = c1_inputs()
    losses, _, _ = _libs.oracle_mlp_train([784, 1000, 1000, 10], params, x, t, 2, opt="adam", lr=1e-3, hook_wd=1e-4)
    assert np.array_equal(losses, g["c1_losses"][:2])
    assert abs(float(g["c1_losses"][0]) - np.log(10)) < 0.5   # untrained 10-class model


def test_reference_is_chaotic_on_the_mnist_shaped_configuration():
    """The sensitivity yardstick in the golden file, made by the unmodified reference itself: its 200-step curve with one
    input element moved by one unit in the last place agrees with the original for the first steps (same program, same
    seeds), then leaves the 1e-3 band before step 30 and ends far outside it -- so "within 1e-3 over 200 steps" on this
    configuration can only be met by a bit-identical implementation, and the GPU test holds the CUDA path to the
    reference's own spread instead."""
    g = np.load(GOLDEN / "reference_vectors.npz")
    ref, ulp = g["c1_losses"], g["c1_losses_ulp"]
    assert len(ref) == len(ulp) == 200
    spread = np.abs(ref - ulp)
    assert spread[:4].max() == 0.0                     # a 1-ulp change of one of 401 408 inputs is invisible at first
    assert spread[:10].max() <= 1e-3
    first_out = int(np.nonzero(spread > 1e-3)[0][0])
    assert 10 < first_out < 30
    assert spread.max() > 0.1
