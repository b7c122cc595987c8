"""Generate tests/golden/reference_vectors.npz by running the UNMODIFIED reference (oracle/_ref/libodl_ref.so).

Needs the reference tree (to build the library); the produced file is committed so that the GPU box, where the
tree does not exist, can still check the CUDA path against numbers that came out of the reference itself.
Inputs are seeded numpy draws with the shapes and distributions of the benchmark configurations (synthetic data;
no dataset is involved).  Run:  python tests/golden/make_golden.py [--c1-steps 200]
"""
import argparse
import ctypes
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import _libs  # noqa: E402

OUT = Path(__file__).resolve().parent / "reference_vectors.npz"
fptr = _libs.fptr


def c1_inputs(n_batches=4, B=512, sizes=(784, 1000, 1000, 10), seed=42):
    """MNIST-shaped MLP configuration: X ~ U[0,1), labels ~ U{0..9}, Kaiming-uniform weights, zero biases."""
    rng = np.random.default_rng(seed)
    params = _libs.mlp_params(rng, sizes)
    x = rng.uniform(0, 1, (n_batches, B, sizes[0])).astype(np.float32)
    t = rng.integers(0, sizes[-1], size=(n_batches, B)).astype(np.int32)
    return params, x, t


def stable_inputs(n_batches=4, B=256, sizes=(784, 256, 256, 10), seed=42):
    """A well-conditioned 200-step configuration: MNIST-shaped inputs, labels from a fixed random linear teacher
    (so the loss falls smoothly), trained with SGD lr 0.003 momentum 0.9."""
    rng = np.random.default_rng(seed)
    params = _libs.mlp_params(rng, sizes)
    x = rng.uniform(0, 1, (n_batches, B, sizes[0])).astype(np.float32)
    teacher = rng.standard_normal((sizes[0], sizes[-1])).astype(np.float32)
    t = np.argmax((x - 0.5) @ teacher, axis=-1).astype(np.int32)
    return params, x, t


def mlp_curve_float64(sizes, params, xs, ts, steps, opt, lr, momentum=0.0, hook_wd=0.0):
    """The same training step in float64 numpy (exact-arithmetic yardstick: how far does a run that makes NO fp32
    rounding error drift from the reference's fp32 curve?)."""
    sizes = [int(v) for v in sizes]
    L = len(sizes) - 1
    p = params.astype(np.float64)
    views, off = [], 0
    for l in range(L):
        nw, nb = sizes[l] * sizes[l + 1], sizes[l + 1]
        views.append((slice(off, off + nw), slice(off + nw, off + nw + nb)))
        off += nw + nb
    m, v = np.zeros_like(p), np.zeros_like(p)
    B = xs.shape[1]
    losses = []
    for s in range(steps):
        x, t = xs[s % len(xs)].astype(np.float64), ts[s % len(ts)]
        acts = [x]
        for l, (ws, bs) in enumerate(views):
            y = acts[-1] @ p[ws].reshape(sizes[l], sizes[l + 1]) + p[bs]
            acts.append(np.maximum(y, 0) if l + 1 < L else y)
        z = acts[-1] - acts[-1].max(1, keepdims=True)
        pr = np.exp(z) / np.exp(z).sum(1, keepdims=True)
        losses.append(-np.log(pr[np.arange(B), t] + 1e-8).sum() / B)
        g = pr.copy()
        g[np.arange(B), t] -= 1
        g /= B
        grads = np.zeros_like(p)
        for l in range(L - 1, -1, -1):
            ws, bs = views[l]
            if l + 1 < L:
                g = g * (acts[l + 1] > 0)
            grads[ws] = (acts[l].T @ g).ravel()
            grads[bs] = g.sum(0)
            g = g @ p[ws].reshape(sizes[l], sizes[l + 1]).T
        grads += hook_wd * p
        if opt == "adam":
            m = 0.9 * m + 0.1 * grads
            v = 0.999 * v + 0.001 * grads * grads
            p = p - lr * (m / (1 - 0.9 ** (s + 1))) / (np.sqrt(v / (1 - 0.999 ** (s + 1))) + 1e-8)
        else:
            m = momentum * m + grads
            p = p - lr * m
    return np.array(losses, np.float64)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--c1-steps", type=int, default=200)
    ap.add_argument("--reuse", action="store_true", help="keep arrays already in the output file, add missing ones")
    args = ap.parse_args()
    ref = _libs.reference()
    if ref is None:
        raise SystemExit("reference library unavailable")
    out = {}
    have = dict(np.load(OUT)) if (args.reuse and OUT.exists()) else {}

    # ---- Linear forward + backward, both weight layouts, with ReLU (N(0,1) inputs, b ~ N(0,0.1))
    for tag, (M, N, K) in {"lin_a": (96, 80, 72), "lin_b": (130, 33, 257)}.items():
        for w_layout in (0, 1):
            rng = np.random.default_rng(1000 + M + w_layout)
            x = rng.standard_normal((M, K), dtype=np.float32)
            w = rng.standard_normal((N, K) if w_layout == 0 else (K, N), dtype=np.float32)
            b = (0.1 * rng.standard_normal(N)).astype(np.float32)
            dy = rng.standard_normal((M, N), dtype=np.float32)
            y, dx, dw, db = np.empty((M, N), np.float32), np.empty_like(x), np.empty_like(w), np.empty(N, np.float32)
            _libs.ref_check(ref.odlref_linear_fwd_bwd(x, w, fptr(b), fptr(dy), M, N, K, w_layout, 1, y, fptr(dx),
                                                      fptr(dw), fptr(db)))
            k = f"{tag}_l{w_layout}_"
            out.update({k + "x": x, k + "w": w, k + "b": b, k + "dy": dy, k + "y": y, k + "dx": dx, k + "dw": dw,
                        k + "db": db})

    # ---- softmax cross-entropy
    rng = np.random.default_rng(3)
    x = (2 * rng.standard_normal((64, 1000))).astype(np.float32)
    t = rng.integers(0, 1000, 64).astype(np.int32)
    loss, d = ctypes.c_float(), np.empty_like(x)
    _libs.ref_check(ref.odlref_softmax_ce(x, t, 64, 1000, ctypes.byref(loss), fptr(d)))
    out.update({"ce_x": x, "ce_t": t, "ce_loss": np.float32(loss.value), "ce_dx": d})

    # ---- optimizer trajectories (7 steps from zero state)
    rng = np.random.default_rng(4)
    p0 = rng.standard_normal(1000).astype(np.float32)
    grads = rng.standard_normal((7, 1000)).astype(np.float32)
    out.update({"opt_p0": p0, "opt_grads": grads})
    for tag, (opt, lr, mom, swd, nes, hwd) in {"adam_wd": (1, 1e-3, 0.0, 0.0, 0, 1e-4), "sgd_mom": (0, 1e-2, 0.9, 0.0, 0, 0.0),
                                               "sgd_nes_wd": (0, 1e-2, 0.9, 1e-2, 1, 0.0)}.items():
        p = p0.copy()
        _libs.ref_check(ref.odlref_optim_replay(p, grads, 1000, 7, opt, lr, mom, swd, nes, hwd))
        out["opt_" + tag] = p

    # ---- conv2d forward + backward as the reference computes them (3 -> 8 channels, k3 s2 p1)
    rng = np.random.default_rng(5)
    N, C, H, W, OC, k, s, p = 2, 3, 16, 16, 8, 3, 2, 1
    x = rng.uniform(0, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = (0.1 * rng.standard_normal(OC)).astype(np.float32)
    OH = (H + 2 * p - k) // s + 1
    dy = rng.standard_normal((N, OC, OH, OH)).astype(np.float32)
    y, dx, dw, db = np.empty_like(dy), np.empty_like(x), np.empty_like(w), np.empty_like(b)
    _libs.ref_check(ref.odlref_conv2d_fwd_bwd(x, w, fptr(b), fptr(dy), N, C, H, W, OC, k, k, s, p, y, fptr(dx), fptr(dw),
                                              fptr(db)))
    out.update({"conv_x": x, "conv_w": w, "conv_b": b, "conv_dy": dy, "conv_y": y, "conv_dx_reflayout": dx,
                "conv_dw_reflayout": dw, "conv_db": db, "conv_cfg": np.array([N, C, H, W, OC, k, s, p], np.int32)})

    # ---- small MLP training runs (both optimizers), losses + final parameters
    sizes = np.array([20, 48, 32, 10], np.int32)
    rng = np.random.default_rng(6)
    params0 = _libs.mlp_params(rng, sizes)
    xs = rng.uniform(0, 1, (3, 16, 20)).astype(np.float32)
    ts = rng.integers(0, 10, (3, 16)).astype(np.int32)
    out.update({"mlp_sizes": sizes, "mlp_params0": params0, "mlp_x": xs, "mlp_t": ts})
    for tag, (opt, lr, mom, hwd) in {"adam": (1, 1e-3, 0.0, 1e-4), "sgd": (0, 5e-2, 0.9, 0.0)}.items():
        params = params0.copy()
        losses = np.empty(12, np.float32)
        grads = np.empty_like(params)
        _libs.ref_check(ref.odlref_mlp_train(sizes, len(sizes), params, xs, ts, 16, 3, 12, opt, lr, mom, hwd, losses,
                                             fptr(grads)))
        out.update({f"mlp_{tag}_losses": losses, f"mlp_{tag}_params": params, f"mlp_{tag}_lastgrads": grads})

    # ---- the MNIST-shaped configuration: loss curve of the reference over --c1-steps Adam steps (lr 1e-3, wd 1e-4)
    if "c1_losses" in have:
        out.update({"c1_losses": have["c1_losses"], "c1_param_sample": have["c1_param_sample"]})
    elif args.c1_steps > 0:
        sizes = np.array([784, 1000, 1000, 10], np.int32)
        params, x, t = c1_inputs()
        losses = np.empty(args.c1_steps, np.float32)
        _libs.ref_check(ref.odlref_mlp_train(sizes, 4, params, x, t, 512, 4, args.c1_steps, 1, 1e-3, 0.0, 1e-4, losses,
                                             None))
        # final parameters are 1.8 M floats; keep a strided sample (every 257th) for a cheap check
        out.update({"c1_losses": losses, "c1_param_sample": params[::257].copy()})
    if "c1_losses" in out and "c1_losses_fp64" not in have:
        params, x, t = c1_inputs()
        out["c1_losses_fp64"] = mlp_curve_float64([784, 1000, 1000, 10], params, x, t, len(out["c1_losses"]), "adam", 1e-3,
                                                  hook_wd=1e-4)
    elif "c1_losses_fp64" in have:
        out["c1_losses_fp64"] = have["c1_losses_fp64"]

    # ---- sensitivity of the REFERENCE ITSELF on that configuration: the same run with one input element moved by one
    #      unit in the last place.  The spread between the two reference curves is the yardstick for "how close can any
    #      implementation that is not bit-identical stay to the reference's curve" on this (random-label) problem.
    if "c1_losses_ulp" in have:
        out["c1_losses_ulp"] = have["c1_losses_ulp"]
    elif "c1_losses" in out:
        sizes = np.array([784, 1000, 1000, 10], np.int32)
        params, x, t = c1_inputs()
        x[0, 0, 0] = np.nextafter(x[0, 0, 0], np.float32(2.0))
        losses = np.empty(len(out["c1_losses"]), np.float32)
        _libs.ref_check(ref.odlref_mlp_train(sizes, 4, params, x, t, 512, 4, len(losses), 1, 1e-3, 0.0, 1e-4, losses, None))
        out["c1_losses_ulp"] = losses

    # ---- the well-conditioned 200-step configuration (SGD momentum, teacher labels)
    if "stable_losses" in have:
        out.update({k: have[k] for k in ("stable_losses", "stable_param_sample")})
    else:
        sizes = np.array([784, 256, 256, 10], np.int32)
        params, x, t = stable_inputs()
        losses = np.empty(200, np.float32)
        _libs.ref_check(ref.odlref_mlp_train(sizes, 4, params, x, t, 256, 4, 200, 0, 3e-3, 0.9, 0.0, losses, None))
        out.update({"stable_losses": losses, "stable_param_sample": params[::101].copy()})
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
