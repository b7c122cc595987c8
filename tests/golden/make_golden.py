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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--c1-steps", type=int, default=200)
    args = ap.parse_args()
    ref = _libs.reference()
    if ref is None:
        raise SystemExit("reference library unavailable")
    out = {}

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
    if args.c1_steps > 0:
        sizes = np.array([784, 1000, 1000, 10], np.int32)
        params, x, t = c1_inputs()
        losses = np.empty(args.c1_steps, np.float32)
        _libs.ref_check(ref.odlref_mlp_train(sizes, 4, params, x, t, 512, 4, args.c1_steps, 1, 1e-3, 0.0, 1e-4, losses,
                                             None))
        # final parameters are 1.8 M floats; keep a strided sample (every 257th) for a cheap check
        out.update({"c1_losses": losses, "c1_param_sample": params[::257].copy()})
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
