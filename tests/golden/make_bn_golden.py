"""Golden outputs of the UNMODIFIED reference for BatchNorm (+ReLU / SiLU), nn::BatchNorm2d's running statistics and
SiLU, written to tests/golden/reference_bn_vectors.npz.  Inputs are functions of fixed seeds (`case_inputs`), so only
the reference's OUTPUTS are stored.  Run where the reference library is built:  python tests/golden/make_bn_golden.py

What the reference can and cannot produce (observed through its public API):
* forward in training and evaluation mode, with the batch mean / biased variance in training mode;
* backward ONLY after an evaluation-mode forward: in training mode the operator returns three outputs and its own
  backward then throws "BatchNorm backward requires exactly 1 gradient, but got 3"
  (src/operators/normalization/batch_norm.cpp:78-92).  The backward arithmetic (cpu::batch_norm_backward) is the same
  in both modes, so the evaluation-mode vectors pin it.
"""
from __future__ import annotations

import ctypes
import sys
from ctypes import c_float, c_int, c_int64
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

# name: (N, C, HW)
CASES = {"bn2d_small": (4, 3, 10), "bn2d_conv": (2, 16, 400), "bn1d": (32, 5, 1), "bn2d_single_channel": (3, 1, 7)}
ACTS = {"none": 0, "relu": 1, "silu": 2}
EPS = 1e-5


def case_inputs(name: str) -> dict:
    n, c, hw = CASES[name]
    rng = np.random.default_rng(sum(map(ord, name)))  # a seed that depends on the case name only
    return {
        "x": (rng.standard_normal((n, c, hw)) * 2.0 + rng.standard_normal((1, c, 1))).astype(np.float32),
        "gamma": (1.0 + 0.5 * rng.standard_normal(c)).astype(np.float32),
        "beta": (0.3 * rng.standard_normal(c)).astype(np.float32),
        "running_mean": (0.2 * rng.standard_normal(c)).astype(np.float32),
        "running_var": (0.5 + rng.random(c)).astype(np.float32),
        "dy": rng.standard_normal((n, c, hw)).astype(np.float32),
    }


def layer_inputs() -> dict:
    rng = np.random.default_rng(99)
    n, c, hw, steps = 4, 6, 25, 3
    return {"xs": (rng.standard_normal((steps, n, c, hw)) * 1.5 + 0.7).astype(np.float32),
            "probe": rng.standard_normal((n, c, hw)).astype(np.float32), "steps": steps, "momentum": 0.1}


def silu_inputs() -> dict:
    rng = np.random.default_rng(3)
    return {"x": np.concatenate([rng.standard_normal(200) * 3, [0.0, -20.0, 20.0, -88.0, 50.0]]).astype(np.float32),
            "dy": rng.standard_normal(205).astype(np.float32)}


def declare(ref) -> None:
    f = np.ctypeslib.ndpointer(np.float32, flags="C")
    p = ctypes.c_void_p
    ref.odlref_batch_norm_fwd_bwd.argtypes = [f, f, f, f, f, c_int, c_float, c_int64, c_int64, c_int64, c_int, p, f, p, p,
                                              p, p, p]
    ref.odlref_batch_norm2d_layer.argtypes = [f, c_int, f, c_int64, c_int64, c_int64, c_float, c_float, f]
    ref.odlref_silu_fwd_bwd.argtypes = [f, p, c_int64, f, p]


def vp(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def ref_batch_norm(ref, inp: dict, training: bool, act: int, backward: bool) -> dict:
    from _libs import ref_check

    n, c, hw = inp["x"].shape
    y, gx = np.empty_like(inp["x"]), np.empty_like(inp["x"])
    mean, var, dg, db = (np.zeros(c, np.float32) for _ in range(4))
    ref_check(ref.odlref_batch_norm_fwd_bwd(inp["x"], inp["gamma"], inp["beta"], inp["running_mean"], inp["running_var"],
                                            int(training), EPS, n, c, hw, act, vp(inp["dy"]) if backward else None, y,
                                            vp(mean), vp(var), vp(gx) if backward else None, vp(dg) if backward else None,
                                            vp(db) if backward else None))
    out = {"y": y}
    if training:
        out.update(mean=mean, var=var)
    if backward:
        out.update(gx=gx, dgamma=dg, dbeta=db)
    return out


def ref_layer(ref, inp: dict) -> np.ndarray:
    from _libs import ref_check

    steps, n, c, hw = inp["xs"].shape
    y = np.empty((n, c, hw), np.float32)
    ref_check(ref.odlref_batch_norm2d_layer(inp["xs"], steps, inp["probe"], n, c, hw, EPS, inp["momentum"], y))
    return y


def ref_silu(ref, inp: dict):
    from _libs import ref_check

    y, gx = np.empty_like(inp["x"]), np.empty_like(inp["x"])
    ref_check(ref.odlref_silu_fwd_bwd(inp["x"], vp(inp["dy"]), inp["x"].size, y, vp(gx)))
    return y, gx


def main() -> None:
    from _libs import reference

    ref = reference()
    if ref is None or not hasattr(ref, "odlref_batch_norm_fwd_bwd"):
        raise SystemExit("the reference library (make -C oracle ref) is needed to write the vectors")
    declare(ref)
    out = {}
    for name in CASES:
        inp = case_inputs(name)
        for act_name, act in ACTS.items():
            for k, v in ref_batch_norm(ref, inp, True, act, False).items():
                out[f"{name}/train/{act_name}/{k}"] = v
            for k, v in ref_batch_norm(ref, inp, False, act, True).items():
                out[f"{name}/eval/{act_name}/{k}"] = v
    out["layer/y"] = ref_layer(ref, layer_inputs())
    out["silu/y"], out["silu/gx"] = ref_silu(ref, silu_inputs())
    np.savez_compressed(HERE / "reference_bn_vectors.npz", **out)
    print("wrote", HERE / "reference_bn_vectors.npz", f"({len(out)} arrays)")


if __name__ == "__main__":
    main()
