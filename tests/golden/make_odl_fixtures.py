"""Writes the `.odl` / `.ckpt` fixtures of tests/golden/ with the UNMODIFIED reference (oracle/_ref/libodl_ref.so):

    tests/golden/ref_state.odl          origin::save of a 4-tensor state dict (ranks 1, 2, 2 and 4)
    tests/golden/ref_checkpoint/        origin::save(Checkpoint) of an nn::MLP({4, 8, 2}): model.odl + metadata.json

The tensors are functions of fixed seeds (`state_tensors`, `checkpoint_params`), so the tests rebuild the expected
values without storing them.  Run where the reference tree is mounted:  python tests/golden/make_odl_fixtures.py
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

CKPT_SIZES = [4, 8, 2]
CKPT_META = dict(epoch=5, step=100, loss=0.5, optimizer_type="Adam", lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8)


def state_tensors() -> dict:
    rng = np.random.default_rng(20240611)
    return {
        "layer_0.weight": rng.standard_normal((3, 5)).astype(np.float32),
        "layer_0.bias": rng.standard_normal((1, 5)).astype(np.float32),
        "head.scale": rng.standard_normal((7,)).astype(np.float32),
        "conv.weight": rng.standard_normal((2, 3, 2, 2)).astype(np.float32),
    }


def checkpoint_params() -> np.ndarray:
    rng = np.random.default_rng(77)
    n = sum(CKPT_SIZES[i] * CKPT_SIZES[i + 1] + CKPT_SIZES[i + 1] for i in range(len(CKPT_SIZES) - 1))
    return rng.standard_normal(n).astype(np.float32)


def ref_save_state(ref, path: str, tensors: dict) -> None:
    from _libs import ref_check

    names = list(tensors)
    arrs = [np.ascontiguousarray(tensors[n], np.float32) for n in names]
    c_names = (ctypes.c_char_p * len(names))(*[n.encode() for n in names])
    ranks = np.array([a.ndim for a in arrs], np.int32)
    dims = np.array([d for a in arrs for d in a.shape], np.int64)
    ptrs = (ctypes.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
    ref_check(ref.odlref_save_state(path.encode(), len(names), c_names, ranks, dims, ptrs))


def ref_save_checkpoint(ref, path: str) -> None:
    from _libs import ref_check

    m = CKPT_META
    ref_check(ref.odlref_save_checkpoint(path.encode(), np.array(CKPT_SIZES, np.int32), len(CKPT_SIZES), checkpoint_params(),
                                         m["epoch"], m["step"], m["loss"], m["optimizer_type"].encode(), m["lr"],
                                         m["beta1"], m["beta2"], m["eps"]))


def main() -> None:
    from _libs import reference

    ref = reference()
    if ref is None or not hasattr(ref, "odlref_save_state"):
        raise SystemExit("the reference library (make -C oracle ref) is needed to write the fixtures")
    ref_save_state(ref, str(HERE / "ref_state.odl"), state_tensors())
    ref_save_checkpoint(ref, str(HERE / "ref_checkpoint.ckpt"))
    print("wrote", HERE / "ref_state.odl", "and", HERE / "ref_checkpoint")


if __name__ == "__main__":
    main()
