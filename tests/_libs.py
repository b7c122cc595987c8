"""Loaders for the two CPU checkers used by the tests (test infrastructure, never imported by the package):

* ``oracle()``    -- oracle/liboracle.so, the plain-C restatement of the reference CPU arithmetic (built on demand
                     with gcc through oracle/Makefile).
* ``reference()`` -- oracle/_ref/libodl_ref.so, the unmodified OriginDL reference behind a thin extern "C" driver.
                     It is built by ``make -C oracle ref`` where the reference tree is mounted and travels prebuilt
                     elsewhere; returns None when it is not available.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_float, c_int, c_int32, c_int64
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
_F = np.ctypeslib.ndpointer(np.float32, flags="C")
_I = np.ctypeslib.ndpointer(np.int32, flags="C")
_FN = ctypes.c_void_p  # nullable float pointer

_oracle = None
_reference = False


def fptr(a):
    """Nullable float32 array argument."""
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def oracle() -> ctypes.CDLL:
    global _oracle
    if _oracle is None:
        lib = ORACLE_DIR / "liboracle.so"
        src = ORACLE_DIR / "oracle.c"
        if not lib.exists() or lib.stat().st_mtime < src.stat().st_mtime:
            subprocess.run(["make", "-C", str(ORACLE_DIR), "oracle"], check=True, capture_output=True)
        L = ctypes.CDLL(str(lib))
        L.oracle_matmul.argtypes = [_F, _F, _F, c_int64, c_int64, c_int64]
        L.oracle_colsum.argtypes = [_F, _F, c_int64, c_int64]
        L.oracle_linear_forward.argtypes = [_F, _F, _FN, _F, c_int64, c_int64, c_int64, c_int, c_int]
        L.oracle_linear_backward.argtypes = [_F, _F, _FN, _F, _FN, _FN, _FN, c_int64, c_int64, c_int64, c_int, c_int]
        L.oracle_softmax_ce.argtypes = [_F, _I, c_int64, c_int64, ctypes.POINTER(c_float), _FN]
        L.oracle_softmax_ce.restype = c_int
        L.oracle_adam_step.argtypes = [_F, _F, _F, _F, c_int64, c_int, c_float, c_float, c_float, c_float, c_float]
        L.oracle_sgd_step.argtypes = [_F, _F, _FN, c_int64, c_float, c_float, c_float, c_int, c_float]
        L.oracle_im2col.argtypes = [_F, _F, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int]
        L.oracle_col2im.argtypes = [_F, _F, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int]
        L.oracle_conv2d_forward.argtypes = [_F, _F, _FN, _F, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                            c_int, c_int]
        L.oracle_conv2d_backward.argtypes = [_F, _F, _F, _FN, _FN, _FN, c_int64, c_int64, c_int64, c_int64, c_int64,
                                             c_int, c_int, c_int, c_int, c_int]
        for name in dir(L):
            pass
        _oracle = L
    return _oracle


def reference():
    """The unmodified reference library, or None if it is not built and cannot be built here."""
    global _reference
    if _reference is False:
        lib = ORACLE_DIR / "_ref" / "libodl_ref.so"
        if not lib.exists() and Path(os.environ.get("ODL_REFERENCE_TREE", ROOT.parent / "reference")).exists():
            subprocess.run(["make", "-C", str(ORACLE_DIR), "ref", "-j8"], check=False, capture_output=True)
        if not lib.exists():
            _reference = None
            return None
        try:
            L = ctypes.CDLL(str(lib))
        except OSError:
            _reference = None
            return None
        L.odlref_last_error.restype = ctypes.c_char_p
        L.odlref_matmul.argtypes = [_F, _F, _F, c_int64, c_int64, c_int64]
        L.odlref_matmul_backward.argtypes = [_F, _F, _F, _F, _F, c_int64, c_int64, c_int64]
        L.odlref_custom_linear.argtypes = [_F, _F, _FN, _F, c_int64, c_int64, c_int64]
        L.odlref_linear_fwd_bwd.argtypes = [_F, _F, _FN, _FN, c_int64, c_int64, c_int64, c_int, c_int, _F, _FN, _FN, _FN]
        L.odlref_softmax_ce.argtypes = [_F, _I, c_int64, c_int64, ctypes.POINTER(c_float), _FN]
        L.odlref_conv2d_fwd_bwd.argtypes = [_F, _F, _FN, _FN, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                            c_int64, c_int, c_int, _F, _FN, _FN, _FN]
        L.odlref_mlp_train.argtypes = [_I, c_int, _F, _F, _I, c_int64, c_int, c_int, c_int, c_float, c_float, c_float,
                                       _F, _FN]
        L.odlref_optim_replay.argtypes = [_F, _F, c_int64, c_int, c_int, c_float, c_float, c_float, c_int, c_float]
        if hasattr(L, "odlref_save_state"):  # a prebuilt library may predate the state-dict entry points
            cp, ip = ctypes.c_char_p, ctypes.POINTER(c_int)
            L.odlref_save_state.argtypes = [cp, c_int, ctypes.POINTER(cp), _I, np.ctypeslib.ndpointer(np.int64, flags="C"),
                                            ctypes.POINTER(ctypes.c_void_p)]
            L.odlref_load_state_names.argtypes = [cp, cp, c_int64, ip]
            L.odlref_load_state_tensor.argtypes = [cp, cp, ip, np.ctypeslib.ndpointer(np.int64, flags="C"), _FN]
            L.odlref_save_checkpoint.argtypes = [cp, _I, c_int, _F, c_int, c_int, c_float, cp, c_float, c_float, c_float,
                                                 c_float]
            L.odlref_load_checkpoint_meta.argtypes = [cp, ip, ip, ctypes.POINTER(c_float), cp, c_int64, _F, ip]
        _reference = L
    return _reference


def ref_check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError("reference driver failed: " + reference().odlref_last_error().decode())


# ---------------------------------------------------------------- seeded synthetic inputs shared by tests and bench
def kaiming_uniform(rng: np.random.Generator, fan_in: int, shape) -> np.ndarray:
    bound = np.sqrt(6.0 / fan_in)
    return rng.uniform(-bound, bound, size=shape).astype(np.float32)


def mlp_params(rng: np.random.Generator, sizes) -> np.ndarray:
    """Concatenated [W_0 {in,out}, b_0 {1,out}, W_1, b_1, ...] with Kaiming-uniform weights and zero biases."""
    parts = []
    for i in range(len(sizes) - 1):
        parts.append(kaiming_uniform(rng, sizes[i], (sizes[i], sizes[i + 1])).ravel())
        parts.append(np.zeros(sizes[i + 1], np.float32))
    return np.concatenate(parts)


def max_rel_err(a, b) -> float:
    """max|a-b| / max|b| -- the metric the tolerances of this repository are stated in."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    denom = np.abs(b).max()
    return float(np.abs(a - b).max() / (denom if denom > 0 else 1.0))


# ---------------------------------------------------------------- MLP training composed from the oracle functions
def oracle_mlp_train(sizes, params, xs, ts, steps, opt="adam", lr=1e-3, momentum=0.0, hook_wd=0.0, grad_hook=None):
    """Train with the oracle's Linear / softmax-CE / optimizer functions, following nn::MLP + the reference loop.

    params: packed [W_0 {in,out}, b_0, ...]; xs[n_batches, B, in], ts[n_batches, B].  `grad_hook(list_of_grads)` is
    called after backward and before the optimizer (used by the data-parallel tests to all-reduce).  Returns
    (losses, final packed params, last gradients as the optimizer left them)."""
    orc = oracle()
    sizes = [int(s) for s in sizes]
    L = len(sizes) - 1
    views, off = [], 0
    params = params.copy()
    for l in range(L):
        nw, nb = sizes[l] * sizes[l + 1], sizes[l + 1]
        views.append((off, nw, off + nw, nb))
        off += nw + nb
    m, v = np.zeros_like(params), np.zeros_like(params)
    B = xs.shape[1]
    losses = np.empty(steps, np.float32)
    grads = np.zeros_like(params)
    for s in range(steps):
        x = np.ascontiguousarray(xs[s % xs.shape[0]])
        t = np.ascontiguousarray(ts[s % ts.shape[0]])
        acts = [x]
        for l, (wo, nw, bo, nb) in enumerate(views):
            y = np.empty((B, sizes[l + 1]), np.float32)
            orc.oracle_linear_forward(acts[-1], params[wo:wo + nw], fptr(params[bo:bo + nb]), y, B, sizes[l + 1],
                                      sizes[l], 1, int(l + 1 < L))
            acts.append(y)
        loss = ctypes.c_float()
        g = np.empty_like(acts[-1])
        assert orc.oracle_softmax_ce(acts[-1], t, B, sizes[-1], ctypes.byref(loss), fptr(g)) == 0
        losses[s] = loss.value
        grads = np.zeros_like(params)
        for l in range(L - 1, -1, -1):
            wo, nw, bo, nb = views[l]
            dx = np.empty_like(acts[l]) if l > 0 else None
            # the ReLU of layer l sits between its Linear and layer l+1: mask the incoming gradient with y_l > 0
            relu = int(l + 1 < L)
            orc.oracle_linear_backward(acts[l], params[wo:wo + nw], fptr(acts[l + 1]), g, fptr(dx),
                                       fptr(grads[wo:wo + nw]), fptr(grads[bo:bo + nb]), B, sizes[l + 1], sizes[l], 1, relu)
            g = dx
        if grad_hook is not None:
            grad_hook(grads)
        if opt == "adam":
            orc.oracle_adam_step(params, grads, m, v, params.size, s + 1, lr, 0.9, 0.999, 1e-8, hook_wd)
        else:
            orc.oracle_sgd_step(params, grads, fptr(m), params.size, lr, momentum, 0.0, 0, hook_wd)
    return losses, params, grads
