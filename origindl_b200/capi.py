"""ctypes binding of libodl_b200.so (the C ABI declared in include/odl_b200.h).

The library is loaded from this package directory; if it has not been built the import of `lib()` raises
with the build command.  There is no fallback path: every function here ends in a CUDA kernel of the library.
Pointers are passed as integers (`tensor.data_ptr()`), streams as `torch.cuda.current_stream().cuda_stream`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libodl_b200.so"

OK = 0
ERR_STALE_GRAPH = 7
ERR_COMM, ERR_COMM_TIMEOUT = 8, 9
PRECISION_3XTF32 = 0
PRECISION_TF32 = 1
EPI_BIAS, EPI_RELU, EPI_MASK, EPI_COLSUM, EPI_SMALL = 1, 2, 4, 8, 16
W_OUT_IN, W_IN_OUT = 0, 1
ACT_NONE, ACT_RELU, ACT_SILU = 0, 1, 2

_lib = None


class OdlError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"odl status {status}: {message}")
        self.status = status


_P = c_void_p
_I64 = c_int64

_SIGNATURES = {
    "odl_init": [c_int],
    "odl_device_status": [_P],
    "odl_debug_set_tile_n": [c_int],
    "odl_debug_set_chunk": [c_int],
    "odl_matmul": [_P, _P, _P, _I64, _I64, _I64, _I64, c_int, c_int, _P],
    "odl_gemm_ex": [c_int, c_int, _I64, _I64, _I64, _P, _P, _I64, _P, _P, _I64, _P, _P, _I64, _P, _P, _I64, _P,
                    c_int, c_int, _P],
    "odl_split_tf32": [_P, _I64, _I64, _I64, _P, _I64, _P, _P, _I64, _P, _P],
    "odl_debug_set_split_k": [c_int],
    "odl_debug_set_bk": [c_int],
    "odl_debug_set_pair_mode": [c_int],
    "odl_debug_set_persistent_pairs": [c_int],
    "odl_debug_set_stream_k": [c_int],
    "odl_debug_set_conv_mode": [c_int],
    "odl_binary": [c_int, _P, _P, _P, _I64, _P],
    "odl_scale": [_P, c_float, _P, _I64, _P],
    "odl_axpy": [c_float, _P, _P, _I64, _P],
    "odl_fill": [_P, c_float, _I64, _P],
    "odl_sum_all": [_P, _P, _I64, _P],
    "odl_linear_forward": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, c_int, c_int, c_int, _P],
    "odl_linear_backward": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, c_int, c_int, _P],
    "odl_linear_backward_chain": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, c_int, c_int, _P],
    "odl_relu_forward": [_P, _P, _I64, _P],
    "odl_relu_backward": [_P, _P, _P, _I64, _P],
    "odl_add_bias": [_P, _P, _P, _I64, _I64, _P],
    "odl_sum_to_row": [_P, _P, _I64, _I64, _P],
    "odl_softmax_cross_entropy": [_P, _P, c_int, _I64, _I64, _P, _P, c_float, _P],
    "odl_adam_step": [_P, _P, _P, _P, _P, _I64, c_int, c_float, c_float, c_float, c_float, c_float, c_float, _P],
    "odl_sgd_step": [_P, _P, _P, _P, _I64, c_float, c_float, c_float, c_int, c_float, c_float, _P],
    "odl_im2col": [_P, _P, _I64, _I64, _I64, _I64, c_int, c_int, c_int, c_int, _P],
    "odl_col2im": [_P, _P, _I64, _I64, _I64, _I64, c_int, c_int, c_int, c_int, _P],
    "odl_conv2d_forward": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "odl_conv2d_backward": [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, c_int, c_int, c_int, c_int, c_int,
                            c_int, _P],
}


def declared_symbols() -> list[str]:
    """Names of every function declared in include/*.h (parsed from the headers: the product ABI odl_b200.h and the
    test-only overrides odl_b200_test.h)."""
    import re

    text = "".join(h.read_text() for h in sorted((_HERE.parent / "include").glob("*.h")))
    return sorted(set(re.findall(r"\b(odl_[a-z0-9_]+)\s*\(", text)))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m origindl_b200.build` (needs nvcc, sm_100a)")
        L = ctypes.CDLL(str(LIB_PATH))
        L.odl_last_error.restype = c_char_p
        L.odl_last_error.argtypes = []
        L.odl_scratch_bytes.restype = c_int64
        L.odl_scratch_bytes.argtypes = []
        for name, args in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int
        _declare_extra(L)
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise OdlError(status, lib().odl_last_error().decode(errors="replace"))


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args))


def ptr(t) -> int | None:
    """Device address of a torch tensor (None passes NULL)."""
    return None if t is None else t.data_ptr()


def stream_handle() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


_initialized = False


def init(device: int = 0) -> None:
    global _initialized
    if not _initialized:
        call("odl_init", device)
        _initialized = True


def device_status() -> None:
    call("odl_device_status", stream_handle())


# ---- MLP training state -----------------------------------------------------------------------------------------
_MLP_SIGNATURES = {
    "odl_mlp_create": [ctypes.POINTER(ctypes.c_int32), c_int, _I64, c_int, c_float, c_float, c_float, c_int,
                       ctypes.POINTER(c_void_p)],
    "odl_mlp_destroy": [_P],
    "odl_mlp_set_params": [_P, _P, _P],
    "odl_mlp_get_packed": [_P, c_int, _P, _P],
    "odl_mlp_forward_loss": [_P, _P, _P, c_int, _P],
    "odl_mlp_backward_layer": [_P, c_int, _P],
    "odl_mlp_optimizer_step": [_P, c_float, _P],
    "odl_mlp_optimizer_step_layer": [_P, c_int, c_float, c_int, _P],
    "odl_mlp_capture": [_P, _P, _P, c_int, _P],
    "odl_mlp_replay": [_P, _P],
    "odl_mlp_train_step": [_P, _P, _P, c_int, _P],
    "odl_mlp_grad_bucket": [_P, c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64)],
    "odl_mlp_set_optimizer_state": [_P, _P, _P, c_int, _P],
    "odl_batch_norm_forward": [_P, _P, _P, _P, _P, c_int, c_float, c_float, _I64, _I64, _I64, c_int, _P, _P, _P, _P],
    "odl_batch_norm_backward": [_P, _P, _P, _P, _P, _P, c_float, _I64, _I64, _I64, c_int, _P, _P, _P, _P],
    "odl_batch_norm_fold": [_P, _P, _P, _P, _P, c_float, _I64, _P, _P, _P],
    "odl_silu_forward": [_P, _P, _I64, _P],
    "odl_silu_backward": [_P, _P, _P, _I64, _P],
    "odl_conv2d_bn_act_forward": [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, c_int, c_int, c_int, c_int, c_int,
                                  c_int, _P],
    "odl_gather_rows": [_P, _I64, _I64, _P, _I64, _I64, _P, _I64, _P, _P, _P],
    "odl_comm_unique_id": [_P],
    "odl_comm_create": [_P, c_int, c_int, ctypes.POINTER(c_void_p)],
    "odl_comm_destroy": [_P],
    "odl_comm_allreduce": [_P, _P, _I64, _P],
    "odl_comm_status": [_P],
    "odl_mlp_dp_attach": [_P, _P, c_int],
    "odl_mlp_train_step_dp": [_P, _P, _P, c_int, _P],
    "odl_mlp_dp_wait": [_P, c_int],
}
_SIGNATURES.update(_MLP_SIGNATURES)
_POINTER_RETURNS = {"odl_mlp_loss_ptr": [_P], "odl_mlp_logits_ptr": [_P]}
_I64_RETURNS = {"odl_mlp_param_count": [_P], "odl_mlp_step_count": [_P], "odl_launch_count": [],
                "odl_scratch_generation": []}


def _declare_extra(L: ctypes.CDLL) -> None:
    for name, args in _POINTER_RETURNS.items():
        fn = getattr(L, name)
        fn.argtypes, fn.restype = args, c_void_p
    for name, args in _I64_RETURNS.items():
        fn = getattr(L, name)
        fn.argtypes, fn.restype = args, c_int64
