"""Thin torch-tensor front end over the C ABI (include/odl_b200.h).

torch is used for device memory and streams only; every function below ends in one or more kernels of
libodl_b200.so launched on torch's current stream.  Tensors must be contiguous fp32 CUDA tensors (labels int32 or
int64).  Shapes and argument meaning follow the reference operators named in the header.
"""
from __future__ import annotations

import torch

from . import capi
from .capi import PRECISION_3XTF32, PRECISION_TF32, W_IN_OUT, W_OUT_IN  # noqa: F401

_p = capi.ptr


def _chk(*tensors):
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("odl ops need contiguous CUDA tensors")
        if t.dtype != torch.float32:
            raise TypeError(f"odl ops compute in float32, got {t.dtype}")


def _s():
    return capi.stream_handle()


def matmul(a: torch.Tensor, b: torch.Tensor, precision: int = PRECISION_3XTF32) -> torch.Tensor:
    """a[M,K] @ b[K,N], a[B,M,K] @ b[K,N] or a[B,M,K] @ b[B,K,N] (origin::cuda::matmul)."""
    _chk(a, b)
    if a.dim() == 2 and b.dim() == 2:
        if a.shape[1] != b.shape[0]:
            raise ValueError(f"Matrix dimensions must be compatible for multiplication. A shape: {tuple(a.shape)}, "
                             f"B shape: {tuple(b.shape)}")
        batch, M, K, N, bb = 1, a.shape[0], a.shape[1], b.shape[1], 0
        out = torch.empty((M, N), device=a.device, dtype=torch.float32)
    elif a.dim() == 3 and b.dim() == 2:
        if a.shape[2] != b.shape[0]:
            raise ValueError("Matrix dimensions must be compatible for multiplication")
        batch, M, K, N, bb = a.shape[0], a.shape[1], a.shape[2], b.shape[1], 0
        out = torch.empty((batch, M, N), device=a.device, dtype=torch.float32)
    elif a.dim() == 3 and b.dim() == 3:
        if a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
            raise ValueError("Matrix dimensions must be compatible for multiplication")
        batch, M, K, N, bb = a.shape[0], a.shape[1], a.shape[2], b.shape[2], 1
        out = torch.empty((batch, M, N), device=a.device, dtype=torch.float32)
    else:
        raise ValueError("Matrix multiplication requires compatible dimensions")
    capi.call("odl_matmul", _p(a), _p(b), _p(out), M, N, K, batch, bb, precision, _s())
    return out


def gemm(a, b, trans_a=False, trans_b=False, bias=None, relu=False, mask_src=None, colsum=None, want_small=False,
         a_small=None, b_small=None, precision: int = PRECISION_3XTF32):
    """D = op(a) @ op(b) with the fused epilogue of odl_gemm_ex; returns D or (D, D_small)."""
    _chk(a, b, bias, mask_src, colsum, a_small, b_small)
    M = a.shape[1] if trans_a else a.shape[0]
    K = a.shape[0] if trans_a else a.shape[1]
    N = b.shape[0] if trans_b else b.shape[1]
    Kb = b.shape[1] if trans_b else b.shape[0]
    if K != Kb:
        raise ValueError("gemm: inner dimensions differ")
    d = torch.empty((M, N), device=a.device, dtype=torch.float32)
    ds = torch.empty_like(d) if want_small else None
    flags = (capi.EPI_BIAS if bias is not None else 0) | (capi.EPI_RELU if relu else 0) | \
            (capi.EPI_MASK if mask_src is not None else 0) | (capi.EPI_COLSUM if colsum is not None else 0) | \
            (capi.EPI_SMALL if want_small else 0)
    capi.call("odl_gemm_ex", int(trans_a), int(trans_b), M, N, K, _p(a), _p(a_small), a.shape[1], _p(b), _p(b_small),
              b.shape[1], _p(d), _p(ds), N, _p(bias), _p(mask_src), N, _p(colsum), flags, precision, _s())
    return (d, ds) if want_small else d


def split_tf32(x: torch.Tensor) -> torch.Tensor:
    """Low part of the 3xTF32 split of a 2-D tensor."""
    _chk(x)
    x2 = x.reshape(-1, x.shape[-1])
    out = torch.empty_like(x2)
    capi.call("odl_split_tf32", _p(x2), x2.shape[1], x2.shape[0], x2.shape[1], None, 0, None, _p(out), x2.shape[1], None,
              _s())
    return out.reshape(x.shape)


def linear_forward(x, w, b=None, relu=False, w_layout=W_OUT_IN, precision=PRECISION_3XTF32, x_small=None, w_small=None,
                   want_small=False):
    _chk(x, w, b, x_small, w_small)
    M, K = x.shape
    N = w.shape[0] if w_layout == W_OUT_IN else w.shape[1]
    Kw = w.shape[1] if w_layout == W_OUT_IN else w.shape[0]
    if K != Kw:
        raise ValueError(f"linear: input features {K} do not match weight {tuple(w.shape)}")
    if b is not None and b.numel() != N:
        raise ValueError("linear: bias size mismatch")
    y = torch.empty((M, N), device=x.device, dtype=torch.float32)
    ys = torch.empty_like(y) if want_small else None
    capi.call("odl_linear_forward", _p(x), _p(x_small), _p(w), _p(w_small), _p(b), _p(y), _p(ys), M, N, K, w_layout,
              int(relu), precision, _s())
    return (y, ys) if want_small else y


def linear_backward(x, w, dy, y=None, w_layout=W_OUT_IN, precision=PRECISION_3XTF32, need_dx=True, need_dw=True,
                    need_db=True, x_small=None, w_small=None):
    """Returns (dx, dw, db); `y` is the forward output when the layer had a fused ReLU."""
    _chk(x, w, dy, y, x_small, w_small)
    M, K = x.shape
    N = dy.shape[1]
    dx = torch.empty_like(x) if need_dx else None
    dw = torch.empty_like(w) if need_dw else None
    db = torch.empty((N,), device=x.device, dtype=torch.float32) if need_db else None
    capi.call("odl_linear_backward", _p(x), _p(x_small), _p(w), _p(w_small), _p(dy), _p(y), _p(dx), _p(dw), _p(db), M, N,
              K, w_layout, precision, _s())
    return dx, dw, db


def relu(x):
    _chk(x)
    y = torch.empty_like(x)
    capi.call("odl_relu_forward", _p(x), _p(y), x.numel(), _s())
    return y


def relu_backward(gy, x_or_y):
    _chk(gy, x_or_y)
    gx = torch.empty_like(gy)
    capi.call("odl_relu_backward", _p(gy), _p(x_or_y), _p(gx), gy.numel(), _s())
    return gx


def add_bias(x, b):
    _chk(x, b)
    y = torch.empty_like(x)
    capi.call("odl_add_bias", _p(x), _p(b), _p(y), x.shape[0], x.shape[1], _s())
    return y


def sum_to_row(g):
    _chk(g)
    out = torch.empty((1, g.shape[1]), device=g.device, dtype=torch.float32)
    capi.call("odl_sum_to_row", _p(g), _p(out), g.shape[0], g.shape[1], _s())
    return out


def softmax_cross_entropy(logits, labels, need_grad=True, grad_scale=1.0):
    """Returns (loss 0-dim tensor on the device, dlogits or None)."""
    _chk(logits)
    if labels.dtype not in (torch.int32, torch.int64) or not labels.is_cuda or not labels.is_contiguous():
        raise TypeError("labels must be a contiguous int32/int64 CUDA tensor")
    if logits.dim() != 2 or labels.dim() != 1 or labels.shape[0] != logits.shape[0]:
        raise ValueError("SoftmaxCrossEntropy expects x (N, C) and target (N,)")
    B, C = logits.shape
    loss = torch.empty((1,), device=logits.device, dtype=torch.float32)
    d = torch.empty_like(logits) if need_grad else None
    capi.call("odl_softmax_cross_entropy", _p(logits), labels.data_ptr(), int(labels.dtype == torch.int64), B, C,
              _p(loss), _p(d), float(grad_scale), _s())
    return loss.reshape(()), d


def adam_step(p, g, m, v, t, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, hook_weight_decay=0.0, grad_scale=1.0,
              p_small=None):
    _chk(p, g, m, v, p_small)
    capi.call("odl_adam_step", _p(p), _p(g), _p(m), _p(v), _p(p_small), p.numel(), int(t), lr, beta1, beta2, eps,
              hook_weight_decay, grad_scale, _s())


def sgd_step(p, g, buf=None, lr=1e-2, momentum=0.0, weight_decay=0.0, nesterov=False, hook_weight_decay=0.0,
             grad_scale=1.0, p_small=None):
    _chk(p, g, buf, p_small)
    capi.call("odl_sgd_step", _p(p), _p(g), _p(buf), _p(p_small), p.numel(), lr, momentum, weight_decay, int(nesterov),
              hook_weight_decay, grad_scale, _s())


def conv_out_size(size, k, s, p):
    return (size + 2 * p - k) // s + 1


def im2col(x, k, stride, pad):
    _chk(x)
    N, C, H, W = x.shape
    OH, OW = conv_out_size(H, k, stride, pad), conv_out_size(W, k, stride, pad)
    col = torch.empty((N * OH * OW, C * k * k), device=x.device, dtype=torch.float32)
    capi.call("odl_im2col", _p(x), _p(col), N, C, H, W, k, k, stride, pad, _s())
    return col


def col2im(col, shape, k, stride, pad):
    _chk(col)
    N, C, H, W = shape
    x = torch.empty(shape, device=col.device, dtype=torch.float32)
    capi.call("odl_col2im", _p(col), _p(x), N, C, H, W, k, k, stride, pad, _s())
    return x


def conv2d_forward(x, w, b=None, stride=1, pad=0, relu=False, precision=PRECISION_3XTF32):
    _chk(x, w, b)
    if x.dim() != 4 or w.dim() != 4:
        raise ValueError("conv2d: x must be 4D (N, C, H, W) and W 4D (OC, C, KH, KW)")
    N, C, H, W = x.shape
    OC, C2, KH, KW = w.shape
    if C != C2:
        raise ValueError(f"conv2d: channel mismatch - x has {C} channels, but W expects {C2} channels")
    OH, OW = conv_out_size(H, KH, stride, pad), conv_out_size(W, KW, stride, pad)
    if OH <= 0 or OW <= 0:
        raise ValueError(f"conv2d: invalid output size OH={OH}, OW={OW}")
    y = torch.empty((N, OC, OH, OW), device=x.device, dtype=torch.float32)
    capi.call("odl_conv2d_forward", _p(x), _p(w), _p(b), _p(y), N, C, H, W, OC, KH, KW, stride, pad, int(relu), precision,
              _s())
    return y


def conv2d_backward(gy, x, w, stride=1, pad=0, gy_layout=0, need_gb=True, precision=PRECISION_3XTF32, need_gx=True,
                    need_gw=True):
    """Returns (gx, gw, gb); a gradient that is not asked for is None and is not computed.  gy_layout 0: true gradient;
    1: the reference's reinterpretation of gy."""
    _chk(gy, x, w)
    N, C, H, W = x.shape
    OC, _, KH, KW = w.shape
    gx = torch.empty_like(x) if need_gx else None
    gw = torch.empty_like(w) if need_gw else None
    gb = torch.empty((OC,), device=x.device, dtype=torch.float32) if need_gb else None
    capi.call("odl_conv2d_backward", _p(gy), _p(x), _p(w), _p(gx), _p(gw), _p(gb), N, C, H, W, OC, KH, KW, stride, pad,
              gy_layout, precision, _s())
    return gx, gw, gb


# ---- BatchNorm (+ activation), SiLU, conv -> BatchNorm -> activation -------------------------------------------------
def _bn_dims(x):
    if x.dim() == 2:
        return x.shape[0], x.shape[1], 1
    if x.dim() == 4:
        return x.shape[0], x.shape[1], x.shape[2] * x.shape[3]
    raise ValueError(f"batch_norm: x must have 2 or 4 dimensions, but got shape {tuple(x.shape)}")


def batch_norm_forward(x, gamma, beta, running_mean=None, running_var=None, training=True, eps=1e-5, momentum=0.1,
                       act=capi.ACT_NONE):
    """Returns (y, save_mean, save_var).  Training mode updates running_mean / running_var in place when given (the
    reference layer's rule: running = momentum * running + (1 - momentum) * batch)."""
    _chk(x, gamma, beta, running_mean, running_var)
    N, C, HW = _bn_dims(x)
    for t in (gamma, beta, running_mean, running_var):
        if t is not None and tuple(t.shape) != (C,):
            raise ValueError(f"batch_norm: gamma, beta, running_mean, running_var must have shape ({C})")
    y = torch.empty_like(x)
    mean, var = torch.empty(C, device=x.device), torch.empty(C, device=x.device)
    capi.call("odl_batch_norm_forward", _p(x), _p(gamma), _p(beta), _p(running_mean), _p(running_var), int(training), eps,
              momentum, N, C, HW, act, _p(y), _p(mean), _p(var), _s())
    return y, mean, var


def batch_norm_backward(gy, x, gamma, beta, save_mean, save_var, eps=1e-5, act=capi.ACT_NONE):
    """Returns (gx, dgamma, dbeta) for the statistics the forward pass used."""
    _chk(gy, x, gamma, beta, save_mean, save_var)
    N, C, HW = _bn_dims(x)
    gx, dg, db = torch.empty_like(x), torch.empty(C, device=x.device), torch.empty(C, device=x.device)
    capi.call("odl_batch_norm_backward", _p(gy), _p(x), _p(gamma), _p(beta), _p(save_mean), _p(save_var), eps, N, C, HW,
              act, _p(gx), _p(dg), _p(db), _s())
    return gx, dg, db


def batch_norm_fold(gamma, beta, mean, var, bias=None, eps=1e-5):
    """(scale, shift) of evaluation-mode BatchNorm applied to conv(x) + bias."""
    _chk(gamma, beta, mean, var, bias)
    C = gamma.numel()
    scale, shift = torch.empty(C, device=gamma.device), torch.empty(C, device=gamma.device)
    capi.call("odl_batch_norm_fold", _p(gamma), _p(beta), _p(mean), _p(var), _p(bias), eps, C, _p(scale), _p(shift), _s())
    return scale, shift


def silu(x):
    _chk(x)
    y = torch.empty_like(x)
    capi.call("odl_silu_forward", _p(x), _p(y), x.numel(), _s())
    return y


def silu_backward(gy, x):
    _chk(gy, x)
    gx = torch.empty_like(x)
    capi.call("odl_silu_backward", _p(gy), _p(x), _p(gx), x.numel(), _s())
    return gx


def conv2d_bn_act_forward(x, w, scale, shift, stride=1, pad=0, act=capi.ACT_RELU, precision=PRECISION_3XTF32):
    """act(scale[oc] * conv2d(x, w) + shift[oc]) in one GEMM (scale / shift from batch_norm_fold)."""
    _chk(x, w, scale, shift)
    N, C, H, W = x.shape
    OC, C2, KH, KW = w.shape
    if C != C2:
        raise ValueError(f"conv2d: channel mismatch - x has {C} channels, but W expects {C2} channels")
    OH, OW = conv_out_size(H, KH, stride, pad), conv_out_size(W, KW, stride, pad)
    y = torch.empty((N, OC, OH, OW), device=x.device, dtype=torch.float32)
    capi.call("odl_conv2d_bn_act_forward", _p(x), _p(w), _p(scale), _p(shift), _p(y), N, C, H, W, OC, KH, KW, stride, pad,
              act, precision, _s())
    return y
