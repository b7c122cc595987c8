"""GPU: a conv -> BatchNorm(training) -> SiLU -> conv -> Linear -> softmax-CE chain, forward and backward through the
C ABI, against the same chain composed from the oracle's functions (the reference's CPU arithmetic).  This is the shape
of one block of the reference's CNN examples (Conv2d, BatchNorm2d, activation) feeding a Linear head; it checks that the
layouts the kernels hand each other (NCHW activations, per-channel statistics, flattened features) agree with the
reference's, not only each kernel on its own.  Tolerance 2e-5 (3xTF32 GEMMs chained through a normalisation)."""
import ctypes
from ctypes import c_float, c_int, c_int64

import numpy as np
import pytest
import torch

import _libs
from _libs import fptr, max_rel_err

pytestmark = pytest.mark.gpu
EPS = 1e-5
_F = np.ctypeslib.ndpointer(np.float32, flags="C")
_P = ctypes.c_void_p


def oracle_chain(x, w1, b1, gamma, beta, w2, b2, wl, bl, labels):
    """Forward and backward of the block with the oracle; returns (loss, grads dict)."""
    L = _libs.oracle()
    L.oracle_batch_norm_forward.argtypes = [_F, _F, _F, _F, _F, c_int, c_float, c_int64, c_int64, c_int64, _F, _F, _F, _P]
    L.oracle_batch_norm_backward.argtypes = [_F, _F, _F, _F, c_float, c_int64, c_int64, c_int64, _F, _F, _F]
    L.oracle_silu_forward.argtypes = [_F, _F, c_int64]
    L.oracle_silu_backward.argtypes = [_F, _F, _F, c_int64]
    N, C, H, W = x.shape
    OC1, OC2 = w1.shape[0], w2.shape[0]
    y1 = np.empty((N, OC1, H, W), np.float32)                      # 3x3, stride 1, pad 1
    L.oracle_conv2d_forward(x, w1, fptr(b1), y1, N, C, H, W, OC1, 3, 3, 1, 1)
    z, xn = np.empty_like(y1), np.empty_like(y1)
    mean, var = np.empty(OC1, np.float32), np.empty(OC1, np.float32)
    L.oracle_batch_norm_forward(y1.reshape(N, OC1, H * W), gamma, beta, np.zeros(OC1, np.float32), np.ones(OC1, np.float32),
                                1, EPS, N, OC1, H * W, z.reshape(N, OC1, H * W), mean, var, xn.ctypes.data_as(_P))
    a = np.empty_like(z)
    L.oracle_silu_forward(z, a, z.size)
    H2, W2 = (H + 2 - 3) // 2 + 1, (W + 2 - 3) // 2 + 1
    y2 = np.empty((N, OC2, H2, W2), np.float32)                    # 3x3, stride 2, pad 1
    L.oracle_conv2d_forward(a, w2, fptr(b2), y2, N, OC1, H, W, OC2, 3, 3, 2, 1)
    feat = y2.reshape(N, -1)
    K, NC = feat.shape[1], wl.shape[0]
    logits = np.empty((N, NC), np.float32)
    L.oracle_linear_forward(feat, wl, fptr(bl), logits, N, NC, K, 0, 0)
    loss, dlogits = c_float(), np.empty_like(logits)
    L.oracle_softmax_ce(logits, labels, N, NC, ctypes.byref(loss), fptr(dlogits))
    dfeat, dwl, dbl = np.empty_like(feat), np.empty_like(wl), np.empty_like(bl)
    L.oracle_linear_backward(feat, wl, None, dlogits, fptr(dfeat), fptr(dwl), fptr(dbl), N, NC, K, 0, 0)
    da, dw2, db2 = np.empty_like(a), np.empty_like(w2), np.empty_like(b2)
    L.oracle_conv2d_backward(dfeat.reshape(y2.shape), a, w2, fptr(da), fptr(dw2), fptr(db2), N, OC1, H, W, OC2, 3, 3, 2, 1, 0)
    dz = np.empty_like(z)
    L.oracle_silu_backward(da, z, dz, z.size)
    dy1, dgamma, dbeta = np.empty_like(y1), np.empty(OC1, np.float32), np.empty(OC1, np.float32)
    L.oracle_batch_norm_backward(dz.reshape(N, OC1, H * W), gamma, var, xn.reshape(N, OC1, H * W), EPS, N, OC1, H * W,
                                 dy1.reshape(N, OC1, H * W), dgamma, dbeta)
    dx, dw1, db1 = np.empty_like(x), np.empty_like(w1), np.empty_like(b1)
    L.oracle_conv2d_backward(dy1, x, w1, fptr(dx), fptr(dw1), fptr(db1), N, C, H, W, OC1, 3, 3, 1, 1, 0)
    return loss.value, dict(dx=dx, dw1=dw1, db1=db1, dgamma=dgamma, dbeta=dbeta, dw2=dw2, db2=db2, dwl=dwl, dbl=dbl,
                            logits=logits, mean=mean, var=var)


@pytest.mark.parametrize("shape", [(4, 3, 12, 12, 8, 6, 5), (2, 5, 9, 11, 40, 12, 7)])
def test_cnn_block_forward_and_backward(shape):
    from origindl_b200 import capi, ops

    capi.init(0)
    N, C, H, W, OC1, OC2, NC = shape
    rng = np.random.default_rng(sum(shape))
    H2, W2 = (H + 2 - 3) // 2 + 1, (W + 2 - 3) // 2 + 1
    host = dict(x=rng.standard_normal((N, C, H, W)), w1=rng.standard_normal((OC1, C, 3, 3)) * (2 / (C * 9)) ** 0.5,
                b1=0.1 * rng.standard_normal(OC1), gamma=1 + 0.2 * rng.standard_normal(OC1), beta=0.1 * rng.standard_normal(OC1),
                w2=rng.standard_normal((OC2, OC1, 3, 3)) * (2 / (OC1 * 9)) ** 0.5, b2=0.1 * rng.standard_normal(OC2),
                wl=rng.standard_normal((NC, OC2 * H2 * W2)) * (1 / (OC2 * H2 * W2)) ** 0.5, bl=0.1 * rng.standard_normal(NC))
    host = {k: np.ascontiguousarray(v, np.float32) for k, v in host.items()}
    labels = rng.integers(0, NC, N).astype(np.int32)
    want_loss, want = oracle_chain(labels=labels, **host)

    d = {k: torch.from_numpy(v).cuda() for k, v in host.items()}
    t = torch.from_numpy(labels).cuda()
    y1 = ops.conv2d_forward(d["x"], d["w1"], d["b1"], 1, 1)
    a, mean, var = ops.batch_norm_forward(y1, d["gamma"], d["beta"], training=True, eps=EPS, act=capi.ACT_SILU)
    y2 = ops.conv2d_forward(a, d["w2"], d["b2"], 2, 1)
    feat = y2.reshape(N, -1)
    logits = ops.linear_forward(feat, d["wl"], d["bl"])
    loss, dlogits = ops.softmax_cross_entropy(logits, t)
    dfeat, dwl, dbl = ops.linear_backward(feat, d["wl"], dlogits)
    da, dw2, db2 = ops.conv2d_backward(dfeat.reshape(y2.shape), a, d["w2"], 2, 1)
    dy1, dgamma, dbeta = ops.batch_norm_backward(da, y1, d["gamma"], d["beta"], mean, var, eps=EPS, act=capi.ACT_SILU)
    dx, dw1, db1 = ops.conv2d_backward(dy1, d["x"], d["w1"], 1, 1)
    capi.device_status()

    assert abs(loss.item() - want_loss) <= 2e-5 * max(1.0, abs(want_loss))
    got = dict(dx=dx, dw1=dw1, db1=db1, dgamma=dgamma, dbeta=dbeta, dw2=dw2, db2=db2, dwl=dwl, dbl=dbl, logits=logits,
               mean=mean, var=var)
    for k, v in got.items():
        if k == "db1":
            # a per-channel shift in front of a training-mode BatchNorm cannot change the loss: the exact gradient is 0
            # and both sides only hold rounding noise
            assert np.abs(v.cpu().numpy()).max() <= 1e-5 * np.abs(want["dbeta"]).max()
            assert np.abs(want[k]).max() <= 1e-5 * np.abs(want["dbeta"]).max()
            continue
        assert max_rel_err(v.cpu().numpy().reshape(want[k].shape), want[k]) <= 2e-5, k
