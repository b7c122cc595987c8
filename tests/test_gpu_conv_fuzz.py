"""GPU: seeded random sweep of conv2d forward / backward geometries (channels 1..300, kernels 1..7, strides 1..3, paddings,
ragged image sizes) against float64 autograd of the same convolution.  The library picks among the direct fp32 forward
(small layers), the implicit-GEMM forward (one CTA or a K-splitting cluster), im2col + GEMM, direct and implicit-GEMM
gradient kernels from the geometry alone;
this sweep walks through those choices.  True-gradient layout; 3xTF32 tolerance 1e-5 (max|a-b| / max|ref|)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_conv_geometries(seed):
    from origindl_b200 import capi, ops

    capi.init(0)
    rng = np.random.default_rng(seed)
    done = 0
    while done < 40:
        N = int(rng.integers(1, 5))
        C = int(rng.choice([1, 2, 3, 5, 8, 16, 24, 32, 48, 64, 96, 130, 256, 300]))
        OC = int(rng.choice([1, 3, 8, 16, 20, 32, 40, 64, 70, 128, 136, 256]))
        k = int(rng.choice([1, 1, 2, 3, 3, 3, 4, 5, 6, 7]))
        s = int(rng.choice([1, 1, 1, 2, 2, 3]))
        p = int(rng.integers(0, k))
        H, W = int(rng.integers(k, 40)), int(rng.integers(k, 40))
        if C * k * k * OC > 3e6 or N * C * H * W > 2e6:
            continue
        OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        if OH <= 0 or OW <= 0:
            continue
        done += 1
        g = torch.Generator(device="cuda").manual_seed(100 * seed + done)
        x = torch.randn(N, C, H, W, device="cuda", generator=g)
        w = torch.randn(OC, C, k, k, device="cuda", generator=g) * (2.0 / (C * k * k)) ** 0.5
        b = torch.randn(OC, device="cuda", generator=g)
        gy = torch.randn(N, OC, OH, OW, device="cuda", generator=g)
        y = ops.conv2d_forward(x, w, b, s, p)
        capi.lib().odl_debug_set_conv_mode(3)          # small layers on the implicit-GEMM forward instead of the direct kernel
        try:
            y_tc = ops.conv2d_forward(x, w, b, s, p)
        finally:
            capi.lib().odl_debug_set_conv_mode(0)
        gx, gw, gb = ops.conv2d_backward(gy, x, w, s, p, gy_layout=0)
        capi.lib().odl_debug_set_conv_mode(7)          # small layers: weight gradient from image tiles wherever the window fits
        try:
            _, gw_tile, gb_tile = ops.conv2d_backward(gy, x, w, s, p, gy_layout=0, need_gx=False)
        finally:
            capi.lib().odl_debug_set_conv_mode(0)
        capi.device_status()
        x64, w64, b64 = x.double().requires_grad_(), w.double().requires_grad_(), b.double().requires_grad_()
        y64 = torch.nn.functional.conv2d(x64, w64, b64, stride=s, padding=p)
        y64.backward(gy.double())
        case = (seed, done, N, C, H, W, OC, k, s, p)
        for got, want in ((y, y64.detach()), (y_tc, y64.detach()), (gx, x64.grad), (gw, w64.grad), (gb, b64.grad),
                          (gw_tile, w64.grad), (gb_tile, b64.grad)):
            assert ((got.double() - want).abs().max() / want.abs().max().clamp_min(1e-30)).item() <= 1e-5, case
