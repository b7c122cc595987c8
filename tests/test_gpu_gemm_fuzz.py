"""GPU: seeded random sweep of odl_gemm_ex over shapes (ragged and tile-aligned, tiny to 8192-wide), the four operand
layouts, both precisions and every combination of epilogue flags, against float64 -- the launcher picks among one-CTA
tiles of three widths, CTA pairs, the 256 x 512 plain-TF32 tile, cluster split-K and sliced split-K, 2-D or 3-D operand
copies from the shape alone, and this sweep walks through all of those choices.  Tolerances: 3xTF32 1e-5, TF32 5e-3
(max|a-b| / max|ref|); elements within the tolerance of a ReLU kink are exempt."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DIMS = [1, 7, 31, 32, 33, 64, 96, 100, 127, 128, 129, 160, 255, 256, 257, 300, 384, 511, 512, 513, 640, 768, 1000, 1024,
        1536, 2048, 2080, 4096]


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_gemm_configurations(seed):
    from origindl_b200 import capi, ops

    capi.init(0)
    rng = np.random.default_rng(seed)
    for it in range(90):
        M, N, K = (int(rng.choice(DIMS)) for _ in range(3))
        if it % 7 == 0:  # large outputs: CTA pairs, wide TF32 tiles
            M, N = int(rng.choice([2048, 4096, 6144])), int(rng.choice([2048, 2560, 4096, 8192]))
        if M * N * K > 4e10:
            K = int(rng.choice([32, 64, 100, 256]))
        ta, tb, prec = int(rng.integers(2)), int(rng.integers(2)), int(rng.integers(2))
        g = torch.Generator(device="cuda").manual_seed(1000 * seed + it)
        a = torch.randn((K, M) if ta else (M, K), device="cuda", generator=g)
        b = torch.randn((N, K) if tb else (K, N), device="cuda", generator=g)
        use_bias, use_relu, use_mask, use_cs, use_small = (bool(rng.integers(2)) for _ in range(5))
        bias = torch.randn(N, device="cuda", generator=g) if use_bias else None
        mask = torch.randn(M, N, device="cuda", generator=g) if use_mask else None
        cs = torch.zeros(N, device="cuda") if use_cs else None
        out = ops.gemm(a, b, trans_a=bool(ta), trans_b=bool(tb), bias=bias, relu=use_relu, mask_src=mask, colsum=cs,
                       want_small=use_small, precision=prec)
        capi.device_status()
        d = out[0] if use_small else out
        ref = (a.t() if ta else a).double() @ (b.t() if tb else b).double()
        if use_bias:
            ref = ref + bias.double()
        pre = ref
        if use_relu:
            ref = torch.clamp(ref, min=0)
        if use_mask:
            ref = ref * (mask > 0)
        tol = (5e-3 if prec else 1e-5) * max(pre.abs().max().item(), 1e-30)
        err = (d.double() - ref).abs()
        if use_relu:
            err = err * (pre.abs() > tol)
        case = (seed, it, M, N, K, ta, tb, prec, use_bias, use_relu, use_mask, use_cs, use_small)
        assert err.max().item() <= tol, case
        if use_cs:
            assert (cs.double() - ref.sum(0)).abs().max().item() <= 20 * tol * max(1.0, M ** 0.5), case
        if use_small:
            assert torch.equal(out[1], ops.split_tf32(d)), case
