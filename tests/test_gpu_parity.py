"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle, the golden vectors that came out of the
unmodified reference, and size-independent properties at the benchmark's full sizes.

Tolerances (metric: max|a-b| / max|ref|, the one the north-star states):
  3xTF32 (default)  <= 1e-5      plain TF32  <= 5e-3
Optimizer steps use exactly-rounded fp32 operations in the reference's order and are held to 1e-6.
"""
import ctypes
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import _libs
from _libs import fptr, max_rel_err

pytestmark = pytest.mark.gpu

TOL = {0: 1e-5, 1: 5e-3}
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def ops():
    from origindl_b200 import capi, ops as _ops

    capi.init(0)
    yield _ops
    capi.device_status()


@pytest.fixture(scope="module")
def orc():
    return _libs.oracle()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


# ------------------------------------------------------------------------------------------------ known answers
def test_known_answers_from_reference_unit_tests(ops):
    ka = json.loads((GOLDEN / "known_answers.json").read_text())
    for c in ka["matmul"]:
        a = dev(np.array(c["a"], np.float32).reshape(c["M"], c["K"]))
        b = dev(np.array(c["b"], np.float32).reshape(c["K"], c["N"]))
        assert np.allclose(host(ops.matmul(a, b)).ravel(), c["c"], atol=1e-3), c["source"]
    for c in ka["matmul_backward_ones"]:
        a = dev(np.array(c["a"], np.float32).reshape(c["M"], c["K"]))
        b = dev(np.array(c["b"], np.float32).reshape(c["K"], c["N"]))
        gy = torch.ones((c["M"], c["N"]), device="cuda")
        ga = ops.gemm(gy, b, trans_b=True)      # gy . b^T
        gb = ops.gemm(a, gy, trans_a=True)      # a^T . gy
        assert np.allclose(host(ga).ravel(), c["ga"], atol=1e-3) and np.allclose(host(gb).ravel(), c["gb"], atol=1e-3)
    for c in ka["custom_linear"]:
        x = dev(np.array(c["x"], np.float32).reshape(c["M"], c["K"]))
        w = dev(np.array(c["w"], np.float32).reshape(c["N"], c["K"]))
        b = None if c["b"] is None else dev(np.array(c["b"], np.float32))
        assert np.allclose(host(ops.linear_forward(x, w, b)).ravel(), c["y"], atol=1e-3), c["source"]
    for c in ka["relu"]:
        x = dev(np.array(c["x"], np.float32))
        assert np.array_equal(host(ops.relu(x)), np.array(c["y"], np.float32))
        if "gx" in c:
            assert np.array_equal(host(ops.relu_backward(torch.ones_like(x), x)), np.array(c["gx"], np.float32))
    for c in ka["softmax_ce"]:
        x = dev(np.array(c["x"], np.float32).reshape(c["B"], c["C"]))
        t = dev(np.array(c["t"], np.int32))
        loss, _ = ops.softmax_cross_entropy(x, t)
        assert abs(loss.item() - c["loss"]) < c["tol"]
    for c in ka["conv2d_forward"]:
        x = dev(np.array(c["x"], np.float32).reshape(c["N"], c["C"], c["H"], c["W"]))
        w = dev(np.array(c["w"], np.float32).reshape(c["OC"], c["C"], c["KH"], c["KW"]))
        b = None if c["b"] is None else dev(np.array(c["b"], np.float32))
        y = ops.conv2d_forward(x, w, b, c["stride"], c["pad"])
        assert np.allclose(host(y).ravel(), c["y"], atol=1e-3), c["source"]
    for c in ka["weight_decay_hook"]:
        p, g = dev(np.array(c["p"], np.float32)), dev(np.array(c["g"], np.float32))
        ops.sgd_step(p, g, None, lr=0.01, hook_weight_decay=c["rate"])
        assert np.allclose(host(g), c["g_after"], atol=1e-5)


# ------------------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (2, 3, 5), (31, 127, 1), (127, 31, 1000), (300, 200, 100), (256, 520, 2080),
                                   (1, 1000, 1), (1024, 1024, 1024)])
def test_gemm_all_layouts_vs_oracle(ops, orc, M, N, K, ta, tb, precision):
    rng = np.random.default_rng(M * 7 + N * 3 + K + ta * 2 + tb)
    a = rng.standard_normal((K, M) if ta else (M, K), dtype=np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32)
    d = host(ops.gemm(dev(a), dev(b), trans_a=bool(ta), trans_b=bool(tb), precision=precision))
    opa = np.ascontiguousarray(a.T) if ta else a
    opb = np.ascontiguousarray(b.T) if tb else b
    if M * N * K <= 128 * 128 * 1100:
        ref = np.empty((M, N), np.float32)
        orc.oracle_matmul(opa, opb, ref, M, N, K)   # the reference's own fp32 loop
    else:
        ref = opa.astype(np.float64) @ opb.astype(np.float64)
    assert max_rel_err(d, ref) <= TOL[precision]


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("chunk", [1, 3, 0])
def test_gemm_tile_widths_and_accumulator_drains(ops, bn, chunk):
    from origindl_b200 import capi

    rng = np.random.default_rng(bn + chunk)
    M, N, K = 257, 515, 1500
    a, b = rng.standard_normal((M, K), dtype=np.float32), rng.standard_normal((K, N), dtype=np.float32)
    capi.call("odl_debug_set_tile_n", bn)
    capi.call("odl_debug_set_chunk", chunk)
    try:
        d = host(ops.gemm(dev(a), dev(b)))
    finally:
        capi.call("odl_debug_set_tile_n", 0)
        capi.call("odl_debug_set_chunk", 0)
    assert max_rel_err(d, a.astype(np.float64) @ b.astype(np.float64)) <= 1e-5


@pytest.mark.parametrize("splits", [1, 5, 0])
def test_gemm_split_k(ops, splits):
    from origindl_b200 import capi

    rng = np.random.default_rng(splits)
    M, N, K = 16, 108, 40000          # conv weight-gradient shape: tiny output, long reduction
    a, b = rng.standard_normal((K, M), dtype=np.float32), rng.standard_normal((K, N), dtype=np.float32)
    capi.call("odl_debug_set_split_k", splits)
    try:
        d = host(ops.gemm(dev(a), dev(b), trans_a=True))
    finally:
        capi.call("odl_debug_set_split_k", 0)
    assert max_rel_err(d, a.T.astype(np.float64) @ b.astype(np.float64)) <= 1e-5


@pytest.mark.parametrize("cluster", [2, 4, 0])
@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(512, 1000, 784), (200, 70, 1000), (130, 300, 96), (512, 10, 1000)])
def test_gemm_split_k_inside_a_cluster(ops, M, N, K, ta, tb, bn, cluster):
    """Split-K across the CTAs of a thread-block cluster (partial tiles combined through distributed shared memory by the
    CTA that runs the epilogue): every epilogue flag at once, all operand layouts, all tile widths (a cluster of 4 falls
    back to 2 where the staging area of the wider tiles holds only one partial tile), K ranges that leave the last rank
    short or empty, and the automatic choice (0).  Same bits on every run."""
    from origindl_b200 import capi

    rng = np.random.default_rng(M + N + K + 2 * ta + tb + bn)
    a = rng.standard_normal((K, M) if ta else (M, K), dtype=np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32)
    bias = rng.standard_normal(N, dtype=np.float32)
    aux = rng.standard_normal((M, N), dtype=np.float32)
    ref = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64) + bias
    ref = np.where(aux > 0, np.maximum(ref, 0), 0)
    capi.call("odl_debug_set_split_k", -cluster)
    capi.call("odl_debug_set_tile_n", bn)
    try:
        outs = []
        for _ in range(2):
            cs = torch.zeros(N, device="cuda")
            d, d_small = ops.gemm(dev(a), dev(b), trans_a=bool(ta), trans_b=bool(tb), bias=dev(bias), relu=True,
                                  mask_src=dev(aux), colsum=cs, want_small=True)
            outs.append((d, d_small, cs))
    finally:
        capi.call("odl_debug_set_split_k", 0)
        capi.call("odl_debug_set_tile_n", 0)
    capi.device_status()
    d, d_small, cs = outs[0]
    assert max_rel_err(host(d), ref) <= 1e-5
    assert max_rel_err(host(cs), ref.sum(0)) <= 1e-5
    assert torch.equal(d_small, ops.split_tf32(d))
    assert all(torch.equal(x, y) for x, y in zip(outs[0], outs[1]))


@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(129, 256, 32), (256, 300, 64), (300, 520, 100), (1024, 1024, 1024), (2048, 768, 515)])
def test_gemm_cta_pair_kernel(ops, M, N, K, ta, tb, precision):
    """The 2-CTA (cta_group::2) kernel, forced on shapes with ragged row / column / K tails, with the full epilogue."""
    from origindl_b200 import capi

    rng = np.random.default_rng(M + N + K + 2 * ta + tb)
    a = rng.standard_normal((K, M) if ta else (M, K), dtype=np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    mask = rng.standard_normal((M, N)).astype(np.float32)
    colsum = torch.zeros(N, device="cuda")
    capi.call("odl_debug_set_pair_mode", 2)
    capi.call("odl_debug_set_tile_n", 256)
    try:
        d, ds = ops.gemm(dev(a), dev(b), trans_a=bool(ta), trans_b=bool(tb), bias=dev(bias), relu=True, mask_src=dev(mask),
                         colsum=colsum, want_small=True, precision=precision)
    finally:
        capi.call("odl_debug_set_pair_mode", 0)
        capi.call("odl_debug_set_tile_n", 0)
    opa = a.T.astype(np.float64) if ta else a.astype(np.float64)
    opb = b.T.astype(np.float64) if tb else b.astype(np.float64)
    pre = opa @ opb + bias
    ref = np.maximum(pre, 0) * (mask > 0)
    # elements whose pre-activation is within the tolerance of zero may legitimately fall on either side of the ReLU
    tol = TOL[precision] * np.abs(pre).max()
    safe = np.abs(pre) > tol
    assert np.abs(host(d) - ref)[safe].max() <= tol
    assert np.abs(host(d) - ref).max() <= 2 * tol
    assert max_rel_err(host(colsum), ref.sum(0)) <= 10 * TOL[precision]
    assert torch.equal(ds, ops.split_tf32(d))


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K,pairs", [(129, 256, 32, 0), (300, 520, 100, 4), (1024, 1024, 1024, 3), (1024, 1024, 1024, 7),
                                         (1024, 1024, 1024, 16), (2048, 768, 515, 5), (2048, 768, 515, 11), (1500, 1300, 700, 9),
                                         (1024, 1024, 1024, -7), (2048, 768, 515, -5)])
def test_gemm_persistent_pair_kernel(ops, M, N, K, pairs, ta, tb):
    """The persistent 3xTF32 pair kernel, forced on small shapes with a small number of CTA pairs so that every pair
    walks several tiles (drawn from the global unit counter, or -- negative `pairs` -- by the fixed assignment; epilogue of
    tile i overlapping the main loop of tile i + 1, stage ring and accumulator buffers carried across tiles) and, where the last round is short, its tiles are split along K between two pairs (partial
    tiles parked in scratch, the second arriver combines).  Ragged row / column / K tails, all four operand layouts,
    the full epilogue -- once with column sums (transpose-slab stores) and once without (rows written straight from
    registers with 256-bit stores where D's rows are 32-byte aligned).  Checked against float64; where no tile is split
    the result must be bit-identical to the one-tile-per-pair kernel (same products, same order), and a second launch
    must give the same bits (tickets reset)."""
    from origindl_b200 import capi

    rng = np.random.default_rng(M + N + K + 2 * ta + tb + pairs)
    a = rng.standard_normal((K, M) if ta else (M, K), dtype=np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    mask = rng.standard_normal((M, N)).astype(np.float32)
    opa = a.T.astype(np.float64) if ta else a.astype(np.float64)
    opb = b.T.astype(np.float64) if tb else b.astype(np.float64)
    pre = opa @ opb + bias
    ref = np.maximum(pre, 0) * (mask > 0)
    tol = TOL[0] * np.abs(pre).max()
    safe = np.abs(pre) > tol
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    p_eff = abs(pairs) if pairs else 74
    r = tiles % p_eff
    split = r > 0 and 2 * r <= p_eff and (K + 31) // 32 >= 8
    for with_colsum in (True, False):
        outs = []
        capi.call("odl_debug_set_tile_n", 256)
        try:
            for mode, n_pairs in ((7, pairs), (7, pairs), (2, 0)):
                capi.call("odl_debug_set_pair_mode", mode)
                capi.call("odl_debug_set_persistent_pairs", n_pairs)
                colsum = torch.zeros(N, device="cuda") if with_colsum else None
                d, ds = ops.gemm(dev(a), dev(b), trans_a=bool(ta), trans_b=bool(tb), bias=dev(bias), relu=True,
                                 mask_src=dev(mask), colsum=colsum, want_small=True)
                outs.append((d, ds) + ((colsum,) if with_colsum else ()))
        finally:
            capi.call("odl_debug_set_pair_mode", 0)
            capi.call("odl_debug_set_tile_n", 0)
            capi.call("odl_debug_set_persistent_pairs", 0)
        capi.device_status()
        d, ds = outs[0][:2]
        assert np.abs(host(d) - ref)[safe].max() <= tol
        assert np.abs(host(d) - ref).max() <= 2 * tol
        if with_colsum:
            assert max_rel_err(host(outs[0][2]), ref.sum(0)) <= 10 * TOL[0]
        assert torch.equal(ds, ops.split_tf32(d))
        assert all(torch.equal(x, y) for x, y in zip(outs[0], outs[1]))          # same bits on a second launch
        if not split:
            assert all(torch.equal(x, y) for x, y in zip(outs[0][:2], outs[2][:2]))  # identical to one tile per pair
            if with_colsum:   # (the column sums add the same 32-row slabs in another fixed order: butterfly vs slab)
                assert max_rel_err(host(outs[0][2]), host(outs[2][2])) <= 1e-5


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K,pairs", [(512, 512, 2048, 3), (1024, 1024, 1024, 7), (2048, 768, 515, 5), (300, 520, 100, 4),
                                         (1500, 1300, 700, 9), (256, 1024, 4096, 0), (640, 512, 96, 74)])
def test_gemm_stream_k(ops, M, N, K, pairs, ta, tb):
    """Stream-K in the persistent pair kernel, forced: the accumulator chunks of the whole problem are cut into one
    contiguous range per CTA pair, so pairs work on tails, whole tiles and heads; every tile cut by a range boundary is
    parked part by part and finished by whichever contributor takes the last ticket, adding the parts in part order.
    Shapes with two to five parts per tile, ragged tails, more pairs than chunks, all operand layouts, the full epilogue
    with and without column sums; against float64, and the same bits on a second launch (arrival order must not matter)."""
    from origindl_b200 import capi

    rng = np.random.default_rng(M + N + K + 2 * ta + tb + pairs + 1)
    a = rng.standard_normal((K, M) if ta else (M, K), dtype=np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    mask = rng.standard_normal((M, N)).astype(np.float32)
    opa = a.T.astype(np.float64) if ta else a.astype(np.float64)
    opb = b.T.astype(np.float64) if tb else b.astype(np.float64)
    pre = opa @ opb + bias
    ref = np.maximum(pre, 0) * (mask > 0)
    tol = TOL[0] * np.abs(pre).max()
    safe = np.abs(pre) > tol
    for with_colsum in (True, False):
        outs = []
        capi.call("odl_debug_set_tile_n", 256)
        capi.call("odl_debug_set_pair_mode", 7)
        capi.call("odl_debug_set_stream_k", 1)
        capi.call("odl_debug_set_persistent_pairs", pairs)
        try:
            for _ in range(2):
                colsum = torch.zeros(N, device="cuda") if with_colsum else None
                d, ds = ops.gemm(dev(a), dev(b), trans_a=bool(ta), trans_b=bool(tb), bias=dev(bias), relu=True,
                                 mask_src=dev(mask), colsum=colsum, want_small=True)
                outs.append((d, ds) + ((colsum,) if with_colsum else ()))
        finally:
            capi.call("odl_debug_set_pair_mode", 0)
            capi.call("odl_debug_set_tile_n", 0)
            capi.call("odl_debug_set_stream_k", 0)
            capi.call("odl_debug_set_persistent_pairs", 0)
        capi.device_status()
        d, ds = outs[0][:2]
        assert np.abs(host(d) - ref)[safe].max() <= tol
        assert np.abs(host(d) - ref).max() <= 2 * tol
        if with_colsum:
            assert max_rel_err(host(outs[0][2]), ref.sum(0)) <= 10 * TOL[0]
        assert torch.equal(ds, ops.split_tf32(d))
        assert all(torch.equal(x, y) for x, y in zip(outs[0], outs[1]))


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(129, 256, 32), (256, 300, 64), (300, 520, 100), (1024, 1024, 1024), (2048, 768, 515),
                                   (512, 1600, 288)])
def test_gemm_wide_tf32_pair_tile(ops, M, N, K, ta, tb):
    """Plain TF32 on the 256 x 512 pair tile (two 256-column MMAs per K-step into one 512-column accumulator), forced on
    shapes with ragged row / column / K tails and second halves that are partly or wholly outside the matrix, with the
    full epilogue; against float64 within the TF32 bound and bit-identical to the 256 x 256 pair tile."""
    from origindl_b200 import capi

    rng = np.random.default_rng(M + N + K + 2 * ta + tb + 5)
    a = rng.standard_normal((K, M) if ta else (M, K), dtype=np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    mask = rng.standard_normal((M, N)).astype(np.float32)
    outs = {}
    capi.call("odl_debug_set_tile_n", 256)
    try:
        for mode in (5, 2):
            capi.call("odl_debug_set_pair_mode", mode)
            colsum = torch.zeros(N, device="cuda")
            d, ds = ops.gemm(dev(a), dev(b), trans_a=bool(ta), trans_b=bool(tb), bias=dev(bias), relu=True,
                             mask_src=dev(mask), colsum=colsum, want_small=True, precision=1)
            outs[mode] = (d, ds, colsum)
    finally:
        capi.call("odl_debug_set_pair_mode", 0)
        capi.call("odl_debug_set_tile_n", 0)
    capi.device_status()
    d, ds, colsum = outs[5]
    opa = a.T.astype(np.float64) if ta else a.astype(np.float64)
    opb = b.T.astype(np.float64) if tb else b.astype(np.float64)
    pre = opa @ opb + bias
    ref = np.maximum(pre, 0) * (mask > 0)
    tol = TOL[1] * np.abs(pre).max()
    safe = np.abs(pre) > tol
    assert np.abs(host(d) - ref)[safe].max() <= tol
    assert max_rel_err(host(colsum), ref.sum(0)) <= 10 * TOL[1]
    assert torch.equal(ds, ops.split_tf32(d))
    assert torch.equal(d, outs[2][0]) and torch.equal(colsum, outs[2][2])  # same products, same accumulation order


def test_gemm_epilogues(ops):
    rng = np.random.default_rng(3)
    M, N, K = 200, 333, 150
    a, b = rng.standard_normal((M, K), dtype=np.float32), rng.standard_normal((K, N), dtype=np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    mask = rng.standard_normal((M, N)).astype(np.float32)
    colsum = torch.zeros(N, device="cuda")
    d, ds = ops.gemm(dev(a), dev(b), bias=dev(bias), relu=True, mask_src=dev(mask), colsum=colsum, want_small=True)
    ref = np.maximum(a.astype(np.float64) @ b + bias, 0) * (mask > 0)
    assert max_rel_err(host(d), ref) <= 1e-5
    assert max_rel_err(host(colsum), ref.sum(0)) <= 1e-5
    big = host(d).view(np.uint32) & np.uint32(0xFFFFE000)
    resid = host(d) - big.view(np.float32)
    # the low part is the residual rounded to tf32: within 2^-11 of it and with 13 zero low bits
    assert np.all(np.abs(host(ds) - resid) <= np.abs(resid) * 2.0 ** -11 + 1e-45)
    assert np.all(host(ds).view(np.uint32) & np.uint32(0x1FFF) == 0)


def test_batched_matmul_forms(ops, orc):
    rng = np.random.default_rng(9)
    a = rng.standard_normal((3, 17, 20), dtype=np.float32)
    b2 = rng.standard_normal((20, 9), dtype=np.float32)
    b3 = rng.standard_normal((3, 20, 9), dtype=np.float32)
    assert max_rel_err(host(ops.matmul(dev(a), dev(b2))), a.astype(np.float64) @ b2) <= 1e-5
    assert max_rel_err(host(ops.matmul(dev(a), dev(b3))), a.astype(np.float64) @ b3) <= 1e-5
    with pytest.raises(ValueError):
        ops.matmul(dev(a[0]), dev(b2[:5]))


def test_invalid_arguments_are_rejected(ops):
    from origindl_b200 import capi

    x = torch.zeros((4, 4), device="cuda")
    with pytest.raises(capi.OdlError):
        capi.call("odl_gemm_ex", 0, 0, 4, 4, 4, x.data_ptr(), None, 2, x.data_ptr(), None, 4, x.data_ptr(), None, 4, None,
                  None, 0, None, 0, 0, capi.stream_handle())          # lda < K
    with pytest.raises(capi.OdlError):
        capi.call("odl_gemm_ex", 0, 0, 4, 4, 4, x.data_ptr(), None, 4, x.data_ptr(), None, 4, x.data_ptr(), None, 4, None,
                  None, 0, None, capi.EPI_BIAS, 0, capi.stream_handle())  # flag without pointer
    with pytest.raises(capi.OdlError):
        capi.call("odl_matmul", None, x.data_ptr(), x.data_ptr(), 4, 4, 4, 1, 0, 0, capi.stream_handle())
    with pytest.raises(ValueError):
        ops.conv2d_forward(torch.zeros((1, 1, 2, 2), device="cuda"), torch.zeros((1, 1, 3, 3), device="cuda"))
    logits, bad = torch.zeros((2, 3), device="cuda"), torch.tensor([0, 3], device="cuda", dtype=torch.int32)
    ops.softmax_cross_entropy(logits, bad)
    with pytest.raises(capi.OdlError):
        capi.device_status()                                       # label out of range, like the reference's throw
    capi.device_status()


# ------------------------------------------------------------------------------------------------ Linear
@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("w_layout", [0, 1])
@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("M,N,K", [(5, 3, 4), (64, 48, 40), (130, 257, 65), (512, 1000, 784), (512, 10, 1000)])
def test_linear_fwd_bwd_vs_oracle(ops, orc, M, N, K, w_layout, relu, precision):
    rng = np.random.default_rng(M + N + K + w_layout)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = rng.standard_normal((N, K) if w_layout == 0 else (K, N), dtype=np.float32)
    b = (0.1 * rng.standard_normal(N)).astype(np.float32)
    dy = rng.standard_normal((M, N), dtype=np.float32)
    y_o, dx_o, dw_o, db_o = np.empty((M, N), np.float32), np.empty_like(x), np.empty_like(w), np.empty(N, np.float32)
    orc.oracle_linear_forward(x, w, fptr(b), y_o, M, N, K, w_layout, int(relu))
    y = ops.linear_forward(dev(x), dev(w), dev(b), relu=relu, w_layout=w_layout, precision=precision)
    tol = TOL[precision]
    assert max_rel_err(host(y), y_o) <= tol
    # backward takes the mask from the forward output of the SAME implementation, so feed it the oracle's y:
    # elements within rounding of zero would otherwise flip the mask and dominate the comparison
    orc.oracle_linear_backward(x, w, fptr(y_o), dy, fptr(dx_o), fptr(dw_o), fptr(db_o), M, N, K, w_layout, int(relu))
    dx, dw, db = ops.linear_backward(dev(x), dev(w), dev(dy), dev(y_o) if relu else None, w_layout=w_layout,
                                     precision=precision)
    assert max_rel_err(host(dx), dx_o) <= tol
    assert max_rel_err(host(dw), dw_o) <= tol
    assert max_rel_err(host(db), db_o) <= 1e-5


def test_linear_golden_vectors_from_reference(ops):
    g = np.load(GOLDEN / "reference_vectors.npz")
    for tag in ("lin_a", "lin_b"):
        for wl in (0, 1):
            k = f"{tag}_l{wl}_"
            y = ops.linear_forward(dev(g[k + "x"]), dev(g[k + "w"]), dev(g[k + "b"]), relu=True, w_layout=wl)
            assert max_rel_err(host(y), g[k + "y"]) <= 1e-5
            dx, dw, db = ops.linear_backward(dev(g[k + "x"]), dev(g[k + "w"]), dev(g[k + "dy"]), dev(g[k + "y"]),
                                             w_layout=wl)
            assert max_rel_err(host(dx), g[k + "dx"]) <= 1e-5
            assert max_rel_err(host(dw), g[k + "dw"]) <= 1e-5
            assert max_rel_err(host(db), g[k + "db"].ravel()) <= 1e-5


def test_chained_backward_matches_unfused(ops):
    """dx epilogue with the previous layer's mask / bias gradient / low part == separate passes."""
    from origindl_b200 import capi

    rng = np.random.default_rng(21)
    M, N, K = 192, 160, 224
    x = np.maximum(rng.standard_normal((M, K), dtype=np.float32), 0)     # previous layer's ReLU output
    w = rng.standard_normal((K, N), dtype=np.float32)
    dy = rng.standard_normal((M, N), dtype=np.float32)
    xd, wd, dyd = dev(x), dev(w), dev(dy)
    dx_ref, dw_ref, db_ref = ops.linear_backward(xd, wd, dyd, None, w_layout=1)
    masked = ops.relu_backward(dx_ref, xd)
    prev_db_ref = ops.sum_to_row(masked)
    dx, dxs = torch.empty_like(xd), torch.empty_like(xd)
    dw, db, pdb = torch.empty_like(wd), torch.empty(N, device="cuda"), torch.empty(K, device="cuda")
    capi.call("odl_linear_backward_chain", xd.data_ptr(), None, wd.data_ptr(), None, dyd.data_ptr(), None, None,
              dx.data_ptr(), dxs.data_ptr(), xd.data_ptr(), pdb.data_ptr(), dw.data_ptr(), db.data_ptr(), M, N, K, 1, 0,
              capi.stream_handle())
    assert torch.equal(dx, masked)
    assert max_rel_err(host(pdb), host(prev_db_ref).ravel()) <= 1e-5
    assert torch.equal(dw, dw_ref) and torch.equal(dxs, ops.split_tf32(masked))


# ------------------------------------------------------------------------------------------------ loss / optimizers
@pytest.mark.parametrize("B,C", [(1, 3), (512, 10), (300, 1000), (64, 1024)])
def test_softmax_ce_vs_oracle(ops, orc, B, C):
    rng = np.random.default_rng(B + C)
    x = (3 * rng.standard_normal((B, C))).astype(np.float32)
    t = rng.integers(0, C, B).astype(np.int32)
    l_o, d_o = ctypes.c_float(), np.empty_like(x)
    assert orc.oracle_softmax_ce(x, t, B, C, ctypes.byref(l_o), fptr(d_o)) == 0
    for labels in (dev(t), dev(t.astype(np.int64))):
        loss, d = ops.softmax_cross_entropy(dev(x), labels)
        assert abs(loss.item() - l_o.value) <= 1e-5 * max(1.0, abs(l_o.value))
        assert max_rel_err(host(d), d_o) <= 1e-5


def test_optimizer_trajectories_vs_reference_golden(ops):
    g = np.load(GOLDEN / "reference_vectors.npz")
    p0, grads = g["opt_p0"], g["opt_grads"]
    cases = {"adam_wd": dict(opt=1, lr=1e-3, hook=1e-4), "sgd_mom": dict(opt=0, lr=1e-2, mom=0.9),
             "sgd_nes_wd": dict(opt=0, lr=1e-2, mom=0.9, wd=1e-2, nes=True)}
    for tag, c in cases.items():
        p = dev(p0)
        m, v, buf = torch.zeros_like(p), torch.zeros_like(p), torch.zeros_like(p)
        for s in range(grads.shape[0]):
            gr = dev(grads[s])
            if c["opt"] == 1:
                ops.adam_step(p, gr, m, v, s + 1, lr=c["lr"], hook_weight_decay=c.get("hook", 0.0))
            else:
                ops.sgd_step(p, gr, buf, lr=c["lr"], momentum=c.get("mom", 0.0), weight_decay=c.get("wd", 0.0),
                             nesterov=c.get("nes", False))
        assert max_rel_err(host(p), g["opt_" + tag]) <= 1e-6, tag


def test_optimizer_steps_vs_oracle_odd_sizes(ops, orc):
    rng = np.random.default_rng(8)
    for n in (1, 3, 1027):
        p0, g0 = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
        m0, v0 = rng.standard_normal(n).astype(np.float32) * 0.1, rng.uniform(0, 1, n).astype(np.float32)
        p, g, m, v = p0.copy(), g0.copy(), m0.copy(), v0.copy()
        orc.oracle_adam_step(p, g, m, v, n, 3, 1e-3, 0.9, 0.999, 1e-8, 1e-4)
        pd, gd, md, vd, ps = dev(p0), dev(g0), dev(m0), dev(v0), torch.empty(n, device="cuda")
        ops.adam_step(pd, gd, md, vd, 3, hook_weight_decay=1e-4, p_small=ps)
        assert max_rel_err(host(pd), p) <= 1e-6 and np.array_equal(host(gd), g)
        assert np.array_equal(host(md), m) and np.array_equal(host(vd), v)
        assert torch.equal(ps, ops.split_tf32(pd.reshape(1, -1)).reshape(-1))


# ------------------------------------------------------------------------------------------------ Conv2d
CONV_CASES = [(1, 1, 3, 3, 1, 2, 1, 0), (2, 3, 9, 7, 4, 3, 1, 1), (2, 3, 16, 16, 8, 3, 2, 1), (1, 2, 12, 12, 5, 6, 2, 2),
              (2, 4, 5, 5, 3, 1, 1, 0), (2, 16, 20, 20, 32, 3, 2, 1), (1, 64, 10, 10, 64, 3, 1, 1)]


@pytest.mark.parametrize("N,C,H,W,OC,k,s,p", CONV_CASES)
def test_conv2d_vs_oracle(ops, orc, N, C, H, W, OC, k, s, p):
    rng = np.random.default_rng(N + C + H + OC + k)
    x = rng.uniform(0, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = (0.1 * rng.standard_normal(OC)).astype(np.float32)
    OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    dy = rng.standard_normal((N, OC, OH, OW)).astype(np.float32)
    y_o = np.empty_like(dy)
    orc.oracle_conv2d_forward(x, w, fptr(b), y_o, N, C, H, W, OC, k, k, s, p)
    y = ops.conv2d_forward(dev(x), dev(w), dev(b), s, p)
    assert max_rel_err(host(y), y_o) <= 1e-5
    for mode in (0, 1):
        dx_o, dw_o, db_o = np.empty_like(x), np.empty_like(w), np.empty_like(b)
        orc.oracle_conv2d_backward(dy, x, w, fptr(dx_o), fptr(dw_o), fptr(db_o), N, C, H, W, OC, k, k, s, p, mode)
        gx, gw, gb = ops.conv2d_backward(dev(dy), dev(x), dev(w), s, p, gy_layout=mode)
        assert max_rel_err(host(gx), dx_o) <= 1e-5
        assert max_rel_err(host(gw), dw_o) <= 1e-5
        assert max_rel_err(host(gb), db_o) <= 1e-5


IGEMM_CASES = CONV_CASES + [(3, 3, 33, 29, 16, 6, 2, 2),      # ragged pixel count, K = 108 (not a multiple of 32)
                            (2, 5, 11, 13, 70, 3, 1, 1),      # K = 45 (not a multiple of 4: padded weights), 64 < OC
                            (1, 8, 14, 14, 130, 3, 2, 0),     # OC > 128: two column tiles
                            (1, 64, 6, 6, 32, 3, 1, 1),       # K = 576, the longest reduction one CTA keeps in TMEM
                            (1, 128, 6, 6, 32, 3, 1, 1),      # K = 1152: a cluster of two CTAs splits K
                            (1, 130, 6, 6, 8, 3, 1, 1),       # K = 1170: three CTAs (37 K-blocks: 13 + 13 + 11)
                            (2, 256, 7, 9, 200, 3, 1, 1),     # K = 2304 = 256 channels x 3 x 3: four CTAs, the longest implicit reduction
                            (1, 260, 5, 5, 12, 3, 1, 1)]      # K = 2340: falls back to the explicit path


@pytest.mark.parametrize("N,C,H,W,OC,k,s,p", IGEMM_CASES)
@pytest.mark.parametrize("precision", ["3xtf32", "tf32"])
def test_conv2d_forward_implicit_and_explicit_paths(ops, orc, N, C, H, W, OC, k, s, p, precision):
    """The forward pass has three implementations -- a direct fp32 kernel for small layers (OC <= 32, C*KH*KW <= 256: mode 0
    takes it where it applies), implicit GEMM (tiles of the column matrix gathered in shared memory; mode 3 sends the small
    layers there too) and im2col + GEMM (mode 1); all against the oracle, with and without bias, with the fused
    activations.  The direct kernel computes in plain fp32 whatever the precision argument says."""
    from origindl_b200 import capi

    prec, tol = (capi.PRECISION_3XTF32, 1e-5) if precision == "3xtf32" else (capi.PRECISION_TF32, 5e-3)
    rng = np.random.default_rng(N * 7 + C + H + OC + k)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = (0.1 * rng.standard_normal(OC)).astype(np.float32)
    OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    y_o, y_nb = np.empty((N, OC, OH, OW), np.float32), np.empty((N, OC, OH, OW), np.float32)
    orc.oracle_conv2d_forward(x, w, fptr(b), y_o, N, C, H, W, OC, k, k, s, p)
    orc.oracle_conv2d_forward(x, w, None, y_nb, N, C, H, W, OC, k, k, s, p)
    xd, wd, bd = dev(x), dev(w), dev(b)
    try:
        for mode in (0, 3, 1):
            capi.lib().odl_debug_set_conv_mode(mode)
            assert max_rel_err(host(ops.conv2d_forward(xd, wd, bd, s, p, precision=prec)), y_o) <= tol
            assert max_rel_err(host(ops.conv2d_forward(xd, wd, None, s, p, precision=prec)), y_nb) <= tol
            relu = host(ops.conv2d_forward(xd, wd, bd, s, p, relu=1, precision=prec))
            assert max_rel_err(relu, np.maximum(y_o, 0)) <= tol
            silu = host(ops.conv2d_forward(xd, wd, bd, s, p, relu=2, precision=prec))
            z = y_o.astype(np.float64)
            assert max_rel_err(silu, z / (1 + np.exp(-z))) <= tol
    finally:
        capi.lib().odl_debug_set_conv_mode(0)
    capi.device_status()


@pytest.mark.parametrize("N,C,H,W,OC,k,s,p", IGEMM_CASES + [(2, 6, 17, 15, 12, 5, 3, 2), (1, 2, 9, 9, 3, 4, 2, 1),
                                                            (1, 20, 9, 9, 300, 1, 1, 0),   # 1x1, 300 products per gx element
                                                            (2, 40, 8, 10, 48, 3, 1, 0),   # stride 1 without padding
                                                            (1, 40, 8, 8, 40, 3, 1, 2),    # stride 1, pad = k - 1
                                                            (3, 3, 40, 36, 16, 6, 2, 2),   # gw over 3 images x 12 pixel blocks
                                                            (2, 24, 16, 16, 200, 3, 1, 1),  # two output-channel tiles, 216 k-rows
                                                            (2, 16, 21, 19, 32, 3, 2, 1),  # the compile-time gx shapes of the CNN:
                                                            (2, 32, 9, 11, 32, 1, 1, 0),   # 16 -> 32 3x3 / 2, 32 -> 32 1x1,
                                                            (2, 6, 12, 10, 16, 3, 1, 1),   # 16 output channels 3x3 / 1 and / 2
                                                            (2, 7, 13, 12, 16, 3, 2, 0),   # (ragged channel groups)
                                                            (2, 12, 10, 12, 16, 3, 1, 1)]) # eight channels per thread, ragged
def test_conv2d_input_gradient_direct_and_gemm_paths(ops, orc, N, C, H, W, OC, k, s, p):
    """gx has three implementations: a direct fp32 kernel (few products per output; the reference's summation order, so
    BIT-EXACT against the oracle); for stride 1 in the correct gradient layout the implicit-GEMM convolution of gy with the
    flipped, transposed weights; and GEMM + gather col2im (both 3xTF32, 1e-5).  gw: a direct fp32 kernel for small layers,
    the implicit GEMM over pixels (correct layout, OH*OW a multiple of 4) and im2col + split-K GEMM.  Both gradient
    layouts, with the implicit paths on and forced off."""
    from origindl_b200 import capi

    rng = np.random.default_rng(N * 11 + C + H + OC + k + s)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    dy = rng.standard_normal((N, OC, OH, OW)).astype(np.float32)
    direct = OC * (-(-k // s)) ** 2 <= 256
    try:
        for layout in (0, 1):
            dx_o, dw_o = np.empty_like(x), np.empty_like(w)
            orc.oracle_conv2d_backward(dy, x, w, fptr(dx_o), fptr(dw_o), None, N, C, H, W, OC, k, k, s, p, layout)
            capi.lib().odl_debug_set_conv_mode(0)
            gx, gw, _ = ops.conv2d_backward(dev(dy), dev(x), dev(w), s, p, gy_layout=layout, need_gb=False)
            if direct:
                assert np.array_equal(host(gx), dx_o)
                for conv_mode in (4, 5, 8):  # 4: the generic direct kernel where a compile-time shape exists; 5: that shape
                    # with one position per thread instead of two; 8: four input channels per thread instead of eight
                    capi.lib().odl_debug_set_conv_mode(conv_mode)
                    gx4, _, _ = ops.conv2d_backward(dev(dy), dev(x), dev(w), s, p, gy_layout=layout, need_gb=False)
                    assert np.array_equal(host(gx4), dx_o), conv_mode
            else:
                assert max_rel_err(host(gx), dx_o) <= 1e-5
            assert max_rel_err(host(gw), dw_o) <= 1e-5  # direct fp32 kernel when OC <= 32 and C*KH*KW <= 256
            for conv_mode in (6, 7, 2, 1):  # 6 / 7: gw of small layers from gathered column blocks / from image tiles always;
                # 2: small layers through the implicit-GEMM gw kernel too; 1: explicit paths only
                capi.lib().odl_debug_set_conv_mode(conv_mode)
                gx, gw, _ = ops.conv2d_backward(dev(dy), dev(x), dev(w), s, p, gy_layout=layout, need_gb=False)
                assert max_rel_err(host(gx), dx_o) <= 1e-5 and max_rel_err(host(gw), dw_o) <= 1e-5
    finally:
        capi.lib().odl_debug_set_conv_mode(0)
    capi.device_status()


@pytest.mark.parametrize("N,C,H,W,OC,k,s,p", [(4, 3, 64, 64, 16, 6, 2, 2), (4, 16, 40, 40, 32, 3, 2, 1), (4, 64, 20, 20, 64, 3, 1, 1),
                                              (2, 20, 9, 9, 300, 1, 1, 0)])
def test_conv2d_backward_is_reproducible(ops, N, C, H, W, OC, k, s, p):
    """Same inputs, same bits, in every path and both gradient layouts: the reductions over pixels (bias gradient, direct
    and implicit-GEMM weight gradients, split-K) add their partial sums in a fixed order."""
    from origindl_b200 import capi

    g = torch.Generator(device="cuda").manual_seed(N + C + OC)
    x = torch.randn(N, C, H, W, device="cuda", generator=g)
    w = torch.randn(OC, C, k, k, device="cuda", generator=g)
    OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    gy = torch.randn(N, OC, OH, OW, device="cuda", generator=g)
    try:
        for conv_mode in (0, 6, 7, 2, 1):
            capi.lib().odl_debug_set_conv_mode(conv_mode)
            for layout in (0, 1):
                runs = [ops.conv2d_backward(gy, x, w, s, p, gy_layout=layout) for _ in range(3)]
                for other in runs[1:]:
                    assert all(torch.equal(a, b) for a, b in zip(runs[0], other)), (conv_mode, layout)
    finally:
        capi.lib().odl_debug_set_conv_mode(0)
    capi.device_status()


@pytest.mark.parametrize("C,OC,k,s,p,hw", [(3, 16, 6, 2, 2, 320), (16, 32, 3, 2, 1, 160), (32, 32, 1, 1, 0, 80), (64, 64, 3, 1, 1, 40)])
def test_conv2d_benchmark_layers_at_full_size(ops, orc, C, OC, k, s, p, hw):
    """The four conv shapes of the benchmark at batch 16: forward against the oracle (the reference's CPU arithmetic);
    backward -- where the scalar oracle needs tens of seconds per layer -- against float64 gradients of the same
    convolution (torch autograd as the checker), all three gradients within 1e-5."""
    N = 16
    rng = np.random.default_rng(C + OC + hw)
    x = rng.uniform(0, 1, (N, C, hw, hw)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = (0.1 * rng.standard_normal(OC)).astype(np.float32)
    OH = (hw + 2 * p - k) // s + 1
    y_o = np.empty((N, OC, OH, OH), np.float32)
    orc.oracle_conv2d_forward(x, w, fptr(b), y_o, N, C, hw, hw, OC, k, k, s, p)
    xd, wd, bd = dev(x), dev(w), dev(b)
    assert max_rel_err(host(ops.conv2d_forward(xd, wd, bd, s, p)), y_o) <= 1e-5
    gy = torch.randn(N, OC, OH, OH, device="cuda", generator=torch.Generator(device="cuda").manual_seed(hw))
    gx, gw, gb = ops.conv2d_backward(gy, xd, wd, s, p, gy_layout=0)
    x64, w64 = xd.double().requires_grad_(), wd.double().requires_grad_()
    torch.nn.functional.conv2d(x64, w64, None, stride=s, padding=p).backward(gy.double())
    for got, want in ((gx, x64.grad), (gw, w64.grad), (gb, gy.double().sum((0, 2, 3)))):
        assert ((got.double() - want).abs().max() / want.abs().max()).item() <= 1e-5
    ops_capi = __import__("origindl_b200.capi", fromlist=["capi"])
    ops_capi.device_status()


def test_conv2d_golden_vectors_from_reference(ops):
    g = np.load(GOLDEN / "reference_vectors.npz")
    N, C, H, W, OC, k, s, p = (int(v) for v in g["conv_cfg"])
    y = ops.conv2d_forward(dev(g["conv_x"]), dev(g["conv_w"]), dev(g["conv_b"]), s, p)
    assert max_rel_err(host(y), g["conv_y"]) <= 1e-5
    gx, gw, gb = ops.conv2d_backward(dev(g["conv_dy"]), dev(g["conv_x"]), dev(g["conv_w"]), s, p, gy_layout=1)
    assert max_rel_err(host(gx), g["conv_dx_reflayout"]) <= 1e-5
    assert max_rel_err(host(gw), g["conv_dw_reflayout"]) <= 1e-5
    assert max_rel_err(host(gb), g["conv_db"]) <= 1e-5


def test_im2col_col2im_pair(ops, orc):
    rng = np.random.default_rng(2)
    N, C, H, W, k, s, p = 2, 4, 9, 11, 3, 2, 1
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    col_o = np.empty((N * OH * OW, C * k * k), np.float32)
    orc.oracle_im2col(x, col_o, N, C, H, W, k, k, s, p)
    col = ops.im2col(dev(x), k, s, p)
    assert np.array_equal(host(col), col_o)                          # pure data movement: bit exact
    back_o = np.empty_like(x)
    orc.oracle_col2im(col_o, back_o, N, C, H, W, k, k, s, p)
    assert np.array_equal(host(ops.col2im(col, x.shape, k, s, p)), back_o)   # same (kh, kw) accumulation order


# ------------------------------------------------------------------------------------------------ full-size properties
def test_full_size_linearity_and_row_samples(ops):
    """M = N = K = 8192: sampled rows against float64, and linearity D(a1 + a2) == D(a1) + D(a2) to 3xTF32 accuracy."""
    torch.manual_seed(0)
    n = 8192
    a, b = torch.randn(n, n, device="cuda"), torch.randn(n, n, device="cuda")
    d = ops.gemm(a, b, trans_b=True)
    rows = torch.randint(0, n, (48,), device="cuda")
    ref = a[rows].double() @ b.double().t()
    assert ((d[rows].double() - ref).abs().max() / ref.abs().max()).item() <= 1e-5
    a2 = torch.randn(n, n, device="cuda")
    d2 = ops.gemm(a2, b, trans_b=True)
    d12 = ops.gemm(a + a2, b, trans_b=True)
    assert ((d12 - (d + d2)).abs().max() / d12.abs().max()).item() <= 2e-5
    # plain TF32 stays inside its own bound
    dt = ops.gemm(a, b, trans_b=True, precision=1)
    assert ((dt[rows].double() - ref).abs().max() / ref.abs().max()).item() <= 5e-3


@pytest.mark.parametrize("M,N,K", [(65536, 1024, 1024), (256, 8192, 8192)])
def test_skinny_linear_backward_row_samples(ops, M, N, K):
    torch.manual_seed(1)
    x, w = torch.randn(M, K, device="cuda"), torch.randn(N, K, device="cuda")
    dy = torch.randn(M, N, device="cuda")
    dx, dw, db = ops.linear_backward(x, w, dy, None, w_layout=0)
    r = torch.randint(0, M, (32,), device="cuda")
    ref = dy[r].double() @ w.double()
    assert ((dx[r].double() - ref).abs().max() / ref.abs().max()).item() <= 1e-5
    c = torch.randint(0, N, (32,), device="cuda")
    ref = dy[:, c].double().t() @ x.double()
    assert ((dw[c].double() - ref).abs().max() / ref.abs().max()).item() <= 1e-5
    ref = dy.double().sum(0)
    assert ((db.double() - ref).abs().max() / ref.abs().max()).item() <= 1e-5


@pytest.mark.parametrize("n", [2048, 4096, 8192])
def test_full_size_linear_forward_backward_rows_against_the_oracle(ops, orc, n):
    """M = N = K = n of the benchmark's Linear sweep, every operand layout of the layer (forward x.W^T, dX = g.W with an
    MN-major B, dW = g^T.x with both operands MN-major) against the ORACLE ITSELF, by row subset: row i of a product of
    the reference depends only on row i of its left operand, one fp32 accumulator, k ascending
    (src/mat/origin/cpu/math/matmul.cpp:29-41), so calling the oracle on 16 sampled rows of the left operand gives the
    reference's exact values for those rows of y and dX, and -- with the left operand g^T -- of dW; db is compared in
    full.  The ReLU mask comes from the same y on both sides (y is an input of the backward call), so a value within
    rounding of zero cannot flip one side's mask."""
    gen = torch.Generator(device="cuda").manual_seed(n)
    x, w = torch.randn((n, n), device="cuda", generator=gen), torch.randn((n, n), device="cuda", generator=gen)
    b, dy = 0.1 * torch.randn((n,), device="cuda", generator=gen), torch.randn((n, n), device="cuda", generator=gen)
    y = ops.linear_forward(x, w, b, relu=True)
    dx, dw, db = ops.linear_backward(x, w, dy, y)
    rows = np.sort(np.random.default_rng(n).choice(n, 16, replace=False))
    xh, wh, bh, yh = host(x), host(w), host(b), host(y)
    gh = host(dy) * (yh > 0)                                            # ReLU::backward: gy * mask, exact in fp32
    r = len(rows)
    # forward: y[rows] = relu(x[rows] . W^T + b)
    y_o = np.empty((r, n), np.float32)
    orc.oracle_linear_forward(np.ascontiguousarray(xh[rows]), wh, fptr(bh), y_o, r, n, n, 0, 1)
    assert max_rel_err(yh[rows], y_o) <= 1e-5
    # dX[rows] = g[rows] . W     (W is [N, K]: already the [reduce, out] matrix)
    dx_o = np.empty((r, n), np.float32)
    orc.oracle_matmul(np.ascontiguousarray(gh[rows]), wh, dx_o, r, n, n)
    assert max_rel_err(host(dx[torch.from_numpy(rows).cuda()]), dx_o) <= 1e-5
    # dW[rows] = (g^T)[rows] . x  (rows of g^T = columns of g)
    dw_o = np.empty((r, n), np.float32)
    orc.oracle_matmul(np.ascontiguousarray(gh[:, rows].T), xh, dw_o, r, n, n)
    assert max_rel_err(host(dw[torch.from_numpy(rows).cuda()]), dw_o) <= 1e-5
    # db = column sums of g, all of it (one fp32 accumulator over m, ascending, on the oracle)
    db_o = np.empty(n, np.float32)
    orc.oracle_colsum(gh, db_o, n, n)
    assert max_rel_err(host(db), db_o) <= 1e-5
