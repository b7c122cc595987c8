"""GPU: the device-resident MLP training step (odl_mlp_*) against the reference's own loss curves and parameters
(golden vectors from the unmodified reference) and against the oracle at other sizes."""
from pathlib import Path

import numpy as np
import pytest
import torch

import _libs
from _libs import max_rel_err

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def trainer_cls():
    from origindl_b200 import capi
    from origindl_b200.trainer import MLPTrainer

    capi.init(0)
    yield MLPTrainer
    capi.device_status()


def run(tr, xs, ts, steps):
    xd, td = torch.from_numpy(xs).cuda(), torch.from_numpy(ts).cuda()
    losses = []
    for s in range(steps):
        losses.append(tr.train_step(xd[s % xd.shape[0]], td[s % td.shape[0]]).item())
    return np.array(losses, np.float32)


@pytest.mark.parametrize("tag,kw", [("adam", dict(optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)),
                                    ("sgd", dict(optimizer="sgd", lr=5e-2, momentum=0.9))])
def test_small_mlp_tracks_reference(trainer_cls, tag, kw):
    g = np.load(GOLDEN / "reference_vectors.npz")
    tr = trainer_cls(g["mlp_sizes"], 16, **kw)
    tr.set_params(g["mlp_params0"])
    losses = run(tr, g["mlp_x"], g["mlp_t"], 12)
    assert np.abs(losses - g[f"mlp_{tag}_losses"]).max() <= 1e-5
    assert max_rel_err(tr.get_params(), g[f"mlp_{tag}_params"]) <= 2e-5
    # gradients of the last step as Parameter::grad() shows them after the hook ran
    _, _, grads = _libs.oracle_mlp_train(g["mlp_sizes"], g["mlp_params0"], g["mlp_x"], g["mlp_t"], 12,
                                         opt=tag, lr=kw["lr"], momentum=kw.get("momentum", 0.0),
                                         hook_wd=kw.get("hook_weight_decay", 0.0))
    assert max_rel_err(tr.get_grads(), grads) <= 1e-4
    tr.close()


def test_stable_200_step_curve_tracks_reference_within_1e3(trainer_cls):
    """784-256-256-10, batch 256, teacher labels, SGD lr 3e-3 momentum 0.9: a well-conditioned run, where the
    reference's 200-step fp32 loss curve is tracked within 1e-3 at every step."""
    from golden.make_golden import stable_inputs

    g = np.load(GOLDEN / "reference_vectors.npz")
    params, x, t = stable_inputs()
    tr = trainer_cls([784, 256, 256, 10], 256, optimizer="sgd", lr=3e-3, momentum=0.9)
    tr.set_params(params)
    losses = run(tr, x, t, 200)
    assert np.abs(losses - g["stable_losses"]).max() <= 1e-3
    # parameters after 200 steps: a loose sanity bound (the stated tolerance is on the loss curve)
    assert max_rel_err(tr.get_params()[::101], g["stable_param_sample"]) <= 1e-2
    tr.close()


def test_mnist_shaped_adam_curve_tracks_reference_like_exact_arithmetic(trainer_cls):
    """784-1000-1000-10, batch 512, Adam lr 1e-3, weight decay 1e-4, random labels, seed 42 (the MNIST-shaped
    benchmark configuration).  This run is chaotic, and two yardsticks in the golden file say so:
      * `c1_losses_ulp`: the UNMODIFIED REFERENCE run again with ONE input element moved by one unit in the last place
        leaves the 1e-3 band around its own original curve at step 19 and ends 0.39 away from it;
      * `c1_losses_fp64`: a float64 restatement of the same step (no fp32 rounding at all) leaves it at step 19 too.
    No implementation that is not bit-identical to the reference can therefore hold 1e-3 over 200 steps here.  The bar:
    inside 1e-3 while the reference's own perturbed run is (first 10 steps, with margin), in the band for at least as
    long as that run minus a few steps, and over all 200 steps no further from the reference than twice the reference's
    own spread.  (A well-conditioned 200-step run is held to 1e-3 at every step in the test above.)"""
    from golden.make_golden import c1_inputs

    g = np.load(GOLDEN / "reference_vectors.npz")
    ref, f64, ulp = g["c1_losses"], g["c1_losses_fp64"], g["c1_losses_ulp"]
    params, x, t = c1_inputs()
    tr = trainer_cls([784, 1000, 1000, 10], 512, optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)
    tr.set_params(params)
    losses = run(tr, x, t, len(ref))
    dev, spread = np.abs(losses - ref), np.abs(ulp - ref)

    def steps_in_band(d):
        out = np.nonzero(d > 1e-3)[0]
        return len(d) if out.size == 0 else int(out[0])

    assert np.abs(f64[:10] - ref[:10]).max() <= 1e-3 and spread[:10].max() <= 1e-3   # the yardsticks are inside here
    assert dev[:10].max() <= 1e-3
    assert steps_in_band(dev) >= steps_in_band(spread) - 5
    assert dev.max() <= max(1e-3, 2.0 * spread.max())
    assert dev.max() <= max(1e-3, 2.0 * np.abs(f64 - ref).max())
    assert losses[-1] < 0.5 * losses[0]                  # and it trains
    tr.close()


def test_tf32_mode_and_odd_widths(trainer_cls):
    """Widths that are not multiples of 4 (staged through padded scratch) and the opt-in plain-TF32 mode."""
    rng = np.random.default_rng(12)
    sizes = [37, 50, 21, 7]
    params = _libs.mlp_params(rng, sizes)
    xs = rng.standard_normal((2, 24, 37)).astype(np.float32)
    ts = rng.integers(0, 7, (2, 24)).astype(np.int32)
    ref_losses, ref_params, _ = _libs.oracle_mlp_train(sizes, params, xs, ts, 6, opt="sgd", lr=0.05, momentum=0.9)
    for precision, tol in ((0, 1e-5), (1, 5e-3)):
        tr = trainer_cls(sizes, 24, optimizer="sgd", lr=0.05, momentum=0.9, precision=precision)
        tr.set_params(params)
        losses = run(tr, xs, ts, 6)
        assert np.abs(losses - ref_losses).max() <= max(tol, 1e-5) * 10
        assert max_rel_err(tr.get_params(), ref_params) <= tol * 10
        tr.close()


def test_int64_labels_and_logits_view(trainer_cls):
    rng = np.random.default_rng(3)
    sizes = [16, 32, 10]
    tr = trainer_cls(sizes, 8)
    params = _libs.mlp_params(rng, sizes)
    tr.set_params(params)
    x = torch.from_numpy(rng.standard_normal((8, 16)).astype(np.float32)).cuda()
    t = torch.from_numpy(rng.integers(0, 10, 8)).cuda()          # int64
    l64 = tr.train_step(x, t).item()
    logits = tr.logits().clone()
    tr.set_params(params)
    l32 = tr.train_step(x, t.to(torch.int32)).item()
    assert l64 == l32 and torch.equal(logits, tr.logits())
    tr.close()


def test_cuda_graph_step_equals_eager_step(trainer_cls):
    """forward + loss + backward replayed from one CUDA graph (optimizer launched after it) trains like eager steps."""
    rng = np.random.default_rng(31)
    sizes = [64, 128, 96, 10]
    params = _libs.mlp_params(rng, sizes)
    x = torch.from_numpy(rng.standard_normal((32, 64)).astype(np.float32)).cuda()
    t = torch.from_numpy(rng.integers(0, 10, 32).astype(np.int32)).cuda()
    eager = trainer_cls(sizes, 32, optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)
    eager.set_params(params)
    ref = [eager.train_step(x, t).item() for _ in range(8)]
    graphed = trainer_cls(sizes, 32, optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)
    graphed.set_params(params)
    step = graphed.capture(x, t)                 # runs two real warm-up steps eagerly
    got = [step().item() for _ in range(6)]
    assert np.abs(np.array(got) - np.array(ref[2:])).max() <= 1e-5
    assert max_rel_err(graphed.get_params(), eager.get_params()) <= 1e-5
    eager.close()
    graphed.close()


def test_training_and_reductions_are_reproducible_bit_for_bit(trainer_cls):
    """Same inputs, same bits: bias gradients (column sums in the dY pass and in the dX GEMM's epilogue) and split-K
    GEMMs add their partial sums in a fixed order, as the reference's sequential CPU loops do -- no floating-point
    atomics on this path."""
    from origindl_b200 import ops

    rng = np.random.default_rng(8)
    sizes, batch = [200, 384, 256, 10], 512
    params = _libs.mlp_params(rng, sizes)
    xs = rng.standard_normal((2, batch, sizes[0])).astype(np.float32)
    ts = rng.integers(0, 10, (2, batch)).astype(np.int32)
    runs = []
    for _ in range(3):
        tr = trainer_cls(sizes, batch, optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)
        tr.set_params(params)
        losses = run(tr, xs, ts, 6)
        runs.append((losses, tr.get_grads(), tr.get_params()))
        tr.close()
    for other in runs[1:]:
        for a, b in zip(runs[0], other):
            assert np.array_equal(a, b)
    # split-K (few output tiles, long reduction) and the masked column sums of Linear's backward, each run three times
    a, b = torch.randn(256, 16384, device="cuda"), torch.randn(192, 16384, device="cuda")
    outs = [ops.gemm(a, b, trans_b=True).clone() for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ref = a.double() @ b.double().t()
    assert ((outs[0].double() - ref).abs().max() / ref.abs().max()).item() <= 1e-5
    x, w = torch.randn(4096, 300, device="cuda"), torch.randn(520, 300, device="cuda")
    y, dy = torch.randn(4096, 520, device="cuda"), torch.randn(4096, 520, device="cuda")
    grads = [[t.clone() for t in ops.linear_backward(x, w, dy, y=y)] for _ in range(3)]
    for other in grads[1:]:
        assert all(torch.equal(p, q) for p, q in zip(grads[0], other))
    # column sums taken in a GEMM's epilogue (ragged M and N)
    a, b = torch.randn(1000, 264, device="cuda"), torch.randn(264, 300, device="cuda")
    sums = []
    for _ in range(3):
        cs = torch.zeros(300, device="cuda")
        d = ops.gemm(a, b, colsum=cs)
        sums.append(cs)
    assert torch.equal(sums[0], sums[1]) and torch.equal(sums[0], sums[2])
    want = (a.double() @ b.double()).sum(0)
    assert ((sums[0].double() - want).abs().max() / want.abs().max()).item() <= 1e-5


def test_library_recorded_graph_step_equals_eager_step(trainer_cls):
    """odl_mlp_capture / odl_mlp_replay (the whole-step graph recorded inside the library, for C++ hosts): bit-identical
    to eager steps, inputs refilled in place between replays, optimizer state advanced once per replay."""
    rng = np.random.default_rng(41)
    sizes, batch = [784, 300, 100, 10], 128
    params = _libs.mlp_params(rng, sizes)
    xs = torch.from_numpy(rng.standard_normal((3, batch, 784)).astype(np.float32)).cuda()
    ts = torch.from_numpy(rng.integers(0, 10, (3, batch)).astype(np.int32)).cuda()
    eager = trainer_cls(sizes, batch, optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)
    eager.set_params(params)
    want = [eager.train_step(xs[i % 3], ts[i % 3]).item() for i in range(7)]
    graphed = trainer_cls(sizes, batch, optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)
    graphed.set_params(params)
    x, t = xs[0].clone(), ts[0].clone()
    step = graphed.capture_native(x, t)          # records; parameters and optimizer state untouched
    got = []
    for i in range(7):
        x.copy_(xs[i % 3]), t.copy_(ts[i % 3])
        got.append(step().item())
    assert got == want
    assert np.array_equal(graphed.get_params(), eager.get_params())
    from origindl_b200 import capi

    capi.device_status()
    eager.close()
    graphed.close()


def test_replay_refuses_a_graph_whose_scratch_was_replaced(trainer_cls):
    """A recorded step holds raw addresses inside the library's scratch blocks (staged copies of operands whose pitch
    breaks the 16-byte rule -- the 10-wide head here -- and the column-sum scratch).  A later call that needs more
    scratch replaces those blocks; replaying the old graph would then write freed memory.  Both graph front ends must
    refuse instead (ODL_ERR_STALE_GRAPH, nothing launched) and work again after a new capture."""
    from origindl_b200 import capi, ops

    rng = np.random.default_rng(43)
    sizes, batch = [64, 48, 10], 32
    params = _libs.mlp_params(rng, sizes)
    x = torch.from_numpy(rng.standard_normal((batch, 64)).astype(np.float32)).cuda()
    t = torch.from_numpy(rng.integers(0, 10, batch).astype(np.int32)).cuda()
    native = trainer_cls(sizes, batch, optimizer="adam", lr=1e-3)
    native.set_params(params)
    step_native = native.capture_native(x, t)
    torch_graph = trainer_cls(sizes, batch, optimizer="adam", lr=1e-3)
    torch_graph.set_params(params)
    step_torch = torch_graph.capture(x, t)
    first = step_native().item()
    step_torch()                                                    # (its capture ran two eager warm-up steps of its own)
    gen = capi.lib().odl_scratch_generation()
    # an unaligned GEMM far larger than anything so far: its staged operand copies make the arena grow
    need = max(int(capi.lib().odl_scratch_bytes()), 1 << 20)
    rows = need // (4 * 1001) + 64
    a, b = torch.randn(rows, 1001, device="cuda"), torch.randn(1001, 3, device="cuda")
    ops.gemm(a, b)
    assert capi.lib().odl_scratch_generation() > gen
    launches = capi.lib().odl_launch_count()
    params_before = native.get_params()
    with pytest.raises(capi.OdlError) as e1:
        step_native()
    assert e1.value.status == capi.ERR_STALE_GRAPH
    with pytest.raises(capi.OdlError) as e2:
        step_torch()
    assert e2.value.status == capi.ERR_STALE_GRAPH
    assert capi.lib().odl_launch_count() == launches               # nothing ran
    assert np.array_equal(native.get_params(), params_before)
    step_native = native.capture_native(x, t)                       # record again: works, and continues the same run
    eager = trainer_cls(sizes, batch, optimizer="adam", lr=1e-3)
    eager.set_params(params)
    want = [eager.train_step(x, t).item() for _ in range(3)]
    assert [first, step_native().item(), step_native().item()] == want
    capi.device_status()
    for tr in (native, torch_graph, eager):
        tr.close()


def test_nvtx_ranges_follow_the_environment_switch():
    """ODL_NVTX=1 wraps forward + loss, each layer's backward and the optimizer in NVTX ranges (for timeline tools); the
    default run opens none.  The switch is read once per process, so each setting runs in a process of its own."""
    import subprocess
    import sys
    import textwrap

    code = textwrap.dedent(f"""
        import ctypes, sys
        sys.path.insert(0, {str(Path(__file__).resolve().parent.parent)!r})
        import numpy as np, torch
        from origindl_b200 import capi
        from origindl_b200.trainer import MLPTrainer
        capi.init(0)
        tr = MLPTrainer([32, 48, 24, 10], 16, optimizer="adam")
        tr.set_params(np.zeros(tr.param_count, np.float32))
        x, t = torch.randn(16, 32, device="cuda"), torch.zeros(16, dtype=torch.int32, device="cuda")
        for _ in range(2):
            tr.train_step(x, t)
        torch.cuda.synchronize()
        fn = capi.lib().odl_debug_nvtx_ranges
        fn.restype = ctypes.c_longlong
        print("ranges", fn())
    """)
    import os

    counts = {}
    for setting in ("0", "1"):
        r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, ODL_NVTX=setting), capture_output=True,
                           text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        counts[setting] = int(r.stdout.split("ranges")[1])
    assert counts["0"] == 0
    assert counts["1"] == 2 * (1 + 3 + 1)        # per step: forward + loss, three layers' backward, the optimizer

