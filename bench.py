#!/usr/bin/env python
"""Benchmark of the dense hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per rank by torch.distributed.run)
    python bench.py --impl reference --gpus N --steps K --warmup W

Workload (config.workload): data-parallel MLP training, 4 x (8192 -> 8192, ReLU) + 8192 -> 1024 head, softmax-CE, Adam
(lr 1e-3), 8192 samples per GPU (weak scaling: global batch 8192 x N), fp32 parameters, 3xTF32 GEMMs, synthetic
N(0,1) inputs and uniform labels, seed 0.  `value` = samples/s over all ranks with inputs resident in HBM; `e2e` =
the same step fed from pinned HOST buffers through the public API (H2D copy of every batch and a D2H read of the loss
inside the timed region).  At N = 1 the line also carries the second half of the headline metric, Linear
forward+backward at M = N = K = 8192 (`linear_fwd_bwd`), the roofline of the dominant kernel (the tcgen05 GEMM) and
the reference's CPU backend timed on the host (`cpu_baseline`).

One step = forward (5 GEMMs), loss, backward (9 GEMMs), all-reduce of the gradient buckets (N > 1), one fused Adam
launch; nothing is skipped.  Inputs (2 x 256 MiB per rank, alternated) exceed the 126 MB L2.  The two headline loops
are alternated (resident K/2, end-to-end K/2, twice) so that both see the same power and thermal state.

Beyond the headline the line carries, each outside the headline's timed region and each with the SM clock sampled during
exactly that leg (`sm_mhz`, `ms_x_mhz`): `dp_parity` (N > 1: replicas bit-identical, equal to full-batch training on one
GPU; a miss fails the run), `strong_scaling` (every N: global batch 65536 split over the ranks), and on rank 0
`linear_sweep` (all six Linear shapes of benchmark config 2: forward, dX, dW, db pass, forward + backward), `roofline`,
`mnist_mlp_step` (config 1, eager and CUDA graph), `deep_mlp_step` (config 3), `conv_layers` (config 4, forward and
backward) and `cpu_baseline` (N = 1).  `--no-extras` keeps only the headline loops.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "MLP train samples/s @1/2/4/8 B200; Linear fwd+bwd TFLOP/s vs TF32 peak"
SIZES = [8192, 8192, 8192, 8192, 8192, 1024]
PER_GPU_BATCH = 8192  # weak scaling (default); --global-batch B switches to strong scaling with B / N samples per GPU
SCALING = "weak"
LR = 1e-3
LIN = 8192  # M = N = K of the Linear forward+backward leg


def flops_per_sample(sizes):
    return 6 * sum(a * b for a, b in zip(sizes[:-1], sizes[1:]))


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------ clock sampling
class ClockSampler:
    """nvidia-smi polled every 100 ms for the whole run (read-only: nothing here sets a clock).  Every sample carries its
    wall-clock time, so each timed leg gets the clocks and throttle reasons seen DURING that leg (`window`)."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, device_index: int):
        import torch

        self.uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
        self.proc = None
        self.tmp = None

    def start(self):
        try:
            self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.tmp,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def _rows(self):
        import datetime

        out = []
        if self.tmp is None:
            return out
        for line in Path(self.tmp.name).read_text().splitlines():
            r = [c.strip() for c in line.split(",")]
            try:
                t = datetime.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                out.append((t, float(r[1]), float(r[2]), float(r[3]),
                            [n for n, v in zip(self.NAMES, r[4:8]) if v.lower() == "active"]))
            except (ValueError, IndexError):
                continue
        return out

    def window(self, t0: float, t1: float):
        """Clocks seen between two time.time() stamps (the sampler's stamps are local wall-clock time as well)."""
        rows = [r for r in self._rows() if t0 - 0.05 <= r[0] <= t1 + 0.05]
        out = {"sm_mhz": None, "sm_max_mhz": None, "power_w": None, "reasons": [], "samples": len(rows)}
        if rows:
            out.update({"sm_mhz": statistics.median(r[1] for r in rows), "sm_max_mhz": max(r[2] for r in rows),
                        "power_w": statistics.median(r[3] for r in rows), "reasons": sorted({n for r in rows for n in r[4]})})
        return out

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.proc = None

    def close(self):
        self.stop()
        if self.tmp is not None:
            try:
                os.unlink(self.tmp.name)
            except OSError:
                pass
            self.tmp = None


# ------------------------------------------------------------------------------------------------ reference (CPU) arm
def time_reference_cpu(steps: int, warmup: int):
    """Times the UNMODIFIED reference (oracle/_ref/libodl_ref.so: nn::MLP + softmax_cross_entropy + backward + Adam on
    its CPU backend, one host thread -- the reference has no threading) on a bounded sample of the workload:
    the same depth and optimizer at width/8 and 32 samples per step, then scaled to the full-size unit by the ratio
    of flops per sample (the reference's scalar ijk GEMM has the same cost per flop at any width)."""
    sys.path.insert(0, str(ROOT / "tests"))
    import numpy as np

    import _libs

    ref = _libs.reference()
    if ref is None:
        return None
    sizes = [s // 8 for s in SIZES]
    B = 32
    rng = np.random.default_rng(0)
    params = _libs.mlp_params(rng, sizes)
    x = rng.standard_normal((1, B, sizes[0])).astype(np.float32)
    t = rng.integers(0, sizes[-1], (1, B)).astype(np.int32)
    arr = np.array(sizes, np.int32)
    losses = np.empty(max(steps, warmup, 1), np.float32)
    if warmup > 0:
        _libs.ref_check(ref.odlref_mlp_train(arr, len(sizes), params, x, t, B, 1, warmup, 1, LR, 0.0, 0.0, losses, None))
    t0 = time.perf_counter()
    _libs.ref_check(ref.odlref_mlp_train(arr, len(sizes), params, x, t, B, 1, steps, 1, LR, 0.0, 0.0, losses, None))
    dt = time.perf_counter() - t0
    twin_sps = B * steps / dt
    full_sps = twin_sps * flops_per_sample(sizes) / flops_per_sample(SIZES)
    return {"value": full_sps, "unit": "samples/s", "cores": 1, "kind": "reference",
            "sample": f"reference CPU backend, {steps} Adam steps of the width/8 twin {sizes} at batch {B} "
                      f"({dt:.1f} s, {twin_sps:.1f} samples/s), extrapolated to full width by flops per sample",
            "host_cores_available": os.cpu_count(), "seconds": dt}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 20))
    res = time_reference_cpu(steps, max(1, min(args.warmup, 2)))
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libodl_ref.so is not built on this machine"}))
        return
    line = {"impl": "reference", "metric": METRIC, "value": res["value"], "unit": "samples/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * res["seconds"] / steps,
            "higher_is_better": True, "scaling": SCALING, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": res["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(n):
    return {"workload": f"data-parallel MLP training (benchmark config 5: five 8192-wide layers + 1024 classes, {PER_GPU_BATCH} "
                        "samples per GPU) + Linear fwd+bwd M=N=K=8192 (benchmark config 2)",
            "layers": SIZES, "per_gpu_batch": PER_GPU_BATCH, "global_batch": PER_GPU_BATCH * n, "optimizer": "adam",
            "precision": "3xTF32", "parallelism": f"dp{n}", "l2": f"inputs (2 x {PER_GPU_BATCH * SIZES[0] * 4 >> 20} MiB per rank) larger than L2"}


# ------------------------------------------------------------------------------------------------ our arm
_PARAM_CACHE = {}


def kaiming_params(sizes, seed=0):
    """Kaiming-uniform weights {in,out} and zero biases in the packed order of Module::named_parameters."""
    import numpy as np

    key = (tuple(sizes), seed)
    if key in _PARAM_CACHE:
        return _PARAM_CACHE[key]
    rng, parts = np.random.default_rng(seed), []
    for a, b in zip(sizes[:-1], sizes[1:]):
        bound = np.sqrt(6.0 / a)
        parts.append(rng.uniform(-bound, bound, a * b).astype(np.float32))
        parts.append(np.zeros(b, np.float32))
    _PARAM_CACHE.clear()  # keep one set at a time: the headline model's parameters are 1.1 GB
    _PARAM_CACHE[key] = np.concatenate(parts)
    return _PARAM_CACHE[key]


class Legs:
    """Times the extra legs of the line: CUDA events on the current stream, and for every leg the wall-clock window so
    that the clocks sampled during exactly that leg can be printed beside its figure (ms x median SM MHz compares legs
    that ran at different clocks under the power cap)."""

    def __init__(self, sampler):
        self.sampler = sampler

    def run(self, fn, iters, warmup=2, min_seconds=0.35):
        import torch

        from origindl_b200 import capi

        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        # keep going (untimed) until the leg has lasted long enough for the 100 ms clock sampler to have seen it
        while time.time() - t0 < min_seconds:
            fn()
            torch.cuda.synchronize()
        t1 = time.time()
        capi.device_status()
        out = {"ms": ms}
        if self.sampler is not None:
            c = self.sampler.window(t0, t1)
            out["sm_mhz"] = c["sm_mhz"]
            out["ms_x_mhz"] = None if c["sm_mhz"] is None else ms * c["sm_mhz"]
            out["reasons"] = c["reasons"]
        return out


def dp_parity_check(rank, world, local, pg):
    """Correctness of the data-parallel step at this N, outside every timed region: a small MLP (256-384-256-10, six Adam
    steps with the weight-decay hook) trained on a global batch sharded over the ranks must leave bit-identical
    parameters on all ranks and must equal rank 0 training the whole batch alone (loss and parameters within 1e-5)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from origindl_b200.trainer import MLPTrainer

    sizes, per, steps = [256, 384, 256, 10], 128, 6
    kw = dict(optimizer="adam", lr=1e-3, hook_weight_decay=1e-4)
    rng = np.random.default_rng(77)
    params = kaiming_params(sizes, 77)
    xs = rng.standard_normal((2, world * per, sizes[0])).astype(np.float32)
    ts = rng.integers(0, sizes[-1], (2, world * per)).astype(np.int32)
    lo, hi = rank * per, (rank + 1) * per
    xd, td = torch.from_numpy(xs[:, lo:hi].copy()).cuda(), torch.from_numpy(ts[:, lo:hi].copy()).cuda()
    tr = MLPTrainer(sizes, per, device=local, process_group=pg, dw0_panels=2, **kw)
    tr.set_params(params)
    losses = torch.stack([tr.train_step(xd[s % 2], td[s % 2]).clone() for s in range(steps)])
    tr.wait(30000)
    torch.cuda.synchronize()
    dist.all_reduce(losses)
    losses = (losses / world).cpu().numpy()
    mine = tr.get_params()
    tr.close()
    # replicas identical: compare the raw bits through two integer checksums gathered from every rank
    bits = torch.from_numpy(mine.view(np.int32).astype(np.int64)).cuda()
    digest = torch.stack([bits.sum(), (bits * torch.arange(1, bits.numel() + 1, device="cuda")).sum()])
    gathered = [torch.empty_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    identical = all(bool(torch.equal(g, gathered[0])) for g in gathered)
    out = {"world": world, "sizes": sizes, "steps": steps, "replicas_identical": identical}
    if rank == 0:
        full = MLPTrainer(sizes, world * per, device=local, **kw)
        full.set_params(params)
        xf, tf = torch.from_numpy(xs).cuda(), torch.from_numpy(ts).cuda()
        want = np.array([full.train_step(xf[s % 2], tf[s % 2]).item() for s in range(steps)], np.float32)
        pf = full.get_params()
        full.close()
        out["loss_max_abs_diff_vs_full_batch"] = float(np.abs(losses - want).max())
        out["param_max_rel_err_vs_full_batch"] = float(np.abs(mine - pf).max() / np.abs(pf).max())
        out["tolerance"] = 1e-5
        out["ok"] = bool(identical and out["loss_max_abs_diff_vs_full_batch"] <= 1e-5 and
                         out["param_max_rel_err_vs_full_batch"] <= 1e-5)
    flag = torch.tensor([1 if out.get("ok", True) else 0], device="cuda")
    dist.broadcast(flag, src=0)
    out["ok"] = bool(flag.item()) and identical
    return out


def run_ours(args):
    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local)
    pg = None
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        pg = dist.group.WORLD
    from origindl_b200 import capi, ops
    from origindl_b200.trainer import MLPTrainer

    capi.init(local)
    L = capi.lib()
    dev = torch.device("cuda", local)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()

    # ---- synthetic inputs: identical parameters on every rank (seed 0), rank-specific batches
    tr = MLPTrainer(SIZES, PER_GPU_BATCH, optimizer="adam", lr=LR, device=local, process_group=pg)
    tr.set_params(kaiming_params(SIZES, 0))
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    n_batches = 2
    xs = torch.randn((n_batches, PER_GPU_BATCH, SIZES[0]), device=dev, generator=g)
    ts = torch.randint(0, SIZES[-1], (n_batches, PER_GPU_BATCH), device=dev, generator=g, dtype=torch.int32)

    # ---- end to end through the public API: host data set -> DataLoader (staged mode: page-locked data set, a worker
    #      thread issuing the H2D copy of the following batches on a copy stream) -> train_step -> loss D2H
    from origindl_b200.loader import DataLoader

    e2e_batches = 4 if PER_GPU_BATCH <= 8192 else 2
    hx = torch.randn((e2e_batches * PER_GPU_BATCH, SIZES[0]), generator=torch.Generator().manual_seed(2000 + rank))
    ht = torch.randint(0, SIZES[-1], (e2e_batches * PER_GPU_BATCH,), generator=torch.Generator().manual_seed(3000 + rank))
    loader = DataLoader(hx.numpy(), ht.numpy(), PER_GPU_BATCH, shuffle=False, resident=False, device=local)
    host_loss = torch.empty((1,), dtype=torch.float32).pin_memory()
    state = {"s": 0, "loss": None}

    def resident_loop(n_steps):
        for _ in range(n_steps):
            state["loss"] = tr.train_step(xs[state["s"] % n_batches], ts[state["s"] % n_batches])
            state["s"] += 1

    def e2e_loop(n_steps):
        for _ in range(n_steps):
            if not loader.has_next():
                loader.reset()  # epoch boundary: the worker is already staging the next epoch
            bx, bt = loader.next()
            lv = tr.train_step(bx, bt)
            loader.release()
            host_loss.copy_(lv.reshape(1), non_blocking=True)
        torch.cuda.synchronize()

    # ---- the two headline loops, alternated (resident / end-to-end / resident / end-to-end) so that both see the same
    #      thermal and power state; each bracket has a barrier + synchronize on both sides, the K timed steps of each
    #      loop are the sum of its two brackets, max over ranks per bracket
    resident_loop(args.warmup)
    e2e_loop(min(2, args.warmup))
    capi.device_status()
    halves = [args.steps // 2, args.steps - args.steps // 2]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ms_total, e2e_ms, launches = 0.0, 0.0, 0
    windows = []
    for n_steps in halves:
        if n_steps == 0:
            continue
        barrier()
        l0, t0 = L.odl_launch_count(), time.time()
        e0.record()
        resident_loop(n_steps)
        e1.record()
        barrier()
        windows.append((t0, time.time()))
        launches += L.odl_launch_count() - l0
        ms_total += max_over_ranks(e0.elapsed_time(e1))
        barrier()
        e0.record()
        e2e_loop(n_steps)
        e1.record()
        barrier()
        e2e_ms += max_over_ranks(e0.elapsed_time(e1))
    capi.device_status()
    final_loss = float(state["loss"].item())
    ms_per_step = ms_total / args.steps
    value = world * PER_GPU_BATCH * args.steps / (ms_total / 1e3)
    e2e_value = world * PER_GPU_BATCH * args.steps / (e2e_ms / 1e3)
    h2d = PER_GPU_BATCH * SIZES[0] * 4 + PER_GPU_BATCH * 8  # fp32 inputs + int64 labels of one batch
    loader.close()
    tr.close()
    del xs, hx, loader
    torch.cuda.empty_cache()

    line = {"metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": SCALING,
            "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core products, fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": 4 * world, "ms_per_step": e2e_ms / args.steps,
                    "order": "alternated with the device-resident loop: resident K/2, end-to-end K/2, twice"},
            "gpu_launches": int(launches), "final_loss": final_loss,
            "mlp_tflops_per_gpu": flops_per_sample(SIZES) * PER_GPU_BATCH / (ms_per_step / 1e3) / 1e12}
    if sampler is not None:
        w = [sampler.window(a, b) for a, b in windows]
        mhz = [c["sm_mhz"] for c in w if c["sm_mhz"] is not None]
        line["clocks"] = {"sm_mhz": statistics.median(mhz) if mhz else None,
                          "sm_max_mhz": max((c["sm_max_mhz"] or 0) for c in w) if w else None,
                          "reasons": sorted({r for c in w for r in c["reasons"]}), "samples": sum(c["samples"] for c in w),
                          "region": "the device-resident timed brackets"}
        if mhz:
            line["ms_per_step_x_sm_mhz"] = ms_per_step * line["clocks"]["sm_mhz"]

    # ---- N > 1: parity of the data-parallel step (not timed); a miss fails the run
    parity_ok = True
    if world > 1:
        parity = dp_parity_check(rank, world, local, pg)
        parity_ok = parity["ok"]
        line["dp_parity"] = parity

    # ---- every N: the benchmark's strong-scaling point (global batch 65536 split over the ranks), a few steps
    if SCALING == "weak" and not args.no_extras and STRONG_GLOBAL_BATCH % world == 0:
        per = STRONG_GLOBAL_BATCH // world
        st = MLPTrainer(SIZES, per, optimizer="adam", lr=LR, device=local, process_group=pg)
        st.set_params(kaiming_params(SIZES, 0))
        sx = torch.randn((per, SIZES[0]), device=dev, generator=g)
        stt = torch.randint(0, SIZES[-1], (per,), device=dev, generator=g, dtype=torch.int32)
        for _ in range(2):
            st.train_step(sx, stt)
        barrier()
        k_strong = 3
        e0.record()
        for _ in range(k_strong):
            st.train_step(sx, stt)
        e1.record()
        barrier()
        strong_ms = max_over_ranks(e0.elapsed_time(e1)) / k_strong
        capi.device_status()
        st.close()
        del sx, st
        torch.cuda.empty_cache()
        line["strong_scaling"] = {"global_batch": STRONG_GLOBAL_BATCH, "per_gpu_batch": per, "steps": k_strong,
                                  "ms_per_step": strong_ms, "value": STRONG_GLOBAL_BATCH / (strong_ms / 1e3),
                                  "unit": "samples/s", "note": "same model and step as the headline, total work fixed"}

    # ---- rank 0 extras: the other benchmark configurations and the roofline of the GEMM (every N; the other ranks wait
    #      at the barrier below, so each kernel is timed on a GPU that runs nothing else); CPU baseline at N = 1 only
    if rank == 0 and not args.no_extras:
        extras(line, args, sampler, dev, g, world, ms_per_step)
    if sampler is not None:
        sampler.close()
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        barrier()
        dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit("bench.py: the data-parallel parity check failed (see dp_parity in the line above)")


CONV_LAYERS = {"L1": (3, 16, 6, 2, 2, 320), "L2": (16, 32, 3, 2, 1, 160), "L3": (32, 32, 1, 1, 0, 80),
               "L4": (64, 64, 3, 1, 1, 40)}  # C, OC, k, stride, pad, H = W; batch 16
C2_SHAPES = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (65536, 1024, 1024),
             (256, 8192, 8192)]
STRONG_GLOBAL_BATCH = 65536


def extras(line, args, sampler, dev, g, world, ms_per_step):
    import torch

    from origindl_b200 import capi, ops
    from origindl_b200.trainer import MLPTrainer

    legs = Legs(sampler)
    peaks = measured_peaks()
    tf32_peak = peaks["bf16_tflops"] / 2.0           # dense TF32 issues at half the bf16 rate
    peak = tf32_peak / 3.0                           # three MMAs per algorithmic product in 3xTF32
    hbm = peaks["hbm_gbs"]
    k = max(3, min(args.steps, 10))

    # ---- Linear forward + backward sweep (benchmark config 2): W [N, K], fused bias + ReLU; forward, dX, dW GEMMs and the
    #      dY pass (ReLU mask + db column sums + low part) timed apart, then the whole forward + backward with the splits
    sweep = []
    for (M, N, K) in C2_SHAPES:
        x, w = torch.randn((M, K), device=dev, generator=g), torch.randn((N, K), device=dev, generator=g)
        b, dy = 0.1 * torch.randn((N,), device=dev, generator=g), torch.randn((M, N), device=dev, generator=g)
        xs_, ws_ = ops.split_tf32(x), ops.split_tf32(w)
        y = ops.linear_forward(x, w, b, relu=True, x_small=xs_, w_small=ws_)
        gm = ops.relu_backward(dy, y)
        gs_ = ops.split_tf32(gm)
        db, gbuf, gsm = torch.zeros((N,), device=dev), torch.empty_like(dy), torch.empty_like(dy)
        it = k if M * N * K >= 2 ** 33 else 4 * k

        def whole():
            a_, b_ = ops.split_tf32(x), ops.split_tf32(w)
            yy = ops.linear_forward(x, w, b, relu=True, x_small=a_, w_small=b_)
            return ops.linear_backward(x, w, dy, yy, x_small=a_, w_small=b_)

        r = {"M": M, "N": N, "K": K}
        f = 2.0 * M * N * K
        for name, fn in (("fwd", lambda: ops.linear_forward(x, w, b, relu=True, x_small=xs_, w_small=ws_)),
                         ("dx", lambda: ops.gemm(gm, w, a_small=gs_, b_small=ws_)),
                         ("dw", lambda: ops.gemm(gm, x, trans_a=True, a_small=gs_, b_small=xs_))):
            t = legs.run(fn, it)
            t.update({"tflops": f / (t["ms"] / 1e3) / 1e12, "frac": f / (t["ms"] / 1e3) / 1e12 / peak})
            r[name] = t
        t = legs.run(lambda: capi.call("odl_split_tf32", dy.data_ptr(), N, M, N, y.data_ptr(), N, gbuf.data_ptr(),
                                       gsm.data_ptr(), N, db.data_ptr(), capi.stream_handle()), it)
        t.update({"gbs": 16.0 * M * N / (t["ms"] / 1e3) / 1e9, "frac_hbm": 16.0 * M * N / (t["ms"] / 1e3) / 1e9 / hbm,
                  "bytes": "8 read (dY, y) + 8 written (masked dY, its low part) per element"})
        r["db_pass"] = t
        t = legs.run(whole, it)
        t.update({"tflops": 3 * f / (t["ms"] / 1e3) / 1e12, "frac": 3 * f / (t["ms"] / 1e3) / 1e12 / peak})
        r["fwd_bwd"] = t
        sweep.append(r)
        if (M, N, K) == (LIN, LIN, LIN):
            line["linear_fwd_bwd"] = {"M": M, "N": N, "K": K, "ms": t["ms"], "tflops": t["tflops"],
                                      "frac_of_tf32_roofline_div3": t["frac"], "sm_mhz": t.get("sm_mhz"),
                                      "ms_x_mhz": t.get("ms_x_mhz"),
                                      "includes": "operand splits of x and W, fused bias+ReLU forward, mask/db pass, dX, dW"}
            # the GEMM alone (operands already split): CUDA events around each launch, on the launching stream
            d = torch.empty((M, N), device=dev)
            s_ = capi.stream_handle()
            durations = []
            layouts = [(0, 1), (0, 0), (1, 0)]  # forward (x.W^T), dX (g.W), dW (g^T.x): the three GEMMs of a Linear layer
            t0 = time.time()
            for i in range(3 + 3 * k):
                ta, tb = layouts[i % 3]
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                capi.call("odl_gemm_ex", ta, tb, M, N, K, x.data_ptr(), xs_.data_ptr(), K, w.data_ptr(), ws_.data_ptr(), K,
                          d.data_ptr(), None, N, None, None, 0, None, 0, capi.PRECISION_3XTF32, s_)
                a1.record()
                durations.append((a0, a1))
            torch.cuda.synchronize()
            t1 = time.time()
            gemm_ms = statistics.mean(a.elapsed_time(b_) for a, b_ in durations[3:])
            capi.device_status()
            achieved = 2 * M * N * K / (gemm_ms / 1e3) / 1e12
            c = sampler.window(t0, t1) if sampler is not None else {"sm_mhz": None}
            line["roofline"] = {"bound": "tensor",
                                "kernel": "tcgen05 GEMM on persistent CTA pairs (gemm_tc2_persistent_kernel, cta_group::2), 3xTF32, M=N=K=8192, mean over the "
                                          "forward / dX / dW layouts",
                                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                                "peak_source": f"{peaks['source']}: bf16 burst {peaks['bf16_tflops']} TF/s / 2 (TF32) / 3 (3xTF32)",
                                "traffic": GEMM_DRAM_TRAFFIC_BYTES, "ms": gemm_ms, "sm_mhz": c["sm_mhz"],
                                "ms_x_mhz": None if c["sm_mhz"] is None else gemm_ms * c["sm_mhz"]}
            if peaks.get("bf16_tflops_sustained"):
                # context: the same kernel against the SUSTAINED library figure (seconds-long loop under the power cap),
                # which is the regime the training step runs in; `peak` / `frac` above stay on the stricter burst figure
                sustained = peaks["bf16_tflops_sustained"] / 6.0
                line["roofline"]["peak_sustained"] = sustained
                line["roofline"]["frac_sustained"] = achieved / sustained
                gemm_flops_per_step = 2.0 * PER_GPU_BATCH * (sum(a * b_ for a, b_ in zip(SIZES[:-1], SIZES[1:])) * 3
                                                             - SIZES[0] * SIZES[1])  # no dX for the first layer
                line["mlp_gemm_tflops_per_gpu"] = gemm_flops_per_step / (ms_per_step / 1e3) / 1e12

            # the opt-in plain-TF32 mode on the same Linear layer (no operand splits, one MMA per product): context only
            def lin_step_tf32():
                yy = ops.linear_forward(x, w, b, relu=True, precision=capi.PRECISION_TF32)
                return ops.linear_backward(x, w, dy, yy, precision=capi.PRECISION_TF32)

            t = legs.run(lin_step_tf32, k)
            line["linear_fwd_bwd_tf32_mode"] = {"ms": t["ms"], "tflops": 3 * f / (t["ms"] / 1e3) / 1e12,
                                                "frac_of_tf32_roofline": 3 * f / (t["ms"] / 1e3) / 1e12 / tf32_peak,
                                                "sm_mhz": t.get("sm_mhz"), "tolerance": "5e-3 (opt-in mode)"}
        del x, w, dy, xs_, ws_, y, gm, gs_, gbuf, gsm
        torch.cuda.empty_cache()
    line["linear_sweep"] = {"config": "benchmark config 2: X [M,K], W [N,K] ~ N(0,1), b ~ N(0,0.1), dY ~ N(0,1), 3xTF32",
                            "frac_is": "TFLOP/s over bf16 burst / 2 / 3", "shapes": sweep}

    # ---- the MNIST-shaped step (benchmark config 1) eager and from the library-recorded CUDA graph
    c1 = [784, 1000, 1000, 10]
    t1_ = MLPTrainer(c1, 512, optimizer="adam", lr=1e-3, hook_weight_decay=1e-4, device=dev.index)
    t1_.set_params(kaiming_params(c1, 42))
    x1 = torch.rand((512, 784), device=dev, generator=g)
    l1 = torch.randint(0, 10, (512,), device=dev, generator=g, dtype=torch.int32)
    eager = legs.run(lambda: t1_.train_step(x1, l1), 200, warmup=5)
    step = t1_.capture_native(x1, l1)
    graph = legs.run(step, 200, warmup=5)
    t1_.close()
    for t in (eager, graph):
        t["samples_per_s"] = 512 / (t["ms"] / 1e3)
    line["mnist_mlp_step"] = {"config": "benchmark config 1: 784-1000-1000-10, batch 512, Adam 1e-3, weight decay 1e-4",
                              "eager": eager, "graph": graph}

    # ---- the deep wide MLP (benchmark config 3): batch 8192, 6 x 4096 + 1000 classes, SGD momentum 0.9
    c3 = [4096] * 7 + [1000]
    t3 = MLPTrainer(c3, 8192, optimizer="sgd", lr=1e-2, momentum=0.9, device=dev.index)
    t3.set_params(kaiming_params(c3, 0))
    x3 = torch.randn((8192, 4096), device=dev, generator=g)
    l3 = torch.randint(0, 1000, (8192,), device=dev, generator=g, dtype=torch.int32)
    r3 = legs.run(lambda: t3.train_step(x3, l3), k, warmup=3)
    t3.close()
    fl = 8192.0 * (flops_per_sample(c3) - 2 * c3[0] * c3[1])
    r3.update({"samples_per_s": 8192 / (r3["ms"] / 1e3), "tflops": fl / (r3["ms"] / 1e3) / 1e12,
               "frac": fl / (r3["ms"] / 1e3) / 1e12 / peak})
    line["deep_mlp_step"] = {"config": "benchmark config 3: batch 8192, 6 x (4096 -> 4096) + 4096 -> 1000, SGD momentum 0.9, 3xTF32",
                             **r3}
    del x3, t3
    torch.cuda.empty_cache()

    # ---- the four convolution layers (benchmark config 4), batch 16, forward and backward (gx, gw, gb)
    convs = {}
    for name, (C, OC, kk, s, p, hw) in CONV_LAYERS.items():
        x = torch.rand((16, C, hw, hw), device=dev, generator=g)
        w = torch.randn((OC, C, kk, kk), device=dev, generator=g) * (2.0 / (C * kk * kk)) ** 0.5
        b = torch.zeros((OC,), device=dev)
        y = ops.conv2d_forward(x, w, b, s, p)
        gy = torch.randn(y.shape, device=dev, generator=g)
        fw = legs.run(lambda: ops.conv2d_forward(x, w, b, s, p), 50, warmup=3)
        bw = legs.run(lambda: ops.conv2d_backward(gy, x, w, s, p), 50, warmup=3)
        ideal_f = 4.0 * (x.numel() + w.numel() + y.numel())                # read x, W; write y
        ideal_b = 4.0 * (2 * x.numel() + 2 * w.numel() + y.numel() + OC)   # read gy, x, W; write gx, gw, gb
        flops = 2.0 * y.numel() * C * kk * kk
        fw.update({"gbs_of_ideal_traffic": ideal_f / (fw["ms"] / 1e3) / 1e9, "frac_hbm": ideal_f / (fw["ms"] / 1e3) / 1e9 / hbm,
                   "tflops": flops / (fw["ms"] / 1e3) / 1e12, "frac_tensor": flops / (fw["ms"] / 1e3) / 1e12 / peak})
        bw.update({"gbs_of_ideal_traffic": ideal_b / (bw["ms"] / 1e3) / 1e9, "frac_hbm": ideal_b / (bw["ms"] / 1e3) / 1e9 / hbm,
                   "tflops": 2 * flops / (bw["ms"] / 1e3) / 1e12, "frac_tensor": 2 * flops / (bw["ms"] / 1e3) / 1e12 / peak})
        convs[name] = {"shape": f"{C}->{OC} k{kk} s{s} p{p} on {hw}x{hw}", "forward": fw, "backward": bw}
    line["conv_layers"] = {"config": "benchmark config 4: batch 16, NCHW, 3xTF32; times include the Python + ctypes call "
                                     "path (about 0.02 ms per call)", "layers": convs}

    if world == 1:
        try:
            cb = time_reference_cpu(4, 1)
        except Exception as ex:  # the checker must never take the measured arm down
            cb = {"error": repr(ex)}
        if cb is not None:
            cb.pop("seconds", None)
            line["cpu_baseline"] = cb


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one 8192^3 3xTF32 GEMM launch, mean of the three
# layouts, from a one-pass ncu capture of that kernel (algorithmic: 1.34e9).
GEMM_DRAM_TRAFFIC_BYTES = 5.64e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline loops (and dp_parity at N > 1): skip the other benchmark configurations")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="strong scaling: fix the global batch (e.g. 65536) and give every rank global / N samples; "
                         "default 0 = weak scaling with 8192 samples per GPU")
    args = ap.parse_args()
    if args.global_batch:
        global PER_GPU_BATCH, SCALING
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if args.global_batch % world:
            raise SystemExit(f"--global-batch {args.global_batch} is not divisible by {world} ranks")
        PER_GPU_BATCH, SCALING = args.global_batch // world, "strong"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
