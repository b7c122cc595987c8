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
launch; nothing is skipped.  Inputs (2 x 256 MiB per rank, alternated) exceed the 126 MB L2.
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
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
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

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.tmp.flush()
        rows = [r.strip().split(",") for r in Path(self.tmp.name).read_text().splitlines() if r.strip()]
        os.unlink(self.tmp.name)
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(self.NAMES, r[3:7]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update({"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                        "samples": len(sm)})
        return out


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

    # ---- synthetic inputs: identical parameters on every rank (seed 0), rank-specific batches
    rng = np.random.default_rng(0)
    parts = []
    for a, b in zip(SIZES[:-1], SIZES[1:]):
        bound = np.sqrt(6.0 / a)
        parts.append(rng.uniform(-bound, bound, a * b).astype(np.float32))
        parts.append(np.zeros(b, np.float32))
    params = np.concatenate(parts)
    del parts
    tr = MLPTrainer(SIZES, PER_GPU_BATCH, optimizer="adam", lr=LR, device=local, process_group=pg)
    tr.set_params(params)
    del params
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    n_batches = 2
    xs = torch.randn((n_batches, PER_GPU_BATCH, SIZES[0]), device=dev, generator=g)
    ts = torch.randint(0, SIZES[-1], (n_batches, PER_GPU_BATCH), device=dev, generator=g, dtype=torch.int32)

    # ---- device-resident timing
    for s in range(args.warmup):
        tr.train_step(xs[s % n_batches], ts[s % n_batches])
    capi.device_status()
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()
    launches0 = L.odl_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(args.steps):
        loss = tr.train_step(xs[s % n_batches], ts[s % n_batches])
    e1.record()
    barrier()
    launches = L.odl_launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    capi.device_status()
    final_loss = float(loss.item())
    ms_per_step = ms_total / args.steps
    value = world * PER_GPU_BATCH * args.steps / (ms_total / 1e3)

    # ---- end to end through the public API: host data set -> DataLoader (staged mode: page-locked data set, a worker
    #      thread issuing the H2D copy of the following batches on a copy stream) -> train_step -> loss D2H
    from origindl_b200.loader import DataLoader

    e2e_batches = 4 if PER_GPU_BATCH <= 8192 else 2
    hx = torch.randn((e2e_batches * PER_GPU_BATCH, SIZES[0]), generator=torch.Generator().manual_seed(2000 + rank))
    ht = torch.randint(0, SIZES[-1], (e2e_batches * PER_GPU_BATCH,), generator=torch.Generator().manual_seed(3000 + rank))
    loader = DataLoader(hx.numpy(), ht.numpy(), PER_GPU_BATCH, shuffle=False, resident=False, device=local)
    host_loss = torch.empty((1,), dtype=torch.float32).pin_memory()

    def e2e_loop(n_steps):
        h2d0 = loader.h2d_bytes
        for _ in range(n_steps):
            if not loader.has_next():
                loader.reset()  # epoch boundary: the worker is already staging the next epoch
            bx, bt = loader.next()
            lv = tr.train_step(bx, bt)
            loader.release()
            host_loss.copy_(lv.reshape(1), non_blocking=True)
        torch.cuda.synchronize()
        return float(host_loss.item()), loader.h2d_bytes - h2d0

    e2e_loop(min(2, args.warmup))
    barrier()
    e0.record()
    e2e_loop(args.steps)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
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
                    "d2h_bytes_per_step": 4 * world},
            "gpu_launches": int(launches), "final_loss": final_loss,
            "mlp_tflops_per_gpu": flops_per_sample(SIZES) * PER_GPU_BATCH / (ms_per_step / 1e3) / 1e12}
    if clocks is not None:
        line["clocks"] = clocks

    # ---- rank 0 extras: Linear fwd+bwd at 8192^3 and the roofline of the GEMM (every N; the other ranks wait at the
    #      barrier below, so the kernel is timed on a GPU that runs nothing else); CPU baseline at N = 1 only
    if rank == 0:
        peaks = measured_peaks()
        n = LIN
        x = torch.randn((n, n), device=dev, generator=g)
        w = torch.randn((n, n), device=dev, generator=g)
        b = 0.1 * torch.randn((n,), device=dev, generator=g)
        dy = torch.randn((n, n), device=dev, generator=g)

        def lin_step():
            # everything a caller needs for one Linear forward + backward in 3xTF32, operand splits included
            xs_ = ops.split_tf32(x)
            ws_ = ops.split_tf32(w)
            y = ops.linear_forward(x, w, b, relu=True, x_small=xs_, w_small=ws_)
            return ops.linear_backward(x, w, dy, y, x_small=xs_, w_small=ws_)

        for _ in range(max(3, args.warmup)):
            lin_step()
        torch.cuda.synchronize()
        k = max(3, min(args.steps, 10))
        e0.record()
        for _ in range(k):
            lin_step()
        e1.record()
        torch.cuda.synchronize()
        lin_ms = e0.elapsed_time(e1) / k
        lin_tflops = 6 * n ** 3 / (lin_ms / 1e3) / 1e12
        # the GEMM alone (operands already split): CUDA events around each launch, on the launching stream
        xs_, ws_ = ops.split_tf32(x), ops.split_tf32(w)
        d = torch.empty((n, n), device=dev)
        s_ = capi.stream_handle()
        durations = []
        layouts = [(0, 1), (0, 0), (1, 0)]  # forward (x.W^T), dX (g.W), dW (g^T.x): the three GEMMs of a Linear layer
        for i in range(3 + 3 * k):
            ta, tb = layouts[i % 3]
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            capi.call("odl_gemm_ex", ta, tb, n, n, n, x.data_ptr(), xs_.data_ptr(), n, w.data_ptr(), ws_.data_ptr(), n,
                      d.data_ptr(), None, n, None, None, 0, None, 0, capi.PRECISION_3XTF32, s_)
            a1.record()
            durations.append((a0, a1))
        torch.cuda.synchronize()
        gemm_ms = statistics.mean(a.elapsed_time(b_) for a, b_ in durations[3:])
        capi.device_status()
        achieved = 2 * n ** 3 / (gemm_ms / 1e3) / 1e12
        tf32_peak = peaks["bf16_tflops"] / 2.0           # dense TF32 issues at half the bf16 rate
        peak = tf32_peak / 3.0                           # three MMAs per algorithmic product in 3xTF32
        line["linear_fwd_bwd"] = {"M": n, "N": n, "K": n, "ms": lin_ms, "tflops": lin_tflops,
                                  "frac_of_tf32_roofline_div3": lin_tflops / peak,
                                  "includes": "operand splits of x and W, fused bias+ReLU forward, mask/db pass, dX, dW"}
        line["roofline"] = {"bound": "tensor",
                            "kernel": "tcgen05 GEMM on CTA pairs (gemm_tc2_kernel<256>, cta_group::2), 3xTF32, M=N=K=8192, "
                                      "mean over the forward / dX / dW layouts",
                            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                            "peak_source": f"{peaks['source']}: bf16 burst {peaks['bf16_tflops']} TF/s / 2 (TF32) / 3 (3xTF32)",
                            "traffic": GEMM_DRAM_TRAFFIC_BYTES}
        # the opt-in plain-TF32 mode on the same Linear layer (no operand splits, one MMA per product): context only,
        # the headline above stays on the default fp32-accurate mode
        def lin_step_tf32():
            y = ops.linear_forward(x, w, b, relu=True, precision=capi.PRECISION_TF32)
            return ops.linear_backward(x, w, dy, y, precision=capi.PRECISION_TF32)

        for _ in range(3):
            lin_step_tf32()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(k):
            lin_step_tf32()
        e1.record()
        torch.cuda.synchronize()
        tf32_ms = e0.elapsed_time(e1) / k
        capi.device_status()
        line["linear_fwd_bwd_tf32_mode"] = {"ms": tf32_ms, "tflops": 6 * n ** 3 / (tf32_ms / 1e3) / 1e12,
                                            "frac_of_tf32_roofline": 6 * n ** 3 / (tf32_ms / 1e3) / 1e12 / tf32_peak,
                                            "tolerance": "5e-3 (opt-in mode)"}
        if peaks.get("bf16_tflops_sustained"):
            # context: the same kernel against the SUSTAINED library figure (seconds-long loop under the power cap), which
            # is the regime the training step runs in; `peak` / `frac` above stay on the stricter burst figure
            sustained = peaks["bf16_tflops_sustained"] / 6.0
            line["roofline"]["peak_sustained"] = sustained
            line["roofline"]["frac_sustained"] = achieved / sustained
            gemm_flops_per_step = 2.0 * PER_GPU_BATCH * (sum(a * b for a, b in zip(SIZES[:-1], SIZES[1:])) * 3
                                                         - SIZES[0] * SIZES[1])  # no dX for the first layer
            line["mlp_gemm_tflops_per_gpu"] = gemm_flops_per_step / (ms_per_step / 1e3) / 1e12
        cb = None
        if world == 1:
            try:
                cb = time_reference_cpu(4, 1)
            except Exception as ex:  # the checker must never take the measured arm down
                cb = {"error": repr(ex)}
        if cb is not None:
            cb.pop("seconds", None)
            line["cpu_baseline"] = cb
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        barrier()
        dist.destroy_process_group()


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one 8192^3 3xTF32 GEMM launch, mean of the three
# layouts, from the one-pass ncu capture summarised in profiles/gemm_tc_3xtf32_n8192_dram.md (algorithmic: 1.34e9).
GEMM_DRAM_TRAFFIC_BYTES = 4.85e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
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
