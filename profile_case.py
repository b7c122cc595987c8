"""Small, self-terminating cases of each kernel of the library, sized for profiler captures.

    python profile_case.py gemm    --n 4096 [--precision 3xtf32|tf32] [--layout nt|nn|tn] [--iters 3]
    python profile_case.py split   --n 8192
    python profile_case.py adam    --n 67108864
    python profile_case.py softmax --rows 8192 --cols 1024
    python profile_case.py conv    --layer 1          (the four conv shapes of the benchmark, batch 16)
    python profile_case.py linear  --m 8192 --n 8192 --k 8192   (forward, dX, dW, dY pass timed apart)
    python profile_case.py batchnorm --n 64 --cols 64 --rows 25600   (N x C x HW, training fwd + bwd, fused SiLU)
    python profile_case.py gather  --rows 65536 --cols 1024       (batch assembly from a resident data set)
    python profile_case.py mlp --sizes 4096,4096,4096,4096,4096,4096,4096,1000 --batch 8192 --optimizer sgd --iters 10
    python profile_case.py checkpoint --n 4096 --layers 4        (save / load of an Adam-trained MLP, host wall clock)

Each case keeps its inputs above the 126 MB L2 where the kernel is HBM-bound, holds well under a few GB on the
device, launches the kernel `--iters` times after one warm-up launch and prints the CUDA-event time per launch.
"""
from __future__ import annotations

import argparse

import torch

from origindl_b200 import capi, ops

# 1-4: the benchmark's conv shapes; 5: a deep 256 -> 256 3x3 layer (K = 2304: the implicit forward splits K over a CTA pair)
CONV_LAYERS = {1: (3, 16, 6, 2, 2, 320), 2: (16, 32, 3, 2, 1, 160), 3: (32, 32, 1, 1, 0, 80), 4: (64, 64, 3, 1, 1, 40),
               5: (256, 256, 3, 1, 1, 20)}


def timed(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    capi.device_status()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "split", "adam", "softmax", "conv", "linear", "checkpoint", "gather", "batchnorm", "mlp"])
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=1024)
    ap.add_argument("--layer", type=int, default=1)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--precision", default="3xtf32")
    ap.add_argument("--layout", default="nt")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--explicit", action="store_true", help="conv: force the im2col + GEMM forward path")
    ap.add_argument("--batch", type=int, default=16, help="conv: images per batch")
    ap.add_argument("--conv-mode", type=int, default=0, help="conv: 2 = implicit-GEMM weight gradient also for small layers")
    ap.add_argument("--sizes", default="4096,4096,4096,4096,4096,4096,4096,1000", help="mlp: layer widths")
    ap.add_argument("--optimizer", default="sgd", help="mlp: sgd (momentum 0.9) or adam")
    ap.add_argument("--graph", action="store_true", help="mlp: also time the step replayed from the library's CUDA graph")
    ap.add_argument("--yardstick", action="store_true", help="gemm: also time torch.matmul (TF32 and fp32) for context")
    ap.add_argument("--rect", action="store_true", help="gemm: an M x N x K problem from --m / --n / --k instead of n cubed")
    a = ap.parse_args()
    capi.init(0)
    torch.manual_seed(0)
    prec = capi.PRECISION_3XTF32 if a.precision == "3xtf32" else capi.PRECISION_TF32
    if a.case == "checkpoint":
        import shutil
        import tempfile
        import time

        import numpy as np

        from origindl_b200.trainer import MLPTrainer

        sizes = [a.n] * (a.layers + 1)
        tr = MLPTrainer(sizes, 128)
        tr.set_params(np.random.default_rng(0).standard_normal(tr.param_count).astype(np.float32) * 0.01)
        x = torch.randn(128, a.n, device="cuda")
        t = torch.randint(0, a.n, (128,), device="cuda", dtype=torch.int32)
        tr.train_step(x, t)
        torch.cuda.synchronize()
        d = tempfile.mkdtemp(prefix="odl_ckpt_")
        nbytes = 3 * 4 * tr.param_count  # parameters + both Adam moments
        t0 = time.perf_counter()
        tr.save_checkpoint(d + "/run.ckpt", epoch=1, step=1, loss=float(tr.loss_tensor()))
        t1 = time.perf_counter()
        tr2 = MLPTrainer(sizes, 128)
        t2 = time.perf_counter()
        tr2.load_checkpoint(d + "/run.ckpt")
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        same = bool(np.array_equal(tr.get_params(), tr2.get_params()))
        shutil.rmtree(d)
        print(f"checkpoint {len(sizes) - 1} x {a.n}^2 ({tr.param_count / 1e6:.1f} M parameters, {nbytes / 1e9:.2f} GB with Adam state): "
              f"save {t1 - t0:.3f} s ({nbytes / (t1 - t0) / 1e9:.2f} GB/s), load {t3 - t2:.3f} s ({nbytes / (t3 - t2) / 1e9:.2f} GB/s), "
              f"parameters identical after reload: {same}")
    elif a.case == "mlp":
        import numpy as np

        from origindl_b200.trainer import MLPTrainer

        sizes = [int(v) for v in a.sizes.split(",")]
        kw = dict(optimizer="sgd", lr=1e-2, momentum=0.9) if a.optimizer == "sgd" else dict(optimizer="adam", lr=1e-3)
        tr = MLPTrainer(sizes, a.batch, precision=prec, **kw)
        rng, parts = np.random.default_rng(0), []
        for i, o in zip(sizes[:-1], sizes[1:]):  # Kaiming-uniform weights {in,out}, zero biases
            parts += [rng.uniform(-np.sqrt(6.0 / i), np.sqrt(6.0 / i), i * o).astype(np.float32), np.zeros(o, np.float32)]
        tr.set_params(np.concatenate(parts))
        x = torch.randn(a.batch, sizes[0], device="cuda")
        t = torch.randint(0, sizes[-1], (a.batch,), device="cuda", dtype=torch.int32)
        for _ in range(2):
            tr.train_step(x, t)
        ms = timed(lambda: tr.train_step(x, t), a.iters)
        flops = 6.0 * a.batch * sum(i * o for i, o in zip(sizes[:-1], sizes[1:])) - 2.0 * a.batch * sizes[0] * sizes[1]
        if a.graph:
            step = tr.capture_native(x, t)
            ms_g = timed(step, a.iters)
            print(f"mlp {a.sizes} batch {a.batch}: {ms_g:.3f} ms per step from the library-recorded CUDA graph "
                  f"({a.batch / ms_g * 1e3:.0f} samples/s)")
        print(f"mlp {a.sizes} batch {a.batch} {a.optimizer} {a.precision}: {ms:.3f} ms per training step, "
              f"{a.batch / ms * 1e3:.0f} samples/s, {flops / ms / 1e9:.1f} TFLOP/s (no dX for the first layer), "
              f"loss {float(tr.loss_tensor()):.4f}")
        tr.close()
    elif a.case == "batchnorm":
        N, C, HW = a.n, a.cols, a.rows
        x, dy = torch.randn(N, C, HW, 1, device="cuda"), torch.randn(N, C, HW, 1, device="cuda")
        gamma, beta = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda")
        rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
        _, mean, var = ops.batch_norm_forward(x, gamma, beta, rm, rv, act=capi.ACT_SILU)
        nb = 4.0 * x.numel()
        t_f = timed(lambda: ops.batch_norm_forward(x, gamma, beta, rm, rv, act=capi.ACT_SILU), a.iters)
        t_e = timed(lambda: ops.batch_norm_forward(x, gamma, beta, rm, rv, training=False, act=capi.ACT_SILU), a.iters)
        t_b = timed(lambda: ops.batch_norm_backward(dy, x, gamma, beta, mean, var, act=capi.ACT_SILU), a.iters)
        print(f"batchnorm+silu {N}x{C}x{HW} ({nb / 1e6:.0f} MB per tensor): training forward {t_f:.4f} ms "
              f"({3 * nb / t_f / 1e6:.0f} GB/s: 2 reads + 1 write), evaluation forward {t_e:.4f} ms ({2 * nb / t_e / 1e6:.0f} GB/s), "
              f"backward {t_b:.4f} ms ({5 * nb / t_b / 1e6:.0f} GB/s: 4 reads + 1 write)")
    elif a.case == "gather":
        n_src = 4 * a.rows
        src = torch.randn(n_src, a.cols, device="cuda")
        lab = torch.randint(0, 10, (n_src,), device="cuda")
        idx = torch.randperm(n_src, device="cuda")[:a.rows].contiguous()
        dst, dl = torch.empty(a.rows, a.cols, device="cuda"), torch.empty(a.rows, dtype=torch.int64, device="cuda")
        ms = timed(lambda: capi.call("odl_gather_rows", src.data_ptr(), a.cols, n_src, idx.data_ptr(), a.rows, a.cols,
                                     dst.data_ptr(), a.cols, lab.data_ptr(), dl.data_ptr(), capi.stream_handle()), a.iters)
        print(f"gather {a.rows} of {n_src} rows x {a.cols}: {ms:.4f} ms/launch, {8 * a.rows * a.cols / ms / 1e6:.1f} GB/s "
              f"(4 B read + 4 B written per element)")
    elif a.case == "gemm":
        n = a.n
        M, N, K = (a.m, a.n, a.k) if a.rect else (n, n, n)
        ta, tb = {"nt": (False, True), "nn": (False, False), "tn": (True, False)}[a.layout]
        A = torch.randn((K, M) if ta else (M, K), device="cuda")
        B = torch.randn((N, K) if tb else (K, N), device="cuda")
        As, Bs = ops.split_tf32(A), ops.split_tf32(B)
        ms = timed(lambda: ops.gemm(A, B, trans_a=ta, trans_b=tb, a_small=As, b_small=Bs, precision=prec), a.iters)
        shape = f"{M}x{N}x{K}" if a.rect else f"n={n}"
        print(f"gemm {a.layout} {a.precision} {shape}: {ms:.4f} ms/launch, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s")
        if a.yardstick:
            # context only: the vendor library's single-pass TF32 and fp32 GEMMs on the same operands
            At, Bt = (A.t() if ta else A), (B.t() if tb else B)
            for name, flag in (("TF32", True), ("fp32", False)):
                torch.backends.cuda.matmul.allow_tf32 = flag
                t = timed(lambda: torch.matmul(At, Bt), a.iters)
                print(f"  yardstick torch.matmul {name}: {t:.4f} ms, {2 * n ** 3 / t / 1e9:.1f} TFLOP/s")
    elif a.case == "split":
        n = a.n
        X = torch.randn(n, n, device="cuda")
        ms = timed(lambda: ops.split_tf32(X), a.iters)
        print(f"split n={n}: {ms:.4f} ms/launch, {8 * n * n / ms / 1e6:.1f} GB/s (4 B read + 4 B written per element)")
    elif a.case == "adam":
        n = a.n
        p, g, m, v = (torch.randn(n, device="cuda") for _ in range(4))
        v.abs_()
        ps = torch.empty_like(p)
        ms = timed(lambda: ops.adam_step(p, g, m, v, 3, hook_weight_decay=1e-4, p_small=ps), a.iters)
        print(f"adam n={n}: {ms:.4f} ms/launch, {36 * n / ms / 1e6:.1f} GB/s (16 B read + 20 B written per parameter)")
    elif a.case == "softmax":
        x = torch.randn(a.rows, a.cols, device="cuda")
        t = torch.randint(0, a.cols, (a.rows,), device="cuda", dtype=torch.int32)
        ms = timed(lambda: ops.softmax_cross_entropy(x, t), a.iters)
        print(f"softmax-CE {a.rows}x{a.cols}: {ms:.4f} ms per loss+gradient")
    elif a.case == "linear":
        # Linear forward+backward, W [N,K]; forward, dX, dW and the dY preparation pass (mask + db + low part) timed apart
        M, N, K = a.m, a.n, a.k
        x, w = torch.randn(M, K, device="cuda"), torch.randn(N, K, device="cuda")
        b, dy = 0.1 * torch.randn(N, device="cuda"), torch.randn(M, N, device="cuda")
        y = ops.linear_forward(x, w, b, relu=True, precision=prec)
        g = ops.relu_backward(dy, y)
        three = prec == capi.PRECISION_3XTF32
        xs, ws, gs = (ops.split_tf32(t) if three else None for t in (x, w, g))
        t_split = timed(lambda: (ops.split_tf32(x), ops.split_tf32(w)), a.iters) if three else 0.0
        t_fwd = timed(lambda: ops.linear_forward(x, w, b, relu=True, precision=prec, x_small=xs, w_small=ws), a.iters)
        db = torch.zeros(N, device="cuda")
        gbuf, gsm = torch.empty_like(dy), torch.empty_like(dy)
        t_prep = timed(lambda: capi.call("odl_split_tf32", dy.data_ptr(), N, M, N, y.data_ptr(), N, gbuf.data_ptr(),
                                         gsm.data_ptr() if three else None, N, db.data_ptr(), capi.stream_handle()), a.iters)
        t_dx = timed(lambda: ops.gemm(g, w, a_small=gs, b_small=ws, precision=prec), a.iters)
        t_dw = timed(lambda: ops.gemm(g, x, trans_a=True, a_small=gs, b_small=xs, precision=prec), a.iters)
        t_all = timed(lambda: ops.linear_backward(x, w, dy, y, precision=prec, x_small=xs, w_small=ws), a.iters)
        f = 2.0 * M * N * K / 1e9
        tot = t_split + t_fwd + t_all
        print(f"linear M={M} N={N} K={K} {a.precision}: split(x,W) {t_split:.3f} ms | fwd {t_fwd:.3f} ms {f / t_fwd:.0f} TF/s | "
              f"dY pass (mask+db+low) {t_prep:.3f} ms {12.0 * M * N / t_prep / 1e6 if three else 8.0 * M * N / t_prep / 1e6:.0f} GB/s | "
              f"dX {t_dx:.3f} ms {f / t_dx:.0f} TF/s | dW {t_dw:.3f} ms {f / t_dw:.0f} TF/s | backward call {t_all:.3f} ms | "
              f"fwd+bwd {tot:.3f} ms = {3 * f / tot:.0f} TFLOP/s")
    else:
        C, OC, k, s, p, hw = CONV_LAYERS[a.layer]
        capi.lib().odl_debug_set_conv_mode(1 if a.explicit else a.conv_mode)
        x = torch.rand(a.batch, C, hw, hw, device="cuda")
        w = torch.randn(OC, C, k, k, device="cuda") * (2.0 / (C * k * k)) ** 0.5
        b = torch.zeros(OC, device="cuda")
        y = ops.conv2d_forward(x, w, b, s, p, precision=prec)
        gy = torch.randn_like(y)
        msf = timed(lambda: ops.conv2d_forward(x, w, b, s, p, precision=prec), a.iters)
        msb = timed(lambda: ops.conv2d_backward(gy, x, w, s, p, precision=prec), a.iters)
        parts = [timed(lambda kw=kw: ops.conv2d_backward(gy, x, w, s, p, precision=prec, **kw), a.iters)
                 for kw in (dict(need_gw=False, need_gb=False), dict(need_gx=False, need_gb=False), dict(need_gx=False, need_gw=False))]
        ideal = 4 * (x.numel() + w.numel() + y.numel())
        print(f"conv layer {a.layer} ({C}->{OC} k{k} s{s} p{p} on {hw}x{hw}, batch {a.batch}, {a.precision}, "
              f"{'im2col + GEMM' if a.explicit else 'implicit GEMM'} forward): forward {msf:.4f} ms "
              f"({ideal / msf / 1e6:.1f} GB/s of ideal traffic), backward {msb:.4f} ms "
              f"(gx {parts[0]:.4f}, gw {parts[1]:.4f}, gb {parts[2]:.4f} when asked for alone)")


if __name__ == "__main__":
    main()
