"""Times the tcgen05 GEMM against torch.matmul (cuBLAS) on the shapes of the LBI Transformer pullback.

    python -m lbi_b200.benchmarks.time_gemm [--rows 131072] [--iters 10]

CUDA events on the launching stream, 3 warm-up launches, a 256 MB write between launches to flush L2.
Prints one line per shape: milliseconds, TFLOP/s of both implementations, and the max abs difference.
"""
from __future__ import annotations

import argparse
import json

import torch

from lbi_b200 import ops


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=131072)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    dev = "cuda"
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    m = args.rows
    # (name, N, K, b_t): forward y = x W^T (b K-major) and dgrad dx = dy W (b MN-major)
    shapes = [
        ("fwd  qkv  ", 3072, 1024, False), ("fwd  out  ", 1024, 1024, False), ("fwd  fc1  ", 5632, 1024, False),
        ("fwd  fc2  ", 1024, 2816, False), ("dgrad qkv ", 1024, 3072, True), ("dgrad out ", 1024, 1024, True),
        ("dgrad fc1 ", 1024, 5632, True), ("dgrad fc2 ", 2816, 1024, True),
    ]
    results = []
    for name, n, k, b_t in shapes:
        a = torch.randn(m, k, device=dev).bfloat16()
        b = torch.randn((k, n) if b_t else (n, k), device=dev).bfloat16()
        ours = lambda: ops.ext().gemm(a, b, False, b_t, False, None, 1)
        lib = (lambda: a @ b) if b_t else (lambda: a @ b.t())
        t_ours, t_lib = _time(ours, args.iters, flush), _time(lib, args.iters, flush)
        diff = (ours().float() - lib().float()).abs().max().item()
        flops = 2.0 * m * n * k
        row = {"shape": name.strip(), "M": m, "N": n, "K": k, "ms_tcgen05": t_ours, "ms_cublas": t_lib,
               "tflops_tcgen05": flops / t_ours / 1e9, "tflops_cublas": flops / t_lib / 1e9, "max_abs_diff": diff}
        results.append(row)
        print(f"{name} M={m} N={n} K={k}: ours {t_ours:.3f} ms ({row['tflops_tcgen05']:.0f} TF)  "
              f"cuBLAS {t_lib:.3f} ms ({row['tflops_cublas']:.0f} TF)  diff {diff:.3g}")
        del a, b
    # wgrad form: dW = dy^T x with split-K
    rows, out_f, in_f = 8192, 1024, 2816
    dy = torch.randn(rows, out_f, device=dev).bfloat16()
    x = torch.randn(rows, in_f, device=dev).bfloat16()
    acc = torch.zeros(out_f, in_f, device=dev)
    t_ours = _time(lambda: ops.linear_wgrad(dy, x, accumulate_into=acc), args.iters, flush)
    t_lib = _time(lambda: acc.addmm_(dy.t().float(), x.float()) if False else dy.t() @ x, args.iters, flush)
    flops = 2.0 * rows * out_f * in_f
    print(f"wgrad fc2  rows={rows} {out_f}x{in_f}: ours {t_ours:.3f} ms ({flops / t_ours / 1e9:.0f} TF)  "
          f"cuBLAS {t_lib:.3f} ms ({flops / t_lib / 1e9:.0f} TF)")
    print(json.dumps(results))


if __name__ == "__main__":
    main()
