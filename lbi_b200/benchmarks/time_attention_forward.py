"""Causal attention forward: this package's tcgen05 kernel against the flash_attn library kernel.

    python -m lbi_b200.benchmarks.time_attention_forward [--batch 8 --heads 16 --seq-lens 512 2048 8192]

CUDA-event timing after warm-up, L2 flushed between iterations; FLOPs counted as 4 * B * H * T^2 * Dh / 2 (causal).
Prints one JSON line per (T, kernel) and a final line with the speed-ups.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from lbi_b200.ops.attention import flash_forward_packed


def time_ms(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq-lens", type=int, nargs="+", default=[512, 2048, 8192])
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    speedups = {}
    for t in args.seq_lens:
        b = max(1, args.batch * 2048 // max(t, 2048))
        qkv = torch.randn(b * t, 3 * args.heads * 64, device="cuda").bfloat16()
        scale = 1.0 / math.sqrt(64)
        flops = 4.0 * b * args.heads * t * t * 64 / 2
        ms = {}
        for mode in ("tcgen05", "fa2"):
            ms[mode] = time_ms(lambda: flash_forward_packed(qkv, b, t, args.heads, args.heads, 64, scale, kernel_mode=mode),
                               args.iters, flush)
            print(json.dumps({"seq_len": t, "batch": b, "heads": args.heads, "kernel": mode, "median_ms": ms[mode],
                              "tflops": flops / ms[mode] / 1e9}))
        speedups[f"T{t}"] = ms["fa2"] / ms["tcgen05"]
    print(json.dumps({"speedup_tcgen05_over_fa2": speedups}))


if __name__ == "__main__":
    main()
