"""Mamba-2 SSD chunk scan (forward, or forward + backward with --backward): this package's sm_100a kernels against the chunked PyTorch form and, when the
reference tree is present under baseline/_ref, its Triton pipeline (``mamba_chunk_scan_combined``).

    python -m lbi_b200.benchmarks.time_ssd [--batch 4 --seq-len 8192 --heads 24 --d-state 64 128]

CUDA events after warm-up, L2 flushed between iterations.  Bytes counted per call: x and y (bf16), B and C (bf16), dt
(fp32) once each: the algorithmic minimum the roofline fraction is quoted against.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from lbi_b200.backbones.mamba2.ssd import ssd_chunk_scan
from lbi_b200.ops.ssd import ssd_chunk_scan_cuda


def _reference_triton():
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(root, "backbones")):
        return None
    for name in [m for m in sys.modules if m == "cuda" or m.startswith("cuda.")]:
        del sys.modules[name]
    sys.path.insert(0, root)
    try:
        from backbones.mamba2.ops.triton.ssd_combined import mamba_chunk_scan_combined

        return mamba_chunk_scan_combined
    except Exception as exc:  # noqa: BLE001
        print(f"[time_ssd] reference Triton path unavailable: {exc!r}", file=sys.stderr)
        return None
    finally:
        sys.path.remove(root)


def time_ms(fn, iters, flush):
    for _ in range(3):
        fn()
    out = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return sorted(out)[len(out) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--groups", type=int, default=1)
    ap.add_argument("--d-state", type=int, nargs="+", default=[64, 128])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip-torch", action="store_true")
    ap.add_argument("--kernel-table", action="store_true", help="with --backward: print the device-time table of one forward + backward")
    ap.add_argument("--backward", action="store_true", help="time forward + backward (all input gradients) instead of the forward")
    args = ap.parse_args()
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    triton_fn = _reference_triton()
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")) as fh:
            peaks = json.load(fh)
    except OSError:
        pass
    for n in args.d_state:
        b, l, h, g = args.batch, args.seq_len, args.heads, args.groups
        x = torch.randn(b, l, h, 64, device=dev).bfloat16()
        dt = torch.rand(b, l, h, device=dev) * 0.1 + 0.001
        A = -(torch.rand(h, device=dev) * 8 + 1)
        B = (torch.randn(b, l, g, n, device=dev) * 0.5).bfloat16()
        C = (torch.randn(b, l, g, n, device=dev) * 0.5).bfloat16()
        D = torch.randn(h, device=dev)
        nbytes = 2 * x.numel() * 2 + 2 * B.numel() * 2 + dt.numel() * 4
        rows = {}
        if args.backward:
            from lbi_b200.ops import ssd as ops_ssd

            leaves = [t.clone().requires_grad_(True) for t in (x, dt, A, B, C, D)]
            gy = torch.randn_like(x)

            def fwd_bwd(fn):
                def run():
                    y = fn(*leaves[:5], D=leaves[5])
                    torch.autograd.grad(y, leaves, gy)
                return run

            rows["tcgen05_fwd_bwd"] = time_ms(fwd_bwd(ssd_chunk_scan_cuda), args.iters, flush)
            if args.kernel_table:
                from torch.profiler import ProfilerActivity, profile

                with profile(activities=[ProfilerActivity.CUDA]) as prof:
                    fwd_bwd(ssd_chunk_scan_cuda)()
                    torch.cuda.synchronize()
                print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=70), file=sys.stderr)
            ops_ssd.BACKWARD_KERNELS = False
            if not args.skip_torch:
                rows["tcgen05_fwd_torch_recompute_bwd"] = time_ms(fwd_bwd(ssd_chunk_scan_cuda), max(2, args.iters // 3), flush)
            ops_ssd.BACKWARD_KERNELS = True
            if triton_fn is not None:
                try:
                    rows["reference_triton_fwd_bwd"] = time_ms(fwd_bwd(lambda *a, D=None: triton_fn(*a, 128, D=D)), args.iters, flush)
                except Exception as exc:  # noqa: BLE001
                    print(f"[time_ssd] reference Triton backward failed: {exc!r}", file=sys.stderr)
            for name, ms in rows.items():
                print(json.dumps({"d_state": n, "batch": b, "seq_len": l, "heads": h, "kernel": name, "median_ms": ms}))
            if "reference_triton_fwd_bwd" in rows:
                print(json.dumps({"d_state": n, "fwd_bwd_speedup_over_reference_triton": rows["reference_triton_fwd_bwd"] / rows["tcgen05_fwd_bwd"]}))
            continue
        with torch.no_grad():
            rows["tcgen05"] = time_ms(lambda: ssd_chunk_scan_cuda(x, dt, A, B, C, D=D), args.iters, flush)
            if triton_fn is not None:
                try:
                    rows["reference_triton"] = time_ms(lambda: triton_fn(x, dt, A, B, C, 128, D=D), args.iters, flush)
                except Exception as exc:  # noqa: BLE001
                    print(f"[time_ssd] reference Triton run failed: {exc!r}", file=sys.stderr)
            if not args.skip_torch:
                rows["torch_chunked"] = time_ms(lambda: ssd_chunk_scan(x, dt, A, B, C, chunk_size=128, D=D), max(2, args.iters // 3), flush)
        for name, ms in rows.items():
            rec = {"d_state": n, "batch": b, "seq_len": l, "heads": h, "kernel": name, "median_ms": ms, "gbytes_per_s": nbytes / ms / 1e6}
            if peaks.get("hbm_gbs"):
                rec["frac_of_measured_hbm"] = rec["gbytes_per_s"] / peaks["hbm_gbs"]
            print(json.dumps(rec))
        if "reference_triton" in rows:
            print(json.dumps({"d_state": n, "speedup_over_reference_triton": rows["reference_triton"] / rows["tcgen05"]}))


if __name__ == "__main__":
    main()
