"""Attention input-pullback microbenchmark (shape sweep).

    python -m lbi_b200.benchmarks.time_attention_pullback [--quick] [--check] [--out-dir out/benchmarks/attention_pullback]

Sweep (the workload of the reference's benchmarks/time_attention_pullback.py, extended to bf16 and head_dim 128):
causal attention, batch 8, 16 heads, seq {128, 512, 2048}, head_dim {64, 128}, basis {4, 16}, fp16 and bf16, inputs
N(0, 1) from seed 0.  Every kernel mode that supports the cell is timed with CUDA events on the launching stream
(3 warm-ups, median of ``--iters``, a 256 MB write between launches to flush L2); peak bytes and, with ``--check``,
the max abs error against the dense fp32 formula are recorded.  Writes ``attention_pullback_<timestamp>.csv``,
``latest.csv`` and ``latest_summary.json`` (speed-ups of the tcgen05 kernel over the library loop).

``--reference-dir DIR`` adds the reference's own CUDA kernel as a third arm where it applies (its WMMA "pblock4" kernel,
cuda/transformer/attention_pullback_mma.cu: fp16, head_dim 64, T <= 1024, at most four directions per launch; more
directions are timed as consecutive launches of four, the way its engine blocks them).  DIR is an unmodified install of
the reference whose ``cuda/transformer`` extension has been built for sm_100a; the arm calls
``cuda.transformer.attention_input_pullback_basis(kernel_mode="fa2_mma_pblock4")``, the reference's public entry.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import time
from pathlib import Path

import torch

from lbi_b200.ops import reference as ref
from lbi_b200.ops.attention import attention_input_pullback_basis, tcgen05_pullback_supported

FIELDS = ["dtype", "batch", "heads", "seq_len", "head_dim", "basis", "kernel_mode", "median_ms", "best_ms", "tflops",
          "peak_bytes", "max_abs_err", "status"]


CELL_KEYS = ("dtype", "batch", "heads", "seq_len", "head_dim", "basis")


def cell_name(row: dict) -> str:
    """``<dtype>_T<seq>_D<head_dim>_P<basis>``, with ``_B<batch>_H<heads>`` appended away from the default 8 x 16."""
    name = f"{row['dtype']}_T{row['seq_len']}_D{row['head_dim']}_P{row['basis']}"
    return name if (row["batch"], row["heads"]) == (8, 16) else f"{name}_B{row['batch']}_H{row['heads']}"


def pullback_flops(b, h, t, dh, p):
    """Useful work: per direction dV, dP, dQ, dK (4 causal matmuls of 2*T*T/2*Dh) plus S once."""
    one = 2.0 * t * t / 2.0 * dh
    return b * h * (p * 4 * one + one)


def load_reference_pullback(ref_dir: str):
    """The reference's attention_input_pullback_basis, or None with the reason."""
    import importlib
    import sys

    root = Path(ref_dir).resolve()
    ext_dir = root / "cuda" / "transformer"
    if not ext_dir.is_dir():
        return None, f"{ext_dir} not found"
    # an unrelated namespace package called `cuda` (cuda-python) may be registered already; the reference's own top-level
    # `cuda` package has to win for `cuda.transformer` to resolve
    for name in [m for m in sys.modules if m == "cuda" or m.startswith("cuda.")]:
        del sys.modules[name]
    for entry in (str(ext_dir), str(root)):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    try:
        mod = importlib.import_module("cuda.transformer")
    except Exception as exc:  # noqa: BLE001
        return None, f"import failed: {exc!r}"
    if getattr(mod, "transformer_lbi_cuda", None) is None:
        return None, "transformer_lbi_cuda extension not built"
    return mod.attention_input_pullback_basis, ""


def reference_mode(ref_fn, q, k, v, do, scale):
    """The reference's WMMA kernel over P directions: launches of at most four directions each."""
    outs = [ref_fn(q, k, v, do[:, lo : lo + 4], softmax_scale=scale, causal=True, kernel_mode="fa2_mma_pblock4")
            for lo in range(0, do.shape[1], 4)]
    return tuple(torch.cat([o[i] for o in outs], dim=1) for i in range(3)) if len(outs) > 1 else outs[0]


def autograd_mode(q, k, v, do, scale):
    """One SDPA backward per direction over a retained graph: the PyTorch baseline of the reference's ``--include-autograd``."""
    qg, kg, vg = (t.detach().requires_grad_(True) for t in (q, k, v))
    out = torch.nn.functional.scaled_dot_product_attention(qg, kg, vg, is_causal=True, scale=scale)
    grads = [torch.autograd.grad(out, (qg, kg, vg), do[:, i], retain_graph=i + 1 < do.shape[1]) for i in range(do.shape[1])]
    return tuple(torch.stack([g[j] for g in grads], dim=1) for j in range(3))


def time_mode(mode, q, k, v, do, scale, iters, flush, ref_fn=None, warmup=3):
    if mode == "reference_wmma_pblock4":
        fn = lambda: reference_mode(ref_fn, q, k, v, do, scale)
    elif mode == "autograd":
        fn = lambda: autograd_mode(q, k, v, do, scale)
    else:
        fn = lambda: attention_input_pullback_basis(q, k, v, do, scale=scale, causal=True, kernel_mode=mode)
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        out = fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0], torch.cuda.max_memory_allocated(), out


def _ints(text: str) -> tuple[int, ...]:
    return tuple(int(x) for x in text.split(",") if x.strip())


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Attention input-pullback microbenchmark")
    ap.add_argument("--quick", action="store_true", help="seq 512 and 2048, head_dim 64, bf16 only")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3, help="untimed launches per mode (at least 3)")
    ap.add_argument("--atol", type=float, default=3e-2)
    ap.add_argument("--out-dir", type=str, default="out/benchmarks/attention_pullback")
    ap.add_argument("--reference-dir", type=str, default="", help="install of the reference with its CUDA extension built")
    ap.add_argument("--seqs", type=str, default="", help="comma-separated sequence lengths (default: the sweep above)")
    # the sweep flags of the reference's benchmark (benchmarks/time_attention_pullback.py:211-230); each overrides one axis
    ap.add_argument("--seq-lens", type=str, default="", help="same as --seqs")
    ap.add_argument("--batches", type=str, default="", help="comma-separated batch sizes (default 8)")
    ap.add_argument("--heads", type=str, default="", help="comma-separated head counts (default 16)")
    ap.add_argument("--head-dims", type=str, default="", help="comma-separated head dimensions (default 64,128)")
    ap.add_argument("--basis-sizes", type=str, default="", help="comma-separated numbers of directions (default 4,16)")
    ap.add_argument("--dtype", choices=["float32", "float16", "bfloat16"], default="", help="one dtype instead of fp16 and bf16")
    ap.add_argument("--causal", choices=["true"], default="true", help="the kernels here are causal only")
    ap.add_argument("--check-max-tokens", type=int, default=0, help="skip the dense check above this B*H*T*Dh*P (0: T <= 512)")
    ap.add_argument("--include-simple", action="store_true", help="also time the dense fp32 formula")
    ap.add_argument("--include-autograd", action="store_true", help="also time one SDPA backward per direction")
    ap.add_argument("--skip-torch-formula", action="store_true", help="accepted; the dense formula is only timed with --include-simple")
    ap.add_argument("--no-default-kernel", action="store_true", help="do not time the tcgen05 kernel")
    for name in ("--include-fa2-loop", "--include-fa2-p1", "--include-fa2-mma-p1", "--include-fa2-mma-pblock4"):
        ap.add_argument(name, action="store_true", help="accepted; the library loop is always timed, and the reference's own "
                                                         "tensor-core kernel is the --reference-dir arm")
    return ap


def sweep_from_args(args) -> dict:
    """The axes of the sweep after the overrides."""
    seqs = (512, 2048) if args.quick else (128, 512, 2048)
    if args.seqs or args.seq_lens:
        seqs = _ints(args.seqs or args.seq_lens)
    dims = (64,) if args.quick else (64, 128)
    dtypes = (torch.bfloat16,) if args.quick else (torch.float16, torch.bfloat16)
    return {
        "batches": _ints(args.batches) or (8,), "heads": _ints(args.heads) or (16,), "seqs": seqs,
        "dims": _ints(args.head_dims) or dims, "basis": _ints(args.basis_sizes) or (4, 16),
        "dtypes": (getattr(torch, args.dtype),) if args.dtype else dtypes,
    }


def modes_for_cell(args, dtype, dh, heads, t, have_reference: bool) -> list[str]:
    modes = ["fa2_loop"] if dtype in (torch.float16, torch.bfloat16) else []
    if not args.no_default_kernel and tcgen05_pullback_supported(dtype, dh, heads, heads, t):
        modes.insert(0, "tcgen05_pblock")
    if have_reference and dtype == torch.float16 and dh == 64 and t <= 1024 and t % 16 == 0:
        modes.append("reference_wmma_pblock4")
    if args.include_simple or not modes:
        modes.append("dense")
    if args.include_autograd:
        modes.append("autograd")
    return modes


def main(argv: list[str] | None = None) -> None:
    args = build_parser().parse_args(argv)
    ref_fn = None
    if args.reference_dir:
        ref_fn, why = load_reference_pullback(args.reference_dir)
        if ref_fn is None:
            print(json.dumps({"reference_arm": "unavailable", "why": why}), flush=True)
    dev = torch.device("cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    axes = sweep_from_args(args)
    rows = []
    cells = [(dtype, batch, heads, t, dh, p) for dtype in axes["dtypes"] for batch in axes["batches"] for heads in axes["heads"]
             for t in axes["seqs"] for dh in axes["dims"] for p in axes["basis"]]
    for dtype, batch, heads, t, dh, p in cells:
        g = torch.Generator(device=dev).manual_seed(0)
        q, k, v = (torch.randn(batch, heads, t, dh, device=dev, generator=g).to(dtype) for _ in range(3))
        do = torch.randn(batch, p, heads, t, dh, device=dev, generator=g).to(dtype)
        scale = 1.0 / math.sqrt(dh)
        want = None
        small = (batch * heads * t * dh * p <= args.check_max_tokens) if args.check_max_tokens else (t <= 512)
        if args.check and small:
            want = ref.attention_input_pullback_dense(q, k, v, do, scale, True)
        for mode in modes_for_cell(args, dtype, dh, heads, t, ref_fn is not None):
            row = dict(dtype=str(dtype).replace("torch.", ""), batch=batch, heads=heads, seq_len=t, head_dim=dh,
                       basis=p, kernel_mode=mode, max_abs_err="", status="ok")
            try:
                med, best, peak, out = time_mode(mode, q, k, v, do, scale, args.iters, flush, ref_fn, args.warmup)
                row.update(median_ms=med, best_ms=best, peak_bytes=peak,
                           tflops=pullback_flops(batch, heads, t, dh, p) / med / 1e9)
                if want is not None:
                    err = max((a.float() - w).abs().max().item() for a, w in zip(out, want))
                    row["max_abs_err"] = err
                    if err > args.atol * max(w.abs().max().item() for w in want) + 1e-3:
                        row["status"] = "mismatch"
            except Exception as exc:  # noqa: BLE001 - recorded per cell
                row.update(median_ms="", best_ms="", peak_bytes="", tflops="", status=f"error: {exc!r}"[:120])
            rows.append(row)
            print(row, flush=True)
        del q, k, v, do, want
    out_dir = Path(args.out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    stamp = time.strftime("%Y%m%d_%H%M%S")
    for name in (f"attention_pullback_{stamp}.csv", "latest.csv"):
        with (out_dir / name).open("w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=FIELDS)
            w.writeheader()
            w.writerows(rows)
    speedups = {}
    for r in rows:
        if r["kernel_mode"] == "tcgen05_pblock" and r["status"] == "ok":
            base = next((x for x in rows if x["kernel_mode"] == "fa2_loop" and all(x[k] == r[k] for k in CELL_KEYS)), None)
            if base and base["status"] == "ok":
                speedups[cell_name(r)] = base["median_ms"] / r["median_ms"]
    over_ref = {}
    for r in rows:
        if r["kernel_mode"] == "tcgen05_pblock" and r["status"] == "ok":
            base = next((x for x in rows if x["kernel_mode"] == "reference_wmma_pblock4" and all(x[k] == r[k] for k in CELL_KEYS)), None)
            if base and base["status"] == "ok":
                over_ref[cell_name(r)] = base["median_ms"] / r["median_ms"]
    summary = {"speedup_tcgen05_over_fa2_loop": speedups, "speedup_tcgen05_over_reference_wmma": over_ref, "rows": len(rows)}
    (out_dir / "latest_summary.json").write_text(json.dumps(summary, indent=2))
    print(json.dumps(summary))


if __name__ == "__main__":
    main()
