"""Per-op device timing of the fused-op layer (CUDA events around every ``lbi_b200.ops`` call).

    from lbi_b200.ops import profile
    profile.enable(); ...run steps...; print(profile.report())

Events are recorded on the current stream and only read after a device synchronise in ``report``; timing adds
two event records per op and no host synchronisation, so relative shares stay meaningful.
"""
from __future__ import annotations

import functools
from collections import defaultdict

import torch

_RECORDS: list = []
_ORIGINALS: dict = {}
_NAMES = [
    "add_rmsnorm_fwd", "rmsnorm_bwd", "rmsnorm_wgrad", "linear_fwd", "linear_dgrad", "linear_wgrad", "rope_qkv",
    "attention_fwd", "attention_pullback_packed", "swiglu_fwd", "swiglu_bwd", "lm_head_cross_entropy", "embedding_fwd",
    "embedding_scatter_add", "add_condition", "mean_pool_tokens", "sum_tokens", "suffix_scan_pullbacks",
    "affine_suffix_scan", "causal_conv_fwd", "causal_conv_dgrad",
]


# functions of lbi_b200.ops.mamba (called as ``mops.<name>`` by the Mamba lowering)
_MAMBA_NAMES = [
    "gate_silu_fwd", "gate_silu_bwd", "gated_rmsnorm_fwd", "gated_rmsnorm_bwd", "siso_small_fwd", "siso_small_bwd", "siso_wide_fwd",
    "siso_wide_bwd", "siso_scan_fwd", "siso_scan_bwd", "softplus_dt_fwd", "silu_fwd", "silu_bwd",
]


# (module, attribute) pairs outside the two op modules: the SSD entry points of the Mamba-2 lowering
_EXTRA = [
    ("lbi_b200.backends.mamba_structured", "_ssd_forward"), ("lbi_b200.backends.mamba_structured", "_ssd_backward"),
]
_MAMBA_NAMES += ["conv_silu_fwd", "conv_silu_bwd", "conv_silu_wgrad"]


def _wrap(name, fn):
    @functools.wraps(fn)
    def timed(*args, **kwargs):
        if not torch.cuda.is_available():
            return fn(*args, **kwargs)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = fn(*args, **kwargs)
        stop.record()
        _RECORDS.append((name, start, stop))
        return out

    return timed


def enable() -> None:
    import lbi_b200.ops as ops_pkg

    if _ORIGINALS:
        return
    for name in _NAMES:
        fn = getattr(ops_pkg, name, None)
        if fn is None:
            continue
        _ORIGINALS[name] = fn
        setattr(ops_pkg, name, _wrap(name, fn))
    import lbi_b200.ops.mamba as mamba_ops

    for name in _MAMBA_NAMES:
        fn = getattr(mamba_ops, name, None)
        if fn is not None:
            _ORIGINALS["mamba." + name] = fn
            setattr(mamba_ops, name, _wrap("mamba." + name, fn))
    import importlib

    for mod_name, attr in _EXTRA:
        mod = importlib.import_module(mod_name)
        _ORIGINALS[f"extra:{mod_name}:{attr}"] = getattr(mod, attr)
        setattr(mod, attr, _wrap(attr.lstrip("_"), getattr(mod, attr)))


def disable() -> None:
    import lbi_b200.ops as ops_pkg
    import lbi_b200.ops.mamba as mamba_ops

    import importlib

    for name, fn in _ORIGINALS.items():
        if name.startswith("extra:"):
            _, mod_name, attr = name.split(":")
            setattr(importlib.import_module(mod_name), attr, fn)
        elif name.startswith("mamba."):
            setattr(mamba_ops, name[len("mamba."):], fn)
        else:
            setattr(ops_pkg, name, fn)
    _ORIGINALS.clear()


def reset() -> None:
    _RECORDS.clear()


def summary() -> dict:
    torch.cuda.synchronize()
    totals, counts = defaultdict(float), defaultdict(int)
    for name, start, stop in _RECORDS:
        totals[name] += start.elapsed_time(stop)
        counts[name] += 1
    return {name: {"ms": totals[name], "calls": counts[name]} for name in totals}


def report() -> str:
    data = summary()
    total = sum(v["ms"] for v in data.values()) or 1.0
    lines = [f"{'op':28s} {'calls':>8s} {'ms':>12s} {'share':>7s}"]
    for name, v in sorted(data.items(), key=lambda kv: -kv[1]["ms"]):
        lines.append(f"{name:28s} {v['calls']:8d} {v['ms']:12.2f} {100.0 * v['ms'] / total:6.1f}%")
    lines.append(f"{'sum of timed ops':28s} {'':8s} {total:12.2f}")
    return "\n".join(lines)
