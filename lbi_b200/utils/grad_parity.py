"""Gradient-parity harness: scan-based exact backward against ``loss.backward()`` on the same model and batch.

A *case* fixes backbone, region axis, region count, device and dtype; a *trial* is one (seed, batch) pair.  Per
parameter the harness records max |diff|, max relative diff, cosine and relative L2; per trial the loss difference,
global cosine / relative L2 over all parameters, the 95th percentile of the per-parameter relative errors and the
``interface_scan_rms`` diagnostic; per case the worst values over the trials.  The pass criteria are the reference's
(tests/test_lbi_gradient_parity.py in the reference: per-parameter allclose atol 1e-5 / rtol 1e-4 in fp32, loss atol 1e-7,
scan rms < 1e-5).  The report script (scripts/generate_grad_parity_report.py) and the test-suite both use this module.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Any, Sequence

import torch
import torch.nn.functional as F

from ..backbones import BackboneSpec
from ..backward import AutogradEngine, ScanADEngine
from ..interfaces import VectorMLPInterface
from ..models import LBILanguageModel

_HYBRID_LAYERS = ("mamba3", "transformer", "mamba2", "transformer")


@dataclass(frozen=True)
class GradParityCase:
    """One gradient-parity case: backbone, region layout, device / dtype, tolerances."""

    name: str
    backbone_name: str
    region_mode: str                 # single_region | multi_region
    region_axis: str = "depth"
    regions: int = 2
    layers: int = 4
    dim: int = 32
    interface_width: int = 8
    vocab_size: int = 64
    seq_len: int = 32
    batch_size: int = 2
    tie_embeddings: bool = False
    device_type: str = "cpu"
    dtype_name: str = "float32"
    seeds: tuple[int, ...] = (0,)
    batches_per_seed: int = 1
    atol: float = 1e-5
    rtol: float = 1e-4
    loss_atol: float = 1e-7
    scan_rms_tol: float = 1e-5


@dataclass
class ParameterMetrics:
    """Gradient agreement of one parameter in one trial."""

    name: str
    numel: int
    has_ref_grad: bool
    has_native_grad: bool
    max_abs_diff: float = 0.0
    max_rel_diff: float = 0.0
    cosine: float = 1.0
    relative_l2: float = 0.0
    passed: bool = True


@dataclass
class TrialMetrics:
    """One (seed, batch) trial of a case: losses, global gradient metrics, per-parameter metrics."""

    case_name: str
    seed: int
    batch_index: int
    loss_ref: float
    loss_native: float
    global_cosine: float
    relative_l2_error: float
    max_abs_grad_diff: float
    max_rel_grad_diff: float
    p95_rel_grad_diff: float
    interface_scan_rms: float
    trial_passed: bool
    parameter_metrics: list[ParameterMetrics] = field(default_factory=list)

    @property
    def loss_abs_diff(self) -> float:
        return abs(self.loss_ref - self.loss_native)

    def to_summary_row(self) -> dict[str, Any]:
        return {"case_name": self.case_name, "seed": self.seed, "batch_index": self.batch_index, "loss_ref": self.loss_ref,
                "loss_native": self.loss_native, "loss_abs_diff": self.loss_abs_diff, "global_grad_cosine": self.global_cosine,
                "relative_l2_error": self.relative_l2_error, "max_abs_grad_diff": self.max_abs_grad_diff,
                "max_rel_grad_diff": self.max_rel_grad_diff, "p95_rel_grad_diff": self.p95_rel_grad_diff,
                "interface_scan_rms": self.interface_scan_rms}

    def per_parameter_rows(self) -> list[dict[str, Any]]:
        return [{"case_name": self.case_name, "seed": self.seed, "batch_index": self.batch_index, "parameter": m.name,
                 "numel": m.numel, "has_ref_grad": m.has_ref_grad, "has_native_grad": m.has_native_grad,
                 "max_abs_diff": m.max_abs_diff, "max_rel_diff": m.max_rel_diff, "cosine": m.cosine,
                 "relative_l2": m.relative_l2, "passed": m.passed} for m in self.parameter_metrics]


@dataclass
class CaseAggregate:
    """All trials of a case with the worst-case summary the report tables print."""

    case: GradParityCase
    interface_jacobian_mode: str
    jacobian_basis_chunk: int
    trial_metrics: list[TrialMetrics]

    @property
    def backbone(self) -> str:
        return self.case.backbone_name

    @property
    def region_mode(self) -> str:
        return self.case.region_mode

    def to_summary_row(self) -> dict[str, Any]:
        t = self.trial_metrics
        p95 = sorted(x.p95_rel_grad_diff for x in t)
        return {
            "case_name": self.case.name, "backbone": self.case.backbone_name, "region_mode": self.case.region_mode,
            "region_axis": self.case.region_axis, "interface_jacobian_mode": self.interface_jacobian_mode,
            "jacobian_basis_chunk": self.jacobian_basis_chunk, "device": self.case.device_type, "dtype": self.case.dtype_name,
            "num_trials": len(t), "num_trials_passed": sum(x.trial_passed for x in t),
            "worst_loss_abs_diff": max(x.loss_abs_diff for x in t), "min_global_grad_cosine": min(x.global_cosine for x in t),
            "max_relative_l2_error": max(x.relative_l2_error for x in t),
            "worst_max_abs_grad_diff": max(x.max_abs_grad_diff for x in t),
            "worst_max_rel_grad_diff": max(x.max_rel_grad_diff for x in t),
            "median_p95_rel_grad_diff": p95[len(p95) // 2], "worst_interface_scan_rms": max(x.interface_scan_rms for x in t),
        }


def _default_cases() -> list[GradParityCase]:
    out = []
    for backbone in ("transformer", "mamba2", "mamba3", "hybrid"):
        out.append(GradParityCase(f"{backbone}_single_region", backbone, "single_region", regions=1))
        out.append(GradParityCase(f"{backbone}_multi_region", backbone, "multi_region", regions=2))
        out.append(GradParityCase(f"{backbone}_sequence_regions", backbone, "sequence_regions", region_axis="sequence", regions=4))
    out.append(GradParityCase("transformer_multi_region_tied", "transformer", "multi_region_tied", regions=4, tie_embeddings=True))
    out.append(GradParityCase("transformer_multi_region_cuda_bf16", "transformer", "multi_region_lowp", regions=2,
                              device_type="cuda", dtype_name="bfloat16", atol=5e-2, rtol=5e-2, loss_atol=1e-2, scan_rms_tol=5e-2))
    return out


def get_grad_parity_cases(names: Sequence[str] | None = None, *, preset: str = "test") -> list[GradParityCase]:
    """``test``: one seed / one batch per case; ``report``: three seeds x two batches unless the caller overrides them."""
    cases = _default_cases()
    if preset == "report":
        cases = [replace(c, seeds=(1000, 1001, 1002), batches_per_seed=2) for c in cases]
    elif preset != "test":
        raise ValueError("preset must be 'test' or 'report'")
    if names:
        known = {c.name: c for c in cases}
        missing = [n for n in names if n not in known]
        if missing:
            raise KeyError(f"unknown grad parity cases: {missing}; known: {sorted(known)}")
        cases = [known[n] for n in names]
    return cases


def grad_parity_skip_reason(case: GradParityCase) -> str | None:
    if case.device_type == "cuda" and not torch.cuda.is_available():
        return "CUDA device not available"
    return None


def build_case_model(case: GradParityCase, seed: int) -> LBILanguageModel:
    """The model of a gradient-parity case, initialised from ``seed``."""
    torch.manual_seed(seed)
    spec = BackboneSpec(name=case.backbone_name, dim=case.dim, layers=case.layers, n_heads=4, n_kv_heads=2, d_conv=4, d_state=16,
                        headdim=16, chunk_size=8, layer_types=_HYBRID_LAYERS if case.backbone_name == "hybrid" else ())
    iface = VectorMLPInterface(feature_dim=case.dim, num_regions=case.regions, interface_width=case.interface_width,
                               interface_map_hidden_dim=case.dim // 2)
    model = LBILanguageModel(vocab_size=case.vocab_size, layers_per_region=max(1, case.layers // case.regions), backbone_spec=spec,
                             interface=iface, region_axis=case.region_axis, num_sequence_regions=case.regions,
                             tie_embeddings=case.tie_embeddings)
    return model.to(case.device_type)


def _loss(model, ids, tgt, case: GradParityCase, detach: bool):
    ctx = torch.autocast(case.device_type, dtype=torch.bfloat16) if case.dtype_name == "bfloat16" else torch.autocast("cpu", enabled=False)
    with ctx:
        logits, cache = model.forward_with_cache(ids, detach_states=detach)
    return F.cross_entropy(logits.float().reshape(-1, case.vocab_size), tgt.reshape(-1)), cache


def _parameter_metrics(name: str, ref, got, case: GradParityCase) -> ParameterMetrics:
    if ref is None or got is None:
        return ParameterMetrics(name, 0, ref is not None, got is not None, passed=(ref is None) == (got is None))
    r, g = ref.double().flatten(), got.double().flatten()
    diff = (g - r).abs()
    rel = diff / r.abs().clamp_min(1e-12)
    # relative error only where the reference gradient is not itself at round-off level
    mask = r.abs() > case.atol
    denom = float(r.norm() * g.norm())
    return ParameterMetrics(
        name, r.numel(), True, True, max_abs_diff=float(diff.max()), max_rel_diff=float(rel[mask].max()) if mask.any() else 0.0,
        cosine=float(torch.dot(r, g)) / denom if denom > 0 else 1.0, relative_l2=float((g - r).norm() / r.norm().clamp_min(1e-30)),
        passed=bool(torch.allclose(got.float(), ref.float(), atol=case.atol, rtol=case.rtol)))


def compute_grad_parity_trial(case: GradParityCase, seed: int, batch_index: int, *, interface_jacobian_mode: str,
                              jacobian_basis_chunk: int) -> TrialMetrics:
    """One trial: dense autograd against the scan engine on the same batch; losses, global and per-parameter gradient metrics."""
    model = build_case_model(case, seed)
    g = torch.Generator().manual_seed(seed * 7919 + batch_index)
    ids = torch.randint(0, case.vocab_size, (case.batch_size, case.seq_len), generator=g).to(case.device_type)
    tgt = torch.randint(0, case.vocab_size, (case.batch_size, case.seq_len), generator=g).to(case.device_type)
    loss_ref, cache = _loss(model, ids, tgt, case, False)
    ref = AutogradEngine().backward(model=model, loss=loss_ref, cache=cache).grad_map
    ref = {k: (None if v is None else v.detach().clone()) for k, v in ref.items()}
    loss_nat, cache = _loss(model, ids, tgt, case, True)
    engine = ScanADEngine(state_jacobian_mode=interface_jacobian_mode, state_jacobian_basis_chunk=jacobian_basis_chunk)
    res = engine.backward(model=model, loss=loss_nat, cache=cache)
    params = [_parameter_metrics(n, ref[n], res.grad_map.get(n), case) for n in ref]
    both = [(ref[m.name].double().flatten(), res.grad_map[m.name].double().flatten()) for m in params
            if m.has_ref_grad and m.has_native_grad]
    r_all, g_all = torch.cat([a for a, _ in both]), torch.cat([b for _, b in both])
    rels = sorted(m.max_rel_diff for m in params if m.has_ref_grad and m.has_native_grad)
    rms = float(res.diagnostics.get("interface_scan_rms", 0.0))
    loss_ok = abs(float(loss_ref.detach()) - float(loss_nat.detach())) <= case.loss_atol
    return TrialMetrics(
        case.name, seed, batch_index, float(loss_ref.detach()), float(loss_nat.detach()),
        global_cosine=float(torch.dot(r_all, g_all) / (r_all.norm() * g_all.norm()).clamp_min(1e-30)),
        relative_l2_error=float((g_all - r_all).norm() / r_all.norm().clamp_min(1e-30)),
        max_abs_grad_diff=max(m.max_abs_diff for m in params), max_rel_grad_diff=max(m.max_rel_diff for m in params),
        p95_rel_grad_diff=rels[min(len(rels) - 1, int(math.ceil(0.95 * len(rels))) - 1)] if rels else 0.0,
        interface_scan_rms=rms, trial_passed=loss_ok and rms < case.scan_rms_tol and all(m.passed for m in params),
        parameter_metrics=params)


def compute_grad_parity_case_aggregate(case: GradParityCase, *, interface_jacobian_mode: str = "recompute",
                                       jacobian_basis_chunk: int = 32) -> CaseAggregate:
    trials = [compute_grad_parity_trial(case, seed, b, interface_jacobian_mode=interface_jacobian_mode,
                                        jacobian_basis_chunk=jacobian_basis_chunk)
              for seed in case.seeds for b in range(case.batches_per_seed)]
    return CaseAggregate(case, interface_jacobian_mode, jacobian_basis_chunk, trials)


def assert_grad_parity_aggregate(case: GradParityCase, aggregate: CaseAggregate) -> None:
    failed = [t for t in aggregate.trial_metrics if not t.trial_passed]
    if failed:
        t = failed[0]
        worst = max(t.parameter_metrics, key=lambda m: m.max_abs_diff)
        raise AssertionError(f"{case.name}: {len(failed)}/{len(aggregate.trial_metrics)} trials failed; seed {t.seed} batch "
                             f"{t.batch_index}: loss diff {t.loss_abs_diff:.3e}, scan rms {t.interface_scan_rms:.3e}, worst "
                             f"parameter {worst.name} max abs diff {worst.max_abs_diff:.3e}")
