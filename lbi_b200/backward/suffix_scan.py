"""Composition of interface Jacobian transposes.

Convention: ``A_k^T[b, i, j] = d s_{k+1}[b, j] / d s_k[b, i]`` so that ``g_k = A_k^T g_{k+1}`` is
``einsum('bij,bj->bi')``.  Same helper set as the reference's ``backward/suffix_scan.py:10-134`` plus the
affine recursion ``g_k = b_k + A_k^T g_{k+1}`` needed when every region owns loss terms.
"""
from __future__ import annotations

from collections.abc import Sequence

import torch

from .. import ops


def compose_suffix_jacobian_t(state_jacobians_t: Sequence[torch.Tensor]) -> list[torch.Tensor]:
    """K matrices [B, R, R] -> K + 1 suffix products (S_k = A_k^T ... A_{K-1}^T, S_K = I), fp32; none for K = 0."""
    if len(state_jacobians_t) == 0:
        return []
    if state_jacobians_t[0].shape[-1] != state_jacobians_t[0].shape[-2]:
        raise ValueError("interface state Jacobian-transpose tensors must be square.")
    stacked = torch.stack([m for m in state_jacobians_t], dim=1)
    suffix = ops.suffix_scan_pullbacks(stacked)
    return list(suffix.unbind(dim=1))


def apply_jacobian_t(jacobian_t: torch.Tensor, cotangent: torch.Tensor, *, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``J^T g`` per batch row in the wider of the two dtypes; ``out_dtype`` casts the result (default: leave it wide)."""
    dtype = torch.promote_types(jacobian_t.dtype, cotangent.dtype)
    out = torch.einsum("bij,bj->bi", jacobian_t.to(dtype), cotangent.to(device=jacobian_t.device, dtype=dtype))
    return out if out_dtype is None else out.to(out_dtype)


def propagate_state_adjoint_with_jacobian_scan(state_jacobians_t: Sequence[torch.Tensor], g_top_state: torch.Tensor) -> list[torch.Tensor]:
    """Seed at s_K: returns [g_0, ..., g_K] with g_K = g_top_state."""
    if len(state_jacobians_t) == 0:
        return [g_top_state]
    suffix = compose_suffix_jacobian_t(state_jacobians_t)
    return [apply_jacobian_t(s, g_top_state) for s in suffix]


def propagate_state_adjoint_from_last_region_input(state_jacobians_t: Sequence[torch.Tensor], g_last_input_state: torch.Tensor,
                                                   *, num_regions: int | None = None) -> list[torch.Tensor]:
    """Seed at s_{K-1} (the input state of the last region): the last Jacobian is not needed.

    Accepts either K matrices (the last one is dropped, as the reference does) or K - 1; with ``num_regions`` given the
    list must hold exactly that many (reference backward/suffix_scan.py:59-79)."""
    mats = list(state_jacobians_t)
    if num_regions is not None:
        if len(mats) != num_regions:
            raise ValueError("state_jacobians_t length mismatch.")
        if num_regions == 0:
            return []
    return propagate_state_adjoint_with_jacobian_scan(mats[:-1] if mats else mats, g_last_input_state)


def propagate_state_adjoint_affine(state_jacobian_t: Sequence[torch.Tensor], offsets: Sequence[torch.Tensor]) -> list[torch.Tensor]:
    """g_k = offsets_k + A_k^T g_{k+1} for k = K-1 .. 0 with g_K = 0, given A_0..A_{K-2} and b_0..b_{K-1}.

    Returns [g_0, ..., g_{K-1}] (fp32)."""
    k = len(offsets)
    if len(state_jacobian_t) != k - 1:
        raise ValueError("need exactly one Jacobian per region except the last")
    if k == 1:
        return [offsets[0].float()]
    mats = torch.stack(list(state_jacobian_t), dim=1)
    offs = torch.stack(list(offsets[:-1]), dim=1)
    g = ops.affine_suffix_scan(mats, offs, seed=offsets[-1])
    return list(g.unbind(dim=1))


def propagate_state_adjoint_by_autograd_chain(*, states: Sequence[torch.Tensor], top_state_adjoint: torch.Tensor) -> list[torch.Tensor]:
    """Diagnostic: pull the top state's adjoint down the retained forward graph one region at a time, without any
    materialised Jacobian (reference backward/suffix_scan.py:82-102).  Entry k is the adjoint of state k."""
    if len(states) < 2:
        raise ValueError("at least two interface states are required.")
    adjoints = [top_state_adjoint]
    for k in range(len(states) - 2, -1, -1):
        (g,) = torch.autograd.grad(states[k + 1], states[k], adjoints[0], retain_graph=True)
        adjoints.insert(0, g)
    return adjoints


def propagate_state_adjoint_by_chain(state_jacobian_t: Sequence[torch.Tensor], offsets: Sequence[torch.Tensor]) -> list[torch.Tensor]:
    """Sequential mat-vec recursion; the oracle for the scans."""
    k = len(offsets)
    out = [None] * k
    g = offsets[-1].float()
    out[k - 1] = g
    for idx in range(k - 2, -1, -1):
        g = offsets[idx].float() + apply_jacobian_t(state_jacobian_t[idx].float(), g)
        out[idx] = g
    return out


def _matrix_norms(mats: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(spectral, Frobenius) norms of [..., R, R]; on CUDA one kernel (power iteration), else torch.linalg."""
    from .. import ops

    if mats.is_cuda and ops.native_available() and hasattr(ops.ext(), "matrix_norms"):
        return ops.ext().matrix_norms(mats.float().contiguous(), 96)
    return torch.linalg.matrix_norm(mats, ord=2), torch.linalg.matrix_norm(mats, ord="fro")


def interface_state_jacobian_t_stats(state_jacobians_t: Sequence[torch.Tensor], *, include_suffix: bool = False) -> dict[str, float]:
    """Frobenius / spectral norms of the local Jacobians (and optionally of the suffix products)."""
    if len(state_jacobians_t) == 0:
        return {}
    mats = torch.stack([m.float() for m in state_jacobians_t], dim=1)  # [B, K, R, R]
    r = mats.shape[-1]
    spec, frob = _matrix_norms(mats)
    stats = {
        "jac_local_spec_mean": float(spec.mean()),
        "jac_local_spec_max": float(spec.max()),
        "jac_local_frob_mean": float(frob.mean()),
        "jac_local_frob_max": float(frob.max()),
        "jac_local_frob_normed_mean": float((frob / (r ** 0.5)).mean()),
    }
    if include_suffix:
        suffix = torch.stack(compose_suffix_jacobian_t(list(state_jacobians_t))[:-1], dim=1)
        sspec = _matrix_norms(suffix)[0]
        stats["jac_suffix_spec_mean"] = float(sspec.mean())
        stats["jac_suffix_spec_max"] = float(sspec.max())
    return stats
