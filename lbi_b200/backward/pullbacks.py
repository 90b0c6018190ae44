"""Materialisation of the per-region interface Jacobian transposes ``A_k^T = (d s_{k+1} / d s_k)^T``.

Providers (factory ``build_interface_pullback_provider``):

* ``graph``       batched ``autograd.grad`` over the retained forward graph (reference backward/pullbacks.py:37-81)
* ``recompute``   re-run decode -> region -> update on a basis-replicated batch, chunk by chunk (reference :84-149)
* ``structured``  no autograd: closed-form interface J^T, the backend's ``input_pullback_basis`` over a chunk of
                  basis directions, token sum, closed-form decode J^T.  This wires the hooks the reference
                  declares but never calls (interfaces/base.py:68-106, backends/base.py:36-50).
* ``forward``     forward-mode: push R tangent directions of s_k through the region with ``torch.func.jvp``
                  (the reference has no forward-mode code).
"""
from __future__ import annotations

from typing import Any, Protocol, Sequence

import torch

from ..backends.base import autocast_as


class InterfacePullbackProvider(Protocol):
    """``materialize_state_jacobian_t(model=, cache=, regions=None) -> [A_k^T [B, R, R]]`` for the listed regions."""

    name: str

    def materialize_state_jacobian_t(self, *, model: Any, cache: dict, regions: Sequence[int] | None = None) -> list[torch.Tensor]: ...


def _regions(model, regions):
    return list(range(model.num_regions)) if regions is None else list(regions)


def _state_in(cache, k):
    return cache["state_inputs"][k] if "state_inputs" in cache else cache["states"][k]


class TorchGraphInterfacePullbackProvider:
    """One batched VJP of the identity basis through the retained forward graph per region."""

    name = "torch_graph"  # the reference's provider names (backward/pullbacks.py:153, :169)

    def __init__(self, basis_chunk: int = 1) -> None:
        self.basis_chunk = int(basis_chunk)  # unused: one batched VJP covers all directions (kept for the reference's signature)

    def materialize_state_jacobian_t(self, *, model, cache, regions=None):
        out = []
        for k in _regions(model, regions):
            s_in, s_out = _state_in(cache, k), cache["states"][k + 1]
            bsz, r = s_out.shape
            eye = torch.eye(r, device=s_out.device, dtype=s_out.dtype).unsqueeze(1).expand(r, bsz, r)
            try:
                (rows,) = torch.autograd.grad(s_out, s_in, eye, retain_graph=True, is_grads_batched=True)
            except RuntimeError:
                rows = torch.stack(
                    [torch.autograd.grad(s_out, s_in, eye[j].contiguous(), retain_graph=True)[0] for j in range(r)], dim=0
                )
            # rows[j, b, i] = d s_out[b, j] / d s_in[b, i]  ->  A^T[b, i, j]
            out.append(rows.permute(1, 2, 0).contiguous())
        return out


class TorchRecomputeInterfacePullbackProvider:
    """Re-runs decode -> region -> update on a basis-replicated batch, ``basis_chunk`` directions at a time."""

    name = "torch_recompute"

    def __init__(self, basis_chunk: int = 1) -> None:
        if basis_chunk <= 0:
            raise ValueError("basis_chunk must be > 0")
        self.basis_chunk = int(basis_chunk)

    def materialize_state_jacobian_t(self, *, model, cache, regions=None):
        out = []
        for k in _regions(model, regions):
            rc = cache["region_caches"][k]
            s_in = _state_in(cache, k).detach()
            canvas = rc.canvas_features.detach()
            bsz, r = s_in.shape
            cols = []
            for j0 in range(0, r, self.basis_chunk):
                c = min(self.basis_chunk, r - j0)
                s_rep = s_in.repeat_interleave(c, dim=0).requires_grad_(True)
                canvas_rep = canvas.repeat_interleave(c, dim=0)
                with torch.enable_grad(), autocast_as(cache.get("autocast")):
                    cond = model.interface.decode(s_rep, k)
                    region_out, _ = model.region_backend.forward_region(region_input=canvas_rep + cond.unsqueeze(1), region_index=k)
                    s_next = model.interface.update(s_rep, region_out, k).state
                basis = torch.zeros(bsz, c, r, device=s_in.device, dtype=s_next.dtype)
                basis[:, torch.arange(c), j0 + torch.arange(c)] = 1.0
                (g,) = torch.autograd.grad(s_next, s_rep, basis.reshape(bsz * c, r))
                cols.append(g.reshape(bsz, c, r))
            rows = torch.cat(cols, dim=1)  # [B, j, i]
            out.append(rows.transpose(1, 2).contiguous())
        return out


class StructuredInterfacePullbackProvider:
    """No autograd: closed-form interface J^T, the backend's basis pullback, token sum, closed-form decode J^T."""

    name = "structured"

    def __init__(self, basis_chunk: int = 0) -> None:
        self.basis_chunk = int(basis_chunk)

    @torch.no_grad()
    def materialize_state_jacobian_t(self, *, model, cache, regions=None):
        out = []
        iface = model.interface
        for k in _regions(model, regions):
            rc = cache["region_caches"][k]
            s_in = _state_in(cache, k).detach()
            bsz, r = s_in.shape
            seqlen = rc.region_output.shape[1]
            diag = {key: val.detach() for key, val in rc.interface_step.diagnostics.items()}
            eye = torch.eye(r, device=s_in.device, dtype=torch.float32).unsqueeze(0).expand(bsz, r, r)
            upd = iface.update_jacobian_t(k, diag, eye, seqlen)
            g_pooled = upd["g_pooled_features"]  # [B, R, D]
            chunk = self.basis_chunk if self.basis_chunk > 0 else r
            g_cond = []
            for j0 in range(0, r, chunk):
                g_out = (g_pooled[:, j0 : j0 + chunk] / float(seqlen)).unsqueeze(2).expand(-1, -1, seqlen, -1)
                g_in = model.region_backend.input_pullback_basis(cache=rc.backend_cache, output_cotangent_basis=g_out)
                g_cond.append(g_in.float().sum(dim=2))
            g_state = iface.decode_jacobian_t(k, s_in, torch.cat(g_cond, dim=1))
            rows = upd["g_state_skip"] + g_state.float()  # [B, j, i]
            out.append(rows.transpose(1, 2).contiguous())
        return out


class ForwardModeInterfacePullbackProvider:
    """Forward mode: pushes the R tangent directions of the incoming state through the region with ``torch.func.jvp``."""

    name = "forward"

    def __init__(self, basis_chunk: int = 0) -> None:
        self.basis_chunk = int(basis_chunk)

    def materialize_state_jacobian_t(self, *, model, cache, regions=None):
        from torch.func import jvp
        from torch.nn.attention import SDPBackend, sdpa_kernel

        out = []
        for k in _regions(model, regions):
            rc = cache["region_caches"][k]
            s_in = _state_in(cache, k).detach()
            canvas = rc.canvas_features.detach()
            bsz, r = s_in.shape

            def step(s):
                cond = model.interface.decode(s, k)
                region_out, _ = model.region_backend.forward_region(region_input=canvas + cond.unsqueeze(1), region_index=k)
                return model.interface.update(s, region_out, k).state

            cols = []
            # fused attention kernels have no forward-mode formula; the math path does
            with torch.enable_grad(), sdpa_kernel(SDPBackend.MATH):
                for i in range(r):
                    tangent = torch.zeros_like(s_in)
                    tangent[:, i] = 1.0
                    cols.append(jvp(step, (s_in,), (tangent,))[1])  # d s_out[b, :] / d s_in[b, i]
            out.append(torch.stack(cols, dim=1).contiguous())  # [B, i, j]
        return out


def materialize_interface_state_jacobian_t_graph(*, model: Any, cache: dict) -> list[torch.Tensor]:
    """Function form of the graph provider (reference backward/pullbacks.py:37-81)."""
    if len(cache["states"]) != model.num_regions + 1:
        raise ValueError("cache has invalid states length.")
    return TorchGraphInterfacePullbackProvider().materialize_state_jacobian_t(model=model, cache=cache)


def materialize_interface_state_jacobian_t_recompute(*, model: Any, cache: dict, basis_chunk: int) -> list[torch.Tensor]:
    """Function form of the recompute provider (reference backward/pullbacks.py:84-149)."""
    if len(cache["region_caches"]) != model.num_regions:
        raise ValueError("cache has invalid region_caches length.")
    return TorchRecomputeInterfacePullbackProvider(basis_chunk=basis_chunk).materialize_state_jacobian_t(model=model, cache=cache)


def build_interface_pullback_provider(mode: str, *, basis_chunk: int = 1) -> InterfacePullbackProvider:
    """``graph`` / ``recompute`` (also spelled ``torch_graph``, ``pytorch_recompute``, ... as in the reference,
    backward/pullbacks.py:187-197), ``structured``, ``forward``."""
    normalized = str(mode).strip().lower().replace("-", "_")
    if normalized in {"graph", "torch_graph", "pytorch_graph"}:
        return TorchGraphInterfacePullbackProvider(basis_chunk=basis_chunk)
    if normalized in {"recompute", "torch_recompute", "pytorch_recompute"}:
        return TorchRecomputeInterfacePullbackProvider(basis_chunk=basis_chunk)
    if normalized == "structured":
        return StructuredInterfacePullbackProvider(basis_chunk=basis_chunk)
    if normalized in {"forward", "forward_mode"}:
        return ForwardModeInterfacePullbackProvider(basis_chunk=basis_chunk)
    raise ValueError("interface Jacobian mode must be one of: graph, recompute, structured, forward")
