"""Vector interface with MLP maps.

    s_0       = Enc_init(mean_t canvas)
    cond_k    = Dec_k(s_k)                                  broadcast-added to every token of region k
    s_{k+1}   = LayerNorm_k(s_k + tanh(alpha_k) * Enc_k(mean_t region_out_k))

Module and parameter names (``initial_encoder``, ``decoders``, ``encoders``, ``norms``, ``update_scale``,
``net.0`` / ``net.2``) match the reference's ``interfaces/vector_mlp.py:125-161`` so state dicts are
interchangeable.  Differences: the hidden activation is configurable (SiLU default, GELU optional); every
Jacobian-transpose helper, LayerNorm included, is closed-form (the reference re-runs autograd on a
replicated batch for LayerNorm, :34-61); forward-mode (JVP) helpers are provided as well; and
``initialize(..., causal=True)`` starts from a token-independent state for sequence-axis regions, where
pooling the whole canvas would leak future tokens.
"""
from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

from .base import InterfaceModule, InterfaceSpec, InterfaceStep

_ACTIVATIONS = {"silu": nn.SiLU, "gelu": nn.GELU}


class VectorMLPHead(nn.Module):
    """``Linear`` or ``Linear -> act -> Linear``."""

    def __init__(self, in_dim: int, out_dim: int, hidden_dim: int = 0, activation: str = "silu") -> None:
        super().__init__()
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation must be one of: {', '.join(_ACTIVATIONS)}")
        self.activation = activation
        if hidden_dim > 0:
            self.net = nn.Sequential(nn.Linear(in_dim, hidden_dim), _ACTIVATIONS[activation](), nn.Linear(hidden_dim, out_dim))
        else:
            self.net = nn.Linear(in_dim, out_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        weight = self.net.weight if isinstance(self.net, nn.Linear) else self.net[0].weight
        return self.net(x.to(dtype=weight.dtype) if x.dtype != weight.dtype else x)

    def layers(self) -> tuple[nn.Linear, nn.Linear | None]:
        if isinstance(self.net, nn.Linear):
            return self.net, None
        return self.net[0], self.net[2]


def activation_derivative(pre: torch.Tensor, activation: str) -> torch.Tensor:
    if activation == "silu":
        sig = torch.sigmoid(pre)
        return sig * (1.0 + pre * (1.0 - sig))
    if activation == "gelu":
        cdf = 0.5 * (1.0 + torch.erf(pre * 0.7071067811865476))
        pdf = torch.exp(-0.5 * pre * pre) * 0.3989422804014327
        return cdf + pre * pdf
    raise ValueError(activation)


def _jac_kernels(*tensors: torch.Tensor) -> bool:
    """The basis-Jacobian kernels (csrc/interface_jac.cu) serve fp32 CUDA tensors outside of autograd graphs."""
    from .. import ops

    if not (tensors[0].is_cuda and ops.native_available() and hasattr(ops.ext(), "interface_mlp_jac")):
        return False
    if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
        return False
    return all(t.dtype == torch.float32 for t in tensors)


def _activation_diagonal(head: VectorMLPHead, first: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    # the pre-activation through the skinny fp32 kernel where it applies (no library GEMM on the engine's path)
    pre = _linear_forward(x.float(), first, None, False)[0]
    return activation_derivative(pre, head.activation).contiguous()


def head_input_jacobian_t(head: VectorMLPHead, x: torch.Tensor, g_out: torch.Tensor) -> torch.Tensor:
    """J^T of an interface map at input x [B, Din], applied to cotangents g_out [B, P, Dout] -> [B, P, Din]."""
    first, second = head.layers()
    if g_out.dim() == 3 and _jac_kernels(g_out, first.weight, *(() if second is None else (second.weight,))):
        from .. import ops

        ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        if second is None:   # g @ W
            return ops.ext().interface_mlp_jac(g_out.contiguous(), first.weight.detach().contiguous(), None, None, 1.0)
        return ops.ext().interface_mlp_jac(g_out.contiguous(), second.weight.detach().contiguous(), _activation_diagonal(head, first, x),
                                           first.weight.detach().contiguous(), 1.0)
    dtype = torch.promote_types(g_out.dtype, first.weight.dtype)
    g = g_out.to(dtype)
    if second is None:
        return (g @ first.weight.to(dtype)).to(g_out.dtype)
    pre = F.linear(x.to(dtype), first.weight.to(dtype), None if first.bias is None else first.bias.to(dtype))
    g_hidden = (g @ second.weight.to(dtype)) * activation_derivative(pre, head.activation).unsqueeze(1)
    return (g_hidden @ first.weight.to(dtype)).to(g_out.dtype)


def head_input_jacobian(head: VectorMLPHead, x: torch.Tensor, t_in: torch.Tensor) -> torch.Tensor:
    """Forward-mode counterpart: J applied to tangents t_in [B, P, Din] -> [B, P, Dout]."""
    first, second = head.layers()
    if t_in.dim() == 3 and _jac_kernels(t_in, first.weight, *(() if second is None else (second.weight,))):
        from .. import ops

        ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        w1_t = first.weight.detach().t().contiguous()
        if second is None:
            return ops.ext().interface_mlp_jac(t_in.contiguous(), w1_t, None, None, 1.0)
        return ops.ext().interface_mlp_jac(t_in.contiguous(), w1_t, _activation_diagonal(head, first, x),
                                           second.weight.detach().t().contiguous(), 1.0)
    dtype = torch.promote_types(t_in.dtype, first.weight.dtype)
    t = t_in.to(dtype) @ first.weight.to(dtype).t()
    if second is None:
        return t.to(t_in.dtype)
    pre = F.linear(x.to(dtype), first.weight.to(dtype), None if first.bias is None else first.bias.to(dtype))
    t = t * activation_derivative(pre, head.activation).unsqueeze(1)
    return (t @ second.weight.to(dtype).t()).to(t_in.dtype)


def layer_norm_input_jacobian_t(norm: nn.LayerNorm, x: torch.Tensor, g_out: torch.Tensor) -> torch.Tensor:
    """Closed-form LayerNorm J^T at x [B, R] applied to g_out [B, P, R]."""
    if g_out.dim() == 3 and x.dim() == 2 and _jac_kernels(g_out, x, *(() if norm.weight is None else (norm.weight,))):
        from .. import ops

        ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        return ops.ext().layernorm_jac(x.contiguous(), None if norm.weight is None else norm.weight.detach().contiguous(),
                                       g_out.contiguous(), float(norm.eps), True, 1.0)
    dtype = torch.promote_types(g_out.dtype, torch.float32)
    xf = x.to(dtype)
    mu = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + norm.eps)
    xhat = ((xf - mu) * rstd).unsqueeze(1)
    gh = g_out.to(dtype)
    if norm.weight is not None:
        gh = gh * norm.weight.to(dtype)
    out = (gh - gh.mean(dim=-1, keepdim=True) - xhat * (gh * xhat).mean(dim=-1, keepdim=True)) * rstd.unsqueeze(1)
    return out.to(g_out.dtype)


def layer_norm_input_jacobian(norm: nn.LayerNorm, x: torch.Tensor, t_in: torch.Tensor) -> torch.Tensor:
    """Forward-mode LayerNorm Jacobian (the un-weighted core is symmetric, so only the weight moves sides)."""
    if t_in.dim() == 3 and x.dim() == 2 and _jac_kernels(t_in, x, *(() if norm.weight is None else (norm.weight,))):
        from .. import ops

        ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        return ops.ext().layernorm_jac(x.contiguous(), None if norm.weight is None else norm.weight.detach().contiguous(),
                                       t_in.contiguous(), float(norm.eps), False, 1.0)
    dtype = torch.promote_types(t_in.dtype, torch.float32)
    xf = x.to(dtype)
    mu = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + norm.eps)
    xhat = ((xf - mu) * rstd).unsqueeze(1)
    t = t_in.to(dtype)
    out = (t - t.mean(dim=-1, keepdim=True) - xhat * (t * xhat).mean(dim=-1, keepdim=True)) * rstd.unsqueeze(1)
    if norm.weight is not None:
        out = out * norm.weight.to(dtype)
    return out.to(t_in.dtype)


# ---- forward with caches and parameter VJPs in closed form (no autograd, no library GEMM on CUDA) ----------------------
_ACT_CODE = {"silu": 1, "gelu": 2}


def _skinny_kernels(*tensors) -> bool:
    from .. import ops

    return (tensors[0].is_cuda and ops.native_available() and hasattr(ops.ext(), "small_linear_fwd") and not torch.is_grad_enabled()
            and all(t is None or t.dtype == torch.float32 for t in tensors))


def _linear_forward(x: torch.Tensor, lin: nn.Linear, act: str | None, want_pre: bool):
    """y = act(x W^T + b) for a few rows -> (y, pre-activation or None)."""
    if _skinny_kernels(x, lin.weight, lin.bias):
        from .. import ops

        ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        y, pre = ops.ext().small_linear_fwd(x.contiguous(), lin.weight.detach().contiguous(), None if lin.bias is None else lin.bias.detach(),
                                            _ACT_CODE[act] if act else 0, bool(want_pre))
        return y, (pre if want_pre else None)
    pre = F.linear(x.float(), lin.weight.float(), None if lin.bias is None else lin.bias.float())
    if act is None:
        return pre, (pre if want_pre else None)
    return (F.silu(pre) if act == "silu" else F.gelu(pre)), (pre if want_pre else None)


def _linear_vjp(g: torch.Tensor, x: torch.Tensor, lin: nn.Linear, target, want_input: bool):
    """Adds g^T x and sum_b g into the gradient accumulators ``target(param)`` and returns g W (or None)."""
    dw = target(lin.weight)
    db = None if lin.bias is None else target(lin.bias)
    if _skinny_kernels(g, x, lin.weight) and dw.is_contiguous() and (db is None or db.is_contiguous()):
        from .. import ops

        ops.dispatch.KERNEL_LAUNCHES["count"] += 1 + int(want_input)
        ops.ext().small_linear_wgrad_(g.contiguous(), x.contiguous(), dw, db)
        return ops.ext().small_linear_dgrad(g.contiguous(), lin.weight.detach().contiguous()) if want_input else None
    gf, xf = g.float(), x.float()
    dw.add_((gf.t() @ xf).to(dw.dtype))
    if db is not None:
        db.add_(gf.sum(0).to(db.dtype))
    return gf @ lin.weight.detach().float() if want_input else None


def head_forward_cached(head: VectorMLPHead, x: torch.Tensor):
    """-> (y [B, Dout] fp32, cache for ``head_parameter_vjp``)."""
    first, second = head.layers()
    xf = x.float()
    if second is None:
        y, _ = _linear_forward(xf, first, None, False)
        return y, (xf, None, None)
    hid, pre = _linear_forward(xf, first, head.activation, True)
    y, _ = _linear_forward(hid, second, None, False)
    return y, (xf, pre, hid)


def head_parameter_vjp(head: VectorMLPHead, cache, g_out: torch.Tensor, target, want_input: bool = True):
    """Cotangent g_out [B, Dout] of a head evaluated by ``head_forward_cached``: parameter gradients are added into
    ``target(param)``; returns the input cotangent [B, Din] (or None)."""
    first, second = head.layers()
    x, pre, hid = cache
    g = g_out.float()
    if second is None:
        return _linear_vjp(g, x, first, target, want_input)
    g_hid = _linear_vjp(g, hid, second, target, True)
    g_pre = g_hid * activation_derivative(pre, head.activation)
    return _linear_vjp(g_pre, x, first, target, want_input)


def layer_norm_parameter_vjp(norm: nn.LayerNorm, x: torch.Tensor, g_out: torch.Tensor, target) -> torch.Tensor:
    """LayerNorm at x [B, R] with cotangent g_out [B, R]: adds the weight / bias gradients, returns the input cotangent."""
    xf, g = x.float(), g_out.float()
    mu = xf.mean(dim=-1, keepdim=True)
    rstd = torch.rsqrt(xf.var(dim=-1, unbiased=False, keepdim=True) + norm.eps)
    xhat = (xf - mu) * rstd
    if norm.weight is not None:
        target(norm.weight).add_((g * xhat).sum(0))
    if norm.bias is not None:
        target(norm.bias).add_(g.sum(0))
    return layer_norm_input_jacobian_t(norm, x, g.unsqueeze(1)).squeeze(1)


def mean_pool_jacobian_t(g_pooled: torch.Tensor, seq_len: int) -> torch.Tensor:
    """[B, P, D] -> [B, P, L, D]: every token receives g / L (expanded view, no copy)."""
    if seq_len <= 0:
        raise ValueError("seq_len must be positive")
    return (g_pooled / float(seq_len)).unsqueeze(2).expand(-1, -1, seq_len, -1)


def broadcast_condition_jacobian_t(g_region_input: torch.Tensor) -> torch.Tensor:
    """[B, P, L, D] -> [B, P, D]: the condition was added to every token, so cotangents sum over tokens."""
    return g_region_input.sum(dim=2)


class VectorMLPInterface(InterfaceModule):
    """The bounded interface state as a vector of width R: the initial state is an MLP of the mean-pooled canvas, ``decode`` maps the
    state to a per-region condition added to every token, ``update`` is ``LayerNorm_k(s + tanh(scale_k) * MLP_k(mean_t(region output)))``.
    Per-region decoders / encoders / norms and one ``update_scale`` vector; closed-form Jacobian-transpose hooks for the structured engines."""

    def __init__(
        self,
        *,
        feature_dim: int,
        num_regions: int,
        interface_width: int,
        interface_map_hidden_dim: int = 0,
        update_scale_init: float = 0.5,
        activation: str = "silu",
    ) -> None:
        super().__init__()
        for label, value in (("feature_dim", feature_dim), ("num_regions", num_regions), ("interface_width", interface_width)):
            if value <= 0:
                raise ValueError(f"{label} must be > 0")
        if interface_map_hidden_dim < 0:
            raise ValueError("interface_map_hidden_dim must be >= 0")
        if update_scale_init <= 0.0:
            raise ValueError("update_scale_init must be > 0")
        self.spec = InterfaceSpec(state_shape=(interface_width,), state_flat_dim=interface_width, region_condition_dim=feature_dim)
        self.activation = activation
        h = interface_map_hidden_dim
        self.initial_encoder = VectorMLPHead(feature_dim, interface_width, h, activation)
        self.decoders = nn.ModuleList([VectorMLPHead(interface_width, feature_dim, h, activation) for _ in range(num_regions)])
        self.encoders = nn.ModuleList([VectorMLPHead(feature_dim, interface_width, h, activation) for _ in range(num_regions)])
        self.norms = nn.ModuleList([nn.LayerNorm(interface_width) for _ in range(num_regions)])
        self.update_scale = nn.Parameter(torch.full((num_regions,), float(update_scale_init)))

    @property
    def num_regions(self) -> int:
        return len(self.decoders)

    def validate_region_count(self, num_regions: int) -> None:
        if num_regions != self.num_regions:
            raise ValueError(f"vector interface region count must match model region count ({self.num_regions} != {num_regions})")

    @staticmethod
    def summarize_features(features: torch.Tensor) -> torch.Tensor:
        if features.dim() != 3:
            raise ValueError("vector interface features must have shape [B, T, D]")
        return features.mean(dim=1).to(dtype=features.dtype)

    def initialize(self, canvas_features: torch.Tensor, causal: bool = False) -> torch.Tensor:
        if causal:
            pooled = canvas_features.new_zeros(canvas_features.shape[0], canvas_features.shape[-1])
        else:
            pooled = self.summarize_features(canvas_features)
        return self.initial_encoder(pooled)

    def decode(self, state: torch.Tensor, region_index: int) -> torch.Tensor:
        return self.decoders[region_index](state)

    def update_from_pooled(self, state: torch.Tensor, pooled: torch.Tensor, region_index: int) -> InterfaceStep:
        delta = self.encoders[region_index](pooled)
        scale = torch.tanh(self.update_scale[region_index])
        pre_norm = state + scale * delta
        return InterfaceStep(
            state=self.norms[region_index](pre_norm),
            diagnostics={"pooled_features": pooled, "delta_state": delta, "update_scale": scale, "pre_norm_state": pre_norm},
        )

    def update(self, state: torch.Tensor, region_features: torch.Tensor, region_index: int) -> InterfaceStep:
        return self.update_from_pooled(state, self.summarize_features(region_features), region_index)

    def initial_vjp_parameters(self) -> list[nn.Parameter]:
        return [p for p in self.initial_encoder.parameters() if p.requires_grad]

    def region_vjp_parameters(self, region_index: int) -> list[nn.Parameter]:
        mods = (self.decoders[region_index], self.encoders[region_index], self.norms[region_index])
        return [p for m in mods for p in m.parameters() if p.requires_grad]

    def shared_vjp_parameters(self) -> list[nn.Parameter]:
        return [self.update_scale] if self.update_scale.requires_grad else []

    # ---- forward with caches / parameter VJPs without autograd ---------------------------
    def decode_cached(self, state: torch.Tensor, region_index: int):
        """-> (condition [B, D] fp32, cache for ``decode_parameter_vjp``)."""
        return head_forward_cached(self.decoders[region_index], state)

    def decode_parameter_vjp(self, region_index: int, cache, g_condition: torch.Tensor, target) -> None:
        head_parameter_vjp(self.decoders[region_index], cache, g_condition, target, want_input=False)

    def initial_cached(self, pooled: torch.Tensor):
        return head_forward_cached(self.initial_encoder, pooled)

    def initial_parameter_vjp(self, cache, g_state: torch.Tensor, target, want_input: bool = False):
        return head_parameter_vjp(self.initial_encoder, cache, g_state, target, want_input=want_input)

    def update_cached(self, state: torch.Tensor, pooled: torch.Tensor, region_index: int):
        """``update_from_pooled`` without autograd -> (InterfaceStep, encoder cache)."""
        delta, enc_cache = head_forward_cached(self.encoders[region_index], pooled)
        scale = torch.tanh(self.update_scale.detach()[region_index])
        pre_norm = state.float() + scale * delta
        norm = self.norms[region_index]
        out = F.layer_norm(pre_norm, (pre_norm.shape[-1],), None if norm.weight is None else norm.weight.detach().float(),
                           None if norm.bias is None else norm.bias.detach().float(), norm.eps)
        step = InterfaceStep(state=out, diagnostics={"pooled_features": pooled, "delta_state": delta, "update_scale": scale,
                                                     "pre_norm_state": pre_norm})
        return step, enc_cache

    def update_parameter_vjp(self, region_index: int, diagnostics: dict, enc_cache, g_state_out: torch.Tensor, target) -> torch.Tensor:
        """Cotangent of the outgoing state [B, R] -> cotangent of the pooled region output [B, D]; the gradients of the
        encoder, the LayerNorm and ``update_scale[region_index]`` are added into ``target(param)``.  ``enc_cache`` may be
        None (a fused forward kept no pre-activations): the encoder is then re-evaluated at the pooled features."""
        if enc_cache is None:
            _, enc_cache = head_forward_cached(self.encoders[region_index], diagnostics["pooled_features"])
        g_pre = layer_norm_parameter_vjp(self.norms[region_index], diagnostics["pre_norm_state"], g_state_out, target)
        scale = diagnostics["update_scale"].float()
        g_scale = (g_pre * diagnostics["delta_state"].float()).sum()
        target(self.update_scale)[region_index] += g_scale * (1.0 - scale * scale)
        return head_parameter_vjp(self.encoders[region_index], enc_cache, g_pre * scale, target, want_input=True)

    # ---- structured reverse-mode pieces -------------------------------------------------
    def update_jacobian_t(self, region_index: int, diagnostics: dict, g_state_out: torch.Tensor, seq_len: int) -> dict:
        g_pre = layer_norm_input_jacobian_t(self.norms[region_index], diagnostics["pre_norm_state"], g_state_out)
        g_delta = g_pre * diagnostics["update_scale"].to(g_pre.dtype)
        g_pooled = head_input_jacobian_t(self.encoders[region_index], diagnostics["pooled_features"], g_delta)
        return {
            "g_pre_norm_state": g_pre,
            "g_state_skip": g_pre,
            "g_delta_state": g_delta,
            "g_pooled_features": g_pooled,
            "g_region_output": mean_pool_jacobian_t(g_pooled, seq_len),
        }

    def decode_jacobian_t(self, region_index: int, state_in: torch.Tensor, g_condition: torch.Tensor) -> torch.Tensor:
        return head_input_jacobian_t(self.decoders[region_index], state_in, g_condition)

    def apply_update_jacobian_t_to_region_output(self, *, region_cache: Any, state_out_cotangent_basis: torch.Tensor):
        if state_out_cotangent_basis.dim() != 3:
            raise ValueError("state_out_cotangent_basis must have shape [B, P, R].")
        return self.update_jacobian_t(
            region_cache.region_index,
            region_cache.interface_step.diagnostics,
            state_out_cotangent_basis,
            region_cache.region_output.shape[1],
        )

    def apply_decode_jacobian_t_to_state_input(self, *, region_cache: Any, region_input_cotangent_basis: torch.Tensor):
        if region_input_cotangent_basis.dim() != 4:
            raise ValueError("region_input_cotangent_basis must have shape [B, P, L, D].")
        g_condition = broadcast_condition_jacobian_t(region_input_cotangent_basis)
        return {
            "g_condition": g_condition,
            "g_state_input": self.decode_jacobian_t(region_cache.region_index, region_cache.state_in, g_condition),
        }

    # ---- structured forward-mode pieces -------------------------------------------------
    def decode_jacobian(self, region_index: int, state_in: torch.Tensor, t_state: torch.Tensor) -> torch.Tensor:
        """Tangents of the state [B, P, R] -> tangents of the region condition [B, P, D]."""
        return head_input_jacobian(self.decoders[region_index], state_in, t_state)

    def update_jacobian(self, region_index: int, diagnostics: dict, t_state: torch.Tensor, t_pooled: torch.Tensor) -> torch.Tensor:
        """Tangents of (state, pooled region output) -> tangents of the next state."""
        t_delta = head_input_jacobian(self.encoders[region_index], diagnostics["pooled_features"], t_pooled)
        t_pre = t_state + diagnostics["update_scale"].to(t_delta.dtype) * t_delta
        return layer_norm_input_jacobian(self.norms[region_index], diagnostics["pre_norm_state"], t_pre)


@dataclass
class LegacyInterfaceUpdate:
    """Result of an LBI-1 state update under that release's field names."""

    state: torch.Tensor
    pooled_region_output: torch.Tensor
    delta_state: torch.Tensor
    update_scale: torch.Tensor
    pre_norm_state: torch.Tensor


class LegacyVectorMLPInterfaceView(nn.Module):
    """The same formulas over modules owned by someone else (the LBI-1 model keeps its own parameter names)."""

    def __init__(self, *, interface_width: int, initial_encoder: nn.Module, decoders: Sequence[nn.Module],
                 encoders: Sequence[nn.Module], norms: Sequence[nn.Module]) -> None:
        super().__init__()
        if interface_width <= 0:
            raise ValueError("interface_width must be > 0")
        if not (len(decoders) == len(encoders) == len(norms)):
            raise ValueError("interface region module counts must match")
        self.interface_width = int(interface_width)
        # bypass nn.Module registration: the owner already registers these modules under its own names
        object.__setattr__(self, "_initial_encoder", initial_encoder)
        object.__setattr__(self, "_decoders", decoders)
        object.__setattr__(self, "_encoders", encoders)
        object.__setattr__(self, "_norms", norms)

    @staticmethod
    def pool_hidden(hidden: torch.Tensor) -> torch.Tensor:
        return hidden.mean(dim=1).to(dtype=hidden.dtype)

    def initial_state(self, canvas: torch.Tensor) -> torch.Tensor:
        return self._initial_encoder(self.pool_hidden(canvas))

    def decode(self, state: torch.Tensor, region_index: int) -> torch.Tensor:
        return self._decoders[region_index](state)

    def update(self, region_output: torch.Tensor, previous_state: torch.Tensor, region_index: int,
               raw_update_scale: torch.Tensor) -> LegacyInterfaceUpdate:
        pooled = self.pool_hidden(region_output)
        delta = self._encoders[region_index](pooled)
        scale = torch.tanh(raw_update_scale)
        pre_norm = previous_state + scale * delta
        return LegacyInterfaceUpdate(
            state=self._norms[region_index](pre_norm), pooled_region_output=pooled, delta_state=delta,
            update_scale=scale, pre_norm_state=pre_norm,
        )
