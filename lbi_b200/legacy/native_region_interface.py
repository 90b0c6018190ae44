"""LBI-1 model: same computation as ``LBILanguageModel`` on depth regions, with the parameter names of the first
release so that its checkpoints load with ``strict=True`` (reference legacy/native_region_interface.py:92-292).

State-dict quirks kept on purpose: ``blocks`` aliases ``backbone.blocks`` (both prefixes are saved) and a tied model
still saves ``lm_head.weight`` (it is the embedding tensor)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from ..backbones.general import BackboneSpec, apply_backbone_init, build_backbone_stack, init_transformer_module, make_final_norm
from ..interfaces.vector_mlp import (
    LegacyVectorMLPInterfaceView,
    VectorMLPHead,
    head_input_jacobian_t,
    layer_norm_input_jacobian_t,
    mean_pool_jacobian_t,
)
from ..models.region_plan import RegionPlan, build_region_ranges

RegionMessageHead = VectorMLPHead
build_region_slices = lambda layers, region_size: build_region_ranges(layers, region_size)  # noqa: E731


@dataclass
class RegionForwardCache:
    """One region of an LBI-1 forward under that release's field names."""

    region_idx: int
    region_range: tuple[int, int]
    x_static: torch.Tensor
    message_in: torch.Tensor
    hidden_bias: torch.Tensor
    hidden_input: torch.Tensor
    hidden_output: torch.Tensor
    pooled_hidden: torch.Tensor
    delta_message: torch.Tensor
    alpha: torch.Tensor
    pre_norm_message: torch.Tensor
    message_out: torch.Tensor


@dataclass
class RegionInterfaceCache:
    """The interface view of a forward cache with the reference's field names (legacy/native_region_interface.py:83-89);
    ``NativeRegionInterfaceModel.interface_cache`` builds it from the dict ``forward_with_cache`` returns."""
    boundaries: list[torch.Tensor]
    region_hidden_inputs: list[torch.Tensor]
    region_messages: list[torch.Tensor]
    region_ranges: list[tuple[int, int]]
    region_caches: list[RegionForwardCache]


class NativeRegionInterfaceModel(nn.Module):
    """The LBI-1 model (see the module docstring): depth regions, messages instead of states, first-release parameter names."""

    def __init__(self, *, vocab_size: int, region_size: int, message_dim: int, backbone_spec: BackboneSpec,
                 message_hidden_dim: int = 0, message_scale_init: float = 0.5, tie_embeddings: bool = False) -> None:
        super().__init__()
        backbone_spec.validate()
        self.dim, self.layers, self.message_dim = backbone_spec.dim, backbone_spec.layers, message_dim
        self.tie_embeddings = bool(tie_embeddings)
        self.plan = RegionPlan.depth(backbone_spec.layers, region_size)
        self.region_ranges = [tuple(r) for r in self.plan.layer_ranges]
        self.n_regions = self.num_regions = len(self.region_ranges)
        self.region_axis = "depth"
        self.embedding = nn.Embedding(vocab_size, self.dim)
        self.backbone = build_backbone_stack(backbone_spec)
        self.blocks = self.backbone.blocks
        self.norm = make_final_norm(backbone_spec)
        self.lm_head = nn.Linear(self.dim, vocab_size, bias=False)
        h = message_hidden_dim
        self.input_to_message = VectorMLPHead(self.dim, message_dim, hidden_dim=h)
        self.message_to_hidden = nn.ModuleList([VectorMLPHead(message_dim, self.dim, hidden_dim=h) for _ in range(self.n_regions)])
        self.hidden_to_message = nn.ModuleList([VectorMLPHead(self.dim, message_dim, hidden_dim=h) for _ in range(self.n_regions)])
        self.message_norm = nn.ModuleList([nn.LayerNorm(message_dim) for _ in range(self.n_regions)])
        self.message_alpha = nn.Parameter(torch.full((self.n_regions,), float(message_scale_init)))
        self.interface = LegacyVectorMLPInterfaceView(
            interface_width=message_dim, initial_encoder=self.input_to_message, decoders=self.message_to_hidden,
            encoders=self.hidden_to_message, norms=self.message_norm)
        object.__setattr__(self, "region_backend", self.backbone)  # engine hook only; must not add state-dict keys
        if backbone_spec.name in ("transformer", "hybrid"):
            init_transformer_module(self.embedding, n_layers=backbone_spec.layers)
            apply_backbone_init(self.backbone, backbone_spec, blocks=self.blocks)
            init_transformer_module(self.lm_head, n_layers=backbone_spec.layers)
        if self.tie_embeddings:
            nn.init.normal_(self.embedding.weight, std=0.02)
            self.lm_head.weight = self.embedding.weight

    # ---- hooks that let the shared scan engines drive this model
    def output_head_vjp_parameters(self) -> list[nn.Parameter]:
        params = list(self.norm.parameters())
        return params if self.tie_embeddings else [*params, self.lm_head.weight]

    def canvas_vjp_parameters(self) -> list[nn.Parameter]:
        return [self.embedding.weight]

    def shared_local_vjp_parameters(self) -> list[nn.Parameter]:
        return [self.embedding.weight, self.message_alpha]

    def _forward_region_message_map(self, ridx: int, x_static: torch.Tensor, m_in: torch.Tensor) -> torch.Tensor:
        """The local map m_k -> m_{k+1} of region ``ridx``."""
        start, end = self.region_ranges[ridx]
        x_out = self.backbone.forward_range(x_static + self.interface.decode(m_in, ridx).unsqueeze(1), start, end)
        return self.interface.update(x_out, m_in, ridx, self.message_alpha[ridx]).state

    # ---- helpers under the names the first release's tests and tools call (reference legacy/native_region_interface.py:155-157,
    # :172-200, :312-397); each is the closed-form statement over one piece of the interface
    def _pool_hidden(self, x: torch.Tensor) -> torch.Tensor:
        return self.interface.pool_hidden(x)

    def _apply_message_ablation(self, m: torch.Tensor, *, mode: str, next_region_idx: int = 0, noise_std: float = 1.0,
                                mask_keep_prob: float = 0.5, generator: torch.Generator | None = None) -> torch.Tensor:
        return self._ablate(m, mode, noise_std, mask_keep_prob, generator)

    def _module_input_pullback_matrix_autograd(self, module: nn.Module, x: torch.Tensor, g_out: torch.Tensor) -> torch.Tensor:
        """J^T of any module on [B, D] inputs for a basis g_out [B, P, D_out], by one backward pass over a replicated batch."""
        if x.dim() != 2 or g_out.dim() != 3:
            raise ValueError("module input pullback expects x [B, D] and g_out [B, P, D_out].")
        bsz, nbasis = g_out.shape[:2]
        rep = x.detach().repeat_interleave(nbasis, dim=0).requires_grad_(True)
        with torch.enable_grad():
            y = module(rep)
        (g,) = torch.autograd.grad(y, rep, g_out.to(device=y.device, dtype=y.dtype).reshape_as(y))
        return g.reshape(bsz, nbasis, x.shape[-1]).to(device=g_out.device, dtype=g_out.dtype)

    def _linear_input_pullback_matrix(self, linear: nn.Linear, g_out: torch.Tensor) -> torch.Tensor:
        if g_out.dim() != 3:
            raise ValueError("linear pullback expects g_out shaped [B, P, D_out].")
        dtype = torch.promote_types(g_out.dtype, linear.weight.dtype)
        return (g_out.to(device=linear.weight.device, dtype=dtype) @ linear.weight.to(dtype)).to(device=g_out.device, dtype=g_out.dtype)

    def _silu_input_pullback_matrix(self, x: torch.Tensor, g_out: torch.Tensor) -> torch.Tensor:
        if x.dim() != 2 or g_out.dim() != 3:
            raise ValueError("SiLU pullback expects x [B, D] and g_out [B, P, D].")
        from ..interfaces.vector_mlp import activation_derivative

        dtype = torch.promote_types(x.dtype, g_out.dtype)
        slope = activation_derivative(x.to(device=g_out.device, dtype=dtype), "silu")
        return (g_out.to(dtype) * slope.unsqueeze(1)).to(g_out.dtype)

    def _region_message_head_input_pullback_matrix(self, head: VectorMLPHead, x: torch.Tensor, g_out: torch.Tensor) -> torch.Tensor:
        if not isinstance(head, VectorMLPHead):
            raise TypeError(f"unsupported message head type: {type(head).__name__}")
        return head_input_jacobian_t(head, x, g_out).to(device=g_out.device, dtype=g_out.dtype)

    def _mean_pool_pullback_matrix(self, g_pooled: torch.Tensor, seq_len: int) -> torch.Tensor:
        if g_pooled.dim() != 3:
            raise ValueError("mean-pool pullback expects g_pooled shaped [B, P, D].")
        if seq_len <= 0:
            raise ValueError("seq_len must be positive.")
        return mean_pool_jacobian_t(g_pooled, seq_len)

    def _broadcast_message_pullback_matrix(self, g_hidden_input: torch.Tensor) -> torch.Tensor:
        if g_hidden_input.dim() != 4:
            raise ValueError("broadcast pullback expects g_hidden_input shaped [B, P, L, D].")
        return g_hidden_input.sum(dim=2)

    def _materialize_interface_pullback_mats_graph(self, cache: dict[str, Any]) -> list[torch.Tensor]:
        return self.materialize_interface_pullback_mats(cache, mode="graph")

    def _materialize_interface_pullback_mats_recompute(self, cache: dict[str, Any], basis_chunk: int) -> list[torch.Tensor]:
        return self._materialize_recompute(cache, int(basis_chunk))

    @staticmethod
    def _ablate(m, mode, noise_std, keep_prob, generator):
        if mode == "none":
            return m
        if mode == "zero_all":
            return torch.zeros_like(m)
        if mode == "noise":
            if noise_std < 0.0:
                raise ValueError("message_noise_std must be >= 0")
            return m if noise_std == 0.0 else m + noise_std * torch.randn(m.shape, device=m.device, dtype=m.dtype, generator=generator)
        if mode == "mask":
            if keep_prob <= 0.0 or keep_prob > 1.0:
                raise ValueError("message_mask_keep_prob must be in (0, 1]")
            return m if keep_prob == 1.0 else m * (torch.rand(m.shape, device=m.device, generator=generator) < keep_prob).to(m.dtype)
        raise ValueError(f"unsupported message ablation mode: {mode}")

    def forward_with_cache(self, input_ids: torch.Tensor, *, message_ablation: str = "none", message_noise_std: float = 1.0,
                           message_mask_keep_prob: float = 0.5, ablation_generator: torch.Generator | None = None,
                           detach_states: bool = False) -> tuple[torch.Tensor, dict[str, Any]]:
        ab = (message_ablation, message_noise_std, message_mask_keep_prob, ablation_generator)
        x_static = self.embedding(input_ids)
        initial = self.interface.initial_state(x_static)
        m = self._ablate(initial, *ab)
        boundaries, hidden_inputs, messages, state_inputs, caches = [x_static], [], [m], [], []
        cut = detach_states and torch.is_grad_enabled()
        for ridx, (start, end) in enumerate(self.region_ranges):
            m_in = m.detach().requires_grad_(True) if cut else m
            state_inputs.append(m_in)
            bias = self.interface.decode(m_in, ridx)
            x_in = x_static + bias.unsqueeze(1)
            x_out = self.backbone.forward_range(x_in, start, end)
            upd = self.interface.update(x_out, m_in, ridx, self.message_alpha[ridx])
            m = self._ablate(upd.state, *ab)
            hidden_inputs.append(x_in)
            boundaries.append(x_out)
            messages.append(m)
            caches.append(RegionForwardCache(ridx, (start, end), x_static, m_in, bias, x_in, x_out, upd.pooled_region_output,
                                             upd.delta_state, upd.update_scale, upd.pre_norm_state, m))
        normed = self.norm(x_out)
        logits = self.lm_head(normed.to(self.lm_head.weight.dtype))
        return logits, {
            "boundaries": boundaries, "region_hidden_inputs": hidden_inputs, "region_messages": messages,
            "region_ranges": self.region_ranges, "region_caches": caches,
            # keys of the owned model's cache, so the shared engines work on this model too
            "states": messages, "state_inputs": state_inputs, "initial_state": initial, "detached_states": cut,
            "region_axis": "depth",
        }

    @staticmethod
    def interface_cache(cache: dict[str, Any]) -> RegionInterfaceCache:
        """The interface fields of a ``forward_with_cache`` dict as the reference's dataclass."""
        return RegionInterfaceCache(boundaries=list(cache["boundaries"]), region_hidden_inputs=list(cache["region_hidden_inputs"]),
                                    region_messages=list(cache["region_messages"]), region_ranges=[tuple(r) for r in cache["region_ranges"]],
                                    region_caches=list(cache["region_caches"]))

    def forward(self, input_ids: torch.Tensor, *, message_ablation: str = "none", message_noise_std: float = 1.0,
                message_mask_keep_prob: float = 0.5, ablation_generator: torch.Generator | None = None) -> torch.Tensor:
        return self.forward_with_cache(input_ids, message_ablation=message_ablation, message_noise_std=message_noise_std,
                                       message_mask_keep_prob=message_mask_keep_prob, ablation_generator=ablation_generator)[0]

    # ---- closed-form pieces of the region-local pullback (reference legacy/native_region_interface.py:399-457; there the
    # LayerNorm factor is an autograd call on a replicated batch, here every factor is closed-form)
    def region_message_output_pullback_to_hidden_output(self, region_cache: RegionForwardCache, g_message_out: torch.Tensor) -> dict:
        """Cotangents of the outgoing message [B, P, R] -> the skip path to the incoming message and the cotangents of the
        region's hidden output [B, P, L, D] (through LayerNorm, the update scale, the encoder head and the token mean)."""
        if g_message_out.dim() != 3:
            raise ValueError("g_message_out must have shape [B, P, R]")
        ridx = region_cache.region_idx
        g_pre = layer_norm_input_jacobian_t(self.message_norm[ridx], region_cache.pre_norm_message.detach(), g_message_out)
        g_delta = g_pre * region_cache.alpha.detach().to(g_pre.dtype)
        g_pooled = head_input_jacobian_t(self.hidden_to_message[ridx], region_cache.pooled_hidden.detach(), g_delta)
        return {"g_pre_norm_message": g_pre, "g_message_skip": g_pre, "g_delta_message": g_delta, "g_pooled_hidden": g_pooled,
                "g_hidden_output": mean_pool_jacobian_t(g_pooled, region_cache.hidden_output.shape[1])}

    def region_hidden_input_pullback_to_message_input(self, region_cache: RegionForwardCache, g_hidden_input: torch.Tensor) -> dict:
        """Cotangents of the region's hidden input [B, P, L, D] -> cotangents of the incoming message (token sum, decoder head)."""
        if g_hidden_input.dim() != 4:
            raise ValueError("g_hidden_input must have shape [B, P, L, D]")
        g_bias = g_hidden_input.sum(dim=2)
        g_message = head_input_jacobian_t(self.message_to_hidden[region_cache.region_idx], region_cache.message_in.detach(), g_bias)
        return {"g_hidden_bias": g_bias, "g_message_input": g_message}

    def region_outer_message_input_pullback(self, region_cache: RegionForwardCache, g_message_out: torch.Tensor,
                                            g_hidden_input: torch.Tensor) -> dict:
        tail = self.region_message_output_pullback_to_hidden_output(region_cache, g_message_out)
        head = self.region_hidden_input_pullback_to_message_input(region_cache, g_hidden_input)
        return {**tail, **head, "g_message_input_total": tail["g_message_skip"] + head["g_message_input"]}

    # ---- message-chain VJPs: sequential reference, Jacobian materialisers, suffix scan (reference :459-694)
    def interface_vjp_chain(self, cache: dict[str, Any], g_top_message: torch.Tensor) -> list[torch.Tensor]:
        """Sequential pullback of the top message cotangent through the retained graph, one region at a time."""
        messages = cache["region_messages"]
        if len(messages) != self.n_regions + 1:
            raise ValueError("cache has an invalid region_messages length")
        if cache.get("detached_states"):
            raise ValueError("interface_vjp_chain needs a connected graph (forward_with_cache without detach_states)")
        g = [torch.zeros_like(messages[0]) for _ in range(self.n_regions + 1)]
        g[-1] = g_top_message
        for ridx in reversed(range(self.n_regions)):
            (g[ridx],) = torch.autograd.grad(messages[ridx + 1], messages[ridx], g[ridx + 1], retain_graph=True)
        return g

    def materialize_interface_pullback_mats(self, cache: dict[str, Any], *, mode: str = "graph", basis_chunk: int = 1) -> list[torch.Tensor]:
        """A_k^T [B, R, R] for every region (g_k = A_k^T g_{k+1}); ``graph`` differentiates the retained forward graph,
        ``recompute`` re-runs each region's message map on a basis-replicated batch, ``basis_chunk`` directions at a time."""
        from ..backward.pullbacks import build_interface_pullback_provider

        if mode not in ("graph", "recompute"):
            raise ValueError("interface Jacobian mode must be one of: graph, recompute")
        if mode == "recompute":
            return self._materialize_recompute(cache, int(basis_chunk))
        return build_interface_pullback_provider("graph").materialize_state_jacobian_t(model=self, cache=cache)

    def _materialize_recompute(self, cache: dict[str, Any], basis_chunk: int) -> list[torch.Tensor]:
        if basis_chunk <= 0:
            raise ValueError("basis_chunk must be > 0")
        out = []
        for ridx, rc in enumerate(cache["region_caches"]):
            m_in, x_static = rc.message_in.detach(), rc.x_static.detach()
            bsz, r = m_in.shape
            cols = []
            for j0 in range(0, r, basis_chunk):
                c = min(basis_chunk, r - j0)
                m_rep = m_in.repeat_interleave(c, dim=0).requires_grad_(True)
                with torch.enable_grad():
                    m_next = self._forward_region_message_map(ridx, x_static.repeat_interleave(c, dim=0), m_rep)
                basis = torch.zeros(bsz, c, r, device=m_in.device, dtype=m_next.dtype)
                basis[:, torch.arange(c), j0 + torch.arange(c)] = 1.0
                (g,) = torch.autograd.grad(m_next, m_rep, basis.reshape(bsz * c, r))
                cols.append(g.reshape(bsz, c, r))
            out.append(torch.cat(cols, dim=1).transpose(1, 2).contiguous())
        return out

    def compose_pullback_suffix(self, interface_pullback_mats) -> list[torch.Tensor]:
        """Suffix products S_k = A_k^T A_{k+1}^T ... (S_K = I), one [B, R, R] per message index."""
        from ..ops import suffix_scan_pullbacks

        mats = list(interface_pullback_mats)
        if not mats:
            return []
        if any(m.dim() != 3 or m.shape[-1] != m.shape[-2] for m in mats):
            raise ValueError("interface pullback matrices must be square [B, R, R]")
        suffix = suffix_scan_pullbacks(torch.stack(mats, dim=1))
        if suffix.shape[1] != len(mats) + 1:
            raise ValueError("suffix scan returned an unexpected shape")
        return [suffix[:, k].contiguous() for k in range(len(mats) + 1)]

    @staticmethod
    def _apply_pullback_mat(mat: torch.Tensor, vec: torch.Tensor, *, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        dtype = torch.promote_types(mat.dtype, vec.dtype)
        return torch.einsum("bij,bj->bi", mat.to(dtype), vec.to(device=mat.device, dtype=dtype)).to(
            device=vec.device, dtype=vec.dtype if out_dtype is None else out_dtype)

    def interface_vjp_scan_from_mats(self, interface_pullback_mats, g_top_message: torch.Tensor) -> list[torch.Tensor]:
        """Every message cotangent g_k = S_k g_K from the materialised A_k^T and the cotangent of the last message."""
        suffix = self.compose_pullback_suffix(interface_pullback_mats)
        if len(suffix) != self.n_regions + 1:
            raise ValueError("suffix length mismatch")
        return [self._apply_pullback_mat(s, g_top_message) for s in suffix]

    def interface_vjp_scan(self, cache: dict[str, Any], g_top_message: torch.Tensor, *, mode: str = "graph",
                           basis_chunk: int = 1) -> list[torch.Tensor]:
        return self.interface_vjp_scan_from_mats(self.materialize_interface_pullback_mats(cache, mode=mode, basis_chunk=basis_chunk),
                                                 g_top_message)

    def interface_vjp_scan_from_last_input_seed(self, interface_pullback_mats, g_last_input_message: torch.Tensor) -> list[torch.Tensor]:
        """The loss reads only the last region, so its cotangent enters at the last region's *incoming* message: cotangents
        of messages 0 .. K - 1 from A_0^T .. A_{K-2}^T seeded there."""
        mats = list(interface_pullback_mats)
        if len(mats) != self.n_regions:
            raise ValueError("interface_pullback_mats length mismatch")
        if self.n_regions == 0:
            return []
        if self.n_regions == 1:
            return [g_last_input_message]
        suffix = self.compose_pullback_suffix(mats[:-1])
        return [self._apply_pullback_mat(s, g_last_input_message) for s in suffix]
