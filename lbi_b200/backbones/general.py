"""Backbone specification, layer stacks and initialisation.

Same public surface as the reference's ``backbones/general.py`` (BackboneSpec
:15-110, stacks :113-144, init :147-161, builders :164-371) so that configs and
checkpoints carry over; the blocks it builds are this package's own.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Optional

import torch
from torch import nn

from .norms import RMSNorm

SUPPORTED_BACKBONES = ("mamba2", "mamba3", "transformer")
_MAMBA_KINDS = {"mamba2", "mamba3"}


@dataclass
class BackboneSpec:
    """One flat description of any supported layer stack."""

    name: str = "transformer"
    dim: int = 64
    layers: int = 4
    d_state: int = 8
    dt_rank: Optional[int] = None
    # Mamba-family knobs
    expand: int = 2
    d_conv: int = 4
    bias: bool = False
    conv_bias: bool = True
    headdim: int = 128
    ngroups: int = 1
    chunk_size: int = 256
    use_mem_eff_path: bool = True
    # Transformer knobs
    n_heads: int = 8
    n_kv_heads: int = 0
    mlp_ratio: float = 4.0
    d_intermediate: int = 0
    rope_base: float = 10000.0
    attn_head_dim: int = 0
    softmax_scale: float = 0.0
    rope_interleaved: bool = False
    use_flash_attn: bool = True
    residual_in_fp32: bool = True
    fused_add_norm: bool = True
    layer_types: tuple[str, ...] = ()
    extra: Optional[dict[str, Any]] = None

    def resolved_layer_types(self) -> tuple[str, ...]:
        if self.name == "hybrid":
            return tuple(self.layer_types)
        return (self.name,) * self.layers

    def validate(self) -> None:
        allowed = (*SUPPORTED_BACKBONES, "hybrid")
        if self.name not in allowed:
            raise ValueError(f"unsupported backbone '{self.name}', expected one of: {', '.join(allowed)}")
        positive = {
            "dim": self.dim,
            "layers": self.layers,
            "d_state": self.d_state,
            "expand": self.expand,
            "headdim": self.headdim,
            "ngroups": self.ngroups,
            "chunk_size": self.chunk_size,
        }
        for key, value in positive.items():
            if value <= 0:
                raise ValueError(f"{key} must be > 0")
        if self.d_conv < 0:
            raise ValueError("d_conv must be >= 0")
        kinds = {self.name}
        if self.name == "hybrid":
            if not self.layer_types:
                raise ValueError("hybrid backbone requires non-empty layer_types")
            if len(self.layer_types) != self.layers:
                raise ValueError("for hybrid, len(layer_types) must equal layers")
            unknown = sorted(set(self.layer_types) - set(SUPPORTED_BACKBONES))
            if unknown:
                raise ValueError(
                    f"hybrid layer_types must be drawn from: {', '.join(SUPPORTED_BACKBONES)}; got: {', '.join(unknown)}"
                )
            kinds = set(self.layer_types)
        if kinds & _MAMBA_KINDS:
            if self.d_conv <= 0 and "mamba2" in kinds:
                raise ValueError("mamba2 requires d_conv > 0")
            if (self.expand * self.dim) % self.headdim != 0:
                raise ValueError("for mamba2/mamba3/hybrid-mamba layers, expand * dim must be divisible by headdim")
        if "transformer" in kinds:
            if self.n_heads <= 0:
                raise ValueError("transformer requires n_heads > 0")
            if self.n_kv_heads < 0:
                raise ValueError("transformer requires n_kv_heads >= 0")
            if self.attn_head_dim < 0:
                raise ValueError("transformer requires attn_head_dim >= 0")
            if self.attn_head_dim == 0 and self.dim % self.n_heads != 0:
                raise ValueError("for transformer, dim must be divisible by n_heads")
            if self.n_heads % (self.n_kv_heads or self.n_heads) != 0:
                raise ValueError("for transformer, n_heads must be divisible by n_kv_heads")
            if self.mlp_ratio < 0.0:
                raise ValueError("transformer requires mlp_ratio >= 0")
            if self.d_intermediate < 0:
                raise ValueError("transformer requires d_intermediate >= 0")
            if self.rope_base <= 0.0:
                raise ValueError("transformer requires rope_base > 0")
            if self.softmax_scale < 0.0:
                raise ValueError("transformer requires softmax_scale >= 0")


class BackboneStack(nn.Module):
    """A list of blocks that can be run in full or over a layer range."""

    def __init__(self, blocks: nn.ModuleList) -> None:
        super().__init__()
        self.blocks = blocks

    def forward_range(self, x: torch.Tensor, start: int = 0, end: Optional[int] = None) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_range(x, 0, len(self.blocks))


class LayerwiseBackboneStack(BackboneStack):
    """Blocks that map x -> x; a range is their composition."""

    def forward_range(self, x: torch.Tensor, start: int = 0, end: Optional[int] = None) -> torch.Tensor:
        stop = len(self.blocks) if end is None else end
        for index in range(start, stop):
            x = self.blocks[index](x)
        return x


class ResidualBackboneStack(BackboneStack):
    """Blocks exchange ``(branch_output, residual_stream)``; the range output is their sum."""

    def forward_range(self, x: torch.Tensor, start: int = 0, end: Optional[int] = None) -> torch.Tensor:
        stop = len(self.blocks) if end is None else end
        branch, stream = x, None
        for index in range(start, stop):
            branch, stream = self.blocks[index](branch, residual=stream)
        return branch if stream is None else branch + stream


def init_transformer_module(module: nn.Module, *, n_layers: int, n_residuals_per_layer: int = 2) -> None:
    """GPT-2 style init: zero Linear biases, N(0, 0.02) embeddings, residual-output
    projections (``out_proj``/``fc2``) drawn Kaiming-uniform and shrunk by sqrt(residuals * layers)."""
    shrink = math.sqrt(max(1, n_residuals_per_layer * n_layers))

    def visit(sub: nn.Module) -> None:
        if isinstance(sub, nn.Linear):
            if sub.bias is not None and not getattr(sub.bias, "_no_reinit", False):
                nn.init.zeros_(sub.bias)
        elif isinstance(sub, nn.Embedding):
            nn.init.normal_(sub.weight, std=0.02)
        for child_name in ("out_proj", "fc2"):
            child = getattr(sub, child_name, None)
            weight = getattr(child, "weight", None) if isinstance(child, nn.Module) else None
            if isinstance(weight, nn.Parameter) and not isinstance(sub, (nn.Linear, nn.Embedding)):
                nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
                with torch.no_grad():
                    weight /= shrink

    module.apply(visit)


def _transformer_block(spec: BackboneSpec) -> nn.Module:
    from .transformer import TransformerBlock

    return TransformerBlock(
        spec.dim,
        n_heads=spec.n_heads,
        n_kv_heads=spec.n_kv_heads or spec.n_heads,
        head_dim=spec.attn_head_dim or (spec.dim // spec.n_heads),
        d_intermediate=spec.d_intermediate,
        mlp_ratio=spec.mlp_ratio,
        rope_base=spec.rope_base,
        rope_interleaved=spec.rope_interleaved,
        softmax_scale=spec.softmax_scale if spec.softmax_scale > 0.0 else None,
        d_conv=spec.d_conv,
        use_flash_attn=spec.use_flash_attn,
        residual_in_fp32=spec.residual_in_fp32,
        fused_add_norm=spec.fused_add_norm,
        bias=spec.bias,
    )


def _mamba2_block(spec: BackboneSpec) -> nn.Module:
    from .mamba2 import Mamba2Block

    return Mamba2Block(
        spec.dim,
        d_state=spec.d_state,
        d_conv=spec.d_conv,
        expand=spec.expand,
        headdim=spec.headdim,
        ngroups=spec.ngroups,
        chunk_size=spec.chunk_size,
        use_mem_eff_path=spec.use_mem_eff_path,
        bias=spec.bias,
        conv_bias=spec.conv_bias,
    )


def _mamba3_block(spec: BackboneSpec) -> nn.Module:
    from .mamba3 import Mamba3Block

    return Mamba3Block(
        spec.dim,
        d_state=spec.d_state,
        expand=spec.expand,
        headdim=spec.headdim,
        ngroups=spec.ngroups,
        chunk_size=spec.chunk_size,
    )


_BLOCK_FACTORIES = {"transformer": _transformer_block, "mamba2": _mamba2_block, "mamba3": _mamba3_block}


def build_backbone_stack(spec: BackboneSpec) -> BackboneStack:
    spec.validate()
    blocks = nn.ModuleList([_BLOCK_FACTORIES[kind](spec) for kind in spec.resolved_layer_types()])
    return ResidualBackboneStack(blocks)


def build_backbone_blocks(spec: BackboneSpec) -> nn.ModuleList:
    return build_backbone_stack(spec).blocks


def make_final_norm(spec: BackboneSpec) -> nn.Module:
    return RMSNorm(spec.dim, eps=1e-5)


_make_final_norm = make_final_norm


def apply_backbone_init(module: nn.Module, spec: BackboneSpec, *, blocks: nn.ModuleList | None = None) -> None:
    """Transformer-style init for Transformer stacks and for the Transformer layers of a hybrid."""
    if spec.name == "transformer":
        init_transformer_module(module, n_layers=spec.layers, n_residuals_per_layer=2)
    elif spec.name == "hybrid" and blocks is not None:
        for kind, block in zip(spec.layer_types, blocks):
            if kind == "transformer":
                init_transformer_module(block, n_layers=spec.layers, n_residuals_per_layer=2)


class ReferenceLM(nn.Module):
    """Plain dense LM with flat key names (``embedding``, ``blocks``, ``norm``, ``lm_head``)."""

    def __init__(self, *, vocab_size: int, backbone_spec: BackboneSpec, tie_embeddings: bool = False) -> None:
        super().__init__()
        backbone_spec.validate()
        self.vocab_size = int(vocab_size)
        self.backbone_spec = backbone_spec
        self.tie_embeddings = bool(tie_embeddings)
        self.embedding = nn.Embedding(vocab_size, backbone_spec.dim)
        self.backbone = build_backbone_stack(backbone_spec)
        self.blocks = self.backbone.blocks
        self.norm = make_final_norm(backbone_spec)
        self.lm_head = nn.Linear(backbone_spec.dim, vocab_size, bias=False)
        if backbone_spec.name == "transformer":
            init_transformer_module(self, n_layers=backbone_spec.layers)
        elif backbone_spec.name == "hybrid":
            init_transformer_module(self.embedding, n_layers=backbone_spec.layers)
            apply_backbone_init(self.backbone, backbone_spec, blocks=self.blocks)
            init_transformer_module(self.lm_head, n_layers=backbone_spec.layers)
        if self.tie_embeddings:
            nn.init.normal_(self.embedding.weight, std=0.02)
            self.lm_head.weight = self.embedding.weight

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.lm_head(self.norm(self.backbone(self.embedding(input_ids))))


def infer_message_hidden_dim(spec: BackboneSpec, explicit_value: int) -> int:
    if explicit_value < 0:
        raise ValueError("explicit_value must be >= 0")
    return explicit_value if explicit_value > 0 else spec.dim
