"""Model construction from a training config (reference train/model_builders.py:14-131)."""
from __future__ import annotations

from typing import Any

from torch import nn

from ..backbones.general import BackboneSpec, infer_message_hidden_dim
from ..interfaces.vector_mlp import VectorMLPInterface
from ..models.dense_language_model import DenseLanguageModel
from ..models.lbi_language_model import LBILanguageModel
from ..models.region_plan import build_region_ranges
from .config import LEGACY_DENSE_REGIME, LEGACY_LBI_REGIME, normalize_regime_name


def build_backbone_spec(cfg: Any) -> BackboneSpec:
    spec = BackboneSpec(
        name=cfg.backbone, dim=cfg.dim, layers=cfg.layers, d_state=cfg.d_state, dt_rank=cfg.dt_rank, expand=cfg.expand,
        d_conv=cfg.d_conv, headdim=cfg.headdim, ngroups=cfg.ngroups, chunk_size=cfg.chunk_size,
        use_mem_eff_path=cfg.use_mem_eff_path, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, mlp_ratio=cfg.mlp_ratio,
        d_intermediate=cfg.d_intermediate, rope_base=cfg.rope_base, attn_head_dim=cfg.attn_head_dim,
        softmax_scale=cfg.softmax_scale, rope_interleaved=cfg.rope_interleaved, use_flash_attn=cfg.use_flash_attn,
        residual_in_fp32=cfg.residual_in_fp32, fused_add_norm=cfg.fused_add_norm,
        layer_types=tuple(t.strip() for t in cfg.layer_types.split(",") if t.strip()),
    )
    spec.validate()
    return spec


def build_dense_model(cfg: Any, *, backbone_spec: BackboneSpec | None = None) -> DenseLanguageModel:
    return DenseLanguageModel(vocab_size=int(cfg.vocab_size), backbone_spec=backbone_spec or build_backbone_spec(cfg),
                              tie_embeddings=bool(getattr(cfg, "tie_embeddings", False)))


def build_lbi_language_model(cfg: Any, *, backbone_spec: BackboneSpec | None = None) -> LBILanguageModel:
    """The owned LBI model of a config: backbone spec, vector-MLP interface, region plan on the configured axis, tied or own head."""
    spec = backbone_spec or build_backbone_spec(cfg)
    axis = getattr(cfg, "region_axis", "depth")
    n_regions = int(cfg.sequence_regions) if axis == "sequence" else len(build_region_ranges(spec.layers, int(cfg.region_size)))
    interface = VectorMLPInterface(
        feature_dim=spec.dim, num_regions=n_regions, interface_width=int(cfg.message_dim),
        interface_map_hidden_dim=infer_message_hidden_dim(spec, int(cfg.message_hidden_dim)),
        update_scale_init=float(cfg.message_scale_init), activation=getattr(cfg, "interface_activation", "silu"),
    )
    return LBILanguageModel(vocab_size=int(cfg.vocab_size), layers_per_region=int(cfg.region_size), backbone_spec=spec,
                            interface=interface, tie_embeddings=bool(getattr(cfg, "tie_embeddings", False)),
                            region_axis=axis, num_sequence_regions=n_regions if axis == "sequence" else 0)


def build_legacy_lbi_model(cfg: Any, *, backbone_spec: BackboneSpec | None = None) -> nn.Module:
    """Model with the LBI-1 parameter names, for state dicts saved by the first release."""
    from ..legacy.native_region_interface import NativeRegionInterfaceModel

    spec = backbone_spec or build_backbone_spec(cfg)
    return NativeRegionInterfaceModel(
        vocab_size=int(cfg.vocab_size), region_size=int(cfg.region_size), message_dim=int(cfg.message_dim),
        backbone_spec=spec, message_hidden_dim=infer_message_hidden_dim(spec, int(cfg.message_hidden_dim)),
        message_scale_init=float(cfg.message_scale_init), tie_embeddings=bool(getattr(cfg, "tie_embeddings", False)),
    )


build_lbi_model = build_lbi_language_model

_LEGACY_PREFIXES = ("input_to_message.", "message_to_hidden.", "hidden_to_message.", "message_norm.", "message_alpha")


def checkpoint_uses_owned_lbi(checkpoint: dict[str, Any]) -> bool:
    return any(str(k).startswith("interface.") for k in checkpoint.get("model_state_dict", {}))


def checkpoint_uses_legacy_lbi(checkpoint: dict[str, Any]) -> bool:
    keys = [str(k) for k in checkpoint.get("model_state_dict", {})]
    return any(k.startswith(_LEGACY_PREFIXES) for k in keys) and not any(k.startswith("interface.") for k in keys)


def build_model_for_regime(cfg: Any, *, checkpoint: dict[str, Any] | None = None,
                           use_legacy_lbi_checkpoint: bool | None = None, use_owned_lbi: bool | None = None) -> nn.Module:
    """The model class a run needs: dense, owned LBI, or the LBI-1 model when ``checkpoint`` carries first-release parameter names."""
    spec = build_backbone_spec(cfg)
    regime = normalize_regime_name(cfg.regime)
    if regime == LEGACY_DENSE_REGIME:
        return build_dense_model(cfg, backbone_spec=spec)
    if regime == LEGACY_LBI_REGIME:
        if use_owned_lbi is not None:
            use_legacy_lbi_checkpoint = not bool(use_owned_lbi)
        elif use_legacy_lbi_checkpoint is None and checkpoint is not None:
            use_legacy_lbi_checkpoint = checkpoint_uses_legacy_lbi(checkpoint)
        return build_legacy_lbi_model(cfg, backbone_spec=spec) if use_legacy_lbi_checkpoint else build_lbi_model(cfg, backbone_spec=spec)
    raise ValueError(f"unsupported model regime: {cfg.regime}")
