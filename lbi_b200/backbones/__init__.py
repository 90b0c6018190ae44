from .general import (
    SUPPORTED_BACKBONES,
    BackboneSpec,
    BackboneStack,
    LayerwiseBackboneStack,
    ReferenceLM,
    ResidualBackboneStack,
    build_backbone_blocks,
    build_backbone_stack,
    infer_message_hidden_dim,
    init_transformer_module,
    make_final_norm,
)

__all__ = [
    "SUPPORTED_BACKBONES",
    "BackboneSpec",
    "BackboneStack",
    "LayerwiseBackboneStack",
    "ReferenceLM",
    "ResidualBackboneStack",
    "build_backbone_blocks",
    "build_backbone_stack",
    "infer_message_hidden_dim",
    "init_transformer_module",
    "make_final_norm",
]
