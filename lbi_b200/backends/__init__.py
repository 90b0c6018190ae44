from .backbone_stack import BackboneStackRegionBackend
from .base import RegionBackend, RegionForwardCache
from .transformer import (
    StructuredTransformerLowering,
    TorchAutogradTransformerLowering,
    TransformerAttentionCache,
    TransformerLayerCache,
    TransformerLowering,
    TransformerMLPCache,
    TransformerRegionBackend,
    TransformerRegionCache,
)
from .transformer_cuda import CudaTransformerLowering
from .transformer_structured import LayerCache, StructuredRegionCache, StructuredTransformerRegion

__all__ = [
    "BackboneStackRegionBackend",
    "RegionBackend",
    "RegionForwardCache",
    "TransformerLowering",
    "TransformerRegionBackend",
    "TransformerAttentionCache",
    "TransformerMLPCache",
    "TransformerLayerCache",
    "TransformerRegionCache",
    "TorchAutogradTransformerLowering",
    "StructuredTransformerLowering",
    "CudaTransformerLowering",
    "LayerCache",
    "StructuredRegionCache",
    "StructuredTransformerRegion",
]
