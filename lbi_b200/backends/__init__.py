from .backbone_stack import BackboneStackRegionBackend
from .base import RegionBackend, RegionForwardCache
from .transformer import (
    StructuredTransformerLowering,
    TorchAutogradTransformerLowering,
    TransformerLowering,
    TransformerRegionBackend,
)
from .transformer_cuda import CudaTransformerLowering
from .transformer_structured import LayerCache, StructuredRegionCache, StructuredTransformerRegion

__all__ = [
    "BackboneStackRegionBackend",
    "RegionBackend",
    "RegionForwardCache",
    "TransformerLowering",
    "TransformerRegionBackend",
    "TorchAutogradTransformerLowering",
    "StructuredTransformerLowering",
    "CudaTransformerLowering",
    "LayerCache",
    "StructuredRegionCache",
    "StructuredTransformerRegion",
]
