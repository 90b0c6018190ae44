from .base import InterfaceModule, InterfaceSpec, InterfaceStep
from .vector_mlp import LegacyVectorMLPInterfaceView, VectorMLPHead, VectorMLPInterface

__all__ = [
    "InterfaceModule",
    "InterfaceSpec",
    "InterfaceStep",
    "VectorMLPHead",
    "VectorMLPInterface",
    "LegacyVectorMLPInterfaceView",
]
