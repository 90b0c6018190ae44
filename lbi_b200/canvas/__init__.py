from .base import CanvasCache, CanvasModule
from .token_embedding import TokenEmbeddingCanvas

__all__ = ["CanvasCache", "CanvasModule", "TokenEmbeddingCanvas"]
