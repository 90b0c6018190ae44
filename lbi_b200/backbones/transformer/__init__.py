from ..norms import RMSNorm
from .attention import CausalSelfAttention
from .block import TransformerBlock
from .mlp import GatedMLP, SwiGLUMLP
from .rope import apply_rope, rope_tables

__all__ = ["RMSNorm", "CausalSelfAttention", "TransformerBlock", "GatedMLP", "SwiGLUMLP", "apply_rope", "rope_tables"]
