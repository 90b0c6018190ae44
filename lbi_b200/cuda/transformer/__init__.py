"""``attention_input_pullback_basis``: (dQ, dK, dV) of causal attention for a basis of output cotangents
(reference cuda/transformer/__init__.py:279-358; same positional arguments, ``softmax_scale`` / ``causal`` / ``use_cuda`` /
``kernel_mode`` keywords, the reference's mode names accepted)."""
from ...ops.attention import attention_input_pullback_basis

__all__ = ["attention_input_pullback_basis"]
