"""CUDA lowering for Transformer regions.

The reference's class of the same name exposes only the attention kernel and leaves the region-level
methods as stubs (backends/transformer_cuda.py:23-83).  This one is the structured lowering plus the
attention entry point with the reference's argument layout.
"""
from __future__ import annotations

from .transformer import StructuredTransformerLowering


class CudaTransformerLowering(StructuredTransformerLowering):
    """The structured lowering plus the attention basis-pullback entry point with the reference's argument layout."""

    name = "cuda"

    def __init__(self, *, allow_reference_fallback: bool = False) -> None:
        self.allow_reference_fallback = bool(allow_reference_fallback)

    def attention_input_pullback_basis(self, q, k, v, output_cotangent_basis, *, scale=None, softmax_scale=None, causal=True,
                                       kernel_mode: str | None = None):
        """(dQ, dK, dV) for a basis of output cotangents [B, P, H, T, Dh].  ``softmax_scale`` is the reference's keyword for
        ``scale``; its kernel-mode names are accepted as well as this package's, None picks by shape (backends/transformer_cuda.py:23-45)."""
        from ..ops.attention import attention_input_pullback_basis

        scale = softmax_scale if scale is None else scale
        return attention_input_pullback_basis(q, k, v, output_cotangent_basis, scale=scale, causal=causal,
                                              use_cuda=q.is_cuda, kernel_mode=kernel_mode)
