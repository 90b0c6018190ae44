"""Entry points of the fused ops.

Every function takes the same arguments as its fp32 PyTorch statement in
``lbi_b200.ops.reference``.  CUDA tensors are routed to the hand-written sm_100a
kernels of the in-tree extension ``lbi_b200._C``; if that extension cannot be
loaded on a machine that has a GPU, importing this module raises instead of
silently running the PyTorch statements.  CPU tensors use the PyTorch statements.
"""
from __future__ import annotations

import os

import torch

from . import dispatch, reference
from . import reference as ref
from .native import ext, native_available, require_native

from .dispatch import (  # noqa: E402
    adamw_step,
    add_condition,
    add_rmsnorm_fwd,
    affine_suffix_scan,
    attention_bwd_packed,
    attention_fwd,
    attention_pullback_packed,
    causal_conv_dgrad,
    causal_conv_fwd,
    causal_conv_wgrad,
    embedding_fwd,
    embedding_scatter_add,
    gemm_tn,
    linear_dgrad,
    linear_fwd,
    linear_wgrad,
    lm_head_cross_entropy,
    mean_pool_tokens,
    rmsnorm,
    rmsnorm_bwd,
    rmsnorm_wgrad,
    rope_qkv,
    suffix_scan_pullbacks,
    sum_tokens,
    swiglu_bwd,
    swiglu_fwd,
    transpose_2d,
)

__all__ = [name for name in dir() if not name.startswith("_")]
