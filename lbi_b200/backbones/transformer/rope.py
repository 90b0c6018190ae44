"""Rotary position embedding.

Half-split ("non-interleaved") or pairwise ("interleaved") rotation with fp32
trigonometry, as in the reference's ``backbones/transformer/rope.py:6-34``; the
cos/sin tables are cached per (length, head_dim, base, device) instead of being
rebuilt on every call.
"""
from __future__ import annotations

import torch

_TABLE_CACHE: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def rope_tables(seq_len: int, head_dim: int, base: float, device: torch.device, offset: int = 0):
    """Return fp32 ``cos, sin`` of shape [seq_len, head_dim // 2] for positions offset..offset+seq_len-1."""
    key = (int(seq_len), int(head_dim), float(base), str(device), int(offset))
    hit = _TABLE_CACHE.get(key)
    if hit is not None:
        return hit
    half = head_dim // 2
    pos = torch.arange(offset, offset + seq_len, device=device, dtype=torch.float32)
    inv_freq = float(base) ** (-2.0 * torch.arange(half, device=device, dtype=torch.float32) / float(head_dim))
    freqs = torch.outer(pos, inv_freq)
    tables = (freqs.cos().contiguous(), freqs.sin().contiguous())
    if offset != 0:  # single positions of a decode loop: cheap to rebuild, not worth a cache entry each
        return tables
    if len(_TABLE_CACHE) > 64:
        _TABLE_CACHE.clear()
    _TABLE_CACHE[key] = tables
    return tables


def apply_rope(x: torch.Tensor, base: float = 10000.0, interleaved: bool = False, inverse: bool = False,
               offset: int = 0) -> torch.Tensor:
    """Rotate ``x`` of shape [B, H, L, D]; ``inverse=True`` applies the transpose rotation (its VJP); ``offset`` is the position
    of the first of the L tokens (token-by-token decoding)."""
    if x.dim() != 4:
        raise ValueError("RoPE expects x shaped [B, H, L, D].")
    head_dim = x.shape[-1]
    if head_dim % 2 != 0:
        raise ValueError("RoPE requires an even head dimension.")
    cos, sin = rope_tables(x.shape[-2], head_dim, base, x.device, offset)
    if inverse:
        sin = -sin
    xf = x.float()
    if interleaved:
        pairs = xf.unflatten(-1, (head_dim // 2, 2))
        a, b = pairs[..., 0], pairs[..., 1]
        out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)
    else:
        a, b = xf[..., : head_dim // 2], xf[..., head_dim // 2 :]
        out = torch.cat((a * cos - b * sin, a * sin + b * cos), dim=-1)
    return out.to(dtype=x.dtype)
