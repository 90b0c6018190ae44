"""Causal self-attention with fused qkv projection, optional depthwise causal
conv on qkv, RoPE and grouped-query heads.

Parameter names (``in_proj``, ``conv1d``, ``out_proj``) and the op order match
the reference's ``backbones/transformer/attention.py:19-112``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from .rope import apply_rope


class CausalSelfAttention(nn.Module):
    """Fused qkv projection, optional depthwise causal conv on qkv, RoPE, grouped-query heads, causal softmax attention, output projection."""

    def __init__(
        self,
        dim: int,
        *,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int,
        rope_base: float = 10000.0,
        rope_interleaved: bool = False,
        softmax_scale: float | None = None,
        d_conv: int = 0,
        use_flash_attn: bool = True,
        bias: bool = False,
    ) -> None:
        super().__init__()
        if n_heads % n_kv_heads != 0:
            raise ValueError("n_heads must be divisible by n_kv_heads")
        self.dim = dim
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        self.rope_base = rope_base
        self.rope_interleaved = rope_interleaved
        self.softmax_scale = softmax_scale
        self.d_conv = d_conv
        self.use_flash_attn = use_flash_attn
        self.qkv_dim = head_dim * (n_heads + 2 * n_kv_heads)
        self.out_dim = head_dim * n_heads
        self.in_proj = nn.Linear(dim, self.qkv_dim, bias=bias)
        if d_conv > 0:
            self.conv1d = nn.Conv1d(
                self.qkv_dim, self.qkv_dim, kernel_size=d_conv, padding=d_conv - 1, groups=self.qkv_dim, bias=bias
            )
        self.out_proj = nn.Linear(self.out_dim, dim, bias=bias)

    @property
    def scale(self) -> float:
        return self.softmax_scale if self.softmax_scale is not None else 1.0 / math.sqrt(self.head_dim)

    def split_heads(self, qkv: torch.Tensor):
        """[B, T, qkv_dim] -> q [B, H, T, Dh], k/v [B, Hkv, T, Dh] (views)."""
        bsz, seqlen, _ = qkv.shape
        q_dim, kv_dim = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        q, k, v = qkv.split((q_dim, kv_dim, kv_dim), dim=-1)
        q = q.view(bsz, seqlen, self.n_heads, self.head_dim).transpose(1, 2)
        k = k.view(bsz, seqlen, self.n_kv_heads, self.head_dim).transpose(1, 2)
        v = v.view(bsz, seqlen, self.n_kv_heads, self.head_dim).transpose(1, 2)
        return q, k, v

    def expand_kv(self, x: torch.Tensor) -> torch.Tensor:
        if self.n_kv_heads == self.n_heads:
            return x
        return x.repeat_interleave(self.n_heads // self.n_kv_heads, dim=1)

    _expand_kv = expand_kv  # the reference's name (backbones/transformer/attention.py:61-65)

    def _can_use_flash_attn(self, x: torch.Tensor) -> bool:
        """Whether ``forward`` may take a fused attention kernel for this input (16-bit CUDA tensors with ``use_flash_attn``)."""
        return bool(self.use_flash_attn and x.is_cuda and x.dtype in (torch.float16, torch.bfloat16))

    def _flash_attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Causal attention of [B, H, T, Dh] tensors (kv heads already expanded) -> [B, T, H, Dh], the layout the reference's
        method of this name returns (attention.py:78-85)."""
        return F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=True, scale=self.scale).transpose(1, 2)

    def causal_conv(self, qkv: torch.Tensor) -> torch.Tensor:
        seqlen = qkv.shape[1]
        return self.conv1d(qkv.transpose(1, 2))[..., :seqlen].transpose(1, 2).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bsz, seqlen, _ = x.shape
        qkv = self.in_proj(x)
        if self.d_conv > 0:
            qkv = self.causal_conv(qkv)
        q, k, v = self.split_heads(qkv)
        q = apply_rope(q, base=self.rope_base, interleaved=self.rope_interleaved)
        k = apply_rope(k, base=self.rope_base, interleaved=self.rope_interleaved)
        k, v = self.expand_kv(k), self.expand_kv(v)
        out = F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=True, scale=self.scale)
        out = out.transpose(1, 2).contiguous().view(bsz, seqlen, self.out_dim)
        return self.out_proj(out)

    # ------------------------------------------------------------------ token-by-token decoding
    def allocate_decode_state(self, batch_size: int, max_len: int, device=None, dtype=None) -> dict:
        """Key / value cache for ``max_len`` positions, the last ``d_conv - 1`` pre-convolution qkv rows, the position counter."""
        device = self.in_proj.weight.device if device is None else device
        dtype = self.in_proj.weight.dtype if dtype is None else dtype
        state = {"k": torch.zeros(batch_size, self.n_kv_heads, max_len, self.head_dim, device=device, dtype=dtype),
                 "v": torch.zeros(batch_size, self.n_kv_heads, max_len, self.head_dim, device=device, dtype=dtype), "pos": 0}
        if self.d_conv > 0:
            state["conv"] = torch.zeros(batch_size, self.qkv_dim, self.d_conv - 1, device=device, dtype=dtype)
        return state

    @torch.no_grad()
    def step(self, x: torch.Tensor, state: dict) -> torch.Tensor:
        """One token x [B, D] at position ``state['pos']`` -> [B, D]; equals row ``pos`` of ``forward`` on the whole sequence."""
        bsz, pos = x.shape[0], int(state["pos"])
        if pos >= state["k"].shape[2]:
            raise ValueError("the key / value cache is full")
        qkv = self.in_proj(x)
        if self.d_conv > 0:
            window = torch.cat([state["conv"], qkv.unsqueeze(-1).to(state["conv"].dtype)], dim=-1)  # oldest ... newest
            state["conv"].copy_(window[..., 1:])
            qkv = (window * self.conv1d.weight[:, 0].to(window.dtype)).sum(dim=-1)
            if self.conv1d.bias is not None:
                qkv = qkv + self.conv1d.bias
        q, k, v = self.split_heads(qkv.unsqueeze(1))
        q = apply_rope(q, base=self.rope_base, interleaved=self.rope_interleaved, offset=pos)
        k = apply_rope(k, base=self.rope_base, interleaved=self.rope_interleaved, offset=pos)
        state["k"][:, :, pos] = k[:, :, 0].to(state["k"].dtype)
        state["v"][:, :, pos] = v[:, :, 0].to(state["v"].dtype)
        state["pos"] = pos + 1
        keys, values = self.expand_kv(state["k"][:, :, : pos + 1]), self.expand_kv(state["v"][:, :, : pos + 1])
        out = F.scaled_dot_product_attention(q, keys.to(q.dtype), values.to(q.dtype), dropout_p=0.0, is_causal=False, scale=self.scale)
        return self.out_proj(out.transpose(1, 2).reshape(bsz, self.out_dim))
