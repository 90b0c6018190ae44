"""Closed-form forward, input pullback over a basis and parameter VJP of a Transformer layer range.

This is the lowering that the reference only declares: its ``CudaTransformerLowering.input_pullback_basis``
and ``parameter_vjp`` raise NotImplementedError (backends/transformer_cuda.py:45-83) and the live engine
falls back to autograd over a replicated batch (backward/pullbacks.py:84-149).  Here every op of the block
(backends/transformer.py:118-243 lists them: prenorm, in_proj, optional conv, RoPE, attention, out_proj,
prenorm, fc1, SwiGLU, fc2) has an explicit J^T, chained over cached activations without autograd:

* ``forward``            records one ``LayerCache`` per layer,
* ``input_pullback``     pulls P output cotangents back to the region input in one pass; rows are laid out
                         basis-major ([P, B, T, D] flattened), so cached activations are shared by all P
                         directions and the GEMMs see M = P*B*T rows,
* ``backward``           single-cotangent backward that also produces every parameter gradient.

All tensor work goes through ``lbi_b200.ops`` (sm_100a kernels on CUDA, fp32 PyTorch on CPU).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import ops
from ..backbones.transformer.rope import rope_tables


@dataclass
class LayerCache:
    """Flat activations of one Transformer layer that the closed-form backward reads."""

    stream1: torch.Tensor  # fp32 residual stream entering norm 1          [n, D]
    rstd1: torch.Tensor  # [n]
    normed1: torch.Tensor  # input of in_proj                              [n, D]
    qkv_pre: torch.Tensor | None  # in_proj output before the causal conv (only when d_conv > 0)
    qkv: torch.Tensor  # after conv and RoPE                               [n, (H + 2Hkv) Dh]
    attn_out: torch.Tensor  # [n, H Dh]
    lse: torch.Tensor  # [B, H, T]
    stream2: torch.Tensor
    rstd2: torch.Tensor
    normed2: torch.Tensor
    fc1_out: torch.Tensor  # [n, 2F]  (up | gate)
    act: torch.Tensor  # [n, F]


@dataclass
class StructuredRegionCache:
    """A region forward of the structured Transformer lowering: shapes, input, per-layer caches, output pieces."""

    batch: int
    seq_len: int
    layer_range: tuple[int, int]
    region_input: torch.Tensor  # [n, D] in the activation dtype
    layers: list[LayerCache] = field(default_factory=list)
    output: torch.Tensor | None = None  # fp32 [n, D] = last_branch + last_stream
    last_branch: torch.Tensor | None = None
    last_stream: torch.Tensor | None = None


class LayerWeights:
    """Compute-dtype views of one block's parameters plus transposed copies for K-major dgrad GEMMs."""

    __slots__ = ("block", "norm1", "norm2", "w_qkv", "w_o", "w_fc1", "w_fc2", "w_qkv_t", "w_o_t", "w_fc1_t", "w_fc2_t",
                 "conv_w", "conv_b", "version")

    def __init__(self, block, dtype: torch.dtype, want_transposes: bool, shadow_of=None) -> None:
        self.block = block
        self.version = None
        self.refresh(dtype, want_transposes, shadow_of)

    def refresh(self, dtype: torch.dtype, want_transposes: bool, shadow_of=None) -> None:
        b = self.block
        for lin in (b.attn.in_proj, b.attn.out_proj, b.mlp.fc1, b.mlp.fc2):
            if lin.bias is not None:
                raise NotImplementedError("the structured Transformer lowering supports bias-free projections only")

        def cast(w):
            if shadow_of is not None:
                view = shadow_of(w)
                if view is not None and view.dtype == dtype:
                    return view  # lives in the optimizer's bf16 shadow buffer: refreshed by the AdamW kernel itself
            return w.detach().to(dtype).contiguous()

        self.norm1 = b.norm.weight.detach()
        self.norm2 = b.norm2.weight.detach()
        self.w_qkv, self.w_o = cast(b.attn.in_proj.weight), cast(b.attn.out_proj.weight)
        self.w_fc1, self.w_fc2 = cast(b.mlp.fc1.weight), cast(b.mlp.fc2.weight)
        if want_transposes:
            self.w_qkv_t, self.w_o_t = ops.transpose_2d(self.w_qkv), ops.transpose_2d(self.w_o)
            self.w_fc1_t, self.w_fc2_t = ops.transpose_2d(self.w_fc1), ops.transpose_2d(self.w_fc2)
        else:
            self.w_qkv_t = self.w_o_t = self.w_fc1_t = self.w_fc2_t = None
        if b.attn.d_conv > 0:
            self.conv_w = b.attn.conv1d.weight.detach().squeeze(1).float().contiguous()
            self.conv_b = None if b.attn.conv1d.bias is None else b.attn.conv1d.bias.detach().float()
        else:
            self.conv_w = self.conv_b = None


class StructuredTransformerRegion:
    """Runs layer ranges of a Transformer ``BackboneStack`` without autograd."""

    def __init__(self, blocks, *, act_dtype: torch.dtype | None = None) -> None:
        self.blocks = blocks
        self.act_dtype = act_dtype
        self._weights: dict[tuple, list[LayerWeights]] = {}
        self.shadow_of = None  # callable(param) -> compute-dtype view, set by the flat-buffer optimizer
        self.want_transposes = False  # K-major copies of W^T; only needed when the GEMM's MN-major path is off

    # ------------------------------------------------------------------ weights
    def weights(self, dtype: torch.dtype) -> list[LayerWeights]:
        device = self.blocks[0].norm.weight.device
        key = (dtype, str(device))
        cached = self._weights.get(key)
        if cached is None:
            cached = [LayerWeights(b, dtype, self.want_transposes and device.type == "cuda", self.shadow_of) if hasattr(b, "attn") else None
                      for b in self.blocks]   # None for the non-Transformer blocks of a hybrid stack
            self._weights[key] = cached
        return cached

    def refresh_weights(self) -> None:
        """Call after an optimizer step that did not update the compute-dtype copies in place."""
        for (dtype, dev), layers in self._weights.items():
            for lw in filter(None, layers):
                lw.refresh(dtype, self.want_transposes and dev.startswith("cuda"), self.shadow_of)

    def _dims(self, index: int):
        attn = self.blocks[index].attn
        return attn.n_heads, attn.n_kv_heads, attn.head_dim, attn.scale, attn.rope_base, attn.rope_interleaved

    # ------------------------------------------------------------------ one block, forward
    @torch.no_grad()
    def layer_forward(self, index: int, branch: torch.Tensor, stream: torch.Tensor | None, bsz: int, seqlen: int, dtype: torch.dtype):
        """(branch, fp32 stream or None) entering block ``index`` -> (branch, stream, LayerCache) leaving it."""
        lw = self.weights(dtype)[index]
        heads, kv_heads, head_dim, scale, rope_base, interleaved = self._dims(index)
        cos, sin = rope_tables(seqlen, head_dim, rope_base, branch.device)
        normed1, stream1, rstd1 = ops.add_rmsnorm_fwd(branch, stream, lw.norm1, self.blocks[index].norm.eps, dtype)
        qkv = ops.linear_fwd(normed1, lw.w_qkv)
        qkv_pre = None
        if lw.conv_w is not None:
            qkv_pre = qkv
            qkv = ops.causal_conv_fwd(qkv_pre, lw.conv_w, lw.conv_b, bsz, seqlen)
        qkv = ops.rope_qkv(qkv, cos, sin, heads, kv_heads, head_dim, seqlen, interleaved, inverse=False)
        attn_out, lse = ops.attention_fwd(qkv, bsz, seqlen, heads, kv_heads, head_dim, scale)
        branch = ops.linear_fwd(attn_out, lw.w_o)
        normed2, stream2, rstd2 = ops.add_rmsnorm_fwd(branch, stream1, lw.norm2, self.blocks[index].norm2.eps, dtype)
        fc1_out = ops.linear_fwd(normed2, lw.w_fc1)
        act = ops.swiglu_fwd(fc1_out)
        branch = ops.linear_fwd(act, lw.w_fc2)
        return branch, stream2, LayerCache(stream1, rstd1, normed1, qkv_pre, qkv, attn_out, lse, stream2, rstd2, normed2, fc1_out, act)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, region_input: torch.Tensor, layer_range: tuple[int, int], materialize_output: bool = True):
        """region_input [B, T, D] -> (fp32 output [B, T, D], cache).

        With ``materialize_output=False`` the sum ``branch + stream`` is left to the consumer (the final-norm
        kernel fuses it) and ``None`` is returned in place of the output."""
        bsz, seqlen, dim = region_input.shape
        dtype = self.act_dtype or region_input.dtype
        x = region_input.reshape(bsz * seqlen, dim).to(dtype).contiguous()
        cache = StructuredRegionCache(batch=bsz, seq_len=seqlen, layer_range=tuple(layer_range), region_input=x)
        branch, stream = x, None
        for index in range(*layer_range):
            branch, stream, lc = self.layer_forward(index, branch, stream, bsz, seqlen, dtype)
            cache.layers.append(lc)
        cache.last_branch, cache.last_stream = branch, stream
        if not materialize_output:
            return None, cache
        out = branch.float() if stream is None else branch.float() + stream
        cache.output = out
        return out.reshape(bsz, seqlen, dim), cache

    # ------------------------------------------------------------------ one block, reverse
    @torch.no_grad()
    def layer_reverse(self, index: int, lc: LayerCache, d_stream: torch.Tensor, d_branch: torch.Tensor, grads, bsz: int, seqlen: int,
                      dtype: torch.dtype):
        """Cotangents (fp32 stream, low-precision branch) [P * n, D] leaving block ``index`` -> the pair entering it."""
        lw = self.weights(dtype)[index]
        heads, kv_heads, head_dim, scale, rope_base, interleaved = self._dims(index)
        cos, sin = rope_tables(seqlen, head_dim, rope_base, d_stream.device)
        prefix = f"blocks.{index}."
        # MLP branch
        if grads is not None:
            _wgrad(grads, prefix + "mlp.fc2.weight", d_branch, lc.act)
        d_act = ops.linear_dgrad(d_branch, lw.w_fc2, lw.w_fc2_t)
        d_fc1 = ops.swiglu_bwd(d_act, lc.fc1_out)
        if grads is not None:
            _wgrad(grads, prefix + "mlp.fc1.weight", d_fc1, lc.normed2)
        d_normed2 = ops.linear_dgrad(d_fc1, lw.w_fc1, lw.w_fc1_t)
        if grads is not None:
            _acc(grads, prefix + "norm2.weight", ops.rmsnorm_wgrad(d_normed2, lc.stream2, lc.rstd2))
        d_stream, d_branch = ops.rmsnorm_bwd(d_normed2, lc.stream2, lc.rstd2, lw.norm2, d_stream, lowp_dtype=dtype)
        # attention branch
        if grads is not None:
            _wgrad(grads, prefix + "attn.out_proj.weight", d_branch, lc.attn_out)
        d_attn = ops.linear_dgrad(d_branch, lw.w_o, lw.w_o_t)
        d_qkv = ops.attention_pullback_packed(d_attn, lc.qkv, lc.attn_out, lc.lse, bsz, seqlen, heads, kv_heads, head_dim, scale,
                                              rope=(cos, sin, interleaved))
        if lw.conv_w is not None:
            if grads is not None:
                dw, db = ops.causal_conv_wgrad(d_qkv, lc.qkv_pre, lw.conv_w.shape[1], bsz, seqlen)
                _acc(grads, prefix + "attn.conv1d.weight", dw.unsqueeze(1))
                if lw.conv_b is not None:
                    _acc(grads, prefix + "attn.conv1d.bias", db)
            d_qkv = ops.causal_conv_dgrad(d_qkv, lw.conv_w, bsz, seqlen)
        if grads is not None:
            _wgrad(grads, prefix + "attn.in_proj.weight", d_qkv, lc.normed1)
        d_normed1 = ops.linear_dgrad(d_qkv, lw.w_qkv, lw.w_qkv_t)
        if grads is not None:
            _acc(grads, prefix + "norm.weight", ops.rmsnorm_wgrad(d_normed1, lc.stream1, lc.rstd1))
        d_stream, d_branch = ops.rmsnorm_bwd(d_normed1, lc.stream1, lc.rstd1, lw.norm1, d_stream, lowp_dtype=dtype)
        return d_stream, d_branch

    # ------------------------------------------------------------------ reverse chain
    @torch.no_grad()
    def _reverse(self, cache: StructuredRegionCache, d_out_rows: torch.Tensor, grads: dict | None):
        """d_out_rows [P*n, D] (cotangent of the region output) -> cotangent of the region input [P*n, D] fp32.

        With ``grads`` (a dict name -> fp32 tensor, P must be 1) parameter gradients are accumulated into it."""
        bsz, seqlen = cache.batch, cache.seq_len
        dtype = cache.region_input.dtype
        d_stream = d_out_rows.float()
        d_branch = d_out_rows.to(dtype)
        start, end = cache.layer_range
        for index in range(end - 1, start - 1, -1):
            d_stream, d_branch = self.layer_reverse(index, cache.layers[index - start], d_stream, d_branch, grads, bsz, seqlen, dtype)
        return d_stream

    def input_pullback(self, cache: StructuredRegionCache, d_out_basis_rows: torch.Tensor) -> torch.Tensor:
        """Basis-major cotangents [P*n, D] of the region output -> [P*n, D] fp32 cotangents of the region input."""
        return self._reverse(cache, d_out_basis_rows, None)

    def backward(self, cache: StructuredRegionCache, d_out_rows: torch.Tensor, grads: dict) -> torch.Tensor:
        """Single cotangent [n, D]: accumulates parameter gradients into ``grads`` and returns d(region input)."""
        if d_out_rows.shape[0] != cache.batch * cache.seq_len:
            raise ValueError("backward expects exactly one cotangent per token row")
        return self._reverse(cache, d_out_rows, grads)


def _wgrad(grads, name: str, dy: torch.Tensor, x: torch.Tensor) -> None:
    """dW = dy^T x, accumulated straight into the sink's fp32 buffer when it offers one."""
    target = grads.target(name) if hasattr(grads, "target") else None
    if target is not None:
        ops.linear_wgrad(dy, x, accumulate_into=target)
    else:
        _acc(grads, name, ops.linear_wgrad(dy, x))


def _acc(grads, name: str, value: torch.Tensor) -> None:
    target = grads.target(name) if hasattr(grads, "target") else None
    if target is not None:
        target.add_(value.reshape(target.shape).to(target.dtype))
        return
    prev = grads.get(name)
    if prev is None:
        grads[name] = value.float()
    elif prev.data_ptr() != value.data_ptr():
        prev.add_(value.float())
