"""Closed-form forward, input pullback over a basis and parameter VJP of Mamba-3, Mamba-2 and hybrid layer ranges.

The reference leaves these entry points as stubs: ``BackboneStackRegionBackend.input_pullback_basis`` and
``parameter_vjp`` raise NotImplementedError (backends/backbone_stack.py:12-82), ``Mamba3Block.input_pullback_matrix``
is an autograd loop over a replicated batch (backbones/mamba3/block.py:104-123) and the native namespace meant to hold
the state-mixer pullback is empty (cuda/mamba3/__init__.py:4-11).  Here every op of a block has an explicit J^T that
is chained over cached activations without autograd, exactly as ``transformer_structured`` does for attention blocks:

* ``forward``         records one cache per block (what each J^T needs, nothing more);
* ``input_pullback``  pulls P stacked output cotangents ([P * n, D], direction-major) back to the region input in one
                      pass: everything that depends only on the forward (normalisation statistics, gate values, the
                      rotary / trapezoid preprocessing, decays, chunk states) is computed once in the forward and shared by
                      all P directions; the GEMMs see M = P * n rows;
* ``backward``        the same chain for one cotangent, also producing every parameter gradient.

Block kinds are dispatched per layer, so a hybrid stack (e.g. three Mamba-3 blocks, one attention block, repeated)
runs through the same three entry points.  All tensor work goes through ``lbi_b200.ops`` (sm_100a kernels on CUDA,
fp32 PyTorch statements on CPU).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from .. import ops
from ..ops import mamba as mops
from ..ops import ssd as ops_ssd
from .transformer_structured import StructuredRegionCache, StructuredTransformerRegion, _acc, _wgrad


# ------------------------------------------------------------------------------------------------ caches
@dataclass
class Mamba3LayerCache:
    """Flat activations of one Mamba-3 block that the closed-form backward reads."""

    stream: torch.Tensor          # fp32 residual stream entering the norm                     [n, D]
    rstd: torch.Tensor            # [n]
    normed: torch.Tensor          # input of in_proj                                            [n, D]
    z: torch.Tensor               # gate                                                        [n, d_inner]
    x: torch.Tensor               # V of the scan                                               [n, d_inner]
    b_raw: torch.Tensor           # B / C before their RMSNorm                                  [n * g, N]
    c_raw: torch.Tensor
    b_rstd: torch.Tensor
    c_rstd: torch.Tensor
    b_normed: torch.Tensor        # [b, l, g, N]
    c_normed: torch.Tensor
    small: Any                    # ops.mamba.SisoSmall
    qr: torch.Tensor              # [b, l, h, N]
    kr: torch.Tensor
    skip: torch.Tensor            # gamma <Q, K> + D                                            [b, l, h]
    y: torch.Tensor               # scan output before the gate                                 [n, d_inner]
    y_in: torch.Tensor            # input of out_proj                                           [n, d_inner]
    states: torch.Tensor | None   # incoming chunk states of the forward scan (kernel path)
    norm_rstd: torch.Tensor | None = None   # only with the optional output norm


@dataclass
class Mamba2LayerCache:
    """Flat activations of one Mamba-2 block that the closed-form backward reads."""

    stream: torch.Tensor
    rstd: torch.Tensor
    normed: torch.Tensor
    z: torch.Tensor               # [n, d_inner]
    xbc_pre: torch.Tensor         # conv input                                                  [n, conv_dim]
    xbc_conv: torch.Tensor        # conv output before SiLU
    x: torch.Tensor               # [b, l, h, p]
    b: torch.Tensor               # [b, l, g, N]
    c: torch.Tensor
    dt: torch.Tensor              # softplus(dt_raw + bias)                                     [b, l, h] fp32
    dt_slope: torch.Tensor        # d dt / d dt_raw
    y: torch.Tensor               # scan output                                                 [n, d_inner]
    y_rstd: torch.Tensor
    y_in: torch.Tensor            # gated-norm output = input of out_proj
    states: torch.Tensor | None
    final: torch.Tensor | None


class _MambaWeights:
    """Compute-dtype views of a block's projection matrices (from the optimizer's shadow buffer when there is one) plus the
    fp32 views of everything small."""

    def __init__(self, block, dtype, shadow_of) -> None:
        mixer = block.mixer
        if mixer.in_proj.bias is not None or mixer.out_proj.bias is not None:
            raise NotImplementedError("the structured Mamba lowering supports bias-free projections only")

        def cast(w):
            if shadow_of is not None:
                view = shadow_of(w)
                if view is not None and view.dtype == dtype:
                    return view
            return w.detach().to(dtype).contiguous()

        self.block = block
        self.norm = block.norm.weight.detach()
        self.w_in, self.w_out = cast(mixer.in_proj.weight), cast(mixer.out_proj.weight)
        self.stale = shadow_of is None or self.w_in.data_ptr() != getattr(shadow_of(mixer.in_proj.weight), "data_ptr", lambda: 0)()

    def refresh(self, dtype, shadow_of) -> None:
        self.__init__(self.block, dtype, shadow_of)


def _kind(block) -> str:
    name = type(block).__name__
    if name == "Mamba3Block":
        return "mamba3"
    if name == "Mamba2Block":
        return "mamba2"
    if hasattr(block, "attn"):
        return "transformer"
    raise NotImplementedError(f"no structured lowering for block type {name}")


class StructuredMambaRegion:
    """Runs layer ranges of a Mamba-3 / Mamba-2 / hybrid ``BackboneStack`` without autograd."""

    def __init__(self, blocks, *, act_dtype: torch.dtype | None = None) -> None:
        self.blocks = blocks
        self.kinds = [_kind(b) for b in blocks]
        self.act_dtype = act_dtype
        self._weights: dict[tuple, list] = {}
        self.shadow_of = None
        self._tf = StructuredTransformerRegion(blocks) if "transformer" in self.kinds else None

    # ------------------------------------------------------------------ weights
    def weights(self, dtype: torch.dtype) -> list:
        device = self.blocks[0].norm.weight.device
        key = (dtype, str(device))
        cached = self._weights.get(key)
        if cached is None:
            cached = [None if kind == "transformer" else _MambaWeights(b, dtype, self.shadow_of) for b, kind in zip(self.blocks, self.kinds)]
            self._weights[key] = cached
            if self._tf is not None:
                self._tf.act_dtype, self._tf.shadow_of = self.act_dtype, self.shadow_of
                self._tf._weights.clear()
        return cached

    def refresh_weights(self) -> None:
        for (dtype, _), layers in self._weights.items():
            for lw in filter(None, layers):
                lw.refresh(dtype, self.shadow_of)
        if self._tf is not None:
            self._tf.refresh_weights()

    # ------------------------------------------------------------------ Mamba-3 block
    def _m3_forward(self, index, branch, stream, bsz, seqlen, dtype):
        block, lw = self.blocks[index], self.weights(dtype)[index]
        mx = block.mixer
        n = bsz * seqlen
        h, p, g, ns = mx.nheads, mx.headdim, mx.num_bc_heads, mx.d_state
        normed, stream1, rstd = ops.add_rmsnorm_fwd(branch, stream, lw.norm, block.norm.eps, dtype)
        proj = ops.linear_fwd(normed, lw.w_in)
        z, x, b_raw, c_raw, dd_dt, dd_a, trap, angles = torch.split(
            proj, [mx.d_inner, mx.d_inner, g * ns, g * ns, h, h, h, mx.num_rope_angles], dim=-1)
        z, x = z.contiguous(), x.contiguous()
        b_raw, c_raw = b_raw.reshape(n * g, ns).contiguous(), c_raw.reshape(n * g, ns).contiguous()
        b_normed, b_rstd = mops.gated_rmsnorm_fwd(b_raw, None, mx.B_norm.weight.detach(), mx.B_norm.eps, ns, False)
        c_normed, c_rstd = mops.gated_rmsnorm_fwd(c_raw, None, mx.C_norm.weight.detach(), mx.C_norm.eps, ns, False)
        b_normed, c_normed = b_normed.view(bsz, seqlen, g, ns), c_normed.view(bsz, seqlen, g, ns)
        small = mops.siso_small_fwd(dd_dt, dd_a, trap, angles, mx.dt_bias.detach(), mx.A_floor, bsz, seqlen)
        qr, kr, qk = mops.siso_wide_fwd(c_normed, b_normed, mx.C_bias.detach().squeeze(1), mx.B_bias.detach().squeeze(1),
                                        small.theta, small.gamma, small.scale)
        x4 = x.view(bsz, seqlen, h, p)
        y, states = mops.siso_scan_fwd(x4, kr, qr, small.adt, qk, mx.D.detach())
        y = y.reshape(n, mx.d_inner).contiguous()
        norm_rstd = None
        if mx.is_outproj_norm:
            y_in, norm_rstd = mops.gated_rmsnorm_fwd(y, z, mx.norm.weight.detach(), mx.norm.eps, p, False)
        else:
            y_in = mops.gate_silu_fwd(y, z)
        out = ops.linear_fwd(y_in, lw.w_out)
        skip = qk + mx.D.detach().float()
        return out, stream1, Mamba3LayerCache(stream1, rstd, normed, z, x, b_raw, c_raw, b_rstd, c_rstd, b_normed, c_normed, small,
                                              qr, kr, skip, y, y_in, states, norm_rstd)

    def _m3_reverse(self, index, lc: Mamba3LayerCache, d_stream, d_branch, grads, bsz, seqlen, dtype):
        block, lw = self.blocks[index], self.weights(dtype)[index]
        mx = block.mixer
        h, p, g, ns = mx.nheads, mx.headdim, mx.num_bc_heads, mx.d_state
        rows = d_branch.shape[0]
        reps = rows // (bsz * seqlen)
        pb = reps * bsz
        prefix = f"blocks.{index}."
        if grads is not None:
            _wgrad(grads, prefix + "mixer.out_proj.weight", d_branch, lc.y_in)
        d_yin = ops.linear_dgrad(d_branch, lw.w_out)
        # the in_proj cotangent [z | x | B | C | dd_dt | dd_A | trap | angles]: the two wide parts are written into their column
        # ranges by the kernels that produce them, the narrow ones are copied in
        widths = [mx.d_inner, mx.d_inner, g * ns, g * ns, h, h, h, lc.small.tanh_angle.shape[-1]]
        offs = [0]
        for wdt in widths:
            offs.append(offs[-1] + wdt)
        d_proj = torch.empty(rows, offs[-1], device=d_branch.device, dtype=dtype)
        part = lambda i: d_proj[:, offs[i] : offs[i + 1]]  # noqa: E731
        if mx.is_outproj_norm:
            d_y, d_z, dw = mops.gated_rmsnorm_bwd(d_yin, lc.y, lc.z, mx.norm.weight.detach(), lc.norm_rstd, p, False,
                                                  want_dweight=grads is not None)
            part(0).copy_(d_z)
            if grads is not None:
                _acc(grads, prefix + "mixer.norm.weight", dw)
        else:
            d_y, _ = mops.gate_silu_bwd(d_yin, lc.y, lc.z, dz_out=part(0))
        d_qr, d_kr, d_adt, d_skip, _, reversed_dkr = mops.siso_scan_bwd(lc.qr, lc.kr, lc.small.adt, lc.skip, lc.x.view(bsz, seqlen, h, p),
                                                                        d_y.view(pb, seqlen, h, p), lc.states, dv_out=part(1))
        d_c, d_b, d_cb, d_bb, d_theta, d_gamma, d_scale = mops.siso_wide_bwd(
            lc.c_normed, lc.b_normed, mx.C_bias.detach().squeeze(1), mx.B_bias.detach().squeeze(1), lc.small.theta, lc.small.gamma,
            lc.small.scale, d_qr, d_kr, d_skip, dkr_reversed=reversed_dkr, want_bias=grads is not None)
        d_dd_dt, d_dd_a, d_trap, d_angles = mops.siso_small_bwd(lc.small, d_adt, d_theta, d_gamma, d_scale, out_dtype=dtype)
        want_dw = grads is not None
        d_braw, _, dw_b = mops.gated_rmsnorm_bwd(d_b.reshape(rows * g, ns), lc.b_raw, None, mx.B_norm.weight.detach(), lc.b_rstd, ns, False,
                                                 want_dweight=want_dw)
        d_craw, _, dw_c = mops.gated_rmsnorm_bwd(d_c.reshape(rows * g, ns), lc.c_raw, None, mx.C_norm.weight.detach(), lc.c_rstd, ns, False,
                                                 want_dweight=want_dw)
        if grads is not None:
            _acc(grads, prefix + "mixer.B_norm.weight", dw_b)
            _acc(grads, prefix + "mixer.C_norm.weight", dw_c)
            _acc(grads, prefix + "mixer.B_bias", d_bb.unsqueeze(1))
            _acc(grads, prefix + "mixer.C_bias", d_cb.unsqueeze(1))
            _acc(grads, prefix + "mixer.D", d_skip.float().sum((0, 1)))
            _acc(grads, prefix + "mixer.dt_bias", d_dd_dt.float().sum(0))
        for i, t in enumerate((d_braw.reshape(rows, g * ns), d_craw.reshape(rows, g * ns), d_dd_dt, d_dd_a, d_trap, d_angles), start=2):
            part(i).copy_(t)
        if grads is not None:
            _wgrad(grads, prefix + "mixer.in_proj.weight", d_proj, lc.normed)
        d_normed = ops.linear_dgrad(d_proj, lw.w_in)
        if grads is not None:
            _acc(grads, prefix + "norm.weight", ops.rmsnorm_wgrad(d_normed, lc.stream, lc.rstd))
        return ops.rmsnorm_bwd(d_normed, lc.stream, lc.rstd, lw.norm, d_stream, lowp_dtype=dtype)

    # ------------------------------------------------------------------ Mamba-2 block
    def _m2_forward(self, index, branch, stream, bsz, seqlen, dtype):
        block, lw = self.blocks[index], self.weights(dtype)[index]
        mx = block.mixer
        n = bsz * seqlen
        h, p, g, ns = mx.nheads, mx.headdim, mx.ngroups, mx.d_state
        gn = g * ns
        normed, stream1, rstd = ops.add_rmsnorm_fwd(branch, stream, lw.norm, block.norm.eps, dtype)
        proj = ops.linear_fwd(normed, lw.w_in)
        z, xbc_pre, dt_raw = torch.split(proj, [mx.d_inner, mx.d_inner + 2 * gn, h], dim=-1)
        z, xbc_pre = z.contiguous(), xbc_pre.contiguous()
        dt, dt_slope = (t.view(bsz, seqlen, h) for t in mops.softplus_dt_fwd(dt_raw, mx.dt_bias.detach(), *mx.dt_limit))
        conv_w = mx.conv1d.weight.detach().squeeze(1).float().contiguous()
        conv_b = None if mx.conv1d.bias is None else mx.conv1d.bias.detach().float()
        xbc_conv, (x, b_, c_) = mops.conv_silu_fwd(xbc_pre, conv_w, conv_b, bsz, seqlen, (mx.d_inner, gn, gn))
        x4 = x.view(bsz, seqlen, h, p)
        b4, c4 = b_.view(bsz, seqlen, g, ns), c_.view(bsz, seqlen, g, ns)
        a_neg = -torch.exp(mx.A_log.detach().float())
        y, final, states = _ssd_forward(x4, dt, a_neg, b4, c4, mx.D.detach(), mx.chunk_size)
        y = y.reshape(n, mx.d_inner).contiguous()
        y_in, y_rstd = mops.gated_rmsnorm_fwd(y, z, mx.norm.weight.detach(), mx.norm.eps, mx.norm.group_size or mx.d_inner,
                                              not mx.norm.norm_before_gate)
        out = ops.linear_fwd(y_in, lw.w_out)
        return out, stream1, Mamba2LayerCache(stream1, rstd, normed, z, xbc_pre, xbc_conv, x4, b4, c4, dt, dt_slope, y, y_rstd, y_in,
                                              states, final)

    def _m2_reverse(self, index, lc: Mamba2LayerCache, d_stream, d_branch, grads, bsz, seqlen, dtype):
        block, lw = self.blocks[index], self.weights(dtype)[index]
        mx = block.mixer
        h, p, g, ns = mx.nheads, mx.headdim, mx.ngroups, mx.d_state
        gn = g * ns
        rows = d_branch.shape[0]
        reps = rows // (bsz * seqlen)
        pb = reps * bsz
        prefix = f"blocks.{index}."
        if grads is not None:
            _wgrad(grads, prefix + "mixer.out_proj.weight", d_branch, lc.y_in)
        d_yin = ops.linear_dgrad(d_branch, lw.w_out)
        d_y, d_z, dw = mops.gated_rmsnorm_bwd(d_yin, lc.y, lc.z, mx.norm.weight.detach(), lc.y_rstd, mx.norm.group_size or mx.d_inner,
                                              not mx.norm.norm_before_gate, want_dweight=grads is not None)
        if grads is not None:
            _acc(grads, prefix + "mixer.norm.weight", dw)
        a_neg = -torch.exp(mx.A_log.detach().float())
        dx, ddt, d_a, d_b, d_c, d_dskip = _ssd_backward(lc.x, lc.dt, a_neg, lc.b, lc.c, mx.D.detach(), d_y.view(pb, seqlen, h, p),
                                                        lc.states, lc.final)
        d_parts = (dx.reshape(rows, mx.d_inner), d_b.reshape(rows, gn), d_c.reshape(rows, gn))
        conv_w = mx.conv1d.weight.detach().squeeze(1).float().contiguous()
        conv_dim = mx.d_inner + 2 * gn
        if grads is not None:
            dw_conv, db_conv = mops.conv_silu_wgrad(d_parts, lc.xbc_conv, lc.xbc_pre, conv_w.shape[1], bsz, seqlen)
            _acc(grads, prefix + "mixer.conv1d.weight", dw_conv.unsqueeze(1))
            if mx.conv1d.bias is not None:
                _acc(grads, prefix + "mixer.conv1d.bias", db_conv)
        d_dt_raw = (ddt.float().view(reps, bsz, seqlen, h) * lc.dt_slope).reshape(rows, h)
        if grads is not None:
            _acc(grads, prefix + "mixer.A_log", d_a.float() * a_neg)          # d/dA_log of A = -exp(A_log)
            _acc(grads, prefix + "mixer.D", d_dskip.float())
            _acc(grads, prefix + "mixer.dt_bias", d_dt_raw.float().sum(0))
        d_proj = torch.empty(rows, mx.d_inner + conv_dim + h, dtype=dtype, device=d_branch.device)
        d_proj[:, : mx.d_inner] = d_z
        mops.conv_silu_bwd(d_parts, lc.xbc_conv, conv_w, bsz, seqlen, d_proj, mx.d_inner)   # fills the xBC columns
        d_proj[:, mx.d_inner + conv_dim :] = d_dt_raw
        if grads is not None:
            _wgrad(grads, prefix + "mixer.in_proj.weight", d_proj, lc.normed)
        d_normed = ops.linear_dgrad(d_proj, lw.w_in)
        if grads is not None:
            _acc(grads, prefix + "norm.weight", ops.rmsnorm_wgrad(d_normed, lc.stream, lc.rstd))
        return ops.rmsnorm_bwd(d_normed, lc.stream, lc.rstd, lw.norm, d_stream, lowp_dtype=dtype)

    # ------------------------------------------------------------------ dispatch
    def _layer_forward(self, index, branch, stream, bsz, seqlen, dtype):
        kind = self.kinds[index]
        if kind == "mamba3":
            return self._m3_forward(index, branch, stream, bsz, seqlen, dtype)
        if kind == "mamba2":
            return self._m2_forward(index, branch, stream, bsz, seqlen, dtype)
        self.weights(dtype)
        return self._tf.layer_forward(index, branch, stream, bsz, seqlen, dtype)

    def _layer_reverse(self, index, lc, d_stream, d_branch, grads, bsz, seqlen, dtype):
        kind = self.kinds[index]
        if kind == "mamba3":
            return self._m3_reverse(index, lc, d_stream, d_branch, grads, bsz, seqlen, dtype)
        if kind == "mamba2":
            return self._m2_reverse(index, lc, d_stream, d_branch, grads, bsz, seqlen, dtype)
        return self._tf.layer_reverse(index, lc, d_stream, d_branch, grads, bsz, seqlen, dtype)

    # ------------------------------------------------------------------ public entry points
    @torch.no_grad()
    def forward(self, region_input: torch.Tensor, layer_range: tuple[int, int], materialize_output: bool = True):
        """region_input [B, T, D] -> (fp32 output [B, T, D] or None, cache)."""
        bsz, seqlen, dim = region_input.shape
        dtype = self.act_dtype or region_input.dtype
        x = region_input.reshape(bsz * seqlen, dim).to(dtype).contiguous()
        cache = StructuredRegionCache(batch=bsz, seq_len=seqlen, layer_range=tuple(layer_range), region_input=x)
        branch, stream = x, None
        for index in range(*layer_range):
            branch, stream, lc = self._layer_forward(index, branch, stream, bsz, seqlen, dtype)
            cache.layers.append(lc)
        cache.last_branch, cache.last_stream = branch, stream
        if not materialize_output:
            return None, cache
        out = branch.float() if stream is None else branch.float() + stream
        cache.output = out
        return out.reshape(bsz, seqlen, dim), cache

    @torch.no_grad()
    def _reverse(self, cache: StructuredRegionCache, d_out_rows: torch.Tensor, grads):
        bsz, seqlen = cache.batch, cache.seq_len
        dtype = cache.region_input.dtype
        d_stream, d_branch = d_out_rows.float(), d_out_rows.to(dtype)
        start, end = cache.layer_range
        for index in range(end - 1, start - 1, -1):
            d_stream, d_branch = self._layer_reverse(index, cache.layers[index - start], d_stream, d_branch, grads, bsz, seqlen, dtype)
        return d_stream

    def input_pullback(self, cache: StructuredRegionCache, d_out_basis_rows: torch.Tensor) -> torch.Tensor:
        """Direction-major cotangents [P * n, D] of the region output -> [P * n, D] fp32 cotangents of the region input."""
        return self._reverse(cache, d_out_basis_rows, None)

    def backward(self, cache: StructuredRegionCache, d_out_rows: torch.Tensor, grads) -> torch.Tensor:
        """One cotangent [n, D]: accumulates every parameter gradient into ``grads`` and returns d(region input)."""
        if d_out_rows.shape[0] != cache.batch * cache.seq_len:
            raise ValueError("backward expects exactly one cotangent per token row")
        return self._reverse(cache, d_out_rows, grads)


# ------------------------------------------------------------------------------------------------ SSD helpers
def _ssd_forward(x, dt, a_neg, b, c, d_skip, chunk_size):
    """-> (y [b, l, h, p], final state, incoming chunk states or None)."""
    if ops_ssd.ssd_cuda_supported(x, b) and x.dtype == torch.bfloat16:
        y, final, states = ops_ssd._forward_kernels(x, dt, a_neg, b, c, d_skip, None)
        return y.to(x.dtype), final, states
    from ..backbones.mamba2.ssd import ssd_chunk_scan

    y, final = ssd_chunk_scan(x, dt, a_neg, b, c, chunk_size=chunk_size, D=d_skip, return_final_state=True)
    return y, final, None


def _ssd_backward(x, dt, a_neg, b, c, d_skip, gy, states, final):
    """x, dt, b, c, states, final: forward operands [b, ...]; gy [P * b, l, h, p] -> (dx, ddt, dA [h], dB, dC, dD [h]) for the
    P stacked directions."""
    reps = gy.shape[0] // x.shape[0]
    if ops_ssd.ssd_cuda_supported(x, b) and x.dtype == torch.bfloat16 and states is not None and ops_ssd.chunk_backward_supported(x):
        return ops_ssd.ssd_backward_fused(x, dt, a_neg, b, c, d_skip, gy.to(x.dtype), states)
    if ops_ssd.ssd_cuda_supported(x, b) and x.dtype == torch.bfloat16 and hasattr(ops.ext(), "ssd_decay_grad"):
        tile = lambda t: None if t is None else mops._tile_rows(t, reps)  # noqa: E731
        dx, ddt, d_a, d_b, d_c, d_d, _ = ops_ssd.ssd_backward(tile(x), tile(dt), a_neg, tile(b), tile(c), d_skip, None, tile(final),
                                                            gy.to(x.dtype), None, fwd_states=tile(states))
        return dx, ddt, d_a, d_b, d_c, d_d
    return ops_ssd.ssd_backward_dense(x, dt, a_neg, b, c, d_skip, gy)
