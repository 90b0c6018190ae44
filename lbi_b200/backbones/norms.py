"""Normalisation layers shared by all backbones.

The reference keeps a plain-PyTorch RMSNorm for the Transformer
(backbones/transformer/block.py:12-22) and Triton-only RMSNorm / gated RMSNorm
for the Mamba families (backbones/mamba2/ops/triton/layernorm_gated.py:384-437),
which is why its Mamba models cannot run without a GPU.  Here one set of modules
serves every backbone: on CUDA tensors they call the fused sm_100a kernels in
``lbi_b200.ops``; on CPU they evaluate the same formula in fp32 PyTorch.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


def rms_norm_reference(
    x: torch.Tensor,
    weight: torch.Tensor,
    *,
    eps: float,
    z: torch.Tensor | None = None,
    norm_before_gate: bool = True,
    group_size: int | None = None,
) -> torch.Tensor:
    """fp32 RMSNorm with optional SiLU gate; the oracle for the fused kernels."""
    out_dtype = x.dtype
    xf = x.float()
    zf = z.float() if z is not None else None
    if zf is not None and not norm_before_gate:
        xf = xf * F.silu(zf)
    if group_size is None or group_size == xf.shape[-1]:
        rstd = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
        out = xf * rstd * weight.float()
    else:
        grouped = xf.unflatten(-1, (-1, group_size))
        rstd = torch.rsqrt(grouped.square().mean(dim=-1, keepdim=True) + eps)
        out = (grouped * rstd).flatten(-2) * weight.float()
    if zf is not None and norm_before_gate:
        out = out * F.silu(zf)
    return out.to(out_dtype)


class _GatedRMSNormFunction(torch.autograd.Function):
    """Forward and backward on the gated / grouped RMSNorm kernels (csrc/gated_norm.cu)."""

    @staticmethod
    def forward(ctx, x, z, weight, eps, group_size, gate_first):
        from lbi_b200.ops import dispatch, ext

        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        z2 = None if z is None else z.to(x.dtype).reshape(-1, shape[-1]).contiguous()
        w = weight.float().contiguous()
        y, rstd = ext().gated_rmsnorm_fwd(x2, z2, w, float(eps), int(group_size), bool(gate_first))
        dispatch.KERNEL_LAUNCHES["count"] += 1
        ctx.save_for_backward(x2, z2 if z2 is not None else x2.new_empty(0), w, rstd)
        ctx.meta = (shape, z is not None, int(group_size), bool(gate_first), weight.dtype, None if z is None else z.dtype)
        return y.view(shape)

    @staticmethod
    def backward(ctx, gy):
        from lbi_b200.ops import dispatch, ext

        x2, z2, w, rstd = ctx.saved_tensors
        shape, has_z, group_size, gate_first, w_dtype, z_dtype = ctx.meta
        dy = gy.to(x2.dtype).reshape(-1, shape[-1]).contiguous()
        dx, dz, dw = ext().gated_rmsnorm_bwd(dy, x2, z2 if has_z else None, w, rstd, group_size, gate_first)
        dispatch.KERNEL_LAUNCHES["count"] += 1
        return dx.view(shape), (dz.view(shape).to(z_dtype) if has_z else None), dw.to(w_dtype), None, None, None


def gated_rms_norm(x, weight, *, eps, z=None, norm_before_gate=True, group_size=None):
    """Kernel path for bf16 / fp32 CUDA tensors (``LBI_B200_TORCH_NORMS=1`` keeps the PyTorch form), else the oracle."""
    import os

    in_transform = torch._C._functorch.maybe_current_level() is not None     # jvp / vmap: the PyTorch form has the rules
    if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and not in_transform
            and os.environ.get("LBI_B200_TORCH_NORMS", "0") != "1"):
        from lbi_b200.ops import ext, native_available

        gs = x.shape[-1] if group_size is None else int(group_size)
        if native_available() and hasattr(ext(), "gated_rmsnorm_fwd") and x.shape[-1] <= 12288 and x.shape[-1] % gs == 0 and gs % 8 == 0:
            return _GatedRMSNormFunction.apply(x, z, weight, eps, gs, not norm_before_gate)
    return rms_norm_reference(x, weight, eps=eps, z=z, norm_before_gate=norm_before_gate, group_size=group_size)


def rms_norm_ref(x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True, upcast=True):
    """The oracle with the argument list of the reference's function (backbones/mamba2/ops/triton/layernorm_gated.py:18-39);
    always evaluated in fp32 (``upcast`` is accepted for that signature)."""
    if bias is None:
        return rms_norm_reference(x, weight, eps=eps, z=z, norm_before_gate=norm_before_gate, group_size=group_size)
    gate_first = z is not None and not norm_before_gate
    xin = (x.float() * F.silu(z.float())) if gate_first else x.float()
    out = rms_norm_reference(xin, weight, eps=eps, group_size=group_size) + bias.float()
    if z is not None and norm_before_gate:
        out = out * F.silu(z.float())
    return out.to(x.dtype)


def rmsnorm_fn(x, weight, bias=None, z=None, eps=1e-6, group_size=None, norm_before_gate=True):
    """Functional gated / grouped RMSNorm (reference layernorm_gated.py:384-385): the kernels of ``gated_rms_norm`` when there
    is no bias, the fp32 PyTorch form otherwise."""
    if bias is None:
        return gated_rms_norm(x, weight, eps=eps, z=z, norm_before_gate=norm_before_gate, group_size=group_size)
    return rms_norm_ref(x, weight, bias, z=z, eps=eps, group_size=group_size, norm_before_gate=norm_before_gate)


def layernorm_fn(x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True, is_rms_norm=False):
    """Functional gated / grouped LayerNorm (mean removed; reference layernorm_gated.py:380-381), fp32 PyTorch; with
    ``is_rms_norm`` it is ``rmsnorm_fn``."""
    if is_rms_norm:
        return rmsnorm_fn(x, weight, bias, z=z, eps=eps, group_size=group_size, norm_before_gate=norm_before_gate)
    xf = x.float()
    zf = None if z is None else z.float()
    if zf is not None and not norm_before_gate:
        xf = xf * F.silu(zf)
    grouped = xf.unflatten(-1, (-1, xf.shape[-1] if group_size is None else group_size))
    centred = grouped - grouped.mean(dim=-1, keepdim=True)
    out = (centred * torch.rsqrt(centred.square().mean(dim=-1, keepdim=True) + eps)).flatten(-2) * weight.float()
    if bias is not None:
        out = out + bias.float()
    if zf is not None and norm_before_gate:
        out = out * F.silu(zf)
    return out.to(x.dtype)


class LayerNormGated(nn.Module):
    """LayerNorm with weight and bias, optional groups and an optional SiLU gate ``z`` (the ``LayerNorm`` of the reference's
    layernorm_gated.py:388-412)."""

    def __init__(self, hidden_size: int, eps: float = 1e-5, group_size: int | None = None, norm_before_gate: bool = True,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(hidden_size, device=device, dtype=dtype))
        self.eps, self.group_size, self.norm_before_gate = float(eps), group_size, bool(norm_before_gate)

    def forward(self, x: torch.Tensor, z: torch.Tensor | None = None) -> torch.Tensor:
        return layernorm_fn(x, self.weight, self.bias, z=z, eps=self.eps, group_size=self.group_size,
                            norm_before_gate=self.norm_before_gate)


class RMSNorm(nn.Module):
    """``y = x / rms(x) * weight`` computed in fp32 and cast back to the input dtype."""

    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.eps = float(eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32):
            from lbi_b200.ops import rmsnorm

            return rmsnorm(x, self.weight, self.eps)
        xf = x.float()
        rstd = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + self.eps)
        return (xf * rstd).to(dtype=x.dtype) * self.weight.to(dtype=x.dtype)


class RMSNormGated(nn.Module):
    """RMSNorm with an optional SiLU gate ``z`` applied before or after normalisation.

    ``norm_before_gate=False`` is the Mamba-2 setting ``norm(x * silu(z))``
    (reference backbones/mamba2/mamba2_simple.py:119); without ``z`` it is a
    plain RMSNorm as used for the Mamba-3 B/C projections
    (reference backbones/mamba3/mamba3.py:116-117).
    """

    def __init__(
        self,
        dim: int,
        eps: float = 1e-5,
        norm_before_gate: bool = True,
        group_size: int | None = None,
        device=None,
        dtype=None,
    ) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.register_parameter("bias", None)
        self.eps = float(eps)
        self.norm_before_gate = bool(norm_before_gate)
        self.group_size = group_size

    def forward(self, x: torch.Tensor, z: torch.Tensor | None = None) -> torch.Tensor:
        return gated_rms_norm(
            x,
            self.weight,
            eps=self.eps,
            z=z,
            norm_before_gate=self.norm_before_gate,
            group_size=self.group_size,
        )
