"""Op-level entry points of the Mamba-2 mixer with the argument lists of the reference's combined ops
(backbones/mamba2/ops/triton/ssd_combined.py:624-643 and :984-1003), for code that calls the scan without the module.

The scan itself is ``ops.ssd.ssd_chunk_scan_cuda`` (tcgen05 kernels) where the shape allows it and the chunked PyTorch form
otherwise; the pieces around it (dt bias / softplus / clamp, gate, packed sequences, convolution, gated norm, projection)
are tensor ops here.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import ssd as ops_ssd
from ..norms import gated_rms_norm
from .ssd import ssd_chunk_scan, ssd_recurrent_reference

_NO_LIMIT = (0.0, float("inf"))


def _effective_dt(dt, dt_bias, dt_softplus, dt_limit):
    dt = dt.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    if dt_softplus:
        dt = F.softplus(dt)
    if tuple(dt_limit) != _NO_LIMIT:
        dt = dt.clamp(dt_limit[0], dt_limit[1])
    return dt


def _scan(x, dt, A, B, C, chunk_size, D, initial_states):
    d_vec = D if (D is not None and D.dim() == 1) else None
    if ops_ssd.ssd_cuda_supported(x, B) and x.dtype == torch.bfloat16:
        y, final = ops_ssd.ssd_chunk_scan_cuda(x, dt, A.float(), B, C, D=d_vec, initial_state=initial_states, return_final_state=True)
    else:
        y, final = ssd_chunk_scan(x, dt, A.float(), B, C, chunk_size=chunk_size, D=d_vec, initial_state=initial_states,
                                  return_final_state=True)
    if D is not None and D.dim() == 2:  # a skip weight per head and channel
        y = y + (x.float() * D.float()[None, None]).to(y.dtype)
    return y, final


def _segments(seq_idx_row: torch.Tensor) -> list[tuple[int, int]]:
    cuts = (torch.nonzero(seq_idx_row[1:] != seq_idx_row[:-1]).flatten() + 1).tolist()
    edges = [0, *cuts, seq_idx_row.numel()]
    return list(zip(edges[:-1], edges[1:]))


def mamba_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None, seq_idx=None,
                              cu_seqlens=None, dt_softplus=False, dt_limit=_NO_LIMIT, return_final_states=False,
                              return_varlen_states=False):
    """x [b, l, h, p]; dt [b, l, h]; A [h]; B, C [b, l, g, n]; D [h] or [h, p]; z [b, l, h, p] (output gate: y silu(z));
    dt_bias [h]; initial_states [b, h, p, n]; seq_idx [b, l] ids of the sequences packed into a row (the state starts from
    zero at every change; the initial state belongs to the first sequence).  Returns y like x, followed by the final state
    [b, h, p, n] when ``return_final_states`` and, when ``return_varlen_states`` (one packed row, boundaries in ``cu_seqlens``
    [num_sequences + 1]), by the state at the end of every sequence [num_sequences, h, p, n]."""
    if return_varlen_states:
        if cu_seqlens is None or x.shape[0] != 1:
            raise ValueError("return_varlen_states needs cu_seqlens and a single packed row")
    dt = _effective_dt(dt, dt_bias, dt_softplus, dt_limit)
    varlen = None
    if seq_idx is None and cu_seqlens is None:
        y, final = _scan(x, dt, A, B, C, chunk_size, D, initial_states)
    else:
        rows, finals, per_sequence = [], [], []
        for b in range(x.shape[0]):
            if cu_seqlens is not None and x.shape[0] == 1:
                edges = [int(v) for v in cu_seqlens.tolist()]
                segments = [(s, e) for s, e in zip(edges[:-1], edges[1:]) if e > s]
            else:
                segments = _segments(seq_idx[b])
            parts = []
            for s, e in segments:
                init = initial_states[b : b + 1] if (initial_states is not None and s == 0) else None
                y_seg, final_seg = _scan(x[b : b + 1, s:e], dt[b : b + 1, s:e], A, B[b : b + 1, s:e], C[b : b + 1, s:e], chunk_size, D,
                                         init)
                parts.append(y_seg)
                per_sequence.append(final_seg)
            rows.append(torch.cat(parts, dim=1))
            finals.append(final_seg)
        y, final = torch.cat(rows, dim=0), torch.cat(finals, dim=0)
        varlen = torch.cat(per_sequence, dim=0)
    if z is not None:
        y = (y.float() * F.silu(z.float())).to(x.dtype)
    out = (y, final) if return_final_states else (y,)
    if return_varlen_states:
        out = (*out, varlen)
    return out if len(out) > 1 else out[0]


def ssd_selective_scan(x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False, dt_limit=_NO_LIMIT):
    """Token-by-token fp64 evaluation of the same op (the oracle; reference ssd_combined.py:724-778)."""
    y, _ = ssd_recurrent_reference(x, _effective_dt(dt, dt_bias, dt_softplus, dt_limit), A, B, C,
                                   D=D if (D is not None and D.dim() == 1) else None)
    if D is not None and D.dim() == 2:
        y = y + x.double() * D.double()[None, None]
    if z is not None:
        y = y * F.silu(z.double())
    return y.to(x.dtype)


def mamba_split_conv1d_scan_combined(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, chunk_size, initial_states=None,
                                     seq_idx=None, dt_limit=_NO_LIMIT, return_final_states=False, activation="silu",
                                     rmsnorm_weight=None, rmsnorm_eps=1e-6, outproj_weight=None, outproj_bias=None, headdim=None,
                                     ngroups=1, norm_before_gate=True):
    """The mixer after ``in_proj`` as one call: zxbcdt [b, l, 2 dim + 2 g n + h] -> split into z | xBC | dt, causal depthwise
    convolution (weight [dim + 2 g n, width]) + SiLU, scan with softplus(dt + dt_bias), then either the gate ``y silu(z)`` or,
    with ``rmsnorm_weight``, the gated RMSNorm, then the output projection when ``outproj_weight`` is given."""
    if activation not in ("silu", "swish"):
        raise ValueError("activation must be silu or swish")
    nheads = D.shape[0]
    if D.dim() == 1:
        if headdim is None:
            raise ValueError("headdim is required when D has one entry per head")
    else:
        headdim = D.shape[1]
    dim = nheads * headdim
    gn = (conv1d_weight.shape[0] - dim) // 2
    if gn <= 0 or gn % ngroups != 0 or zxbcdt.shape[-1] != 2 * dim + 2 * gn + nheads:
        raise ValueError("zxbcdt / conv1d_weight widths do not match dim = nheads * headdim and ngroups")
    bsz, seqlen, _ = zxbcdt.shape
    z, xBC, dt = torch.split(zxbcdt, [dim, dim + 2 * gn, nheads], dim=-1)
    width = conv1d_weight.shape[-1]

    def conv(t):  # [1 or b, l', c]
        out = F.conv1d(t.transpose(1, 2), conv1d_weight.unsqueeze(1).to(t.dtype),
                       None if conv1d_bias is None else conv1d_bias.to(t.dtype), padding=width - 1, groups=t.shape[-1])
        return F.silu(out[..., : t.shape[1]].transpose(1, 2))

    if seq_idx is None:
        xBC = conv(xBC)
    else:  # the window starts afresh with every packed sequence
        xBC = torch.cat([torch.cat([conv(xBC[b : b + 1, s:e]) for s, e in _segments(seq_idx[b])], dim=1) for b in range(bsz)], dim=0)
    x, B, C = torch.split(xBC, [dim, gn, gn], dim=-1)
    gated_norm = rmsnorm_weight is not None
    z4 = z.reshape(bsz, seqlen, nheads, headdim)
    out = mamba_chunk_scan_combined(
        x.reshape(bsz, seqlen, nheads, headdim), dt, A, B.reshape(bsz, seqlen, ngroups, -1), C.reshape(bsz, seqlen, ngroups, -1),
        chunk_size, D=D, z=None if gated_norm else z4, dt_bias=dt_bias, initial_states=initial_states, seq_idx=seq_idx,
        dt_softplus=True, dt_limit=dt_limit, return_final_states=return_final_states)
    y, final = out if return_final_states else (out, None)
    y = y.reshape(bsz, seqlen, dim)
    if gated_norm:
        y = gated_rms_norm(y, rmsnorm_weight, eps=rmsnorm_eps, z=z, norm_before_gate=norm_before_gate)
    if outproj_weight is not None:
        y = F.linear(y.to(outproj_weight.dtype), outproj_weight, outproj_bias)
    return (y, final) if return_final_states else y


__all__ = ["mamba_chunk_scan_combined", "mamba_split_conv1d_scan_combined", "ssd_selective_scan"]
