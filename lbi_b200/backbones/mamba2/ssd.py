"""State-space duality (Mamba-2) scan.

``ssd_chunk_scan`` is the chunked algorithm (in-chunk quadratic form, chunk
states, state passing across chunks, state-to-output) that the reference runs as
Triton kernels (backbones/mamba2/ops/triton/ssd_combined.py:343-393; PyTorch
restatement :683-721).  It is written with plain differentiable tensor ops so it
runs on CPU and CUDA alike; on CUDA the chunk kernels in ``lbi_b200.ops.ssd``
replace the einsums.  ``ssd_recurrent_reference`` is the token-by-token
recurrence used as the test oracle.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def ssd_recurrent_reference(x, dt, A, B, C, D=None, initial_state=None):
    """h_t = exp(dt_t A) h_{t-1} + dt_t x_t B_t^T ;  y_t = h_t C_t + D x_t  (all fp64)."""
    bsz, seqlen, nheads, headdim = x.shape
    ngroups, dstate = B.shape[2], B.shape[3]
    rep = nheads // ngroups
    xf, dtf = x.double(), dt.double()
    Bf = B.double().repeat_interleave(rep, dim=2)
    Cf = C.double().repeat_interleave(rep, dim=2)
    state = (
        torch.zeros(bsz, nheads, headdim, dstate, dtype=torch.float64, device=x.device)
        if initial_state is None
        else initial_state.double().clone()
    )
    ys = []
    for t in range(seqlen):
        decay = torch.exp(dtf[:, t] * A.double())
        state = state * decay[..., None, None] + (dtf[:, t, :, None] * xf[:, t])[..., None] * Bf[:, t, :, None, :]
        y = torch.einsum("bhpn,bhn->bhp", state, Cf[:, t])
        if D is not None:
            y = y + D.double()[None, :, None] * xf[:, t]
        ys.append(y)
    return torch.stack(ys, dim=1), state


def ssd_chunk_scan(x, dt, A, B, C, chunk_size: int, D=None, initial_state=None, return_final_state: bool = False):
    """Chunked SSD.

    x [b, l, h, p]; dt [b, l, h] (already positive); A [h] (negative); B, C [b, l, g, n]; D [h] or None.
    Internal math is fp32; the output has x's dtype.
    """
    bsz, seqlen, nheads, headdim = x.shape
    ngroups, dstate = B.shape[2], B.shape[3]
    rep = nheads // ngroups
    out_dtype = x.dtype
    pad = (-seqlen) % chunk_size
    xf, dtf, Bf, Cf = x.float(), dt.float(), B.float(), C.float()
    if pad:
        xf = F.pad(xf, (0, 0, 0, 0, 0, pad))
        dtf = F.pad(dtf, (0, 0, 0, pad))
        Bf = F.pad(Bf, (0, 0, 0, 0, 0, pad))
        Cf = F.pad(Cf, (0, 0, 0, 0, 0, pad))
    nchunks = (seqlen + pad) // chunk_size
    xc = xf.view(bsz, nchunks, chunk_size, nheads, headdim)
    dtc = dtf.view(bsz, nchunks, chunk_size, nheads)
    Bc = Bf.view(bsz, nchunks, chunk_size, ngroups, dstate)
    Cc = Cf.view(bsz, nchunks, chunk_size, ngroups, dstate)

    dA = dtc * A.float()  # [b, c, q, h]
    cum = torch.cumsum(dA, dim=2)
    total = cum[:, :, -1]  # [b, c, h]

    # in-chunk quadratic form
    diff = cum[:, :, :, None, :] - cum[:, :, None, :, :]  # [b, c, i, j, h]
    causal = torch.ones(chunk_size, chunk_size, dtype=torch.bool, device=x.device).tril()
    decay = torch.exp(diff.masked_fill(~causal[None, None, :, :, None], float("-inf")))
    cb = torch.einsum("bcign,bcjgn->bcijg", Cc, Bc).repeat_interleave(rep, dim=-1)  # [b, c, i, j, h]
    weights = cb * decay * dtc[:, :, None, :, :]
    y = torch.einsum("bcijh,bcjhp->bcihp", weights, xc)

    # per-chunk end states (contribution of the chunk's own tokens)
    to_end = torch.exp(total[:, :, None, :] - cum) * dtc  # [b, c, q, h]
    Bh = Bc.repeat_interleave(rep, dim=3)
    chunk_states = torch.einsum("bcqhn,bcqh,bcqhp->bchpn", Bh, to_end, xc)

    # state passing across chunks
    state = (
        torch.zeros(bsz, nheads, headdim, dstate, dtype=torch.float32, device=x.device)
        if initial_state is None
        else initial_state.float()
    )
    incoming = []
    for c in range(nchunks):
        incoming.append(state)
        state = state * torch.exp(total[:, c])[..., None, None] + chunk_states[:, c]
    prev = torch.stack(incoming, dim=1)  # [b, c, h, p, n]

    Ch = Cc.repeat_interleave(rep, dim=3)
    y = y + torch.einsum("bcqhn,bchpn,bcqh->bcqhp", Ch, prev, torch.exp(cum))
    if D is not None:
        y = y + D.float()[None, None, None, :, None] * xc
    y = y.reshape(bsz, nchunks * chunk_size, nheads, headdim)[:, :seqlen].to(out_dtype)
    if return_final_state:
        return y, state
    return y
