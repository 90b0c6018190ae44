"""Dense (no regions) training step on the same kernels as the region-parallel engine, without autograd.

``DenseFastEngine.step(input_ids, targets)``: embedding gather, the closed-form forward of the whole layer stack with cached
activations, final norm, LM head fused with cross-entropy (forward and backward at once), one closed-form backward of
the stack with weight gradients accumulated by the GEMMs into a flat fp32 buffer, embedding scatter-add, fused clip +
AdamW.  It is the "dense model of the same size" baseline next to ``FastLBIEngine`` (the reference trains its dense
baseline with ``loss.backward()`` and ``torch.optim.AdamW``: train/runners.py:104-289, backward/autograd.py:11-28).
"""
from __future__ import annotations

import torch

from .. import ops
from ..utils import nvtx
from .flat import FlatParams


class DenseFastEngine:
    """The dense model of the same size on the same structured kernels (no regions, no interface): forward with cached activations,
    closed-form backward, fused clip + AdamW on flat buffers.  Single device."""

    def __init__(self, model, *, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, grad_clip: float = 1.0, act_dtype: torch.dtype | None = None) -> None:
        from ..backends.mamba_structured import StructuredMambaRegion
        from ..backends.transformer_structured import StructuredTransformerRegion

        self.model = model
        self.device = next(model.parameters()).device
        self.act_dtype = act_dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.lr, self.betas, self.eps, self.weight_decay, self.grad_clip = lr, betas, eps, weight_decay, grad_clip
        self.flat = FlatParams(model, world_size=1, shadow_dtype=self.act_dtype if self.act_dtype != torch.float32 else None)
        self.flat.ensure_state(0, self.flat.total)
        blocks = model.backbone.blocks
        all_attention = all(hasattr(b, "attn") for b in blocks)
        self.structured = (StructuredTransformerRegion if all_attention else StructuredMambaRegion)(blocks, act_dtype=self.act_dtype)
        self.structured.shadow_of = self._shadow_of
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)

    def _shadow_of(self, p):
        try:
            return self.flat.weight(self.flat.name_of(p))
        except KeyError:
            return None

    def _g(self, p) -> torch.Tensor:
        return self.flat.grad(self.flat.name_of(p))

    def target(self, name: str):
        """Gradient sink of the structured backward: backbone-relative parameter name -> fp32 accumulator."""
        return self.flat.grad("backbone." + name)

    @torch.no_grad()
    def backward(self, input_ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Forward and backward; gradients end up in ``self.flat.grads``.  Returns the mean next-token loss."""
        model = self.model
        self.flat.zero_grad()
        bsz, seqlen = input_ids.shape
        dim = model.backbone_spec.dim
        emb = model.canvas.embedding.weight
        table = self.flat.weight(self.flat.name_of(emb))
        tied = model.tie_embeddings
        head_param = emb if tied else model.readout.lm_head.weight
        head_w = table if tied else self.flat.weight(self.flat.name_of(head_param))
        final = model.readout.norm
        with nvtx.range("dense/forward"):
            rows = ops.embedding_fwd(input_ids, table, self.act_dtype)
            _, cache = self.structured.forward(rows.view(bsz, seqlen, dim), (0, len(model.backbone.blocks)), materialize_output=False)
            normed, out, rstd = ops.add_rmsnorm_fwd(cache.last_branch, cache.last_stream, final.weight.detach(), final.eps, self.act_dtype)
            loss, d_normed, _ = ops.lm_head_cross_entropy(normed, head_w, targets.reshape(-1), 1.0 / float(bsz * seqlen),
                                                          want_dweight=True, dweight_into=self._g(head_param))
        with nvtx.range("dense/backward"):
            self._g(final.weight).add_(ops.rmsnorm_wgrad(d_normed, out, rstd))
            d_out = ops.rmsnorm_bwd(d_normed, out, rstd, final.weight.detach())
            d_in = self.structured.backward(cache, d_out, self)
            ops.embedding_scatter_add(self._g(emb), input_ids, d_in)
        return loss

    @torch.no_grad()
    def step(self, input_ids: torch.Tensor, targets: torch.Tensor, lr: float | None = None) -> torch.Tensor:
        loss = self.backward(input_ids, targets)
        flat = self.flat
        flat.step_count += 1
        lr = self.lr if lr is None else lr
        with nvtx.range("dense/optimizer"):
            use_kernel = self.device.type == "cuda" and ops.native_available()
            self.sumsq.zero_()
            if self.grad_clip > 0:
                if use_kernel:
                    ops.ext().sumsq_(flat.grads, self.sumsq)
                    ops.dispatch.KERNEL_LAUNCHES["count"] += 1
                else:
                    self.sumsq += flat.grads.float().square().sum()
            if use_kernel:
                ops.ext().adamw_step_(flat.params, flat.grads, flat.exp_avg, flat.exp_avg_sq, flat.shadow, lr, self.betas[0], self.betas[1],
                                      self.eps, self.weight_decay, flat.step_count, 1.0, self.sumsq if self.grad_clip > 0 else None,
                                      float(self.grad_clip))
                ops.dispatch.KERNEL_LAUNCHES["count"] += 1
            else:
                scale = 1.0
                if self.grad_clip > 0:
                    scale = torch.clamp(self.grad_clip / (self.sumsq.sqrt() + 1e-6), max=1.0)
                ops.reference.adamw_step(flat.params, flat.grads, flat.exp_avg, flat.exp_avg_sq, lr, self.betas[0], self.betas[1],
                                         self.eps, self.weight_decay, flat.step_count, scale, flat.shadow)
        return loss.detach().clone()

    def named_grads(self) -> dict[str, torch.Tensor]:
        return self.flat.grad_map()
