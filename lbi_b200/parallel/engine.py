"""Region-parallel exact-backprop training engine (no autograd on the hot path).

One step of ``FastLBIEngine.step(input_ids, targets)``:

1. forward chain over this rank's regions: embedding gather, condition add, structured Transformer region
   forward, token pooling, interface update; the boundary state is handed to the rank that owns the next region;
2. for regions with loss terms: final norm, LM head fused with cross-entropy (forward and backward at once);
3. one batched input pullback per region over the R interface basis directions plus (where the region has
   loss) the loss cotangent as an extra direction: yields A_k^T and the offset b_k together;
4. affine suffix scan g_k = b_k + A_k^T g_{k+1} over all regions (inputs exchanged across ranks);
5. one full backward per region with cotangent (loss part + update-path part of g_{k+1}); weight gradients are
   accumulated by the GEMMs straight into the flat fp32 gradient buffer;
6. gradient reduce-scatter, clip + AdamW on this rank's shard (bf16 shadow refreshed by the same kernel),
   all-gather of the updated weights.

Regions are blocks of layers (depth axis, the reference's definition) or blocks of tokens (sequence axis).
The reference performs steps 3-5 with autograd over a retained graph (backward/scan.py:18-97,
backward/pullbacks.py:84-149, backward/local_vjp.py:137-185) and has no multi-device mode.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from .. import ops
from ..models.region_plan import RegionPlacement
from ..utils import nvtx
from .comm import LocalComm
from .flat import FlatParams


@dataclass
class RegionRecord:
    """Per-region forward record kept between the forward chain and the region's turn in the backward."""

    index: int
    token_range: tuple[int, int]
    state_in: torch.Tensor
    pooled: torch.Tensor
    diagnostics: dict
    cache: Any
    ids: torch.Tensor
    out: torch.Tensor | None = None  # fp32 region output (only kept for regions with loss)
    rstd: torch.Tensor | None = None
    normed: torch.Tensor | None = None
    d_out_loss: torch.Tensor | None = None
    state_out: torch.Tensor | None = None
    dec_cache: Any = None   # decoder pre-activations (interface parameter VJP)
    enc_cache: Any = None   # encoder pre-activations; None after the fused update kernel (re-evaluated in the VJP)


@dataclass
class StepResult:
    """What ``backward`` returns: the loss, the state cotangents g_k [B, K, R] and the interface Jacobians when they were kept."""

    loss: torch.Tensor
    state_cotangents: torch.Tensor | None = None
    jacobians: torch.Tensor | None = None
    extras: dict = field(default_factory=dict)


class FastLBIEngine:
    """Autograd-free training step of an ``LBILanguageModel`` on the structured kernels: forward chain over the regions with cached
    activations, interface Jacobians by batched basis pullbacks (the basis directions are split over the ranks), affine suffix scan of
    the state cotangents, one local VJP per region into a flat fp32 gradient buffer, fused clip + AdamW.  One process per GPU;
    regions are placed on ranks in contiguous blocks and states, Jacobians and gradients move through the ``comm`` plane."""

    def __init__(
        self,
        model,
        *,
        lr: float = 1e-3,
        betas: tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 0.0,
        grad_clip: float = 1.0,
        basis_chunk: int = 16,
        act_dtype: torch.dtype | None = None,
        comm=None,
        basis_parallel: bool | None = None,
        recompute_forward: bool = False,
    ) -> None:
        backend = model.region_backend
        if getattr(backend, "structured", None) is None:
            raise NotImplementedError("FastLBIEngine needs a region backend with a closed-form lowering (`structured`: forward with "
                                      "caches, input_pullback, backward); use ScanADEngine otherwise")
        self.model = model
        self.comm = comm or LocalComm()
        self.device = next(model.parameters()).device
        on_cuda = self.device.type == "cuda"
        self.act_dtype = act_dtype or (torch.bfloat16 if on_cuda else torch.float32)
        self.lr, self.betas, self.eps, self.weight_decay, self.grad_clip = lr, betas, eps, weight_decay, grad_clip
        self.basis_chunk = max(1, int(basis_chunk))
        self.placement = RegionPlacement(model.num_regions, self.comm.world_size)
        self.my_regions = list(self.placement.regions_of(self.comm.rank))
        self.flat = FlatParams(model, world_size=self.comm.world_size,
                               shadow_dtype=self.act_dtype if self.act_dtype != torch.float32 else None)
        if hasattr(self.comm, "attach_flat"):
            self.comm.attach_flat(self.flat)  # gradients and bf16 weights move into symmetric (peer-mapped) memory
        lo = self.comm.rank * self.flat.shard
        self.flat.ensure_state(lo, lo + self.flat.shard)
        self.structured = backend.structured
        self.structured.act_dtype = self.act_dtype
        self.structured.shadow_of = self._shadow_of
        self.structured._weights.clear()
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.last: dict = {}
        # Basis-parallel pullback: the (region, block of basis directions) work items are spread evenly over the ranks;
        # a rank that takes items of a region it does not own recomputes that region's forward (1 / R of the pullback).
        # Needs every region's input to be recomputable from tokens and state, i.e. the sequence axis.
        if basis_parallel is None:
            basis_parallel = self.comm.world_size > 1 and model.region_axis == "sequence"
        if basis_parallel and model.region_axis != "sequence":
            raise ValueError("basis_parallel needs sequence-axis regions")
        self.basis_parallel = bool(basis_parallel) and self.comm.world_size > 1
        # Activation recomputation: a region's cached activations are dropped as soon as its forward has produced the outgoing
        # state and the loss cotangent, and rebuilt from its tokens and incoming state right before its pullback and again
        # before its local VJP (two extra region forwards against R + 1 pullback directions).  Sequence axis only.
        if recompute_forward and model.region_axis != "sequence":
            raise ValueError("recompute_forward needs sequence-axis regions (a depth-axis region's input is not recomputable from tokens)")
        self.recompute_forward = bool(recompute_forward)
        self._step_ids: torch.Tensor | None = None

    # ------------------------------------------------------------------ helpers
    def _shadow_of(self, p):
        try:
            return self.flat.weight(self.flat.name_of(p))
        except KeyError:
            return None

    def _w(self, p) -> torch.Tensor:
        return self.flat.weight(self.flat.name_of(p))

    def _g(self, p) -> torch.Tensor:
        return self.flat.grad(self.flat.name_of(p))

    def target(self, name: str):
        """Gradient sink protocol of the structured backward: backbone-relative name -> fp32 accumulator."""
        return self.flat.grad("region_backend.backbone." + name)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def _forward(self, ids: torch.Tensor, targets: torch.Tensor) -> tuple[list[RegionRecord], torch.Tensor]:
        model, iface, comm = self.model, self.model.interface, self.comm
        bsz, seqlen = ids.shape
        sequence_axis = model.region_axis == "sequence"
        token_ranges = model.plan.token_ranges(seqlen)
        table = self._w(model.canvas.embedding.weight)
        dim = model.hidden_dim
        k_regions = model.num_regions
        loss = torch.zeros((), dtype=torch.float32, device=self.device)
        loss_scale = 1.0 / float(bsz * seqlen)
        final_w = model.readout.norm.weight
        final_eps = model.readout.norm.eps
        head_w = table if model.tie_embeddings else self._w(model.readout.lm_head.weight)
        head_grad = self._g(model.canvas.embedding.weight if model.tie_embeddings else model.readout.lm_head.weight)

        full_canvas = None
        if not sequence_axis:
            full_canvas = ops.embedding_fwd(ids, table, self.act_dtype)

        fused_iface = hasattr(comm, "interface_update_handoff") and self.device.type == "cuda"
        if hasattr(comm, "prepare"):
            comm.prepare(bsz, model.interface_width)
        first = self.my_regions[0]
        if first == 0:
            if sequence_axis:
                pooled0 = torch.zeros(bsz, dim, dtype=torch.float32, device=self.device)
            else:
                pooled0 = ops.mean_pool_tokens(full_canvas, bsz, seqlen)
            state, self.last["init_cache"] = iface.initial_cached(pooled0)
            self.last["pooled0"] = pooled0
        else:
            like = torch.empty(bsz, model.interface_width, dtype=torch.float32, device=self.device)
            state = comm.handoff_recv(like, self.placement.owner(first - 1), slot=first)

        records: list[RegionRecord] = []
        for k in self.my_regions:
            t0, t1 = token_ranges[k]
            t_len = t1 - t0
            region_ids = ids[:, t0:t1].contiguous() if sequence_axis else ids
            canvas_rows = ops.embedding_fwd(region_ids, table, self.act_dtype) if sequence_axis else full_canvas
            cond, dec_cache = iface.decode_cached(state, k)
            x_in = ops.add_condition(canvas_rows, cond, t_len)
            _, cache = self.structured.forward(x_in.view(bsz, t_len, dim), model.region_ranges[k], materialize_output=False)
            rec = RegionRecord(index=k, token_range=(t0, t1), state_in=state, pooled=None, diagnostics={}, cache=cache,
                               ids=region_ids, dec_cache=dec_cache)
            if model.plan.region_has_loss(k):
                normed, out, rstd = ops.add_rmsnorm_fwd(cache.last_branch, cache.last_stream, final_w, final_eps, self.act_dtype)
                pooled = ops.mean_pool_tokens(out, bsz, t_len)
                region_targets = targets[:, t0:t1].reshape(-1) if sequence_axis else targets.reshape(-1)
                loss_k, d_normed, _ = ops.lm_head_cross_entropy(normed, head_w, region_targets, loss_scale,
                                                                want_dweight=True, dweight_into=head_grad)
                loss = loss + loss_k
                self._g(final_w).add_(ops.rmsnorm_wgrad(d_normed, out, rstd))
                rec.d_out_loss = ops.rmsnorm_bwd(d_normed, out, rstd, final_w)
                rec.out, rec.rstd = None, None  # not needed again
            else:
                pooled = ops.mean_pool_tokens(cache.last_branch, bsz, t_len)
                if cache.last_stream is not None:
                    pooled = pooled + ops.mean_pool_tokens(cache.last_stream, bsz, t_len)
            remote = k + 1 < k_regions and self.placement.owner(k + 1) != comm.rank
            if fused_iface:
                # interface MLP + LayerNorm in one kernel whose epilogue stores the state into the next owner's mailbox
                new_state, diagnostics = comm.interface_update_handoff(
                    iface, k, state, pooled, self.placement.owner(k + 1) if remote else None)
                rec.pooled, rec.diagnostics, rec.state_out = pooled, diagnostics, new_state
            else:
                step, rec.enc_cache = iface.update_cached(state, pooled, k)
                rec.pooled, rec.diagnostics, rec.state_out = pooled, step.diagnostics, step.state.float()
                if remote:
                    comm.handoff_send(rec.state_out, self.placement.owner(k + 1), slot=k + 1)
            if self.recompute_forward:
                rec.cache = None
            records.append(rec)
            state = rec.state_out
        return records, loss

    def _cache_of(self, rec: RegionRecord):
        """The region's cached activations; rebuilt from its tokens and incoming state when they were dropped."""
        if rec.cache is None:
            rec.cache = self._adopt_region(rec.index, rec.state_in, self._step_ids).cache
        return rec.cache

    # ------------------------------------------------------------------ Jacobian + offset of one region
    @torch.no_grad()
    def _pullback_directions(self, rec: RegionRecord, lo: int, hi: int, include_loss: bool):
        """Pull basis directions [lo, hi) of the outgoing state (and, if asked, the region's loss cotangent) back to the
        incoming state.  Returns (rows [B, hi - lo, R] with rows[b, i] = d s_out[lo + i] / d s_in, or None; b [B, R] or None)."""
        model, iface = self.model, self.model.interface
        k = rec.index
        bsz, r = rec.state_in.shape
        t_len = rec.token_range[1] - rec.token_range[0]
        n = bsz * t_len
        dim = model.hidden_dim
        n_basis = hi - lo
        skip = None
        if n_basis > 0:
            eye = torch.eye(r, device=self.device, dtype=torch.float32)[lo:hi].unsqueeze(0).expand(bsz, n_basis, r)
            upd = iface.update_jacobian_t(k, rec.diagnostics, eye, t_len)
            skip = upd["g_state_skip"]  # [B, n_basis, R]
            g_pooled = upd["g_pooled_features"] / float(t_len)  # [B, n_basis, D]
        has_loss = include_loss and rec.d_out_loss is not None
        total = n_basis + (1 if has_loss else 0)
        if total == 0:
            return None, None
        cond_cots = torch.empty(total, bsz, dim, dtype=torch.float32, device=self.device)
        j = 0
        while j < total:
            c = min(self.basis_chunk, total - j)
            if total - (j + c) == 1:
                c += 1  # a lone trailing direction (the loss cotangent) joins this pass instead of costing one of its own
            rows = torch.empty(c, bsz, t_len, dim, dtype=self.act_dtype, device=self.device)
            nb = max(0, min(c, n_basis - j))
            if nb > 0:
                rows[:nb] = g_pooled[:, j : j + nb].transpose(0, 1).unsqueeze(2).to(self.act_dtype)
            if nb < c:  # the loss direction rides in the last chunk
                rows[nb] = rec.d_out_loss.view(bsz, t_len, dim).to(self.act_dtype)
            g_in = self.structured.input_pullback(self._cache_of(rec), rows.view(c * n, dim))
            cond_cots[j : j + c] = ops.sum_tokens(g_in, c * bsz, t_len).view(c, bsz, dim)
            j += c
        g_state = iface.decode_jacobian_t(k, rec.state_in, cond_cots.transpose(0, 1))  # [B, total, R]
        jac_rows = (skip + g_state[:, :n_basis]) if n_basis > 0 else None
        offset = g_state[:, n_basis].contiguous() if has_loss else None
        return jac_rows, offset

    def _pullback_region(self, rec: RegionRecord, need_jacobian: bool):
        """Returns (A^T [B, R, R] or None, b [B, R])."""
        bsz, r = rec.state_in.shape
        rows, offset = self._pullback_directions(rec, 0, r if need_jacobian else 0, include_loss=True)
        jac = rows.transpose(1, 2).contiguous() if rows is not None else None
        if self.recompute_forward:
            rec.cache = None
        if offset is None:
            offset = torch.zeros(bsz, r, dtype=torch.float32, device=self.device)
        return jac, offset

    # ------------------------------------------------------------------ basis-parallel plan
    def basis_plan(self) -> list[list[tuple[int, int, int]]]:
        """Per rank, the (region, lo, hi) blocks of basis directions it pulls back: the blocks of all regions that need a
        Jacobian, in region order, cut into `world` contiguous runs of equal length.  A rank's run then covers part of
        at most two neighbouring regions beyond whole ones, so it recomputes the forward of at most a few foreign
        regions, and every rank computes the same plan from (regions, width, block size, world) alone."""
        k_regions, r, bc, world = self.model.num_regions, self.model.interface_width, self.basis_chunk, self.comm.world_size
        blocks = [(k, lo, min(r, lo + bc)) for k in range(k_regions - 1) for lo in range(0, r, bc)]
        quota = -(-len(blocks) // world) if blocks else 0
        return [blocks[rank * quota : (rank + 1) * quota] for rank in range(world)]

    @torch.no_grad()
    def _adopt_region(self, k: int, state: torch.Tensor, ids: torch.Tensor) -> RegionRecord:
        """Forward of a region owned by another rank, recomputed here from its tokens and incoming state."""
        model, iface = self.model, self.model.interface
        bsz, seqlen = ids.shape
        t0, t1 = model.plan.token_ranges(seqlen)[k]
        t_len, dim = t1 - t0, model.hidden_dim
        region_ids = ids[:, t0:t1].contiguous()
        table = self._w(model.canvas.embedding.weight)
        canvas_rows = ops.embedding_fwd(region_ids, table, self.act_dtype)
        x_in = ops.add_condition(canvas_rows, iface.decode_cached(state, k)[0], t_len)
        _, cache = self.structured.forward(x_in.view(bsz, t_len, dim), model.region_ranges[k], materialize_output=False)
        if model.plan.region_has_loss(k):
            _, out, _ = ops.add_rmsnorm_fwd(cache.last_branch, cache.last_stream, model.readout.norm.weight, model.readout.norm.eps,
                                            self.act_dtype)
            pooled = ops.mean_pool_tokens(out, bsz, t_len)
        else:
            pooled = ops.mean_pool_tokens(cache.last_branch, bsz, t_len)
            if cache.last_stream is not None:
                pooled = pooled + ops.mean_pool_tokens(cache.last_stream, bsz, t_len)
        step, _ = iface.update_cached(state, pooled, k)
        return RegionRecord(index=k, token_range=(t0, t1), state_in=state, pooled=pooled, diagnostics=step.diagnostics, cache=cache,
                            ids=region_ids)

    @torch.no_grad()
    def _pullback_basis_parallel(self, records: list[RegionRecord], ids: torch.Tensor) -> torch.Tensor:
        """All regions' Jacobians and offsets with the work spread over the ranks -> g [B, K, R]."""
        model, comm = self.model, self.comm
        k_regions, r = model.num_regions, model.interface_width
        bsz = ids.shape[0]
        own = {rec.index: rec for rec in records}
        states = torch.zeros(k_regions, bsz, r, dtype=torch.float32, device=self.device)
        for rec in records:
            states[rec.index] = rec.state_in
        comm.all_reduce_sum(states)   # every rank learns every region's incoming state (K x B x R floats)
        rows_all = torch.zeros(k_regions, bsz, r, r, dtype=torch.float32, device=self.device)   # [k, b, direction, R]
        offs_all = torch.zeros(k_regions, bsz, r, dtype=torch.float32, device=self.device)
        mine = self.basis_plan()[comm.rank]
        by_region: dict[int, list[tuple[int, int]]] = {}
        for k, lo, hi in mine:
            by_region.setdefault(k, []).append((lo, hi))
        loss_done = set()
        for k in sorted(by_region):
            rec = own.get(k) or self._adopt_region(k, states[k], ids)
            blocks = by_region[k]
            for i, (lo, hi) in enumerate(blocks):
                # the owner's loss direction rides with its last block (one direction more in that pass)
                ride = k in own and i == len(blocks) - 1
                rows, off = self._pullback_directions(rec, lo, hi, include_loss=ride)
                rows_all[k, :, lo:hi] = rows
                if off is not None:
                    offs_all[k] = off
                    loss_done.add(k)
            if k not in own or self.recompute_forward:
                rec.cache = None
        for rec in records:   # loss directions that found no block to ride with
            if rec.index not in loss_done and rec.d_out_loss is not None:
                _, off = self._pullback_directions(rec, 0, 0, include_loss=True)
                offs_all[rec.index] = off
        if hasattr(comm, "scan_published") and self.device.type == "cuda":
            g, rows_full = comm.scan_published(rows_all, offs_all, mine, sorted(loss_done | {rec.index for rec in records
                                                                                              if rec.d_out_loss is not None}))
            # A_k^T[b, i, j] = d s_out[j] / d s_in[i]: a view of the gathered rows (valid until the next step publishes)
            self.last["jacobians"], self.last["offsets"] = rows_full.permute(1, 0, 3, 2), None
            return g
        comm.all_reduce_sum(rows_all)
        comm.all_reduce_sum(offs_all)
        mats_all = rows_all.permute(1, 0, 3, 2).contiguous()   # [B, K, R, R] with A_k^T[b, i, j] = d s_out[j] / d s_in[i]
        offs = offs_all.transpose(0, 1).contiguous()           # [B, K, R]
        self.last["jacobians"], self.last["offsets"] = mats_all, offs
        if k_regions == 1:
            return offs
        g = ops.affine_suffix_scan(mats_all[:, : k_regions - 1].contiguous(), offs[:, : k_regions - 1].contiguous(),
                                   seed=offs[:, k_regions - 1].contiguous())
        return g[:, :k_regions]

    # ------------------------------------------------------------------ scan over all regions
    @torch.no_grad()
    def _scan(self, jacobians: list, offsets: list[torch.Tensor]) -> torch.Tensor:
        """Local lists (one entry per owned region; jacobian None for the global last region) -> g [B, K, R]."""
        model, comm = self.model, self.comm
        k_regions = model.num_regions
        bsz, r = offsets[0].shape
        mats = torch.stack(
            [j if j is not None else torch.zeros(bsz, r, r, dtype=torch.float32, device=self.device) for j in jacobians], dim=1
        )
        offs = torch.stack(offsets, dim=1)
        if hasattr(comm, "scan") and self.device.type == "cuda":
            self.last["jacobians"] = None
            return comm.scan(mats, offs)  # peer-loaded matrices, recursion on every rank
        mats_all, offs_all = comm.gather_scan_inputs(mats, offs)  # [B, K, R, R], [B, K, R]
        self.last["jacobians"] = mats_all
        self.last["offsets"] = offs_all
        if k_regions == 1:
            return offs_all
        g = ops.affine_suffix_scan(mats_all[:, : k_regions - 1].contiguous(), offs_all[:, : k_regions - 1].contiguous(),
                                   seed=offs_all[:, k_regions - 1].contiguous())
        return g[:, :k_regions]

    # ------------------------------------------------------------------ local VJPs
    @torch.no_grad()
    def _backward_region(self, rec: RegionRecord, g_next: torch.Tensor | None) -> None:
        model, iface = self.model, self.model.interface
        k = rec.index
        bsz = rec.state_in.shape[0]
        t_len = rec.token_range[1] - rec.token_range[0]
        dim = model.hidden_dim
        cot = rec.d_out_loss
        if g_next is not None:
            g_pooled = iface.update_parameter_vjp(k, rec.diagnostics, rec.enc_cache, g_next, self._g)
            spread = (g_pooled.float() / float(t_len)).unsqueeze(1)  # [B, 1, D] broadcast over tokens
            if cot is None:
                cot = spread.expand(bsz, t_len, dim).reshape(bsz * t_len, dim).contiguous()
            else:
                cot.view(bsz, t_len, dim).add_(spread)
        if cot is None:
            return
        d_in = self.structured.backward(self._cache_of(rec), cot, self)
        d_cond = ops.sum_tokens(d_in, bsz, t_len)
        ops.embedding_scatter_add(self._g(model.canvas.embedding.weight), rec.ids, d_in)
        iface.decode_parameter_vjp(k, rec.dec_cache, d_cond, self._g)

    @torch.no_grad()
    def _backward_initial(self, ids: torch.Tensor, g0: torch.Tensor) -> None:
        model, iface = self.model, self.model.interface
        depth = model.region_axis == "depth"
        g_pooled = iface.initial_parameter_vjp(self.last["init_cache"], g0, self._g, want_input=depth)
        if depth and g_pooled is not None:
            bsz, seqlen = ids.shape
            rows = (g_pooled.float() / float(seqlen)).unsqueeze(1).expand(bsz, seqlen, -1).reshape(bsz * seqlen, -1).contiguous()
            ops.embedding_scatter_add(self._g(model.canvas.embedding.weight), ids, rows)

    # ------------------------------------------------------------------ optimizer
    @torch.no_grad()
    def _optimizer_step(self, lr: float) -> None:
        flat, comm = self.flat, self.comm
        if hasattr(comm, "optimizer_step") and self.device.type == "cuda" and comm.fused_optimizer_ready(flat):
            comm.optimizer_step(flat, lr=lr, betas=self.betas, eps=self.eps, weight_decay=self.weight_decay,
                                grad_clip=self.grad_clip)
            return
        shard = flat.shard
        lo = comm.rank * shard
        g_shard = comm.reduce_scatter_grads(flat.grads, shard) if comm.world_size > 1 else flat.grads
        flat.step_count += 1
        use_kernel = self.device.type == "cuda" and ops.native_available()
        self.sumsq.zero_()
        if self.grad_clip > 0:
            if use_kernel:
                ops.ext().sumsq_(g_shard, self.sumsq)
                ops.dispatch.KERNEL_LAUNCHES["count"] += 1
            else:
                self.sumsq += g_shard.float().square().sum()
            comm.all_reduce_sum(self.sumsq)
        p_shard = flat.params[lo : lo + shard]
        sh_shard = flat.shadow[lo : lo + shard] if flat.shadow is not None else None
        if use_kernel:
            ops.ext().adamw_step_(p_shard, g_shard, flat.exp_avg, flat.exp_avg_sq, sh_shard, lr, self.betas[0], self.betas[1],
                                  self.eps, self.weight_decay, flat.step_count, 1.0,
                                  self.sumsq if self.grad_clip > 0 else None, float(self.grad_clip))
            ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        else:
            scale = 1.0
            if self.grad_clip > 0:
                scale = torch.clamp(self.grad_clip / (self.sumsq.sqrt() + 1e-6), max=1.0)
            ops.reference.adamw_step(p_shard, g_shard, flat.exp_avg, flat.exp_avg_sq, lr, self.betas[0], self.betas[1], self.eps,
                                     self.weight_decay, flat.step_count, scale, sh_shard)
        if comm.world_size > 1:
            comm.all_gather_flat(flat.shadow if flat.shadow is not None else flat.params, shard)

    def _plan_master_sync(self) -> None:
        """Runs of the flat layout that the engine reads from the fp32 master rather than from the compute-dtype shadow:
        every interface parameter, every norm weight, bias and per-head scalar (all but the 2-D projection / embedding
        matrices).  Adjacent slots are merged so that a step moves a few dozen contiguous pieces."""
        runs: list[list[int]] = []
        for name, slot in self.flat.slots.items():
            matrix = len(slot.shape) == 2 and not name.startswith("interface.")
            if matrix:
                continue
            lo, hi = slot.offset, slot.offset + slot.numel
            if runs and lo - runs[-1][1] < 64:
                runs[-1][1] = hi
            else:
                runs.append([lo, hi])
        self._master_runs = [(a, b) for a, b in runs]
        total = sum(b - a for a, b in self._master_runs)
        self._master_buf = torch.zeros(total, dtype=torch.float32, device=self.device)

    @torch.no_grad()
    def _sync_fp32_read_params(self) -> None:
        """Collective, after every optimizer step of a multi-rank run that keeps a low-precision shadow: a rank's AdamW
        updates the fp32 master of its own shard only and the other shards arrive as shadow weights, so the parameters
        that the engine reads in fp32 would otherwise go stale (and differ between ranks).  Their owners' fp32 values are
        exchanged here through one compact buffer (zeros outside the owned part, summed over ranks)."""
        if self.comm.world_size == 1 or self.flat.shadow is None:
            return
        if not hasattr(self, "_master_runs"):
            self._plan_master_sync()
        flat, buf = self.flat, self._master_buf
        lo, hi = self.comm.rank * flat.shard, (self.comm.rank + 1) * flat.shard
        buf.zero_()
        pos = 0
        for a, b in self._master_runs:
            x, y = max(a, lo), min(b, hi)
            if x < y:
                buf[pos + x - a : pos + y - a].copy_(flat.params[x:y])
            pos += b - a
        self.comm.all_reduce_sum(buf)
        pos = 0
        for a, b in self._master_runs:
            flat.params[a:b].copy_(buf[pos : pos + b - a])
            pos += b - a

    # ------------------------------------------------------------------ public API
    def backward(self, input_ids: torch.Tensor, targets: torch.Tensor) -> StepResult:
        """Forward + exact region-local backward; gradients end up in ``self.flat.grads`` (not yet reduced)."""
        model = self.model
        self.flat.zero_grad()
        self._step_ids = input_ids
        with nvtx.range("lbi/forward"):
            records, loss = self._forward(input_ids, targets)
        k_regions = model.num_regions
        if self.basis_parallel:
            with nvtx.range("lbi/pullback/basis_parallel"):
                g = self._pullback_basis_parallel(records, input_ids)  # [B, K, R]
        else:
            jacobians, offsets = [], []
            for rec in records:
                with nvtx.range(f"lbi/pullback/region{rec.index}"):
                    jac, off = self._pullback_region(rec, need_jacobian=rec.index < k_regions - 1)
                jacobians.append(jac)
                offsets.append(off)
            with nvtx.range("lbi/scan"):
                g = self._scan(jacobians, offsets)  # [B, K, R]
        for rec in records:
            g_next = g[:, rec.index + 1] if rec.index + 1 < k_regions else None
            with nvtx.range(f"lbi/local_vjp/region{rec.index}"):
                self._backward_region(rec, g_next)
            rec.cache = None
        if self.my_regions[0] == 0:
            with nvtx.range("lbi/local_vjp/initial"):
                self._backward_initial(input_ids, g[:, 0])
        return StepResult(loss=loss, state_cotangents=g, jacobians=self.last.get("jacobians"))

    def step(self, input_ids: torch.Tensor, targets: torch.Tensor, lr: float | None = None) -> torch.Tensor:
        result = self.backward(input_ids, targets)
        with nvtx.range("lbi/optimizer"):
            self._optimizer_step(self.lr if lr is None else lr)
            self._sync_fp32_read_params()
        loss = result.loss.detach().clone()
        if self.comm.world_size > 1:
            self.comm.all_reduce_sum(loss)
        return loss

    def sync_master_params(self) -> None:
        """Collective: complete the fp32 master copy on every rank (a rank's optimizer updates only its own shard; the
        other shards reach it as bf16 weights).  Needed before evaluating or saving the module's parameters."""
        if self.comm.world_size > 1 and self.flat.shadow is not None:
            self.comm.all_gather_flat(self.flat.params, self.flat.shard)

    def named_grads(self) -> dict[str, torch.Tensor]:
        return self.flat.grad_map()
