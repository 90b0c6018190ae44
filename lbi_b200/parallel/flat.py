"""Flat parameter / gradient / optimizer-state buffers.

All trainable parameters of a model are re-pointed at views of one contiguous fp32 buffer; gradients live
in a second buffer of the same layout, AdamW moments in two more, and a bf16 "shadow" copy (the weights
the tensor-core kernels read) in a fifth.  One fused kernel then does clip-scale + AdamW + bf16 refresh
over a contiguous range, and a rank's optimizer shard is simply ``[rank * shard, (rank + 1) * shard)``.
The flat layout follows ``model.named_parameters()`` order; tied parameters appear once.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn


@dataclass
class Slot:
    """Where a parameter lives in the flat buffers: name, element offset, element count, shape."""

    name: str
    offset: int
    numel: int
    shape: torch.Size


class FlatParams:
    """All trainable parameters of a model as views into one fp32 buffer (aligned slots, padded so that ``world_size`` equal shards
    tile it), with a gradient buffer of the same layout, AdamW moments per shard and an optional low-precision shadow of the weights."""

    def __init__(self, model: nn.Module, *, world_size: int = 1, shadow_dtype: torch.dtype | None = torch.bfloat16,
                 align: int = 64) -> None:
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not named:
            raise ValueError("model has no trainable parameters")
        device = named[0][1].device
        self.device = device
        self.slots: dict[str, Slot] = {}
        self._by_id: dict[int, Slot] = {}
        offset = 0
        for name, p in named:
            slot = Slot(name, offset, p.numel(), p.shape)
            self.slots[name] = slot
            self._by_id[id(p)] = slot
            offset += -(-p.numel() // align) * align
        unit = align * max(1, world_size)
        self.total = -(-offset // unit) * unit
        self.world_size = max(1, world_size)
        self.shard = self.total // self.world_size
        self.params = torch.zeros(self.total, dtype=torch.float32, device=device)
        self.grads = torch.zeros(self.total, dtype=torch.float32, device=device)
        self.exp_avg = None
        self.exp_avg_sq = None
        self.shadow = torch.zeros(self.total, dtype=shadow_dtype, device=device) if shadow_dtype is not None else None
        with torch.no_grad():
            for name, p in named:
                view = self.view(self.params, name)
                view.copy_(p.detach().float())
                p.data = view
        self.refresh_shadow()
        self.step_count = 0

    # ---- views
    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        s = self.slots[name]
        return flat[s.offset : s.offset + s.numel].view(s.shape)

    def grad(self, name: str) -> torch.Tensor:
        return self.view(self.grads, name)

    def weight(self, name: str) -> torch.Tensor:
        """Compute-dtype (shadow) view of a parameter; the fp32 master when no shadow is kept."""
        return self.view(self.shadow if self.shadow is not None else self.params, name)

    def slot_of(self, p: nn.Parameter) -> Slot:
        return self._by_id[id(p)]

    def name_of(self, p: nn.Parameter) -> str:
        return self._by_id[id(p)].name

    def refresh_shadow(self) -> None:
        if self.shadow is not None:
            self.shadow.copy_(self.params)

    def zero_grad(self) -> None:
        self.grads.zero_()

    def grad_map(self) -> dict[str, torch.Tensor]:
        return {name: self.grad(name) for name in self.slots}

    # ---- optimizer state
    def ensure_state(self, lo: int = 0, hi: int | None = None) -> None:
        """Allocate AdamW moments for the range this rank updates (the full buffer by default)."""
        hi = self.total if hi is None else hi
        if self.exp_avg is None:
            self.state_range = (lo, hi)
            self.exp_avg = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)
            self.exp_avg_sq = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)

    def gathered_moments(self, comm=None) -> tuple[torch.Tensor, torch.Tensor]:
        """Full-length AdamW moments.  With sharded state every rank must call this (it is an all-gather)."""
        lo, hi = self.state_range
        if (lo, hi) == (0, self.total):
            return self.exp_avg, self.exp_avg_sq
        if comm is None or comm.world_size != self.world_size:
            raise RuntimeError("gather the moment shards before exporting the optimizer state: pass the communicator")
        return comm._all_gather(self.exp_avg).reshape(-1), comm._all_gather(self.exp_avg_sq).reshape(-1)

    def state_dict_like_torch(self, param_order: list[str], hyper: dict, comm=None) -> dict:
        """Optimizer state in ``torch.optim.AdamW.state_dict()`` layout (consolidated over ranks when sharded)."""
        exp_avg, exp_avg_sq = self.gathered_moments(comm)
        state = {}
        for idx, name in enumerate(param_order):
            s = self.slots[name]
            state[idx] = {
                "step": torch.tensor(float(self.step_count)),
                "exp_avg": exp_avg[s.offset : s.offset + s.numel].view(s.shape).clone(),
                "exp_avg_sq": exp_avg_sq[s.offset : s.offset + s.numel].view(s.shape).clone(),
            }
        group = dict(hyper)
        group["params"] = list(range(len(param_order)))
        return {"state": state, "param_groups": [group]}

    def load_state_dict_like_torch(self, sd: dict, param_order: list[str]) -> None:
        """Load a consolidated state; a rank with sharded moments keeps only the part inside its range."""
        self.ensure_state()
        lo, hi = self.state_range
        for idx, name in enumerate(param_order):
            st = sd["state"].get(idx)
            if st is None:
                continue
            s = self.slots[name]
            a, b = max(lo, s.offset), min(hi, s.offset + s.numel)
            if a < b:
                self.exp_avg[a - lo : b - lo].copy_(st["exp_avg"].reshape(-1)[a - s.offset : b - s.offset])
                self.exp_avg_sq[a - lo : b - lo].copy_(st["exp_avg_sq"].reshape(-1)[a - s.offset : b - s.offset])
            self.step_count = int(float(st["step"]))
