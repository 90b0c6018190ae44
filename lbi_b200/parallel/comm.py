"""Communication plane of the region-parallel engine.

``LocalComm``   single process (world size 1): every exchange is the identity.
``CollectiveComm``  one process per GPU over ``torch.distributed`` (NCCL on GPUs, gloo on CPU ranks).  This is the
                library-collective twin of every fused path: state handoff by send/recv, scan inputs by
                all-gather, gradients by reduce-scatter followed by a separate AdamW kernel and an all-gather of
                the updated weights.  It is the baseline the peer-memory kernels in ``lbi_b200.parallel.symm``
                are measured against, and the fall-back where peer memory is unavailable.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


class LocalComm:
    """The single-process plane: every exchange is the identity."""

    rank = 0
    world_size = 1
    name = "local"

    def handoff_send(self, state: torch.Tensor, dst: int, slot: int = 0) -> None:
        raise RuntimeError("no peers in a single-process run")

    def handoff_recv(self, like: torch.Tensor, src: int, slot: int = 0) -> torch.Tensor:
        raise RuntimeError("no peers in a single-process run")

    def gather_scan_inputs(self, mats: torch.Tensor, offsets: torch.Tensor):
        return mats, offsets

    def reduce_scatter_grads(self, grads: torch.Tensor, shard: int) -> torch.Tensor:
        return grads

    def all_gather_flat(self, flat: torch.Tensor, shard: int) -> None:
        return None

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def barrier(self) -> None:
        return None


class CollectiveComm:
    """Communication plane on library collectives (NCCL on GPUs, gloo on CPUs): state hand-off by send / recv, Jacobian exchange by
    all-gather, gradient reduce-scatter and weight all-gather around the sharded AdamW.  The twin of ``SymmComm``, and the baseline it is timed against."""

    name = "collective"

    def __init__(self, group=None) -> None:
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)

    def handoff_send(self, state: torch.Tensor, dst: int, slot: int = 0) -> None:
        dist.send(state.contiguous(), dst=dst, group=self.group, tag=slot)

    def handoff_recv(self, like: torch.Tensor, src: int, slot: int = 0) -> torch.Tensor:
        buf = torch.empty_like(like)
        dist.recv(buf, src=src, group=self.group, tag=slot)
        return buf

    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[*shape] on every rank -> [world, *shape]."""
        w = self.world_size
        flat = t.contiguous().reshape(-1)
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(flat) for _ in range(w)]
            dist.all_gather(parts, flat, group=self.group)
            return torch.stack(parts).reshape(w, *t.shape)
        out = torch.empty(w * flat.numel(), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, flat, group=self.group)
        return out.reshape(w, *t.shape)

    def gather_scan_inputs(self, mats: torch.Tensor, offsets: torch.Tensor):
        """mats [B, k_local, R, R], offsets [B, k_local, R] -> concatenated over ranks along dim 1."""
        w = self.world_size
        m_all = self._all_gather(mats)
        o_all = self._all_gather(offsets)
        b = mats.shape[0]
        m_cat = m_all.permute(1, 0, 2, 3, 4).reshape(b, w * mats.shape[1], *mats.shape[2:])
        o_cat = o_all.permute(1, 0, 2, 3).reshape(b, w * offsets.shape[1], offsets.shape[2])
        return m_cat.contiguous(), o_cat.contiguous()

    def reduce_scatter_grads(self, grads: torch.Tensor, shard: int) -> torch.Tensor:
        out = grads[self.rank * shard : (self.rank + 1) * shard]
        if dist.get_backend(self.group) == "gloo":
            dist.all_reduce(grads, group=self.group)
            return out
        dist.reduce_scatter_tensor(out, grads, group=self.group)
        return out

    def all_gather_flat(self, flat: torch.Tensor, shard: int) -> None:
        mine = flat[self.rank * shard : (self.rank + 1) * shard]
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(mine) for _ in range(self.world_size)]
            dist.all_gather(parts, mine.clone(), group=self.group)
            for r, part in enumerate(parts):
                flat[r * shard : (r + 1) * shard].copy_(part)
            return
        dist.all_gather_into_tensor(flat, mine.clone(), group=self.group)

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    def barrier(self) -> None:
        dist.barrier(group=self.group)


def init_distributed_from_env(device_type: str = "cuda"):
    """Initialise the default process group from torchrun's environment; returns (rank, local_rank, world)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device_type == "cuda":
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
    return rank, local_rank, world
