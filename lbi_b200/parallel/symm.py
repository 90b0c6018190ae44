"""Peer-memory communication plane: the three fused paths over NVLink 5 / NVSwitch.

Buffers are allocated with ``torch.distributed._symmetric_memory`` (every rank maps every peer's buffer), the kernels
in ``csrc/peer.cu`` receive tables of peer pointers and do the transfers themselves:

1. ``interface_update_handoff``  interface MLP + LayerNorm epilogue stores the bounded state into the next owner's
   mailbox and raises its flag; ``handoff_recv`` is the matching bounded wait;
2. ``scan``                      every rank publishes its Jacobians / offsets in its symmetric buffer, raises its flag
   on all peers, and runs the affine suffix scan over peer-loaded matrices;
3. ``optimizer_step``            gradient reduce-scatter by peer loads (NVLS ``multimem.ld_reduce`` when the buffer has
   a multicast mapping and LBI_B200_MULTIMEM=1) with the gradient-norm partial, a one-float exchange, then
   clip + AdamW fused with the all-gather of the new bf16 weights by peer stores.

``CollectiveComm`` (library collectives) is the baseline twin of all three.  Flags are monotonically increasing
sequence numbers in a symmetric int32 array; every device-side wait is bounded and reports through
``ext.kernel_status``.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import ops
from .comm import CollectiveComm

# flag slots (each block holds one slot per rank)
_SLOT_BARRIER, _SLOT_SCAN, _SLOT_NORM, _SLOT_HANDOFF = 0, 1, 2, 3


_GUARD_BYTES = 256          # canary region before and after every symmetric buffer (keeps 256-byte alignment)
_GUARD_BYTE = 0xA5


class _GuardedHandle:
    """A rendezvous handle seen through the guard offset: peers address the payload, not the canary in front of it."""

    def __init__(self, handle, offset: int) -> None:
        self._handle = handle
        self.buffer_ptrs = [int(p) + offset for p in handle.buffer_ptrs]
        mc = getattr(handle, "multicast_ptr", 0)
        self.multicast_ptr = int(mc) + offset if mc else 0


class SymmComm(CollectiveComm):
    """Communication plane on symmetric (peer-mapped) memory: the kernels of ``csrc/peer.cu`` store states into the next rank's
    mailbox, publish Jacobian pieces into every peer's buffer, reduce-scatter gradients by peer loads and all-gather the updated
    weights by peer stores.  Every device-side wait is bounded; canaries guard the buffers peers write into."""

    name = "symm"

    def __init__(self, group=None) -> None:
        super().__init__(group)
        import torch.distributed._symmetric_memory as symm

        if not ops.native_available():
            raise RuntimeError("the peer-memory plane needs the CUDA extension")
        self._symm = symm
        self._group = group if group is not None else dist.group.WORLD
        self.device = torch.device("cuda", torch.cuda.current_device())
        w = self.world_size
        self.flags, self._flag_handle = self._alloc((4 + 64) * w, torch.int32)
        self.flags.zero_()
        self.flag_ptrs = self._table(self._flag_handle)
        self.norm_vals, h = self._alloc(w, torch.float32)
        self.norm_ptrs = self._table(h)
        self.seq = 0
        self.send_seq = 0
        self.recv_seq = 0
        self._mailboxes: dict[tuple, tuple] = {}
        self._scan_bufs: dict[tuple, tuple] = {}
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.use_multimem = os.environ.get("LBI_B200_MULTIMEM", "0") == "1"
        self._flat_state = None
        self._handle_keepalive = []
        self._setup_barrier()

    # ------------------------------------------------------------------ symmetric allocation
    def _alloc(self, numel: int, dtype: torch.dtype):
        """Symmetric buffer of ``numel`` elements with a canary region on both sides (peers write into these buffers with
        plain stores; a store that runs past an end lands in a canary and ``check_canaries`` reports it)."""
        item = torch.empty((), dtype=dtype).element_size()
        guard = _GUARD_BYTES // item
        payload = -(-int(numel) * item // _GUARD_BYTES) * _GUARD_BYTES // item     # rounded up: the rear canary stays aligned
        full = self._symm.empty(payload + 2 * guard, dtype=dtype, device=self.device)
        handle = self._symm.rendezvous(full, self._group)
        raw = full.view(torch.uint8)
        raw[:_GUARD_BYTES] = _GUARD_BYTE
        raw[_GUARD_BYTES + payload * item:] = _GUARD_BYTE
        if not hasattr(self, "_guarded"):
            self._guarded = []
        self._guarded.append((raw, payload * item))
        return full[guard : guard + int(numel)], _GuardedHandle(handle, _GUARD_BYTES)

    def check_canaries(self) -> list[int]:
        """Indices (allocation order) of the symmetric buffers whose front or rear canary was overwritten."""
        bad = []
        for i, (raw, nbytes) in enumerate(getattr(self, "_guarded", [])):
            front, rear = raw[:_GUARD_BYTES], raw[_GUARD_BYTES + nbytes:]
            if not (bool((front == _GUARD_BYTE).all()) and bool((rear == _GUARD_BYTE).all())):
                bad.append(i)
        return bad

    def _table(self, handle, byte_offset: int = 0) -> torch.Tensor:
        return torch.tensor([int(p) + byte_offset for p in handle.buffer_ptrs], dtype=torch.int64, device=self.device)

    def alloc_flat(self, numel: int, dtype: torch.dtype):
        """Symmetric flat buffer for gradients / bf16 weights; returns (tensor, pointer table, multicast address)."""
        t, handle = self._alloc(numel, dtype)
        t.zero_()
        self._handle_keepalive.append(handle)
        return t, self._table(handle), handle.multicast_ptr

    # ------------------------------------------------------------------ barrier
    def _setup_barrier(self) -> None:
        """Barrier for set-up points, where ranks may be far apart (imports, allocation): meet on the host first."""
        dist.barrier(group=self.group)
        self.barrier()

    def scan_slot_base(self) -> int:
        """First flag word of the scan's per-rank flags (for callers that drive the publish / recursion kernels directly)."""
        return _SLOT_SCAN * self.world_size

    def barrier(self) -> None:
        self.seq += 1
        ops.ext().peer_barrier(self.flag_ptrs, self.rank, self.world_size, _SLOT_BARRIER * self.world_size, self.seq)

    # ------------------------------------------------------------------ (1) forward hand-off
    def _mailbox(self, shape: tuple):
        key = tuple(shape)
        hit = self._mailboxes.get(key)
        if hit is None:
            numel = 1
            for s in shape:
                numel *= int(s)
            t, handle = self._alloc(numel, torch.float32)
            hit = (t.view(*shape), [int(p) for p in handle.buffer_ptrs], handle)
            self._mailboxes[key] = hit
            self._setup_barrier()
        return hit

    def prepare(self, batch: int, width: int) -> None:
        """Collective: create the hand-off mailbox for states of shape [batch, width] (all ranks, same call order)."""
        self._mailbox((batch, width))

    def interface_update_handoff(self, iface, k: int, state: torch.Tensor, pooled: torch.Tensor, dst: int | None):
        """Fused interface update; with ``dst`` the new state also lands in rank dst's mailbox.  Returns (state, diagnostics)."""
        enc, norm = iface.encoders[k], iface.norms[k]
        first, second = enc.layers()
        peer_state = peer_flag = 0
        seq = 0
        if dst is not None:
            _, ptrs, _ = self._mailbox(tuple(state.shape))
            self.send_seq += 1
            seq = self.send_seq
            peer_state = ptrs[dst]
            peer_flag = int(self._flag_handle.buffer_ptrs[dst]) + 4 * (_SLOT_HANDOFF * self.world_size + self.rank)
        act = 0 if iface.activation == "silu" else 1
        delta, pre, out = ops.ext().interface_update_handoff(
            state.contiguous(), pooled.contiguous(), first.weight.detach(), None if first.bias is None else first.bias.detach(),
            None if second is None else second.weight.detach(), None if (second is None or second.bias is None) else second.bias.detach(),
            iface.update_scale.detach()[k : k + 1], norm.weight.detach(), norm.bias.detach(), float(norm.eps), act,
            int(peer_state), int(peer_flag), int(seq), self.done_counter)
        ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        diagnostics = {"pooled_features": pooled, "delta_state": delta, "pre_norm_state": pre,
                       "update_scale": torch.tanh(iface.update_scale.detach()[k])}
        return out, diagnostics

    def handoff_send(self, state: torch.Tensor, dst: int, slot: int = 0) -> None:
        raise RuntimeError("the peer-memory plane hands states off inside interface_update_handoff")

    def handoff_recv(self, like: torch.Tensor, src: int, slot: int = 0) -> torch.Tensor:
        mailbox, _, _ = self._mailbox(tuple(like.shape))
        self.recv_seq += 1
        out = ops.ext().wait_state(mailbox, self.flags, _SLOT_HANDOFF * self.world_size + src, self.recv_seq)
        ops.dispatch.KERNEL_LAUNCHES["count"] += 1
        return out

    # ------------------------------------------------------------------ (2) cross-GPU scan
    def scan(self, mats: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
        """mats [B, k_local, R, R], offsets [B, k_local, R] of this rank -> g [B, K, R] for all regions."""
        key = (tuple(mats.shape), tuple(offsets.shape))
        hit = self._scan_bufs.get(key)
        if hit is None:
            m_buf, mh = self._alloc(mats.numel(), torch.float32)
            o_buf, oh = self._alloc(offsets.numel(), torch.float32)
            hit = (m_buf, o_buf, self._table(mh), self._table(oh), mh, oh)
            self._scan_bufs[key] = hit
            self._setup_barrier()
        m_buf, o_buf, m_ptrs, o_ptrs, _, _ = hit
        # peers may still be reading last step's matrices: the barrier at the end of the optimizer step orders that
        m_buf.copy_(mats.reshape(-1))
        o_buf.copy_(offsets.reshape(-1))
        self.seq += 1
        w = self.world_size
        ops.ext().peer_signal_all(self.flag_ptrs, self.rank, w, _SLOT_SCAN * w, self.seq)
        g = ops.ext().affine_scan_peer(m_ptrs, o_ptrs, self.flags, _SLOT_SCAN * w, self.seq, mats.shape[0], w, mats.shape[1],
                                       mats.shape[-1])
        ops.dispatch.KERNEL_LAUNCHES["count"] += 2
        return g

    def scan_published(self, rows_all: torch.Tensor, offs_all: torch.Tensor, row_blocks, off_regions):
        """Basis-parallel scan, gather form.  rows_all [K, B, R, R] / offs_all [K, B, R] hold this rank's results in the
        blocks ``row_blocks`` = [(region, lo, hi)] of basis directions and the offsets of ``off_regions``; one kernel stores
        exactly those pieces into every rank's symmetric buffer (peer stores) and raises this rank's flag, then the scan
        kernel waits for every rank's flag and recurses over its own, now complete, copy.  Each matrix element crosses
        NVLink once per destination and nothing is summed.  Returns (g [B, K, R], complete rows [K, B, R, R] view)."""
        key = ("published", tuple(rows_all.shape))
        hit = self._scan_bufs.get(key)
        if hit is None:
            m_buf, mh = self._alloc(rows_all.numel(), torch.float32)
            o_buf, oh = self._alloc(offs_all.numel(), torch.float32)
            m_buf.zero_()
            o_buf.zero_()
            hit = (m_buf, o_buf, self._table(mh), self._table(oh), mh, oh, {})
            self._scan_bufs[key] = hit
            self._setup_barrier()
        m_buf, o_buf, m_ptrs, o_ptrs, _, _, seg_cache = hit
        k_total, bsz, r = rows_all.shape[0], rows_all.shape[1], rows_all.shape[-1]
        plan_key = (tuple(row_blocks), tuple(off_regions))
        segs = seg_cache.get(plan_key)
        if segs is None:
            seg_m = [(((k * bsz + b) * r + lo) * r, (hi - lo) * r) for (k, lo, hi) in row_blocks for b in range(bsz)]
            seg_o = [(k * bsz * r, bsz * r) for k in off_regions]
            if r % 4:
                raise ValueError("the published scan moves 16-byte pieces: the interface width must be a multiple of 4")
            as_tensor = lambda seg: torch.tensor(seg or [(0, 0)], dtype=torch.int64, device=self.device).reshape(-1, 2).contiguous()  # noqa: E731
            segs = (as_tensor(seg_m), as_tensor(seg_o))
            seg_cache[plan_key] = segs
        self.seq += 1
        w = self.world_size
        ext = ops.ext()
        # peers may still be reading last step's matrices: the barrier at the end of the optimizer step orders that
        ext.peer_publish(rows_all.contiguous(), m_ptrs, segs[0], offs_all.contiguous(), o_ptrs, segs[1], self.flag_ptrs, self.rank, w,
                         _SLOT_SCAN * w, self.seq, self.done_counter)
        own_m, own_o = m_ptrs[self.rank : self.rank + 1], o_ptrs[self.rank : self.rank + 1]
        g = ext.affine_scan_peer_sum(own_m, own_o, self.flags, _SLOT_SCAN * w, self.seq, bsz, 1, k_total, r, w)
        ops.dispatch.KERNEL_LAUNCHES["count"] += 2
        return g, m_buf.view(rows_all.shape)

    # ------------------------------------------------------------------ (3) gradients + optimizer + weight all-gather
    def attach_flat(self, flat) -> None:
        """Move the gradient and bf16-weight buffers of ``flat`` into symmetric memory (views are re-pointed)."""
        grads, g_ptrs, g_mc = self.alloc_flat(flat.total, torch.float32)
        flat.grads = grads
        shadow_ptrs = None
        if flat.shadow is not None:
            shadow, shadow_ptrs, _ = self.alloc_flat(flat.total, flat.shadow.dtype)
            shadow.copy_(flat.shadow)
            flat.shadow = shadow
        self._flat_state = (g_ptrs, g_mc if self.use_multimem else 0, shadow_ptrs)
        self._setup_barrier()

    def fused_optimizer_ready(self, flat) -> bool:
        """The fused reduce-scatter + AdamW + all-gather kernels move the updated weights as the low-precision shadow.  A
        run without one (fp32 activations) keeps its gradients in symmetric memory but takes the library-collective
        optimizer step, which gathers the fp32 master itself."""
        return self._flat_state is not None and self._flat_state[2] is not None

    def optimizer_step(self, flat, *, lr, betas, eps, weight_decay, grad_clip) -> None:
        g_ptrs, g_mc, shadow_ptrs = self._flat_state
        w, shard = self.world_size, flat.shard
        lo = self.rank * shard
        ext = ops.ext()
        self.barrier()  # every rank has finished writing its gradients
        self.sumsq.zero_()
        ext.grad_reduce_scatter_(g_ptrs, g_mc, self.rank, w, lo, shard, self.sumsq)
        self.seq += 1
        ext.exchange_scalar(self.norm_ptrs, self.flag_ptrs, self.sumsq, self.rank, w, _SLOT_NORM * w, self.seq)
        flat.step_count += 1
        ext.adamw_allgather_(flat.params[lo : lo + shard], flat.grads[lo : lo + shard], flat.exp_avg, flat.exp_avg_sq, shadow_ptrs,
                             w, lo, lr, betas[0], betas[1], eps, weight_decay, flat.step_count, self.norm_vals, float(grad_clip))
        ops.dispatch.KERNEL_LAUNCHES["count"] += 4
        self.barrier()  # all peers' weight shards have landed before the next forward reads them
