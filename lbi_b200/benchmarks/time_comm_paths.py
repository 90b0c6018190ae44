"""Microbenchmark of the three fused communication paths against their library-collective twins.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29631 \
        -m lbi_b200.benchmarks.time_comm_paths [--params 361968776] [--iters 20]

One process per GPU.  Every figure is CUDA-event time on the launching stream, after warm-up, the maximum over ranks:

1. hand-off     the interface update of one region plus the transfer of its bounded state to the next rank and the wait on
                the receiving side, as a ping-pong between ranks 0 and 1 (per hop).  Peer plane: one kernel whose epilogue stores
                into the peer's mailbox + the receiver's wait kernel.  Twin: the update as separate kernels, NCCL send / recv.
2. scan         Jacobian rows of (K regions, width R, batch B) spread over the ranks by the basis-parallel plan -> state
                cotangents on every rank.  Peer plane: publish by peer stores + local recursion.  Twin: two all-reduces + the
                local scan kernel.
3. optimizer    gradient reduce-scatter, global-norm clip, AdamW on the rank's shard, all-gather of the bf16 weights, for a
                flat buffer of ``--params`` elements.  Peer plane: peer-load reduce kernel, scalar exchange, AdamW kernel that
                stores the new weights into every peer.  Twin: NCCL reduce-scatter, all-reduce of the norm, AdamW kernel, NCCL
                all-gather.  GB/s counts the bytes that cross NVLink per rank: (N - 1) / N of the fp32 gradients in, (N - 1) / N
                of the rank's bf16 shard out N - 1 times; the roofline is those bytes at the measured peer-copy bandwidth.
Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist
from torch import nn

PEER_COPY_GBS = 770.0   # measured peer copy on this class of machine, per direction per GPU (nominal 900)


def _timed(fn, iters: int, warmup: int = 3) -> float:
    """Milliseconds per call, maximum over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(stop) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def bench_handoff(symm, coll, iters: int) -> dict:
    from lbi_b200.interfaces import VectorMLPInterface

    rank = symm.rank
    torch.manual_seed(0)
    iface = VectorMLPInterface(feature_dim=1024, num_regions=2, interface_width=128, interface_map_hidden_dim=1024).cuda()
    bsz = 4
    state = torch.randn(bsz, 128, device="cuda")
    pooled = torch.randn(bsz, 1024, device="cuda")
    symm.prepare(bsz, 128)
    out = {}
    if rank > 1:   # ranks beyond the pair only take part in the barriers of the timing helper
        for _ in range(2):
            _timed(lambda: None, iters)
        return out

    peer = 1 - rank

    def fused_hop():
        # rank 0 sends first, rank 1 receives first: one hop each per call
        with torch.no_grad():
            if rank == 0:
                symm.interface_update_handoff(iface, 0, state, pooled, peer)
                symm.handoff_recv(state, peer)
            else:
                symm.handoff_recv(state, peer)
                symm.interface_update_handoff(iface, 1, state, pooled, peer)

    def library_hop():
        with torch.no_grad():
            if rank == 0:
                step, _ = iface.update_cached(state, pooled, 0)
                coll.handoff_send(step.state, peer)
                coll.handoff_recv(state, peer)
            else:
                coll.handoff_recv(state, peer)
                step, _ = iface.update_cached(state, pooled, 1)
                coll.handoff_send(step.state, peer)

    out["handoff_fused_us_per_hop"] = 1e3 * _timed(fused_hop, iters) / 2
    out["handoff_library_us_per_hop"] = 1e3 * _timed(library_hop, iters) / 2
    return out


def bench_scan(symm, coll, iters: int, k: int, r: int, bsz: int, chunk: int = 16) -> dict:
    from lbi_b200 import ops

    world, rank = symm.world_size, symm.rank
    blocks = [(kk, lo, min(r, lo + chunk)) for kk in range(k - 1) for lo in range(0, r, chunk)]
    quota = -(-len(blocks) // world)
    mine = blocks[rank * quota : (rank + 1) * quota]
    g = torch.Generator(device="cuda").manual_seed(1)
    full = torch.randn(k, bsz, r, r, device="cuda", generator=g) * (0.5 / r ** 0.5)
    offs_full = torch.randn(k, bsz, r, device="cuda", generator=g)
    rows = torch.zeros_like(full)
    for kk, lo, hi in mine:
        rows[kk, :, lo:hi] = full[kk, :, lo:hi]
    own_regions = [kk for kk in range(k) if kk * world // k == rank]
    offs = torch.zeros_like(offs_full)
    for kk in own_regions:
        offs[kk] = offs_full[kk]

    def fused():
        return symm.scan_published(rows, offs, mine, own_regions)[0]

    def library():
        a, b = rows.clone(), offs.clone()
        coll.all_reduce_sum(a)
        coll.all_reduce_sum(b)
        mats = a.permute(1, 0, 3, 2).contiguous()
        o = b.transpose(0, 1).contiguous()
        return ops.affine_suffix_scan(mats[:, : k - 1].contiguous(), o[:, : k - 1].contiguous(), seed=o[:, k - 1].contiguous())[:, :k]

    ga, gb = fused(), library()
    torch.cuda.synchronize()
    err = float((ga - gb).abs().max() / (gb.abs().max() + 1e-9))
    symm.barrier()
    bytes_in = 4.0 * (k - 1) * bsz * r * r * (world - 1) / world    # rows this rank receives from its peers
    t_fused = _timed(lambda: (fused(), symm.barrier()), iters)
    t_lib = _timed(library, iters)
    # the parts of the fused path on their own: the barrier, the publish kernel (peer stores + flags; repeating it rewrites
    # the same values), the recursion over the local, complete copy (its flags are already up)
    ext = ops.ext()
    m_buf, o_buf, m_ptrs, o_ptrs, _, _, seg_cache = symm._scan_bufs[("published", tuple(rows.shape))]
    segs = next(iter(seg_cache.values()))
    w = symm.world_size
    slot = symm.scan_slot_base()
    t_barrier = _timed(symm.barrier, iters)
    t_publish = _timed(lambda: ext.peer_publish(rows, m_ptrs, segs[0], offs, o_ptrs, segs[1], symm.flag_ptrs, rank, w, slot, symm.seq,
                                                symm.done_counter), iters)
    own_m, own_o = m_ptrs[rank : rank + 1], o_ptrs[rank : rank + 1]
    t_rec = _timed(lambda: ext.affine_scan_peer_sum(own_m, own_o, symm.flags, slot, symm.seq, bsz, 1, k, r, w), iters)
    t_local = _timed(lambda: ops.affine_suffix_scan(full.permute(1, 0, 3, 2)[:, : k - 1].contiguous(), offs_full.transpose(0, 1)[:, : k - 1].contiguous(),
                                                    seed=offs_full[k - 1].contiguous()), iters)
    return {f"scan_K{k}_R{r}_B{bsz}": {"fused_us": 1e3 * t_fused, "library_us": 1e3 * t_lib, "max_rel_diff": err,
                                        "parts_us": {"barrier": 1e3 * t_barrier, "publish": 1e3 * t_publish, "recursion": 1e3 * t_rec,
                                                     "local_scan_kernel_with_layout_copies": 1e3 * t_local},
                                        "nvlink_bytes_in_per_rank": bytes_in,
                                        "roofline_us": 1e6 * bytes_in / (PEER_COPY_GBS * 1e9)}}


class _Flat(nn.Module):
    def __init__(self, n: int) -> None:
        super().__init__()
        self.w = nn.Parameter(torch.randn(n, device="cuda") * 0.02)


def bench_optimizer(symm, coll, iters: int, n_params: int) -> dict:
    from lbi_b200 import ops
    from lbi_b200.parallel.flat import FlatParams

    world, rank = symm.world_size, symm.rank
    out = {}
    for name, comm in (("fused", symm), ("library", coll)):
        flat = FlatParams(_Flat(n_params), world_size=world, shadow_dtype=torch.bfloat16)
        if name == "fused":
            comm.attach_flat(flat)
        lo = rank * flat.shard
        flat.ensure_state(lo, lo + flat.shard)
        flat.grads.normal_(0.0, 1e-3)
        sumsq = torch.zeros(1, device="cuda")

        def step():
            if name == "fused":
                comm.optimizer_step(flat, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, grad_clip=1.0)
                return
            g_shard = comm.reduce_scatter_grads(flat.grads, flat.shard)
            flat.step_count += 1
            sumsq.zero_()
            ops.ext().sumsq_(g_shard, sumsq)
            comm.all_reduce_sum(sumsq)
            ops.ext().adamw_step_(flat.params[lo : lo + flat.shard], g_shard, flat.exp_avg, flat.exp_avg_sq, flat.shadow[lo : lo + flat.shard],
                                  1e-4, 0.9, 0.999, 1e-8, 0.01, flat.step_count, 1.0, sumsq, 1.0)
            comm.all_gather_flat(flat.shadow, flat.shard)

        ms = _timed(step, iters)
        frac = (world - 1) / world
        nv_bytes = frac * flat.total * 4 + frac * flat.total * 2          # gradients in (reduce-scatter) + bf16 weights out (all-gather)
        out[name] = {"ms": ms, "nvlink_gb_per_rank": nv_bytes / 1e9, "gbs": nv_bytes / 1e9 / (ms / 1e3),
                     "roofline_ms": 1e3 * max(frac * flat.total * 4, frac * flat.total * 2) / (PEER_COPY_GBS * 1e9)}
        del flat
        torch.cuda.empty_cache()
    return {"optimizer": {"params": n_params, **out}}


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--params", type=int, default=361968776)
    p.add_argument("--iters", type=int, default=20)
    args = p.parse_args()
    from lbi_b200.parallel import CollectiveComm, init_distributed_from_env
    from lbi_b200.parallel.symm import SymmComm

    rank, local_rank, world = init_distributed_from_env("cuda")
    if world < 2:
        raise SystemExit("run under torch.distributed.run with at least two processes")
    torch.cuda.set_device(local_rank)
    symm, coll = SymmComm(), CollectiveComm()
    result = {"n_gpus": world, "nvls": os.environ.get("NCCL_NVLS_ENABLE", "default"), "peer_copy_gbs_reference": PEER_COPY_GBS}
    result.update(bench_handoff(symm, coll, args.iters))
    result.update(bench_scan(symm, coll, args.iters, 8, 128, 4))
    result.update(bench_scan(symm, coll, args.iters, 32, 256, 2, chunk=64))
    result.update(bench_optimizer(symm, coll, max(5, args.iters // 2), args.params))
    from lbi_b200 import ops

    result["kernel_status"] = int(ops.ext().kernel_status(torch.zeros(1, device="cuda")))
    if rank == 0:
        print(json.dumps(result))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
