"""Two-rank runs on real GPUs: the peer-memory plane (fused hand-off, cross-GPU scan, fused reduce-scatter + AdamW +
weight all-gather) must reproduce the library-collective plane and the single-GPU engine.  Child processes, one per
GPU; skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model(axis):
    from lbi_b200.backbones import BackboneSpec
    from lbi_b200.interfaces import VectorMLPInterface
    from lbi_b200.models import LBILanguageModel

    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=256, layers=4, n_heads=4, d_conv=0, d_intermediate=512)
    iface = VectorMLPInterface(feature_dim=256, num_regions=4, interface_width=16, interface_map_hidden_dim=64)
    return LBILanguageModel(vocab_size=1024, layers_per_region=1, backbone_spec=spec, interface=iface, region_axis=axis,
                            num_sequence_regions=4, tie_embeddings=True)


def _batch():
    g = torch.Generator().manual_seed(3)
    return torch.randint(0, 1024, (2, 1024), generator=g), torch.randint(0, 1024, (2, 1024), generator=g)


def _worker(rank, world, port, axis, plane, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    import datetime

    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    try:
        from lbi_b200 import ops
        from lbi_b200.parallel import CollectiveComm, FastLBIEngine
        from lbi_b200.parallel.symm import SymmComm

        comm = SymmComm() if plane == "symm" else CollectiveComm()
        model = _model(axis).cuda()
        engine = FastLBIEngine(model, lr=1e-3, grad_clip=1.0, basis_chunk=8, comm=comm)
        ids, tgt = _batch()
        losses = [engine.step(ids.cuda(), tgt.cuda()) for _ in range(2)]
        torch.cuda.synchronize()
        status = ops.ext().kernel_status(losses[0])
        canaries = comm.check_canaries() if plane == "symm" else []
        if rank == 0:
            torch.save({"params": engine.flat.shadow.float().cpu(), "losses": [float(x) for x in losses], "status": int(status),
                        "canaries": canaries},
                       os.path.join(out_dir, f"{plane}.pt"))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("axis", ["sequence", "depth"])
def test_peer_memory_plane_matches_collectives(tmp_path, axis):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    for plane in ("collective", "symm"):
        mp.spawn(_worker, args=(2, _free_port(), axis, plane, str(tmp_path)), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "collective.pt"), torch.load(tmp_path / "symm.pt")
    assert b["status"] == 0, "a bounded wait in a peer-memory kernel ran out"
    assert b["canaries"] == [], f"a peer store ran past the end of symmetric buffer(s) {b['canaries']}"
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 2e-2 * max(1.0, abs(x))
    n = min(a["params"].numel(), b["params"].numel())
    diff = (a["params"][:n] - b["params"][:n]).abs().max().item()
    assert diff < 5e-2, f"weights after two steps differ by {diff}"
