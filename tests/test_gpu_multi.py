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


def _worker(rank, world, port, axis, plane, out_dir, act_dtype=None, steps=2):
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
        engine = FastLBIEngine(model, lr=1e-3, grad_clip=1.0, basis_chunk=8, comm=comm, act_dtype=act_dtype)
        ids, tgt = _batch()
        losses = [engine.step(ids.cuda(), tgt.cuda()) for _ in range(steps)]
        torch.cuda.synchronize()
        status = ops.ext().kernel_status(losses[0])
        canaries = comm.check_canaries() if plane == "symm" else []
        if rank == 0:
            weights = engine.flat.shadow if engine.flat.shadow is not None else engine.flat.params
            torch.save({"params": weights.float().cpu(), "master": engine.flat.params.cpu(), "losses": [float(x) for x in losses], "status": int(status),
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


@pytest.mark.parametrize("plane", ["collective", "symm"])
def test_two_ranks_track_the_single_gpu_engine_over_several_steps(tmp_path, plane):
    """bf16 shadow, four optimizer steps at a large learning rate: a rank that kept reading stale fp32 interface or norm
    weights of the other rank's shard would drift away from the single-GPU run within a few steps."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from lbi_b200.parallel import FastLBIEngine

    steps = 4
    mp.spawn(_worker, args=(2, _free_port(), "sequence", plane, str(tmp_path), None, steps), nprocs=2, join=True)
    got = torch.load(tmp_path / f"{plane}.pt")
    engine = FastLBIEngine(_model("sequence").cuda(), lr=1e-3, grad_clip=1.0, basis_chunk=8)
    ids, tgt = _batch()
    single = [float(engine.step(ids.cuda(), tgt.cuda())) for _ in range(steps)]
    assert got["status"] == 0
    for a, b in zip(got["losses"], single):
        assert abs(a - b) < 5e-3 * max(1.0, abs(b)), (got["losses"], single)
    flat = engine.flat
    for name, slot in flat.slots.items():
        if len(slot.shape) == 2 and not name.startswith("interface."):
            continue
        a = got["master"][slot.offset : slot.offset + slot.numel]
        b = flat.params[slot.offset : slot.offset + slot.numel].cpu()
        assert torch.allclose(a, b, atol=2e-3, rtol=2e-2), f"{name}: fp32-read parameter drifted from the single-GPU run"


def test_peer_memory_plane_trains_with_fp32_activations(tmp_path):
    """No low-precision shadow (float32 is the training config's default dtype): the peer plane still hands states off and
    scans through peer memory, and takes the library-collective optimizer step, which gathers the fp32 weights."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    for plane in ("collective", "symm"):
        mp.spawn(_worker, args=(2, _free_port(), "sequence", plane, str(tmp_path), torch.float32, 2), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "collective.pt"), torch.load(tmp_path / "symm.pt")
    assert b["status"] == 0 and b["canaries"] == []
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 1e-3 * max(1.0, abs(x))
    n = min(a["params"].numel(), b["params"].numel())
    assert (a["params"][:n] - b["params"][:n]).abs().max().item() < 1e-3
