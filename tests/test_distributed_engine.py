"""Region-parallel engine over several ranks (gloo on CPU): gradients and the optimizer step must equal the
single-process run, for both region axes."""
import copy
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lbi_b200.backbones import BackboneSpec
from lbi_b200.interfaces import VectorMLPInterface
from lbi_b200.models import LBILanguageModel


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model(axis, regions):
    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=32, layers=4, n_heads=4, d_conv=0)
    iface = VectorMLPInterface(feature_dim=32, num_regions=regions, interface_width=8, interface_map_hidden_dim=16)
    return LBILanguageModel(vocab_size=64, layers_per_region=4 // regions if axis == "depth" else 1, backbone_spec=spec,
                            interface=iface, region_axis=axis, num_sequence_regions=regions, tie_embeddings=True)


def _worker(rank, world, port, axis, regions, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lbi_b200.parallel import CollectiveComm, FastLBIEngine

        torch.set_num_threads(1)
        model = _model(axis, regions)
        engine = FastLBIEngine(model, lr=1e-2, grad_clip=1.0, basis_chunk=3, comm=CollectiveComm())
        g = torch.Generator().manual_seed(5)
        ids, tgt = torch.randint(0, 64, (2, 32), generator=g), torch.randint(0, 64, (2, 32), generator=g)
        res = engine.backward(ids, tgt)
        grads = engine.flat.grads.clone()
        dist.all_reduce(grads)
        loss = res.loss.clone()
        dist.all_reduce(loss)
        engine._optimizer_step(1e-2)
        if rank == 0:
            torch.save({"grads": grads, "loss": loss, "params": engine.flat.params.clone(), "g": res.state_cotangents},
                       os.path.join(out_dir, "dist.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("axis,regions,world", [("sequence", 4, 2), ("depth", 4, 4), ("sequence", 4, 4)])
def test_multi_rank_engine_matches_single_process(tmp_path, axis, regions, world):
    from lbi_b200.parallel import FastLBIEngine

    port = _free_port()
    mp.spawn(_worker, args=(world, port, axis, regions, str(tmp_path)), nprocs=world, join=True)
    got = torch.load(tmp_path / "dist.pt")
    model = _model(axis, regions)
    engine = FastLBIEngine(copy.deepcopy(model), lr=1e-2, grad_clip=1.0, basis_chunk=3)
    g = torch.Generator().manual_seed(5)
    ids, tgt = torch.randint(0, 64, (2, 32), generator=g), torch.randint(0, 64, (2, 32), generator=g)
    res = engine.backward(ids, tgt)
    n = min(engine.flat.total, got["grads"].numel())
    assert torch.allclose(got["loss"], res.loss, atol=1e-6)
    assert torch.allclose(got["g"], res.state_cotangents, atol=1e-6)
    assert torch.allclose(got["grads"][:n], engine.flat.grads[:n], atol=1e-6, rtol=1e-5)
    engine._optimizer_step(1e-2)
    assert torch.allclose(got["params"][:n], engine.flat.params[:n], atol=1e-5, rtol=1e-5)


def _train_worker(rank, world, port, out_dir, overrides=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from lbi_b200.train.lbi import run_lbi_experiment

    torch.set_num_threads(1)
    try:
        run_lbi_experiment(_train_cfg(out_dir, **(overrides or {})))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _train_cfg(out_dir, **kw):
    from lbi_b200.train.config import LBITrainingConfig

    base = dict(variants="lbi", backbone="transformer", device="cpu", dtype="float32", output_dir=str(out_dir), run_name="run",
                task="copy", vocab_size=32, seq_len=32, train_sequences=32, val_sequences=8, batch_size=2, steps=3, eval_every=3,
                eval_batches=1, log_every=1, save_every=3, layers=2, dim=16, n_heads=2, d_conv=0, region_axis="sequence",
                sequence_regions=4, region_size=2, message_dim=4, message_hidden_dim=8, backward_engine="fast", jacobian_basis_chunk=2)
    base.update(kw)
    return LBITrainingConfig(**base)


def test_training_program_on_two_ranks_matches_one_process(tmp_path, monkeypatch):
    """The training CLI path under a torchrun-style environment: rank 0 writes the run, the checkpoint holds the
    consolidated optimizer state, and losses / weights equal the single-process run."""
    import json

    from lbi_b200.train.lbi import run_lbi_experiment

    for key in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(key, raising=False)
    mp.spawn(_train_worker, args=(2, _free_port(), str(tmp_path / "dist")), nprocs=2, join=True)
    single = run_lbi_experiment(_train_cfg(tmp_path / "single"))
    rows = {}
    for tag in ("dist", "single"):
        path = tmp_path / tag / "run" / "lbi" / "metrics.jsonl"
        rows[tag] = [json.loads(line) for line in path.read_text().splitlines()]
    assert [r["split"] for r in rows["dist"]] == [r["split"] for r in rows["single"]]
    for a, b in zip(rows["dist"], rows["single"]):
        assert a["ce_loss"] == pytest.approx(b["ce_loss"], rel=1e-5, abs=1e-6), (a, b)
    ck_d = torch.load(tmp_path / "dist" / "run" / "lbi" / "checkpoints" / "latest.pt", weights_only=False)
    ck_s = torch.load(tmp_path / "single" / "run" / "lbi" / "checkpoints" / "latest.pt", weights_only=False)
    for name, w in ck_s["model_state_dict"].items():
        assert torch.allclose(ck_d["model_state_dict"][name], w, atol=1e-5, rtol=1e-5), name
    for idx, st in ck_s["optimizer_state_dict"]["state"].items():
        for key in ("exp_avg", "exp_avg_sq"):
            assert torch.allclose(ck_d["optimizer_state_dict"]["state"][idx][key], st[key], atol=1e-6, rtol=1e-4), (idx, key)
    # a single process resumes from the checkpoint the two ranks wrote
    resumed = run_lbi_experiment(_train_cfg(tmp_path / "dist", steps=4, resume_from=str(tmp_path / "dist" / "run")))
    assert resumed["runs"][0]["start_step"] == 3


@pytest.mark.parametrize("overrides", [
    dict(backbone="mamba3", d_state=16, headdim=16, chunk_size=16),
    dict(backbone="hybrid", layer_types="mamba2,transformer", d_state=16, headdim=16, chunk_size=16, d_conv=4, region_axis="depth",
         region_size=1),
])
def test_training_program_on_two_ranks_with_mamba_backbones(tmp_path, monkeypatch, overrides):
    """The same program on the Mamba-3 and hybrid stacks: the two-rank run logs the losses of the one-process run."""
    import json

    from lbi_b200.train.lbi import run_lbi_experiment

    for key in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(key, raising=False)
    mp.spawn(_train_worker, args=(2, _free_port(), str(tmp_path / "dist"), overrides), nprocs=2, join=True)
    run_lbi_experiment(_train_cfg(tmp_path / "single", **overrides))
    rows = {tag: [json.loads(line) for line in (tmp_path / tag / "run" / "lbi" / "metrics.jsonl").read_text().splitlines()]
            for tag in ("dist", "single")}
    assert len(rows["dist"]) == len(rows["single"]) >= 4
    for a, b in zip(rows["dist"], rows["single"]):
        assert a["split"] == b["split"] and a["ce_loss"] == pytest.approx(b["ce_loss"], rel=1e-4, abs=1e-5), (a, b)


def test_basis_plan_is_balanced_and_complete():
    """Every (region, block) of basis directions is assigned exactly once and no rank gets more than its share."""
    from types import SimpleNamespace

    from lbi_b200.models.region_plan import RegionPlacement
    from lbi_b200.parallel import FastLBIEngine

    for k_regions, width, chunk, world in [(8, 128, 16, 8), (8, 128, 16, 2), (8, 128, 16, 4), (4, 8, 3, 2), (4, 8, 3, 4), (2, 16, 16, 2)]:
        fake = SimpleNamespace(model=SimpleNamespace(num_regions=k_regions, interface_width=width), basis_chunk=chunk,
                               comm=SimpleNamespace(world_size=world), placement=RegionPlacement(k_regions, world))
        plan = FastLBIEngine.basis_plan(fake)
        blocks = [b for per_rank in plan for b in per_rank]
        want = [(k, lo, min(width, lo + chunk)) for k in range(k_regions - 1) for lo in range(0, width, chunk)]
        assert sorted(blocks) == sorted(want)
        quota = -(-len(want) // world)
        assert max(len(p) for p in plan) <= quota
    # 8 regions on 8 ranks: 56 blocks, 7 each; no rank touches more than two regions, so at most one foreign forward each
    fake = SimpleNamespace(model=SimpleNamespace(num_regions=8, interface_width=128), basis_chunk=16,
                           comm=SimpleNamespace(world_size=8), placement=RegionPlacement(8, 8))
    plan = FastLBIEngine.basis_plan(fake)
    assert [len(p) for p in plan] == [7] * 8
    assert all(len({k for k, _, _ in per_rank}) <= 2 for per_rank in plan) and {k for k, _, _ in plan[7]} == {6}


def _bf16_worker(rank, world, port, out_dir, steps):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lbi_b200.parallel import CollectiveComm, FastLBIEngine

        torch.set_num_threads(1)
        engine = FastLBIEngine(_model("sequence", 4), lr=3e-2, grad_clip=1.0, basis_chunk=3, comm=CollectiveComm(),
                               act_dtype=torch.bfloat16)
        g = torch.Generator().manual_seed(5)
        ids, tgt = torch.randint(0, 64, (2, 32), generator=g), torch.randint(0, 64, (2, 32), generator=g)
        losses = [float(engine.step(ids, tgt)) for _ in range(steps)]
        torch.save({"losses": losses, "params": engine.flat.params.clone(), "shadow": engine.flat.shadow.clone()},
                   os.path.join(out_dir, f"bf16_rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_low_precision_shadow_run_keeps_every_rank_on_current_weights(tmp_path):
    """With a bf16 shadow a rank's optimizer updates the fp32 master of its own shard only.  The parameters the engine
    reads in fp32 (interface maps, norm weights) must still be current and identical on every rank after each step:
    losses and fp32-read weights of a 2-rank run equal the single-process run over several steps."""
    from lbi_b200.parallel import FastLBIEngine

    steps = 4
    mp.spawn(_bf16_worker, args=(2, _free_port(), str(tmp_path), steps), nprocs=2, join=True)
    ranks = [torch.load(tmp_path / f"bf16_rank{r}.pt") for r in range(2)]
    engine = FastLBIEngine(_model("sequence", 4), lr=3e-2, grad_clip=1.0, basis_chunk=3, act_dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    ids, tgt = torch.randint(0, 64, (2, 32), generator=g), torch.randint(0, 64, (2, 32), generator=g)
    single = [float(engine.step(ids, tgt)) for _ in range(steps)]
    for r in range(2):
        for a, b in zip(ranks[r]["losses"], single):
            assert a == pytest.approx(b, rel=2e-3, abs=2e-3), (r, ranks[r]["losses"], single)
    # both ranks hold the same fp32 values for every parameter the engine reads from the master copy
    flat = engine.flat
    for name, slot in flat.slots.items():
        if len(slot.shape) == 2 and not name.startswith("interface."):
            continue
        a = ranks[0]["params"][slot.offset : slot.offset + slot.numel]
        b = ranks[1]["params"][slot.offset : slot.offset + slot.numel]
        ref = flat.params[slot.offset : slot.offset + slot.numel]
        assert torch.equal(a, b), f"{name}: ranks disagree on an fp32-read parameter"
        assert torch.allclose(a, ref, atol=2e-3, rtol=2e-2), f"{name}: drifted from the single-process run"
    assert torch.equal(ranks[0]["shadow"], ranks[1]["shadow"])
