"""Closed-form Mamba-3 / Mamba-2 / hybrid region lowering: the autograd-free engine must give the gradients of dense
autograd on the same LBI model (the reference's parity bar: per-parameter allclose(atol=1e-5, rtol=1e-4) in fp32,
tests/test_lbi_gradient_parity.py:40-44 there), on one process and on two gloo ranks."""
import copy
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from lbi_b200.backbones import BackboneSpec
from lbi_b200.interfaces import VectorMLPInterface
from lbi_b200.models import LBILanguageModel
from lbi_b200.parallel import FastLBIEngine

VOCAB = 50


def _model(kind: str, axis: str = "sequence", regions: int = 3, layers: int = 2):
    torch.manual_seed(0)
    kw = dict(dim=32, layers=layers, d_state=16, headdim=8, expand=2, d_conv=4, chunk_size=8, ngroups=1)
    if kind == "hybrid":
        spec = BackboneSpec(name="hybrid", layer_types=("mamba3", "transformer", "mamba2")[:layers], n_heads=4, **kw)
    else:
        spec = BackboneSpec(name=kind, **kw)
    iface = VectorMLPInterface(feature_dim=32, num_regions=regions, interface_width=6, interface_map_hidden_dim=16)
    return LBILanguageModel(vocab_size=VOCAB, layers_per_region=max(1, layers // regions) if axis == "depth" else 1, backbone_spec=spec,
                            interface=iface, tie_embeddings=True, region_axis=axis, num_sequence_regions=regions)


def _batch(seq=24):
    g = torch.Generator().manual_seed(3)
    return torch.randint(0, VOCAB, (2, seq), generator=g), torch.randint(0, VOCAB, (2, seq), generator=g)


def _dense_grads(model, ids, tgt):
    ref = copy.deepcopy(model)
    logits, _ = ref.forward_with_cache(ids)
    loss = F.cross_entropy(logits.float().reshape(-1, VOCAB), tgt.reshape(-1))
    loss.backward()
    return loss.detach(), {n: p.grad for n, p in ref.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("kind,axis,layers,regions", [("mamba3", "sequence", 2, 3), ("mamba2", "sequence", 2, 3),
                                                      ("hybrid", "sequence", 3, 2), ("mamba3", "depth", 2, 2),
                                                      ("mamba2", "depth", 2, 2)])
def test_fast_engine_matches_dense_autograd(kind, axis, layers, regions):
    model = _model(kind, axis, regions, layers)
    ids, tgt = _batch()
    loss, want = _dense_grads(model, ids, tgt)
    engine = FastLBIEngine(model, lr=1e-3, basis_chunk=4)
    res = engine.backward(ids, tgt)
    assert torch.allclose(res.loss, loss, atol=1e-6, rtol=1e-6)
    assert set(want) <= set(engine.flat.slots)
    for name, g in want.items():
        assert torch.allclose(engine.flat.grad(name), g, atol=1e-5, rtol=1e-4), name


def test_pullback_of_stacked_directions_equals_one_direction_at_a_time():
    """P directions in one pass share the cached forward: the result must equal P single passes."""
    model = _model("mamba3")
    structured = model.region_backend.structured
    x = torch.randn(2, 16, 32)
    _, cache = structured.forward(x, (0, 2))
    cots = torch.randn(3, 2 * 16, 32)
    stacked = structured.input_pullback(cache, cots.reshape(3 * 32, 32)).view(3, 32, 32)
    for p in range(3):
        single = structured.input_pullback(cache, cots[p])
        assert torch.allclose(stacked[p], single, atol=1e-6, rtol=1e-5)


def test_output_norm_variant_of_mamba3_mixer():
    """``is_outproj_norm`` (grouped RMSNorm before the gate instead of the plain gate) through the structured chain."""
    from lbi_b200.backbones.mamba3.mixer import Mamba3

    model = _model("mamba3")
    for block in model.region_backend.backbone.blocks:
        old = block.mixer
        torch.manual_seed(1)
        block.mixer = Mamba3(d_model=32, d_state=16, expand=2, headdim=8, ngroups=1, chunk_size=8, is_outproj_norm=True)
        del old
    model.region_backend._structured = None
    ids, tgt = _batch()
    loss, want = _dense_grads(model, ids, tgt)
    engine = FastLBIEngine(model, lr=1e-3, basis_chunk=4)
    res = engine.backward(ids, tgt)
    assert torch.allclose(res.loss, loss, atol=1e-6, rtol=1e-6)
    for name, g in want.items():
        assert torch.allclose(engine.flat.grad(name), g, atol=1e-5, rtol=1e-4), name


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, kind, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lbi_b200.parallel import CollectiveComm

        torch.set_num_threads(1)
        engine = FastLBIEngine(_model(kind, regions=4), lr=1e-2, grad_clip=1.0, basis_chunk=3, comm=CollectiveComm())
        ids, tgt = _batch(32)
        res = engine.backward(ids, tgt)
        grads = engine.flat.grads.clone()
        dist.all_reduce(grads)
        loss = res.loss.clone()
        dist.all_reduce(loss)
        if rank == 0:
            torch.save({"grads": grads, "loss": loss}, os.path.join(out_dir, "dist.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["mamba3", "mamba2"])
def test_two_ranks_with_basis_parallel_pullback_match_one_process(tmp_path, kind):
    mp.spawn(_worker, args=(2, _free_port(), kind, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    engine = FastLBIEngine(_model(kind, regions=4), lr=1e-2, grad_clip=1.0, basis_chunk=3)
    ids, tgt = _batch(32)
    res = engine.backward(ids, tgt)
    n = min(engine.flat.total, got["grads"].numel())
    assert torch.allclose(got["loss"], res.loss, atol=1e-6)
    assert torch.allclose(got["grads"][:n], engine.flat.grads[:n], atol=1e-6, rtol=1e-5)


def test_activation_recomputation_gives_the_same_gradients():
    """Dropping every region's cached activations after its forward and rebuilding them before the pullback and the local
    VJP must not change anything."""
    model = _model("mamba2", regions=4)
    ids, tgt = _batch(32)
    a = FastLBIEngine(copy.deepcopy(model), lr=1e-3, basis_chunk=4)
    b = FastLBIEngine(copy.deepcopy(model), lr=1e-3, basis_chunk=4, recompute_forward=True)
    ra, rb = a.backward(ids, tgt), b.backward(ids, tgt)
    assert torch.equal(ra.loss, rb.loss)
    assert torch.allclose(a.flat.grads, b.flat.grads, atol=1e-7, rtol=1e-6)
    with pytest.raises(ValueError):
        FastLBIEngine(_model("mamba2", axis="depth", regions=2), recompute_forward=True)


@pytest.mark.parametrize("kind", ["transformer", "mamba3"])
def test_dense_fast_engine_matches_autograd(kind):
    """The dense (no regions) step on the closed-form chain against loss.backward() of the same dense model."""
    from lbi_b200.models import DenseLanguageModel
    from lbi_b200.parallel import DenseFastEngine

    torch.manual_seed(0)
    kw = dict(dim=32, layers=2, d_state=16, headdim=8, expand=2, chunk_size=8, ngroups=1)
    spec = BackboneSpec(name=kind, n_heads=4, d_conv=0 if kind == "transformer" else 4, **kw)
    model = DenseLanguageModel(vocab_size=VOCAB, backbone_spec=spec, tie_embeddings=True)
    ids, tgt = _batch()
    ref = copy.deepcopy(model)
    loss = F.cross_entropy(ref(ids).float().reshape(-1, VOCAB), tgt.reshape(-1))
    loss.backward()
    engine = DenseFastEngine(model, lr=1e-3)
    got = engine.backward(ids, tgt)
    assert torch.allclose(got, loss.detach(), atol=1e-6, rtol=1e-6)
    for name, p in ref.named_parameters():
        if p.grad is not None and name in engine.flat.slots:
            assert torch.allclose(engine.flat.grad(name), p.grad, atol=1e-5, rtol=1e-4), name
    before = engine.flat.params.clone()
    engine.step(ids, tgt)
    assert not torch.equal(before, engine.flat.params)
