"""Exact-gradient parity: every scan-based engine against ``loss.backward()`` on the same LBI model.

fp32 on the CPU with the reference's tolerances (per-parameter allclose atol 1e-5 / rtol 1e-4, loss atol 1e-7,
interface_scan_rms < 1e-5), for all backbones, both region axes and all Jacobian providers."""
import copy

import pytest
import torch
import torch.nn.functional as F

from lbi_b200.backbones import BackboneSpec
from lbi_b200.backward import AutogradEngine, ReferenceScanEngine, ScanADEngine
from lbi_b200.interfaces import VectorMLPInterface
from lbi_b200.models import LBILanguageModel
from lbi_b200.parallel import FastLBIEngine

VOCAB = 64


def build(backbone="transformer", axis="depth", regions=2, tie=False, layers=4, activation="silu", layer_types=()):
    torch.manual_seed(0)
    spec = BackboneSpec(name=backbone, dim=32, layers=layers, n_heads=4, n_kv_heads=2, d_conv=4, d_state=16, headdim=16,
                        chunk_size=8, layer_types=layer_types)
    k = regions
    iface = VectorMLPInterface(feature_dim=32, num_regions=k, interface_width=8, interface_map_hidden_dim=16, activation=activation)
    return LBILanguageModel(vocab_size=VOCAB, layers_per_region=max(1, layers // k), backbone_spec=spec, interface=iface,
                            region_axis=axis, num_sequence_regions=k, tie_embeddings=tie)


def batch(seed=1, b=2, t=32):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, VOCAB, (b, t), generator=g), torch.randint(0, VOCAB, (b, t), generator=g)


def run(model, engine, ids, tgt, detach):
    logits, cache = model.forward_with_cache(ids, detach_states=detach)
    loss = F.cross_entropy(logits.float().reshape(-1, VOCAB), tgt.reshape(-1))
    return loss.detach(), engine.backward(model=model, loss=loss, cache=cache)


def assert_parity(ref, got, atol=1e-5, rtol=1e-4):
    assert set(ref) == set(got)
    for name, r in ref.items():
        g = got[name]
        assert (r is None) == (g is None), f"{name}: None mismatch"
        if r is not None:
            assert torch.allclose(g, r, atol=atol, rtol=rtol), f"{name}: max err {(g - r).abs().max().item():.3e}"


CASES = [
    ("transformer", "depth", 1), ("transformer", "depth", 2), ("transformer", "depth", 4), ("transformer", "sequence", 4),
    ("mamba2", "depth", 2), ("mamba2", "sequence", 2), ("mamba3", "depth", 2), ("mamba3", "sequence", 4), ("hybrid", "depth", 2),
]


@pytest.mark.parametrize("backbone,axis,regions", CASES)
@pytest.mark.parametrize("mode", ["graph", "recompute", "structured"])
def test_scan_engine_matches_autograd(backbone, axis, regions, mode):
    lt = ("mamba3", "transformer", "mamba2", "transformer") if backbone == "hybrid" else ()
    model = build(backbone, axis, regions, layer_types=lt)
    ids, tgt = batch()
    loss_ref, ref = run(model, AutogradEngine(), ids, tgt, False)
    loss, res = run(model, ScanADEngine(state_jacobian_mode=mode, state_jacobian_basis_chunk=3), ids, tgt, True)
    assert torch.allclose(loss, loss_ref, atol=1e-7, rtol=1e-6)
    assert_parity(ref.grad_map, res.grad_map)
    assert res.diagnostics["interface_scan_rms"] < 1e-5
    for p, (name, g) in zip(model.parameters(), res.grad_map.items()):
        assert (p.grad is None) == (g is None)


def test_forward_mode_provider_and_gelu_interface():
    model = build("transformer", "sequence", 2, activation="gelu")
    ids, tgt = batch()
    _, ref = run(model, AutogradEngine(), ids, tgt, False)
    _, res = run(model, ScanADEngine(state_jacobian_mode="forward"), ids, tgt, True)
    assert_parity(ref.grad_map, res.grad_map)


@pytest.mark.parametrize("axis,regions", [("depth", 2), ("sequence", 4)])
@pytest.mark.parametrize("detach", [True, False])
def test_reference_scan_engine(axis, regions, detach):
    if axis == "sequence" and not detach:
        pytest.skip("sequence-axis regions need region-local graphs")
    model = build("transformer", axis, regions)
    ids, tgt = batch()
    _, ref = run(model, AutogradEngine(), ids, tgt, False)
    _, res = run(model, ReferenceScanEngine(), ids, tgt, detach)
    assert_parity(ref.grad_map, res.grad_map)


def test_connected_graph_scan_follows_reference_hooks():
    model = build("transformer", "depth", 4)
    ids, tgt = batch()
    _, ref = run(model, AutogradEngine(), ids, tgt, False)
    _, res = run(model, ScanADEngine(state_jacobian_mode="graph"), ids, tgt, False)
    assert_parity(ref.grad_map, res.grad_map)
    none_names = sorted(n for n, g in res.grad_map.items() if g is None)
    assert none_names and all(n.startswith(("interface.encoders.3", "interface.norms.3")) for n in none_names)


class _ForeignLocalVJP:
    """A provider written against the reference's hook names only (backward/local_vjp.py:10-62)."""

    name = "foreign"

    def __init__(self):
        self.calls = []

    def _store(self, model, grad_map, params, grads):
        names = {id(p): n for n, p in model.named_parameters()}
        for p, g in zip(params, grads):
            if g is not None:
                n = names[id(p)]
                grad_map[n] = g if grad_map[n] is None else grad_map[n] + g

    def new_grad_map(self, model):
        self.calls.append("new")
        return {n: None for n, p in model.named_parameters() if p.requires_grad}

    def store_output_head_grads(self, *, model, loss, grad_map):
        self.calls.append("head")
        params = model.output_head_vjp_parameters()
        self._store(model, grad_map, params, torch.autograd.grad(loss, params, retain_graph=True, allow_unused=True))

    def state_adjoint_from_loss(self, *, loss, state):
        return torch.autograd.grad(loss, state, retain_graph=True)[0]

    def store_initial_interface_grads(self, *, model, state0, state0_adjoint, grad_map):
        self.calls.append("initial")
        params = model.interface.initial_vjp_parameters()
        self._store(model, grad_map, params, torch.autograd.grad(state0, params, state0_adjoint, retain_graph=True, allow_unused=True))

    def store_region_grads(self, *, model, loss, states, region_index, num_regions, state_adjoints, grad_map):
        self.calls.append(f"region{region_index}")
        params = [*model.region_backend.parameters_for_region(region_index), *model.interface.region_vjp_parameters(region_index)]
        if region_index < num_regions - 1:
            grads = torch.autograd.grad(states[region_index + 1], params, state_adjoints[region_index + 1], retain_graph=True,
                                        allow_unused=True)
        else:
            grads = torch.autograd.grad(loss, params, retain_graph=True, allow_unused=True)
        self._store(model, grad_map, params, grads)

    def store_shared_canvas_grads(self, *, model, loss, grad_map):
        self.calls.append("shared")
        params = model.shared_local_vjp_parameters()
        self._store(model, grad_map, params, torch.autograd.grad(loss, params, allow_unused=True))


class _ForeignPullback:
    """No ``regions`` keyword, as in the reference's protocol (backward/pullbacks.py:9-18)."""

    name = "foreign_graph"

    def materialize_state_jacobian_t(self, *, model, cache):
        from lbi_b200.backward.pullbacks import materialize_interface_state_jacobian_t_graph

        return materialize_interface_state_jacobian_t_graph(model=model, cache=cache)


def test_scan_step_with_providers_and_keywords_of_the_reference():
    from lbi_b200.backward import TorchAutogradLocalVJPProvider, autograd_backward_step, lbi_scan_backward_step
    from lbi_b200.backward.reference_scan import lbi_reference_scan_backward_step

    model = build("transformer", "depth", 4)
    ids, tgt = batch()

    def fresh():
        logits, cache = model.forward_with_cache(ids)
        return F.cross_entropy(logits.float().reshape(-1, VOCAB), tgt.reshape(-1)), cache

    loss, _ = fresh()
    ref = autograd_backward_step(model, ce_loss=loss)
    loss, cache = fresh()
    foreign = _ForeignLocalVJP()
    got = lbi_scan_backward_step(model, ce_loss=loss, cache=cache, pullback_provider=_ForeignPullback(), local_vjp_provider=foreign)
    assert_parity(ref, got.grad_map)
    assert foreign.calls == ["new", "head", "initial", "region0", "region1", "region2", "region3", "shared"]

    # the engine wrapper: a caller's provider makes it ask for the connected graph and is driven hook by hook
    engine = ScanADEngine(state_jacobian_mode="graph", pullback_provider=_ForeignPullback(), local_vjp_provider=_ForeignLocalVJP())
    assert engine.requires_detached_states is False and ScanADEngine().requires_detached_states is True
    _, via_engine = run(model, engine, ids, tgt, engine.requires_detached_states)
    assert_parity(ref, via_engine.grad_map)
    assert engine.local_vjp_provider.calls[0] == "new" and engine.local_vjp_provider.calls[-1] == "shared"
    assert (via_engine.diagnostics["interface_pullback_provider"], via_engine.diagnostics["local_vjp_provider"]) == ("foreign_graph", "foreign")

    # this package's provider through the reference's hook names
    loss, cache = fresh()
    own = TorchAutogradLocalVJPProvider()
    gm = own.new_grad_map(model)
    own.store_output_head_grads(model=model, loss=loss, grad_map=gm)
    states = cache["states"]
    adj = [None] * 5
    adj[3] = own.state_adjoint_from_loss(loss=loss, state=states[3])
    for k in (2, 1, 0):
        (adj[k],) = torch.autograd.grad(states[k + 1], states[k], adj[k + 1], retain_graph=True)
    own.store_initial_interface_grads(model=model, state0=states[0], state0_adjoint=adj[0], grad_map=gm)
    for k in range(4):
        own.store_region_grads(model=model, loss=loss, states=states, region_index=k, num_regions=4, state_adjoints=adj, grad_map=gm)
    own.store_shared_canvas_grads(model=model, loss=loss, grad_map=gm)
    assert_parity(ref, gm)

    for mode in ("graph", "recompute"):
        loss, cache = fresh()
        res = lbi_reference_scan_backward_step(model, ce_loss=loss, cache=cache, state_jacobian_mode=mode,
                                               state_jacobian_basis_chunk=3, compute_interface_jacobian_stats=True,
                                               include_interface_jacobian_suffix=True)
        assert_parity(ref, res.grad_map)
        assert res.interface_jacobian_stats


@pytest.mark.parametrize("axis,regions,tie", [("depth", 2, False), ("depth", 4, True), ("sequence", 4, True), ("sequence", 8, False)])
def test_fast_engine_matches_autograd(axis, regions, tie):
    model = build("transformer", axis, regions, tie=tie, layers=4 if regions <= 4 else 8)
    twin = copy.deepcopy(model)
    ids, tgt = batch(t=64)
    loss_ref, ref = run(twin, AutogradEngine(), ids, tgt, False)
    engine = FastLBIEngine(model, basis_chunk=3)
    res = engine.backward(ids, tgt)
    assert torch.allclose(res.loss, loss_ref, atol=1e-6, rtol=1e-6)
    got = engine.named_grads()
    for name, r in ref.grad_map.items():
        if r is None:
            assert float(got[name].abs().max()) == 0.0
        else:
            assert torch.allclose(got[name], r, atol=1e-5, rtol=1e-4), f"{name}: {(got[name] - r).abs().max().item():.3e}"


def test_tiny_config_one_of_baseline():
    """Vocab 512, seq 1024 in 8 regions of 128, d_model 128, 2 layers, 4 heads, GELU interface 128 -> 64 -> 16, batch 4."""
    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=128, layers=2, n_heads=4, d_conv=0)
    iface = VectorMLPInterface(feature_dim=128, num_regions=8, interface_width=16, interface_map_hidden_dim=64, activation="gelu")
    model = LBILanguageModel(vocab_size=512, layers_per_region=1, backbone_spec=spec, interface=iface, region_axis="sequence",
                             num_sequence_regions=8)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (4, 1025), generator=g)
    x, y = ids[:, :-1], ids[:, 1:]
    logits = model(x)
    loss = F.cross_entropy(logits.float().reshape(-1, 512), y.reshape(-1))
    ref = AutogradEngine().backward(model=model, loss=loss).grad_map
    engine = FastLBIEngine(copy.deepcopy(model), basis_chunk=16)
    engine.backward(x, y)
    got = engine.named_grads()
    worst = 0.0
    for name, r in ref.items():
        if r is not None:
            worst = max(worst, float(((got[name] - r).abs() / torch.maximum(torch.maximum(got[name].abs(), r.abs()), torch.tensor(1e-12))).max())
                        if float(r.abs().max()) > 1e-6 else 0.0)
            assert float((got[name] - r).norm() / (r.norm() + 1e-12)) < 1e-5
