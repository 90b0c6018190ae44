"""Token-shard sampling, the shard writer, the byte-BPE tokenizer, and LBI-1 checkpoint migration."""
import json

import numpy as np
import pytest
import torch

from lbi_b200.backbones import BackboneSpec
from lbi_b200.data.bpe_tokenizer import ByteBPETokenizer, train_byte_bpe_tokenizer
from lbi_b200.data.pretokenize_corpus import write_shards
from lbi_b200.data.token_shards import TokenShardCorpus, corpus_numel, sample_batch_token_shards
from lbi_b200.interfaces import VectorMLPInterface
from lbi_b200.legacy import NativeRegionInterfaceModel, is_lbi1_state_dict, migrate_lbi1_state_dict, native_backward_step
from lbi_b200.models import DenseLanguageModel, LBILanguageModel
from lbi_b200.train.checkpointing import load_model_state


def test_shard_sampling_windows(tmp_path):
    sizes = (50, 7, 120)
    shards, start = [], 0
    for i, n in enumerate(sizes):
        np.arange(start, start + n, dtype=np.int32).tofile(tmp_path / f"train_{i:04d}.bin")
        shards.append({"path": f"train_{i:04d}.bin", "num_tokens": n})
        start += n
    manifest = tmp_path / "train_manifest.json"
    manifest.write_text(json.dumps({"split": "train", "dtype": "int32", "num_tokens_total": start, "shards": shards}))
    corpus = TokenShardCorpus(manifest)
    assert corpus_numel(corpus) == start and corpus.valid_starts_per_shard(10) == [40, 0, 110]
    g = torch.Generator().manual_seed(0)
    x, y = sample_batch_token_shards(corpus, batch_size=16, seq_len=10, generator=g, device=torch.device("cpu"))
    assert x.shape == (16, 10) and torch.equal(x[:, 1:], y[:, :-1])
    assert torch.equal(x[:, 1:] - x[:, :-1], torch.ones(16, 9, dtype=torch.int64))  # windows never straddle shards
    with pytest.raises(ValueError):
        sample_batch_token_shards(corpus, batch_size=1, seq_len=500, generator=g, device=torch.device("cpu"))


def test_tokenizer_and_shard_writer_round_trip(tmp_path):
    text = tmp_path / "t.txt"
    text.write_bytes(b"alpha beta gamma alpha beta delta\n" * 50)
    tok = train_byte_bpe_tokenizer(text, vocab_size=280, max_bytes=10_000)
    assert 256 < tok.vocab_size <= 280
    ids = tok.encode_bytes(text.read_bytes())
    assert tok.decode(ids) == text.read_bytes() and len(ids) < len(text.read_bytes())
    tok.save(tmp_path / "tok.json")
    again = ByteBPETokenizer.load(tmp_path / "tok.json")
    assert again.encode_bytes(b"alpha beta") == tok.encode_bytes(b"alpha beta")
    manifest = write_shards("train", text, tok, tmp_path / "shards", shard_tokens=200)
    meta = json.loads(manifest.read_text())
    assert meta["dtype"] == "int32" and meta["num_tokens_total"] == len(ids) and len(meta["shards"]) > 1
    corpus = TokenShardCorpus(manifest)
    joined = np.concatenate([np.fromfile(tmp_path / "shards" / s["path"], dtype=np.int32) for s in meta["shards"]])
    assert joined.tolist() == ids and corpus.tokenizer_vocab_size == tok.vocab_size


@pytest.mark.parametrize("tie", [False, True])
def test_lbi1_checkpoint_migrates_bit_exactly(tie):
    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=32, layers=4, n_heads=4, d_conv=4)
    old = NativeRegionInterfaceModel(vocab_size=40, region_size=2, message_dim=8, backbone_spec=spec, message_hidden_dim=16,
                                     tie_embeddings=tie)
    sd = old.state_dict()
    assert is_lbi1_state_dict(sd) and "blocks.0.norm.weight" in sd and "backbone.blocks.0.norm.weight" in sd and "lm_head.weight" in sd
    iface = VectorMLPInterface(feature_dim=32, num_regions=2, interface_width=8, interface_map_hidden_dim=16)
    new = LBILanguageModel(vocab_size=40, layers_per_region=2, backbone_spec=spec, interface=iface, tie_embeddings=tie)
    new.load_state_dict(migrate_lbi1_state_dict(sd), strict=True)
    ids = torch.randint(0, 40, (2, 12))
    assert torch.equal(old(ids), new(ids))  # same modules, same op order: bit-identical logits
    with torch.no_grad():  # without autograd the owned model runs its structured kernels path
        assert torch.allclose(old(ids), new(ids), atol=1e-5, rtol=1e-5)
    # the checkpoint loader accepts the raw LBI-1 dict as well
    fresh = LBILanguageModel(vocab_size=40, layers_per_region=2, backbone_spec=spec,
                             interface=VectorMLPInterface(feature_dim=32, num_regions=2, interface_width=8, interface_map_hidden_dim=16),
                             tie_embeddings=tie)
    load_model_state(fresh, sd)
    assert torch.equal(fresh(ids), old(ids))


def test_lbi1_backward_step_matches_autograd():
    torch.manual_seed(1)
    spec = BackboneSpec(name="transformer", dim=32, layers=4, n_heads=4, d_conv=4)
    model = NativeRegionInterfaceModel(vocab_size=40, region_size=2, message_dim=8, backbone_spec=spec, message_hidden_dim=16)
    ids, tgt = torch.randint(0, 40, (2, 12)), torch.randint(0, 40, (2, 12))
    loss = torch.nn.functional.cross_entropy(model(ids).reshape(-1, 40), tgt.reshape(-1))
    loss.backward()
    want = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    logits, cache = model.forward_with_cache(ids, detach_states=True)
    loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 40), tgt.reshape(-1))
    diag = native_backward_step(model, loss, cache)
    assert diag["interface_scan_rms"] < 1e-5
    for n, p in model.named_parameters():
        if n in want:
            assert torch.allclose(p.grad, want[n], atol=1e-5, rtol=1e-4), n


@pytest.mark.parametrize("mode", ["graph", "recompute"])
def test_lbi1_backward_entry_with_the_reference_keywords(mode):
    """``_native_backward_step(model, ce_loss=..., cache=..., ...)`` returns named gradients, the scan residual and, on request,
    the Jacobian statistics with their suffix part; ``.grad`` stays untouched."""
    from lbi_b200.legacy import NativeBackwardResult, RegionInterfaceCache, _native_backward_step, build_region_slices

    assert build_region_slices(5, 2) == [(0, 2), (2, 4), (4, 5)]
    torch.manual_seed(2)
    spec = BackboneSpec(name="transformer", dim=32, layers=3, n_heads=4, d_conv=0)
    model = NativeRegionInterfaceModel(vocab_size=40, region_size=1, message_dim=8, backbone_spec=spec, message_hidden_dim=16)
    ids, tgt = torch.randint(0, 40, (2, 10)), torch.randint(0, 40, (2, 10))
    loss = torch.nn.functional.cross_entropy(model(ids).reshape(-1, 40), tgt.reshape(-1))
    want = dict(zip([n for n, _ in model.named_parameters()], torch.autograd.grad(loss, list(model.parameters()), allow_unused=True)))
    logits, cache = model.forward_with_cache(ids, detach_states=True)
    view = model.interface_cache(cache)
    assert isinstance(view, RegionInterfaceCache) and len(view.region_caches) == 3 and view.region_ranges == [(0, 1), (1, 2), (2, 3)]
    loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 40), tgt.reshape(-1))
    out = _native_backward_step(model, ce_loss=loss, cache=cache, interface_jacobian_mode=mode, jacobian_basis_chunk=4,
                                compute_interface_jacobian_stats=True, include_interface_jacobian_suffix=True)
    assert isinstance(out, NativeBackwardResult) and out.interface_scan_rms < 1e-5
    assert {"jac_local_spec_mean", "jac_local_frob_max", "jac_suffix_spec_max"} <= set(out.interface_jacobian_stats)
    assert all(p.grad is None for p in model.parameters())
    for n, g in want.items():
        if g is not None:
            assert torch.allclose(out.grad_map[n], g, atol=1e-5, rtol=1e-4), n


def test_dense_state_dict_has_both_block_prefixes():
    model = DenseLanguageModel(vocab_size=30, backbone_spec=BackboneSpec(name="transformer", dim=16, layers=1, n_heads=2))
    keys = set(model.state_dict())
    assert "blocks.0.norm.weight" in keys and "backbone.blocks.0.norm.weight" in keys and "canvas.embedding.weight" in keys


def _legacy_model(regions=3):
    from lbi_b200.backbones import BackboneSpec

    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=16, layers=regions * 1, n_heads=2, d_conv=0)
    return NativeRegionInterfaceModel(vocab_size=40, region_size=1, message_dim=6, backbone_spec=spec, message_hidden_dim=8)


def test_legacy_model_recompute_mode_and_scan_helpers():
    """The LBI-1 model's own Jacobian materialisers (graph and recompute), suffix composition and message-cotangent scans
    agree with the sequential autograd chain, and its backward step runs in both modes with the same gradients."""
    model = _legacy_model()
    ids = torch.randint(0, 40, (2, 12))
    logits, cache = model.forward_with_cache(ids)
    g_top = torch.randn_like(cache["region_messages"][-1])
    chain = model.interface_vjp_chain(cache, g_top)
    for mode, chunk in (("graph", 1), ("recompute", 4)):
        mats = model.materialize_interface_pullback_mats(cache, mode=mode, basis_chunk=chunk)
        assert len(mats) == model.n_regions and mats[0].shape == (2, 6, 6)
        scan = model.interface_vjp_scan_from_mats(mats, g_top)
        for a, b in zip(scan, chain):
            assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)
    seeded = model.interface_vjp_scan_from_last_input_seed(mats, chain[-2])
    for a, b in zip(seeded, chain[:-1]):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)
    assert len(model.compose_pullback_suffix(mats)) == model.n_regions + 1
    grads = {}
    tgt = torch.randint(0, 40, (2, 12))
    for mode in ("graph", "recompute"):
        logits, cache = model.forward_with_cache(ids, detach_states=True)
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 40), tgt.reshape(-1))
        native_backward_step(model, loss, cache, interface_jacobian_mode=mode, jacobian_basis_chunk=3)
        grads[mode] = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    assert grads["graph"].keys() == grads["recompute"].keys()
    for n in grads["graph"]:
        assert torch.allclose(grads["graph"][n], grads["recompute"][n], atol=1e-5, rtol=1e-4), n


def test_legacy_model_closed_form_region_pullback_matches_autograd():
    """The closed-form outer pieces of a region's message pullback (LayerNorm, update scale, encoder, token mean on one side;
    token sum, decoder on the other) combined with autograd through the backbone give the graph-mode A_k^T."""
    model = _legacy_model()
    ids = torch.randint(0, 40, (2, 12))
    _, cache = model.forward_with_cache(ids)
    mats = model.materialize_interface_pullback_mats(cache, mode="graph")
    for ridx, rc in enumerate(cache["region_caches"]):
        eye = torch.eye(6).unsqueeze(0).expand(2, 6, 6)
        tail = model.region_message_output_pullback_to_hidden_output(rc, eye)
        g_hidden_in = torch.stack([torch.autograd.grad(rc.hidden_output, rc.hidden_input, tail["g_hidden_output"][:, j].contiguous(),
                                                       retain_graph=True)[0] for j in range(6)], dim=1)
        total = model.region_outer_message_input_pullback(rc, eye, g_hidden_in)["g_message_input_total"]   # [B, j, i]
        assert torch.allclose(total.transpose(1, 2), mats[ridx], atol=1e-5, rtol=1e-4)


def test_legacy_model_helpers_under_the_names_of_the_first_release():
    from lbi_b200.legacy.native_region_interface import RegionMessageHead

    model = _legacy_model()
    torch.manual_seed(11)
    ids = torch.randint(0, 40, (2, 12))
    logits, cache = model.forward_with_cache(ids)
    x_static = cache["boundaries"][0]
    for ridx in range(model.n_regions):  # a region's hidden input is the embedding plus the decoded incoming message
        want = x_static + model.message_to_hidden[ridx](cache["region_messages"][ridx]).unsqueeze(1)
        assert torch.allclose(cache["region_hidden_inputs"][ridx], want, atol=1e-6)
    assert torch.equal(model(ids, message_ablation="none"), logits)
    assert not torch.allclose(model(ids, message_ablation="zero_all"), logits)
    assert torch.equal(model._pool_hidden(x_static), x_static.mean(dim=1))
    m = cache["region_messages"][1]
    assert torch.equal(model._apply_message_ablation(m, mode="zero_all", next_region_idx=1, noise_std=1.0, mask_keep_prob=0.5,
                                                     generator=None), torch.zeros_like(m))
    with pytest.raises(ValueError):
        model._apply_message_ablation(m, mode="drop", next_region_idx=1, noise_std=1.0, mask_keep_prob=0.5, generator=None)

    for hidden_dim in (0, 9):
        head = RegionMessageHead(5, 7, hidden_dim=hidden_dim)
        x, g_out = torch.randn(3, 5, requires_grad=True), torch.randn(3, 4, 7)
        y = head(x)
        want = torch.stack([torch.autograd.grad(y, x, g_out[:, i], retain_graph=True)[0] for i in range(4)], dim=1)
        assert torch.allclose(model._region_message_head_input_pullback_matrix(head, x.detach(), g_out), want, atol=1e-6)
        assert torch.allclose(model._module_input_pullback_matrix_autograd(head, x.detach(), g_out), want, atol=1e-6)
    lin = torch.nn.Linear(5, 7)
    g_out, x = torch.randn(3, 4, 7), torch.randn(3, 7)
    assert torch.allclose(model._linear_input_pullback_matrix(lin, g_out), g_out @ lin.weight, atol=1e-6)
    xg = x.clone().requires_grad_(True)
    (slope,) = torch.autograd.grad(torch.nn.functional.silu(xg).sum(), xg)
    assert torch.allclose(model._silu_input_pullback_matrix(x, g_out), g_out * slope.unsqueeze(1), atol=1e-6)
    pooled = torch.randn(2, 3, 6)
    assert torch.allclose(model._mean_pool_pullback_matrix(pooled, 4), pooled.unsqueeze(2).expand(-1, -1, 4, -1) / 4.0)
    g_hidden = torch.randn(2, 3, 4, 6)
    assert torch.equal(model._broadcast_message_pullback_matrix(g_hidden), g_hidden.sum(dim=2))
    graph = model._materialize_interface_pullback_mats_graph(cache)
    recompute = model._materialize_interface_pullback_mats_recompute(cache, 4)
    assert len(graph) == len(recompute) == model.n_regions and all(torch.allclose(a, b, atol=1e-5) for a, b in zip(graph, recompute))
    vec = torch.randn(2, 6)
    assert model._apply_pullback_mat(graph[0], vec, out_dtype=torch.float64).dtype == torch.float64
    for bad in (lambda: model._mean_pool_pullback_matrix(pooled, 0), lambda: model._broadcast_message_pullback_matrix(pooled),
                lambda: model._linear_input_pullback_matrix(lin, x)):
        with pytest.raises(ValueError):
            bad()


def test_first_release_trainer_entry_and_component_counts(tmp_path):
    from lbi_b200.legacy import train_region_interface as legacy_train
    from lbi_b200.train.model_builders import build_lbi_language_model
    from lbi_b200.train import metrics
    from lbi_b200.train.config import NEW_OUTPUT_NAME_BY_VARIANT, LBITrainingConfig

    cfg = LBITrainingConfig(
        regime="native_region_interface", variants="", backbone="transformer", device="cpu", dtype="float32",
        output_dir=str(tmp_path), run_name="first", task="copy", vocab_size=32, seq_len=16, train_sequences=16,
        val_sequences=4, batch_size=2, steps=2, eval_every=1, eval_batches=1, log_every=1, save_every=2, layers=2, dim=16,
        n_heads=2, region_size=1, message_dim=4, message_hidden_dim=8, seed=3)
    out = legacy_train.run_training(cfg)
    assert cfg.variants == "native_region_interface" and out
    assert set(NEW_OUTPUT_NAME_BY_VARIANT) == {"dense", "lbi"}

    cfg.variants = "lbi"
    model = build_lbi_language_model(cfg)
    total = sum(p.numel() for p in model.parameters())
    parts = (metrics.canvas_component_params(model), metrics.readout_lm_head_component_params(model),
             metrics.readout_norm_component_params(model))
    assert all(0 <= p <= total for p in parts) and parts[0] > 0
    assert isinstance(metrics.readout_uses_tied_output_weight(model), bool)


def test_reference_names_import_from_the_same_modules():
    from lbi_b200.backbones.mamba3.block import Mamba3BlockCache, Mamba3BlockForwardCache
    from lbi_b200.backbones.transformer.block import RMSNorm  # noqa: F401
    from lbi_b200.backends.transformer import (TransformerAttentionCache, TransformerLayerCache,  # noqa: F401
                                               TransformerMLPCache, TransformerRegionCache)
    from lbi_b200.backward.pullbacks import (materialize_interface_state_jacobian_t_graph,  # noqa: F401
                                             materialize_interface_state_jacobian_t_recompute)
    from lbi_b200.backward.scan import ReferenceScanEngine  # noqa: F401
    from lbi_b200.backward.suffix_scan import propagate_state_adjoint_by_autograd_chain  # noqa: F401
    from lbi_b200.models.lbi_language_model import build_region_ranges  # noqa: F401

    assert Mamba3BlockForwardCache is Mamba3BlockCache
    from lbi_b200.backends import TransformerLayerCache as exported_layer_cache, TransformerRegionCache as exported_region_cache
    from lbi_b200.backward import (ScanADEngine, materialize_interface_state_jacobian_t_graph as exported_graph,  # noqa: F401
                                   materialize_interface_state_jacobian_t_recompute as exported_recompute,  # noqa: F401
                                   propagate_state_adjoint_by_autograd_chain as exported_chain, store_named_grads)  # noqa: F401
    from lbi_b200.backward.reference_scan import ScanADEngine as via_reference_scan, lbi_scan_backward_step  # noqa: F401
    from lbi_b200.scripts.plot_jacobian_diagnostics import generate_jacobian_diagnostic_plots  # noqa: F401
    from lbi_b200.scripts.plot_message_ablations import generate_message_ablation_plots  # noqa: F401
    from lbi_b200.scripts.plot_training_curves import generate_training_plots  # noqa: F401
    from lbi_b200.train.config import ALL_REGIME, DENSE_REGIME, LBI_REGIME

    assert exported_layer_cache is TransformerLayerCache and exported_region_cache is TransformerRegionCache
    assert via_reference_scan is ScanADEngine and (DENSE_REGIME, LBI_REGIME, ALL_REGIME) == ("dense", "lbi", "all")


def test_private_step_names_that_subclasses_of_the_reference_override():
    from lbi_b200.backbones import BackboneSpec, build_backbone_stack
    from lbi_b200.backends import BackboneStackRegionBackend, TransformerRegionBackend

    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=16, layers=2, n_heads=4, n_kv_heads=2, d_conv=0)
    backend = TransformerRegionBackend(backbone_spec=spec, region_ranges=[(0, 1), (1, 2)])
    block = backend.backbone.blocks[0]
    x = torch.randn(2, 8, 16)
    normed, stream = block._prenorm(x, None, block.norm)
    assert torch.equal(normed, block.add_norm(x, None, block.norm)[0]) and torch.equal(stream, x)
    q, k, v = block.attn.split_heads(block.attn.in_proj(normed))
    assert block.attn._expand_kv(k).shape == q.shape and not block.attn._can_use_flash_attn(normed)
    heads = block.attn._flash_attention(q, block.attn._expand_kv(k), block.attn._expand_kv(v))
    assert heads.shape == (2, 8, 4, 4)
    out, residual, attn_cache, mlp_cache = backend._block_forward_with_cache(block=block, hidden_states=x, residual=None)
    want_out, want_res = block(x)
    assert torch.allclose(out, want_out, atol=1e-6) and torch.equal(residual, want_res)
    assert torch.equal(attn_cache.norm_input, x) and torch.allclose(mlp_cache.down_output, want_out, atol=1e-6)
    a_out, a_cache = backend._attention_forward_with_cache(block.attn, normed)
    assert torch.allclose(a_out, block.attn(normed), atol=1e-6) and a_cache.norm_output is normed
    m_out, _ = backend._mlp_forward_with_cache(block.mlp, normed)
    assert torch.allclose(m_out, block.mlp(normed), atol=1e-6)
    assert backend._region_range(1) == (1, 2)
    stack = BackboneStackRegionBackend(backbone=build_backbone_stack(spec), region_ranges=[(0, 2)])
    for b in (backend, stack):
        with pytest.raises(IndexError):
            b._region_range(5)


def test_transformer_layer_caches_and_jacobian_function_forms():
    from lbi_b200.backends.transformer import TransformerRegionBackend
    from lbi_b200.backward.pullbacks import (materialize_interface_state_jacobian_t_graph,
                                             materialize_interface_state_jacobian_t_recompute)
    from lbi_b200.backward.suffix_scan import propagate_state_adjoint_by_autograd_chain
    from lbi_b200.train.config import LBITrainingConfig
    from lbi_b200.train.model_builders import build_lbi_language_model

    torch.manual_seed(0)
    cfg = LBITrainingConfig(variants="lbi", backbone="transformer", device="cpu", dtype="float32", vocab_size=32, seq_len=8,
                            layers=4, dim=16, n_heads=2, region_size=2, message_dim=4, message_hidden_dim=8, d_conv=3)
    model = build_lbi_language_model(cfg)
    backend = model.region_backend
    x = torch.randn(2, 8, 16)
    with torch.no_grad():
        want = backend.backbone.forward_range(x, 2, 4)
        got, cache = backend.forward_region_with_layer_caches(region_input=x, region_index=1)
    assert torch.allclose(got, want, atol=1e-6) and [lc.layer_index for lc in cache.layer_caches] == [2, 3]
    first = cache.layer_caches[0]
    assert first.residual_input is None and first.attention.norm_input is not None
    assert first.attention.q_rope.shape == first.attention.k_expanded.shape == (2, 2, 8, 8)
    assert torch.allclose(first.mlp.down_input, first.mlp.up * first.mlp.activation)
    assert torch.allclose(cache.layer_caches[1].mlp.down_output + cache.layer_caches[1].residual_output, got, atol=1e-6)
    shared = TransformerRegionBackend(backbone=backend.backbone, region_ranges=[(0, 4)])
    assert shared.backbone is backend.backbone and shared.count_parameters() == backend.count_parameters()
    with pytest.raises(ValueError):
        TransformerRegionBackend(backbone_spec=None, region_ranges=[(0, 1)])

    tokens = torch.randint(0, 32, (2, 8))
    _, fcache = model.forward_with_cache(tokens)
    graph = materialize_interface_state_jacobian_t_graph(model=model, cache=fcache)
    rec = materialize_interface_state_jacobian_t_recompute(model=model, cache=fcache, basis_chunk=3)
    assert len(graph) == len(rec) == model.num_regions
    for a, b in zip(graph, rec):
        assert torch.allclose(a, b, atol=1e-5)
    top = torch.randn_like(fcache["states"][-1])
    by_graph = propagate_state_adjoint_by_autograd_chain(states=fcache["states"], top_state_adjoint=top)
    assert len(by_graph) == model.num_regions + 1 and torch.equal(by_graph[-1], top)
    expect = torch.einsum("bij,bj->bi", graph[-1], top)
    assert torch.allclose(by_graph[-2], expect, atol=1e-5)
    with pytest.raises(ValueError):
        propagate_state_adjoint_by_autograd_chain(states=fcache["states"][:1], top_state_adjoint=top)


def test_pretokenize_entry_takes_the_keywords_of_the_reference(tmp_path):
    from lbi_b200.data.pretokenize_corpus import pretokenize_text_corpus

    train, val = tmp_path / "corpus.txt", tmp_path / "corpus_val.txt"
    train.write_bytes(b"alpha beta gamma alpha beta delta\n" * 40)
    val.write_bytes(b"gamma delta alpha\n" * 10)
    common = dict(tokenizer_type="byte_bpe", vocab_size=270, tokenizer_train_bytes=4096, train_tokenizer=True, shard_tokens=150)
    tm, vm = pretokenize_text_corpus(text_corpus="", train_text_path=str(train), val_text_path=str(val),
                                     tokenizer_path=str(tmp_path / "tok.json"), output_dir=str(tmp_path / "out"), **common)
    assert tm == tmp_path / "out" / "train_manifest.json" and vm == tmp_path / "out" / "val_manifest.json"
    assert json.loads(tm.read_text())["num_tokens_total"] > json.loads(vm.read_text())["num_tokens_total"] > 0
    with pytest.raises(FileNotFoundError):
        pretokenize_text_corpus(text_corpus="", train_text_path=str(train), val_text_path="", output_dir=str(tmp_path / "o2"),
                                tokenizer_path=str(tmp_path / "tok.json"), **common)
    with pytest.raises(ValueError):
        pretokenize_text_corpus(text_corpus="no_such_corpus", **common)
    tm2, vm2 = pretokenize_text_corpus(train_path=train, val_path=None, out_dir=tmp_path / "o3",
                                       tokenizer_path=tmp_path / "tok.json", **{**common, "train_tokenizer": False})
    assert vm2 is None and json.loads(tm2.read_text()) == json.loads(tm.read_text())


def test_fineweb_export_fills_the_train_budget_before_the_validation_file(tmp_path):
    from lbi_b200.data.export_fineweb_edu import export

    docs = [{"text": f"document number {i} " + "x" * 40} for i in range(50)] + [{"text": ""}, {"other": 1}]
    wt, wv = export(iter(docs), tmp_path / "train.txt", tmp_path / "val.txt", train_bytes=500, val_bytes=200)
    assert (wt, wv) == (500, 200)
    train, val = (tmp_path / "train.txt").read_bytes(), (tmp_path / "val.txt").read_bytes()
    assert len(train) == 500 and len(val) == 200 and train.startswith(b"document number 0 ")
    first_val_doc = int(val.split(b" ")[2])
    assert first_val_doc > int(train.rsplit(b"document number ", 1)[1].split(b" ")[0]) - 1  # validation starts after the train budget
    small = export(iter(docs[:3]), tmp_path / "t2.txt", tmp_path / "v2.txt", train_bytes=10_000, val_bytes=10_000)
    assert small[0] == sum(len(d["text"].strip()) + 1 for d in docs[:3]) and small[1] == 0


def test_every_synthetic_task_has_its_structure():
    from lbi_b200.data.train_data import SYNTHETIC_TASKS, build_synthetic_corpus, sample_batch

    vocab, seq_len = 32, 20
    bos, sep, pad = vocab - 1, vocab - 2, vocab - 3
    for task in SYNTHETIC_TASKS:
        corpus = build_synthetic_corpus(num_sequences=6, seq_len=seq_len, vocab_size=vocab, seed=4, task=task)
        again = build_synthetic_corpus(num_sequences=6, seq_len=seq_len, vocab_size=vocab, seed=4, task=task)
        assert corpus.shape == (6, seq_len + 1) and corpus.dtype == torch.long and torch.equal(corpus, again)
        assert int(corpus.min()) >= 0 and int(corpus.max()) < vocab
    arith = build_synthetic_corpus(num_sequences=4, seq_len=seq_len, vocab_size=vocab, seed=1, task="arith")
    stride = (arith[:, 1] - arith[:, 0]) % vocab
    assert torch.equal((arith[:, 1:] - arith[:, :-1]) % vocab, stride.unsqueeze(1).expand(-1, seq_len)) and int(stride.min()) >= 1
    plen = (seq_len + 1 - 2) // 2
    for task, answer in (("copy", lambda p: p), ("reverse", lambda p: p.flip(dims=(1,))), ("selective_copy", lambda p: p[:, ::2])):
        seq = build_synthetic_corpus(num_sequences=5, seq_len=seq_len, vocab_size=vocab, seed=2, task=task)
        payload = seq[:, 1 : 1 + plen]
        want = answer(payload)
        width = min(want.shape[1], seq_len + 1 - (2 + plen))
        assert torch.all(seq[:, 0] == bos) and torch.all(seq[:, 1 + plen] == sep) and int(payload.max()) < pad
        assert torch.equal(seq[:, 2 + plen : 2 + plen + width], want[:, :width])
    ind = build_synthetic_corpus(num_sequences=5, seq_len=seq_len, vocab_size=vocab, seed=3, task="induction")
    pairs = (seq_len + 1 - 6) // 2
    keys, vals = ind[:, 1 : 1 + 2 * pairs : 2], ind[:, 2 : 2 + 2 * pairs : 2]
    q_key, q_val = ind[:, 2 + 2 * pairs], ind[:, 4 + 2 * pairs]
    assert torch.all(ind[:, 1 + 2 * pairs] == sep) and torch.all(ind[:, 3 + 2 * pairs] == sep)
    for row in range(5):  # the queried key occurs among the keys and its value is (one of) the values stored with it
        hits = (keys[row] == q_key[row]).nonzero().flatten()
        assert len(hits) > 0 and any(int(vals[row, h]) == int(q_val[row]) for h in hits)
    x, y = sample_batch(arith, batch_size=3, generator=torch.Generator().manual_seed(0), device=torch.device("cpu"))
    assert x.shape == y.shape == (3, seq_len) and torch.equal(x[:, 1:], y[:, :-1])
    for bad in (dict(task="sort"), dict(num_sequences=0), dict(seq_len=1), dict(vocab_size=4, task="copy")):
        kw = dict(num_sequences=2, seq_len=8, vocab_size=16, seed=0, task="copy")
        kw.update(bad)
        with pytest.raises(ValueError):
            build_synthetic_corpus(**kw)
