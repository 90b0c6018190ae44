"""Decoding (CPU): token-by-token evaluation equals the training forward for every block type and for sequence-axis LBI models,
in both the recompute and the cached mode; generation is consistent with the full forward."""
import pytest
import torch

from lbi_b200.backbones import BackboneSpec, build_backbone_stack
from lbi_b200.inference import IncrementalLBIDecoder, generate
from lbi_b200.interfaces import VectorMLPInterface
from lbi_b200.models import DenseLanguageModel, LBILanguageModel

STACKS = [
    ("transformer", dict(n_heads=4, n_kv_heads=2, d_conv=4)),
    ("transformer", dict(n_heads=4, n_kv_heads=4, d_conv=0, rope_interleaved=True)),
    ("mamba2", dict(d_state=16, headdim=16, chunk_size=8, d_conv=4)),
    ("mamba3", dict(d_state=16, headdim=16, chunk_size=8)),
    ("hybrid", dict(d_state=16, headdim=16, chunk_size=8, d_conv=4, n_heads=4, layer_types=("mamba3", "transformer", "mamba2"))),
]


@pytest.mark.parametrize("name,extra", STACKS)
def test_block_decode_steps_reproduce_the_stack(name, extra):
    torch.manual_seed(0)
    layers = len(extra.get("layer_types", (0, 0)))
    stack = build_backbone_stack(BackboneSpec(name=name, dim=32, layers=layers, **extra)).eval()
    x = torch.randn(2, 13, 32)
    with torch.no_grad():
        want = stack.forward_range(x, 0, layers)
    states = [block.allocate_decode_state(2, 13) for block in stack.blocks]
    rows = []
    for t in range(13):
        branch, stream = x[:, t], None
        for block, state in zip(stack.blocks, states):
            branch, stream = block.decode_step(branch, stream, state)
        rows.append(branch + stream)
    assert torch.allclose(torch.stack(rows, dim=1), want, atol=5e-6, rtol=1e-5)


def test_attention_cache_refuses_to_overflow():
    torch.manual_seed(1)
    stack = build_backbone_stack(BackboneSpec(name="transformer", dim=32, layers=1, n_heads=4, d_conv=0)).eval()
    block = stack.blocks[0]
    state = block.allocate_decode_state(1, 2)
    for _ in range(2):
        block.decode_step(torch.randn(1, 32), None, state)
    with pytest.raises(ValueError):
        block.decode_step(torch.randn(1, 32), None, state)


def _lbi(name, extra, regions=4, layers=2):
    torch.manual_seed(0)
    spec = BackboneSpec(name=name, dim=32, layers=len(extra.get("layer_types", (0,) * layers)), **extra)
    iface = VectorMLPInterface(feature_dim=32, num_regions=regions, interface_width=8, interface_map_hidden_dim=16)
    return LBILanguageModel(vocab_size=50, layers_per_region=1, backbone_spec=spec, interface=iface, region_axis="sequence",
                            num_sequence_regions=regions, tie_embeddings=True).eval()


@pytest.mark.parametrize("name,extra", [STACKS[0], STACKS[2], STACKS[3], STACKS[4]])
@pytest.mark.parametrize("use_cache", [True, False])
def test_incremental_decoder_matches_the_training_forward(name, extra, use_cache):
    model = _lbi(name, extra)
    ids = torch.randint(0, 50, (2, 22))
    with torch.no_grad():
        want, _ = model.forward_with_cache(ids)
    decoder = IncrementalLBIDecoder(model, 22, use_cache=use_cache)
    got = torch.cat([decoder.append(ids[:, :5]), decoder.append(ids[:, 5:13]), decoder.append(ids[:, 13:])], dim=1)
    assert decoder.position == 22 and decoder.region == 4 and decoder.use_cache is use_cache
    assert torch.allclose(got, want, atol=5e-6, rtol=1e-5)
    with pytest.raises(ValueError):
        decoder.append(ids[:, :1])
    # a prompt that covers whole spans goes through them in one pass each (spans of 22 tokens in 4 regions: 6, 6, 5, 5)
    whole = IncrementalLBIDecoder(model, 22, use_cache=use_cache)
    first = whole.append(ids[:, :14])
    assert whole.region == 2 and whole.position == 14 and (whole._block_states is not None or not use_cache)
    assert torch.allclose(torch.cat([first, whole.append(ids[:, 14:])], dim=1), want, atol=5e-6, rtol=1e-5)


def test_generation_is_consistent_with_the_full_forward_and_between_modes():
    model = _lbi(*STACKS[0])
    prompt = torch.randint(0, 50, (2, 7))
    cached = generate(model, prompt, 15, use_cache=True)
    assert cached.shape == (2, 22) and torch.equal(cached[:, :7], prompt)
    assert torch.equal(cached, generate(model, prompt, 15, use_cache=False))
    with torch.no_grad():
        logits, _ = model.forward_with_cache(cached)
    assert torch.equal(logits[:, 6:-1].argmax(dim=-1), cached[:, 7:])  # every generated token is the arg-max of the full forward
    # the cut of a longer training length: still self-consistent when the rest is filled in later
    longer = generate(model, prompt, 5, total_len=32)
    assert longer.shape == (2, 12)
    sampled = generate(model, prompt, 6, temperature=0.8, top_k=5, generator=torch.Generator().manual_seed(3))
    again = generate(model, prompt, 6, temperature=0.8, top_k=5, generator=torch.Generator().manual_seed(3))
    assert torch.equal(sampled, again) and model.training is False
    with pytest.raises(ValueError):
        generate(model, prompt, 30, total_len=16)
    assert generate(model, prompt[:, :1], 2).shape == (2, 3)  # shorter than the number of regions


def test_generation_of_dense_and_depth_axis_models_by_recomputation():
    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=32, layers=2, n_heads=4, d_conv=0)
    dense = DenseLanguageModel(vocab_size=50, backbone_spec=spec, tie_embeddings=True).train()
    prompt = torch.randint(0, 50, (1, 5))
    out = generate(dense, prompt, 4)
    assert out.shape == (1, 9) and dense.training is True  # the mode is put back
    assert torch.equal(out, generate(dense, prompt, 4, use_cache=False))
    from lbi_b200.inference import IncrementalDenseDecoder

    ids = torch.randint(0, 50, (2, 11))
    decoder = IncrementalDenseDecoder(dense.eval(), 11)
    with torch.no_grad():
        assert torch.allclose(torch.cat([decoder.append(ids[:, :4]), decoder.append(ids[:, 4:])], dim=1), dense(ids), atol=5e-6, rtol=1e-5)
    with pytest.raises(ValueError):
        decoder.append(ids[:, :1])
    dense.train()
    with torch.no_grad():
        assert torch.equal(dense.eval()(out)[:, 4:-1].argmax(dim=-1), out[:, 5:])
    iface = VectorMLPInterface(feature_dim=32, num_regions=2, interface_width=8, interface_map_hidden_dim=16)
    depth = LBILanguageModel(vocab_size=50, layers_per_region=1, backbone_spec=spec, interface=iface, tie_embeddings=True)
    assert generate(depth, prompt, 3).shape == (1, 8)
    with pytest.raises(ValueError):
        IncrementalLBIDecoder(depth, 8)


def test_generation_command_on_trained_runs(tmp_path):
    from lbi_b200 import inference
    from lbi_b200.train.config import LBITrainingConfig
    from lbi_b200.train.lbi import run_lbi_experiment

    base = dict(variants="lbi", backbone="transformer", device="cpu", dtype="float32", output_dir=str(tmp_path), seq_len=16,
                batch_size=2, steps=2, eval_every=2, eval_batches=1, log_every=1, save_every=2, layers=2, dim=16, n_heads=2, d_conv=0,
                region_axis="sequence", sequence_regions=4, message_dim=4, message_hidden_dim=8)
    run_lbi_experiment(LBITrainingConfig(run_name="syn", task="copy", vocab_size=32, train_sequences=16, val_sequences=4, **base))
    out = inference.main([str(tmp_path / "syn" / "lbi"), "--prompt-ids", "1,2,3", "--max-new-tokens", "5", "--device", "cpu"])
    assert out["prompt_ids"] == [1, 2, 3] and len(out["new_ids"]) == 5 and all(0 <= i < 32 for i in out["new_ids"])
    with pytest.raises(SystemExit):
        inference.main([str(tmp_path / "syn" / "lbi"), "--prompt", "text needs a tokenizer", "--device", "cpu"])

    text = tmp_path / "corpus.txt"
    text.write_bytes(b"the quick brown fox jumps over the lazy dog. " * 100)
    run_lbi_experiment(LBITrainingConfig(run_name="bytes", data_mode="text_byte", vocab_size=256, train_text_path=str(text), **base))
    out = inference.main([str(tmp_path / "bytes" / "lbi"), "--prompt", "the quick", "--max-new-tokens", "4", "--temperature", "0.7",
                          "--top-k", "8", "--seed", "1", "--device", "cpu"])
    assert out["prompt_ids"] == list(b"the quick") and len(out["new_ids"]) == 4 and isinstance(out["text"], str)

    pytest.importorskip("sentencepiece")
    tok = tmp_path / "tok.model"
    run_lbi_experiment(LBITrainingConfig(run_name="bpe", data_mode="text_bpe", train_text_path=str(text), tokenizer_path=str(tok),
                                         vocab_size=300, tokenizer_train_bytes=4096, train_tokenizer=True, **base))
    out = inference.main([str(tmp_path / "bpe" / "lbi"), "--prompt", "the lazy", "--max-new-tokens", "3", "--device", "cpu"])
    assert len(out["new_ids"]) == 3 and isinstance(out["text"], str)


def test_generation_service_requests(tmp_path):
    from lbi_b200.serve import GenerationService, build_app
    from lbi_b200.train.config import LBITrainingConfig
    from lbi_b200.train.lbi import run_lbi_experiment

    text = tmp_path / "corpus.txt"
    text.write_bytes(b"the quick brown fox jumps over the lazy dog. " * 100)
    run_lbi_experiment(LBITrainingConfig(
        variants="lbi", backbone="mamba3", device="cpu", dtype="float32", output_dir=str(tmp_path), run_name="svc", seq_len=16,
        batch_size=2, steps=2, eval_every=2, eval_batches=1, log_every=1, save_every=2, layers=2, dim=16, d_state=16, headdim=16,
        chunk_size=16, region_axis="sequence", sequence_regions=4, message_dim=4, message_hidden_dim=8, data_mode="text_byte",
        vocab_size=256, train_text_path=str(text)))
    service = GenerationService.from_run(tmp_path / "svc" / "lbi", device="cpu", max_new_tokens_limit=8)
    assert service.health()["backbone"] == "mamba3" and service.health()["region_axis"] == "sequence"
    reply = service.handle({"prompt": "the quick", "max_new_tokens": 4})
    assert reply["prompt_ids"] == list(b"the quick") and len(reply["new_ids"]) == 4 and isinstance(reply["text"], str)
    assert service.handle({"prompt_ids": [116, 104, 101], "max_new_tokens": 2, "temperature": 0.5, "top_k": 4, "seed": 3}) == \
        service.handle({"prompt_ids": [116, 104, 101], "max_new_tokens": 2, "temperature": 0.5, "top_k": 4, "seed": 3})
    for bad in ({}, {"prompt_ids": [999]}, {"prompt": "x", "max_new_tokens": 0}, {"prompt": "x", "max_new_tokens": 99}):
        with pytest.raises(ValueError):
            service.handle(bad)
    pytest.importorskip("fastapi")
    app = build_app(service)
    assert {"/health", "/generate"} <= {route.path for route in app.routes}


def test_the_python_api_example_of_the_readme_runs():
    """The snippet under "Python API" in README.md is executed as written."""
    from pathlib import Path

    text = (Path(__file__).resolve().parent.parent / "README.md").read_text(encoding="utf-8")
    section = text.split("## Python API", 1)[1]
    code = section.split("```python", 1)[1].split("```", 1)[0]
    scope: dict = {}
    exec(compile(code, "README.md:python-api", "exec"), scope)  # noqa: S102
    assert scope["tokens"].shape == (2, 16) and scope["first"] == scope["first"] and scope["second"] == scope["second"]


def test_decode_benchmark_runs_on_the_cpu():
    from lbi_b200.benchmarks import time_decode

    out = time_decode.main(["--device", "cpu", "--backbone", "mamba2", "--dim", "64", "--layers", "2", "--regions", "2",
                            "--total-len", "32", "--prompt-len", "4", "--new-tokens", "8", "--vocab", "64"])
    assert out["cached_tokens_per_s"] > 0 and out["recompute_tokens_per_s"] > 0 and out["decode_state_bytes"] > 0
