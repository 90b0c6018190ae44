"""End-to-end smoke of the training program on the CPU: artefacts, metric rows, ablations, resume, init-from,
external checkpoint root, no-checkpoint mode, config validation, every backbone and backward engine."""
import csv
import json
from dataclasses import replace
from pathlib import Path

import pytest
import torch

from lbi_b200.train.config import LBITrainingConfig, build_arg_parser, config_from_args
from lbi_b200.train.lbi import run_lbi_experiment


def make_cfg(tmp_path, **kw):
    base = dict(
        variants="lbi", backbone="transformer", device="cpu", dtype="float32", output_dir=str(tmp_path / "out"), run_name="run",
        task="copy", vocab_size=32, seq_len=16, train_sequences=32, val_sequences=8, batch_size=2, steps=2, eval_every=1,
        eval_batches=1, log_every=1, save_every=1, layers=2, dim=16, n_heads=2, d_state=16, headdim=16, chunk_size=16,
        region_size=1, message_dim=4, message_hidden_dim=8,
    )
    base.update(kw)
    return LBITrainingConfig(**base)


def rows(path: Path):
    with path.open() as f:
        return list(csv.DictReader(f))


def test_dense_and_lbi_run_write_all_artefacts(tmp_path):
    cfg = make_cfg(tmp_path, variants="all", eval_all_message_ablations=True, log_interface_jacobian_every=1,
                   log_interface_jacobian_suffix=True)
    summary = run_lbi_experiment(cfg)
    root = Path(summary["root_dir"])
    assert summary["variants"] == ["dense", "lbi"] and (root / "summary.json").exists()
    for variant in ("dense", "lbi"):
        run_dir = root / variant
        for name in ("config.json", "data_info.json", "model_info.json", "metrics.csv", "metrics.jsonl", "summary.json"):
            assert (run_dir / name).exists(), f"{variant}/{name}"
        ckpts = sorted(p.name for p in (run_dir / "checkpoints").iterdir())
        assert "latest.pt" in ckpts and all(not n.startswith("step_") for n in ckpts)
    lbi_rows = rows(root / "lbi" / "metrics.csv")
    splits = {r["split"] for r in lbi_rows}
    assert {"train", "val", "val_zero_all", "val_noise", "val_mask"} <= splits
    train_rows = [r for r in lbi_rows if r["split"] == "train"]
    assert len(train_rows) == 2 and float(train_rows[0]["scan_align"]) < 1e-5 and train_rows[0]["jac_local_spec_mean"] != ""
    assert train_rows[0]["jac_suffix_spec_max"] != ""
    info = json.loads((root / "lbi" / "model_info.json").read_text())
    assert info["n_regions"] == 2 and info["owned_lbi_model"] and "interface.decoders" in info["component_params"]
    ckpt = torch.load(root / "lbi" / "checkpoints" / "latest.pt", weights_only=False)
    for key in ("step", "tokens_seen", "config", "model_state_dict", "optimizer_state_dict", "torch_rng_state",
                "train_generator_state", "eval_generator_state", "owned_lbi_model", "interface_jacobian_mode"):
        assert key in ckpt
    assert ckpt["step"] == 2 and ckpt["tokens_seen"] == 2 * 2 * 16


def test_resume_continues_counters_and_rows(tmp_path):
    cfg = make_cfg(tmp_path)
    first = run_lbi_experiment(cfg)
    run_dir = Path(first["root_dir"]) / "lbi"
    n_before = len(rows(run_dir / "metrics.csv"))
    resumed = run_lbi_experiment(replace(cfg, steps=4, resume_from=str(first["root_dir"])))
    assert resumed["root_dir"] == first["root_dir"]
    run = resumed["runs"][0]
    assert run["start_step"] == 2 and run["total_train_tokens"] == 4 * 2 * 16 and run["resumed_from"].endswith("latest.pt")
    all_rows = rows(run_dir / "metrics.csv")
    assert len(all_rows) > n_before and [r["step"] for r in all_rows if r["split"] == "train"] == ["1", "2", "3", "4"]


def test_resume_reproduces_uninterrupted_run(tmp_path):
    straight = run_lbi_experiment(make_cfg(tmp_path, run_name="a", steps=4, eval_every=4))
    half = run_lbi_experiment(make_cfg(tmp_path, run_name="b", steps=4, eval_every=4, save_every=2))
    # replay b from its step-2 checkpoint by truncating: emulate a crash after step 2
    cfg_b = make_cfg(tmp_path, run_name="c", steps=2, eval_every=4, save_every=2)
    part = run_lbi_experiment(cfg_b)
    cont = run_lbi_experiment(replace(cfg_b, steps=4, resume_from=str(part["root_dir"])))
    a = torch.load(Path(straight["root_dir"]) / "lbi" / "checkpoints" / "latest.pt", weights_only=False)["model_state_dict"]
    c = torch.load(Path(cont["root_dir"]) / "lbi" / "checkpoints" / "latest.pt", weights_only=False)["model_state_dict"]
    # the learning-rate schedule is constant, so a resumed run must land on the same weights
    for key in a:
        assert torch.allclose(a[key], c[key], atol=1e-6), key
    assert half["runs"][0]["steps"] == 4


def test_init_from_and_external_checkpoint_root_and_no_checkpoint(tmp_path):
    src = run_lbi_experiment(make_cfg(tmp_path, run_name="src"))
    init = run_lbi_experiment(make_cfg(tmp_path, run_name="dst", init_from=str(Path(src["root_dir"]) / "lbi"),
                                       checkpoint_root=str(tmp_path / "ckpt_root")))
    run = init["runs"][0]
    assert run["start_step"] == 0 and run["initialized_from"].endswith(".pt")
    assert str(tmp_path / "ckpt_root") in run["latest_checkpoint_path"]
    assert not (Path(init["root_dir"]) / "lbi" / "checkpoints").exists()
    quiet = run_lbi_experiment(make_cfg(tmp_path, run_name="quiet", save_checkpoints=False))
    assert quiet["runs"][0]["latest_checkpoint_path"] == "" and not (Path(quiet["root_dir"]) / "lbi" / "checkpoints").exists()


@pytest.mark.parametrize("kw", [
    dict(backbone="mamba2"), dict(backbone="mamba3"), dict(backbone="hybrid", layer_types="mamba3,transformer"),
    dict(backward_engine="fast", d_conv=0), dict(backward_engine="fast", region_axis="sequence", sequence_regions=4, tie_embeddings=True),
    dict(backward_engine="fast", backbone="mamba2", region_axis="sequence", sequence_regions=2),
    dict(backward_engine="fast", backbone="mamba3"), dict(backward_engine="fast", backbone="hybrid", layer_types="mamba2,transformer"),
    dict(backward_engine="reference_scan"), dict(backward_engine="autograd"), dict(interface_jacobian_mode="recompute", jacobian_basis_chunk=3),
    dict(interface_jacobian_mode="structured"), dict(region_axis="sequence", sequence_regions=2, interface_activation="gelu"),
])
def test_variants_of_the_lbi_run(tmp_path, kw):
    summary = run_lbi_experiment(make_cfg(tmp_path, **kw))
    run = summary["runs"][0]
    assert run["final_train_ce_loss"] == run["final_train_ce_loss"]  # not NaN
    assert run["final_val_ce_loss"] < 10.0


def test_dense_variant_on_the_fast_engine_trains_resumes_and_saves_torch_layout(tmp_path):
    first = run_lbi_experiment(make_cfg(tmp_path, variants="dense", backward_engine="fast", d_conv=0, steps=2))
    run = first["runs"][0]
    assert run["final_train_ce_loss"] == run["final_train_ce_loss"] and run["final_val_ce_loss"] < 10.0
    ckpt = torch.load(Path(first["root_dir"]) / "dense" / "checkpoints" / "latest.pt", weights_only=False)
    from lbi_b200.train.model_builders import build_dense_model

    model = build_dense_model(LBITrainingConfig.from_dict(ckpt["config"]))
    model.load_state_dict(ckpt["model_state_dict"])
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    opt.load_state_dict(ckpt["optimizer_state_dict"])
    resumed = run_lbi_experiment(make_cfg(tmp_path, variants="dense", backward_engine="fast", d_conv=0, steps=3,
                                          resume_from=str(Path(first["root_dir"]))))
    assert resumed["runs"][0]["start_step"] == 2 and resumed["runs"][0]["steps"] == 3
    autograd = run_lbi_experiment(make_cfg(tmp_path, variants="dense", d_conv=0, steps=2, run_name="autograd"))
    assert autograd["runs"][0]["final_train_ce_loss"] == pytest.approx(run["final_train_ce_loss"], rel=2e-3)


def test_fast_engine_checkpoint_round_trips_into_torch_adamw(tmp_path):
    summary = run_lbi_experiment(make_cfg(tmp_path, backward_engine="fast", d_conv=0))
    ckpt = torch.load(Path(summary["root_dir"]) / "lbi" / "checkpoints" / "latest.pt", weights_only=False)
    from lbi_b200.train.model_builders import build_lbi_model

    model = build_lbi_model(LBITrainingConfig.from_dict(ckpt["config"]))
    model.load_state_dict(ckpt["model_state_dict"])
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    opt.load_state_dict(ckpt["optimizer_state_dict"])  # same layout as torch's own AdamW state
    assert len(opt.state_dict()["state"]) == len(list(model.parameters()))


@pytest.mark.parametrize("bad", [
    dict(backbone="rnn"), dict(dtype="float16"), dict(resume_from="a", init_from="b"), dict(data_mode="text_byte", vocab_size=300),
    dict(steps=0), dict(lr_schedule="step"), dict(warmup_steps=10, steps=2), dict(min_lr_ratio=2.0), dict(region_size=0),
    dict(interface_jacobian_mode="magic"), dict(eval_message_ablation="drop"), dict(message_mask_keep_prob=0.0),
    dict(backbone="hybrid", layer_types=""), dict(backbone="mamba3", d_state=8), dict(region_axis="sequence", sequence_regions=0),
    dict(backward_engine="turbo"),
])
def test_config_validation_rejects(tmp_path, bad):
    with pytest.raises(ValueError):
        make_cfg(tmp_path, **bad)


def test_cli_round_trip():
    args = build_arg_parser().parse_args(["--variants", "lbi", "--regime", "native_region_interface", "--dt-rank", "-1",
                                          "--no-save-checkpoints", "--tie-embeddings", "--layers", "2"])
    cfg = config_from_args(args)
    assert cfg.variants == "native_region_interface" and cfg.dt_rank is None and cfg.save_checkpoints is False and cfg.tie_embeddings


def test_text_byte_route(tmp_path):
    text = tmp_path / "corpus.txt"
    text.write_bytes(b"the quick brown fox jumps over the lazy dog. " * 200)
    summary = run_lbi_experiment(make_cfg(tmp_path, data_mode="text_byte", vocab_size=256, train_text_path=str(text)))
    assert summary["runs"][0]["final_val_ce_loss"] < 10.0


def _tiny_corpus(tmp_path):
    train, val = tmp_path / "train.txt", tmp_path / "val.txt"
    train.write_text("hello world\n" * 128 + "bounded interfaces learn\n" * 128, encoding="utf-8")
    val.write_text("hello bounded world\n" * 32, encoding="utf-8")
    return train, val


def test_text_bpe_route_trains_its_tokenizer(tmp_path):
    pytest.importorskip("sentencepiece")
    train, val = _tiny_corpus(tmp_path)
    tok = tmp_path / "tok.model"
    summary = run_lbi_experiment(make_cfg(
        tmp_path, data_mode="text_bpe", train_text_path=str(train), val_text_path=str(val), tokenizer_path=str(tok), vocab_size=320,
        tokenizer_train_bytes=4096, train_tokenizer=True, message_dim=8, message_hidden_dim=16))
    run = summary["runs"][0]
    assert tok.exists() and run["final_train_ce_loss"] == run["final_train_ce_loss"] and run["final_val_ce_loss"] < 10.0
    info = json.loads((Path(summary["root_dir"]) / "lbi" / "data_info.json").read_text())
    assert info["tokenizer_exists"] and info["tokenizer_type"] == "sentencepiece" and info["tokenizer_train_bytes"] == 4096


def test_text_bpe_sharded_route_reads_pretokenized_shards(tmp_path):
    pytest.importorskip("sentencepiece")
    from lbi_b200.data.pretokenize_corpus import pretokenize_text_corpus

    train, val = _tiny_corpus(tmp_path)
    tok, shards = tmp_path / "tok.model", tmp_path / "tokens"
    pretokenize_text_corpus(text_corpus="tiny_shakespeare", train_text_path=str(train), val_text_path=str(val),
                            tokenizer_type="sentencepiece", tokenizer_path=str(tok), vocab_size=320, tokenizer_train_bytes=4096,
                            train_tokenizer=True, shard_tokens=128, output_dir=str(shards))
    assert (shards / "train_manifest.json").exists() and (shards / "val_manifest.json").exists()
    summary = run_lbi_experiment(make_cfg(
        tmp_path, data_mode="text_bpe_sharded", train_text_path=str(train), val_text_path=str(val), tokenizer_path=str(tok),
        token_shards_dir=str(shards), vocab_size=320, save_every=2, message_dim=8, message_hidden_dim=16))
    run = summary["runs"][0]
    assert run["final_train_ce_loss"] == run["final_train_ce_loss"] and run["final_val_ce_loss"] < 10.0
    info = json.loads((Path(summary["root_dir"]) / "lbi" / "data_info.json").read_text())
    assert info["train_manifest_exists"] and info["val_manifest_exists"] and info["token_shards_dir"] == str(shards)


@pytest.mark.parametrize("kind", ["llama", "llama31"])
def test_pretrained_tokenizer_types_cannot_be_trained(tmp_path, kind):
    from lbi_b200.data.bpe_tokenizer import load_text_tokenizer

    train, _ = _tiny_corpus(tmp_path)
    with pytest.raises(ValueError):
        make_cfg(tmp_path, data_mode="text_bpe", train_text_path=str(train), tokenizer_type=kind, train_tokenizer=True, vocab_size=320)
    with pytest.raises(ValueError):
        load_text_tokenizer(tokenizer_type=kind, tokenizer_path=tmp_path / "none", train_path=train, vocab_size=320, train_bytes=1024,
                            force_train=True)
    with pytest.raises(FileNotFoundError):
        load_text_tokenizer(tokenizer_type=kind, tokenizer_path=tmp_path / "none", train_path=train, vocab_size=320, train_bytes=1024)


def test_fineweb_edu_needs_the_sharded_route(tmp_path):
    with pytest.raises(ValueError):
        make_cfg(tmp_path, text_corpus="fineweb_edu", data_mode="text_bpe", vocab_size=320)
    assert make_cfg(tmp_path, text_corpus="fineweb_edu", data_mode="text_bpe_sharded", vocab_size=320).data_mode == "text_bpe_sharded"
