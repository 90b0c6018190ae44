"""Paper tooling on the CPU: launcher presets, post-hoc evaluation, figures/tables from metrics, grad-parity report."""
import csv
import json
from pathlib import Path

import pytest

from lbi_b200.scripts import (evaluate_paper_checkpoints, generate_grad_parity_report, paper_presets, plot_jacobian_diagnostics,
                              plot_message_ablations, plot_training_curves)
from lbi_b200.train.config import LBITrainingConfig, build_arg_parser, config_from_args
from lbi_b200.train.lbi import run_lbi_experiment


def _train(family: Path, run_name: str, variants: str, seed: int, message_dim: int = 4, **kw):
    cfg = LBITrainingConfig(
        variants=variants, backbone="transformer", device="cpu", dtype="float32", output_dir=str(family), run_name=run_name,
        task="copy", vocab_size=32, seq_len=16, train_sequences=32, val_sequences=8, batch_size=2, steps=3, eval_every=1,
        eval_batches=1, log_every=1, save_every=1, layers=2, dim=16, n_heads=2, region_size=1, message_dim=message_dim,
        message_hidden_dim=8, seed=seed, **kw)
    return run_lbi_experiment(cfg)


@pytest.fixture(scope="module")
def family(tmp_path_factory):
    root = tmp_path_factory.mktemp("family")
    _train(root, "dense_seed7", "dense", 7)
    for seed in (7, 8):
        _train(root, f"lbi_r4_seed{seed}", "lbi", seed, eval_all_message_ablations=True, log_interface_jacobian_every=1,
               log_interface_jacobian_suffix=True)
    return root


_LAUNCH_VARS = ("BACKBONE", "MODEL_SCALE", "MESSAGE_DIM", "TOKENIZER_PATH", "OUTPUT_ROOT", "FAMILY_NAME", "FAMILY_DIR", "TARGET_STEPS",
                "TIE_EMBEDDINGS", "TOKENIZER_TYPE", "VOCAB_SIZE", "SEQ_LEN", "FAMILY_SEQ_LEN", "LR_MODEL", "WEIGHT_DECAY", "WARMUP_STEPS",
                "VARIANT_NAME", "RUN_NAME", "OUTPUT_DIR", "SEED", "BACKWARD_ENGINE", "MESSAGE_HIDDEN_DIM", "NPROC_PER_NODE", "MASTER_PORT", "REGION_AXIS", "SEQUENCE_REGIONS")


@pytest.fixture
def launch_env(monkeypatch):
    for var in _LAUNCH_VARS:
        monkeypatch.delenv(var, raising=False)
    monkeypatch.setenv("LBI_LAUNCH_QUIET", "1")
    return monkeypatch


def _parse(cmd):
    at = cmd.index("lbi_b200.train.lbi")
    assert cmd[at - 1] == "-m"
    return config_from_args(build_arg_parser().parse_args(cmd[at + 1:]))


@pytest.mark.parametrize("kind,backbone,dim", [("lbi", "transformer", 64), ("lbi", "hybrid", 32), ("dense", "mamba2", 16),
                                               ("lbi", "mamba3", 16)])
def test_launcher_commands_parse_with_the_training_cli(launch_env, kind, backbone, dim):
    launch_env.setenv("BACKBONE", backbone)
    launch_env.setenv("MESSAGE_DIM", str(dim))
    launch_env.setenv("TOKENIZER_PATH", "/tmp/tok")
    cfg = _parse(paper_presets.build_command(kind))
    arch = paper_presets.ARCHITECTURES[("canonical", backbone)]
    assert (cfg.layers, cfg.dim, cfg.backbone) == (arch.layers, arch.dim, backbone)
    assert cfg.seq_len == 1024 and cfg.batch_size == 1 and cfg.steps == 20000 and cfg.tie_embeddings
    assert cfg.log_every == 20 and cfg.save_every == 5000 and cfg.eval_every == 200 and cfg.eval_batches == 4
    if kind == "lbi":
        assert cfg.message_dim == dim and cfg.region_size == 2 and cfg.interface_jacobian_mode == "recompute"
        assert cfg.jacobian_basis_chunk == 32 and cfg.message_hidden_dim == 0 and cfg.message_scale_init == 0.5
        assert cfg.lr_model == paper_presets.lbi_learning_rate(backbone, dim)
    else:
        assert cfg.lr_model == paper_presets.DENSE_RECIPE[backbone][0]
    if backbone in ("mamba3", "hybrid"):
        assert cfg.device == "cuda" and cfg.dtype == "bfloat16" and cfg.ngroups == 1


def test_launcher_choices_follow_the_tables_of_the_reference_launchers(launch_env):
    """Values read off scripts/train_lbi_paper.sh:44-92 / :146-176 and scripts/train_dense_paper.sh:40-83 of the reference."""
    lr, dense, warm, wd = (paper_presets.lbi_learning_rate, paper_presets.dense_learning_rate, paper_presets.warmup_steps,
                           paper_presets.weight_decay)
    assert [lr("mamba2", 64), lr("mamba3", 64), lr("hybrid", 64), lr("hybrid", 32), lr("hybrid", 16), lr("transformer", 64)] == \
        [8e-4, 3e-4, 3e-4, 3e-4, 6e-4, 6e-4]
    assert [lr("mamba2", 64, "large"), lr("mamba3", 64, "large"), lr("hybrid", 16, "large"), lr("transformer", 8, "large")] == \
        [6e-4, 3e-4, 3e-4, 6e-4]
    assert [dense("mamba2"), dense("mamba3"), dense("hybrid"), dense("transformer"), dense("mamba3", "large"), dense("hybrid", "large")] == \
        [8e-4, 6e-4, 6e-4, 6e-4, 3e-4, 3e-4]
    assert [warm("mamba3"), warm("hybrid"), warm("mamba2"), warm("transformer"), warm("mamba3", "large")] == [500, 500, 1000, 1000, 1000]
    assert [wd("mamba2"), wd("mamba3"), wd("hybrid"), wd("transformer"), wd("mamba3", "large"), wd("mamba2", "large")] == \
        [0.03, 0.03, 0.03, 0.01, 0.1, 0.01]
    assert [paper_presets.step_tag(n) for n in (20000, 2_000_000, 1500)] == ["20ksteps", "2msteps", "1500steps"]
    assert [paper_presets.tokenizer_tag(*a) for a in (("llama", 32000), ("llama31", 128256), ("sentencepiece", 32000), ("llama", 1000))] == \
        ["llama32k", "llama31", "sentencepiece32000", "llama1000"]
    name = paper_presets.family_name(backbone="transformer", scale="canonical", seq_len=1024, steps=20000, tokenizer_tag="llama32k", tied=True)
    assert name == "paper_transformer_12l_512d_llama32k_tied_seq1024_20ksteps"
    assert paper_presets.family_from_env() == ("paper_mamba3_14l_768d_llama32k_tied_seq1024_20ksteps",
                                               "out/region_interface/paper_mamba3_14l_768d_llama32k_tied_seq1024_20ksteps")

    # leading positional arguments: output root, then backbone; runs land in <root>/<family>/<run name>/<variant>
    cmd = paper_presets.build_command("lbi", ["/data/runs", "mamba2", "--eval-every", "7"])
    cfg = _parse(cmd)
    assert cfg.backbone == "mamba2" and cfg.eval_every == 7 and cfg.message_dim == 64 and cfg.run_name == "lbi_r64_seed7"
    assert cfg.output_dir == "/data/runs/paper_mamba2_14l_768d_llama32k_tied_seq1024_20ksteps" and cfg.weight_decay == 0.03
    launch_env.setenv("MODEL_SCALE", "large")
    launch_env.setenv("BACKBONE", "mamba3")
    launch_env.setenv("TIE_EMBEDDINGS", "no")
    launch_env.setenv("BACKWARD_ENGINE", "fast")
    cfg = _parse(paper_presets.build_command("dense"))
    assert (cfg.layers, cfg.lr_model, cfg.weight_decay, cfg.warmup_steps, cfg.tie_embeddings) == (28, 3e-4, 0.1, 1000, False)
    assert cfg.run_name == "dense_seed7" and cfg.output_dir.endswith("paper_mamba3_28l_768d_llama32k_untied_seq1024_20ksteps")
    assert _parse(paper_presets.build_command("lbi")).backward_engine == "fast"
    assert _parse(paper_presets.build_command("dense")).backward_engine == "fast"
    launch_env.setenv("NPROC_PER_NODE", "8")
    multi = paper_presets.build_command("lbi")
    assert multi[1:7] == ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=8", "--master-addr", "127.0.0.1"]
    assert _parse(multi).backward_engine == "fast"
    launch_env.setenv("REGION_AXIS", "sequence")
    cut = _parse(paper_presets.build_command("lbi"))
    assert (cut.region_axis, cut.sequence_regions) == ("sequence", 8)
    launch_env.delenv("REGION_AXIS")
    with pytest.raises(SystemExit):
        paper_presets.build_command("dense")
    launch_env.delenv("NPROC_PER_NODE")
    for var, bad in (("MODEL_SCALE", "huge"), ("BACKBONE", "rnn"), ("TIE_EMBEDDINGS", "maybe"), ("TARGET_STEPS", "0")):
        launch_env.setenv(var, bad)
        with pytest.raises(SystemExit):
            paper_presets.build_command("lbi")
        launch_env.setenv(var, {"MODEL_SCALE": "large", "BACKBONE": "mamba3", "TIE_EMBEDDINGS": "no", "TARGET_STEPS": "20000"}[var])


def test_shell_launchers_share_the_family_name(launch_env, family, tmp_path):
    """train -> evaluate -> plot through the .sh files: the evaluation and plotting launchers find the runs under the family
    directory the training launcher would write to."""
    import shutil
    import subprocess
    import sys

    scripts = Path(paper_presets.__file__).parent
    env = {k: v for k, v in __import__("os").environ.items() if k not in _LAUNCH_VARS}
    env.update(PYTHON_BIN=sys.executable, BACKBONE="transformer", OUTPUT_ROOT=str(tmp_path / "runs"), LBI_LAUNCH_QUIET="1",
               PYTHONPATH=str(scripts.parent.parent) + ":" + env.get("PYTHONPATH", ""))
    dry = subprocess.run(["bash", str(scripts / "train_lbi_paper.sh"), "--dry-run"], env=env, capture_output=True, text=True, check=True)
    name = "paper_transformer_12l_512d_llama32k_tied_seq1024_20ksteps"
    assert f"--output-dir {tmp_path / 'runs' / name}" in dry.stdout and "--run-name lbi_r64_seed7" in dry.stdout
    shutil.copytree(family, tmp_path / "runs" / name)  # stand-in for the trained family
    env.update(EVAL_OUTPUT_ROOT=str(tmp_path / "evals"), EVAL_BATCHES="1", CHECKPOINT="latest", DEVICE="cpu")
    subprocess.run(["bash", str(scripts / "evaluate_paper_checkpoints.sh")], env=env, capture_output=True, text=True, check=True)
    assert len(json.loads((tmp_path / "evals" / name / "lm_eval_summary.json").read_text())) == 3
    env.update(LABEL_MODE="regime", REGIMES="lbi")
    subprocess.run(["bash", str(scripts / "plot_paper_results.sh")], env=env, capture_output=True, text=True, check=True)
    groups = json.loads((tmp_path / "runs" / name / "plots_regime" / "group_summary.json").read_text())
    assert [g["label"] for g in groups] == ["lbi"] and (tmp_path / "runs" / name / "ablation_plots_regime" / "ablation_summary.csv").exists()


def test_posthoc_evaluation_of_named_run_directories(family, tmp_path):
    one = family / "lbi_r4_seed8" / "lbi"
    rows = evaluate_paper_checkpoints.main(["--family", str(family), "--run-dir", str(one), "--run-dir", str(family / "dense_seed7" / "dense"),
                                            "--output-dir", str(tmp_path / "named"), "--eval-batches", "1", "--checkpoint", "latest",
                                            "--device", "cpu"])
    assert [r["label"] for r in rows] == ["lbi_r4_seed8", "dense_seed7"] and (tmp_path / "named" / "lm_eval_summary.csv").exists()
    single = evaluate_paper_checkpoints.main([str(one), "--output-dir", str(tmp_path / "single"), "--eval-batches", "1",
                                              "--checkpoint", "latest", "--device", "cpu"])
    assert len(single) == 1 and single[0]["posthoc_val_ce_loss"] == rows[0]["posthoc_val_ce_loss"]
    with pytest.raises(SystemExit):
        evaluate_paper_checkpoints.main(["--eval-batches", "1"])


def test_posthoc_evaluation_writes_summary(family, tmp_path):
    rows = evaluate_paper_checkpoints.main([str(family), "--output-dir", str(tmp_path / "ev"), "--eval-batches", "2",
                                            "--checkpoint", "latest", "--device", "cpu"])
    assert [r["label"] for r in rows] == ["dense_seed7", "lbi_r4_seed7", "lbi_r4_seed8"]
    stored = json.loads((tmp_path / "ev" / "lm_eval_summary.json").read_text())
    assert len(stored) == 3 and all(r["posthoc_val_ce_loss"] > 0 and r["eval_tokens"] == 2 * 2 * 16 for r in stored)
    assert all(r["posthoc_val_ppl"] == pytest.approx(2.718281828 ** r["posthoc_val_ce_loss"], rel=1e-4) for r in stored)
    with (tmp_path / "ev" / "lm_eval_summary.csv").open() as fh:
        assert len(list(csv.DictReader(fh))) == 3


def test_training_curve_outputs(family, tmp_path):
    out = plot_training_curves.main([str(family), "--output-dir", str(tmp_path / "plots")])
    names = {Path(f).stem for f in out["figures"]}
    assert {"ce_vs_tokens", "ce_vs_step", "paper_val_ce_vs_tokens", "paper_val_ce_vs_step", "paper_ce_vs_tokens",
            "tokens_per_s_vs_step", "message_diagnostics", "val_summary_bar"} <= names
    groups = {g["label"]: g for g in json.loads((tmp_path / "plots" / "group_summary.json").read_text())}
    assert groups["lbi r4"]["num_runs"] == 2 and groups["dense"]["num_runs"] == 1
    lbi = groups["lbi r4"]
    assert (lbi["backbones"], lbi["regimes"], lbi["seeds"], lbi["variants"], lbi["region_sizes"], lbi["seq_lens"]) == \
        ("transformer", "lbi", "7,8", "lbi_r4_seed7,lbi_r4_seed8", "1", "16")
    assert lbi["mean_total_params"] > 0 and lbi["std_total_params"] == 0.0 and lbi["std_final_val_ce"] >= 0.0
    assert lbi["mean_final_val_ce"] == pytest.approx(lbi["final_val_ce_mean"]) and groups["dense"]["region_sizes"] == ""
    assert (tmp_path / "plots" / "group_summary.csv").exists()
    only_lbi = plot_training_curves.main([str(family), "--output-dir", str(tmp_path / "p2"), "--regimes", "native_region_interface",
                                          "--label-mode", "rank_region"])
    assert [g["label"] for g in only_lbi["groups"]] == ["lbi r4"] and only_lbi["groups"][0]["num_runs"] == 2
    for mode, labels in (("backbone", {"transformer"}), ("regime", {"dense", "lbi"}), ("region_size", {"dense", "region=1"}),
                         ("backbone_regime", {"transformer:dense", "transformer:lbi"})):
        got = plot_training_curves.main([str(family), "--output-dir", str(tmp_path / f"p_{mode}"), "--label-mode", mode])
        assert {g["label"] for g in got["groups"]} == labels
    anchored = plot_training_curves.main([str(family), "--output-dir", str(tmp_path / "p_anch"), "--include-variant-regex",
                                          r"^(dense_seed[789]|lbi_r(4|32|64)_seed[78])$", "--exclude-variant-regex", r"^lbi_r4_seed8$"])
    assert {g["label"]: g["num_runs"] for g in anchored["groups"]} == {"dense": 1, "lbi r4": 1}
    assert plot_training_curves.run_variant(family, family / "lbi_r4_seed7" / "lbi", {}) == "lbi_r4_seed7"
    assert plot_training_curves.run_variant(family.parent, family / "lbi_r4_seed7" / "lbi", {}) == family.name
    assert plot_training_curves.run_variant(family / "x", family / "x" / "lbi", {"message_dim": 4, "seed": 7}) == "x"
    out_dir = plot_training_curves.generate_training_plots([family], output_dir=tmp_path / "fn", regimes=["native_region_interface"],
                                                           label_mode="rank_region", smooth_window=1)
    assert out_dir == tmp_path / "fn" and (out_dir / "group_summary.json").exists()
    assert plot_message_ablations.generate_message_ablation_plots([family], output_dir=tmp_path / "fn_abl") == tmp_path / "fn_abl"
    none_left = plot_message_ablations.main([str(family), "--output-dir", str(tmp_path / "abl_none"), "--exclude-variant-regex", "lbi_r4"])
    assert none_left["summary"] == []


def test_ablation_and_jacobian_outputs(family, tmp_path):
    out = plot_message_ablations.main([str(family), "--output-dir", str(tmp_path / "abl")])
    stems = {Path(f).stem for f in out["figures"]}
    assert {"transformer_ablation_ce_vs_tokens", "transformer_ablation_final_ce"} <= stems
    with (tmp_path / "abl" / "ablation_summary.csv").open() as fh:
        abl_rows = list(csv.DictReader(fh))
        splits = {r["split"] for r in abl_rows}
    assert {"backbone", "split", "num_runs", "mean_final_ce", "std_final_ce"} <= set(abl_rows[0])
    assert {"val", "val_zero_all", "val_noise", "val_mask"} <= splits
    out = plot_jacobian_diagnostics.main([str(family), "--output-dir", str(tmp_path / "jac"), "--min-step", "1"])
    assert out["table"][0]["message_dim"] == 4 and out["table"][0]["num_runs"] == 2
    first = out["table"][0]
    assert (first["rank"], first["num_seeds"], first["seeds"]) == (4, 2, "7,8") and "jac_suffix_spec_mean_std" in first
    tex = (tmp_path / "jac" / "jacobian_final_summary.tex").read_text()
    assert tex.count("$\\pm$") == 3 and tex.splitlines()[3].startswith("4 & ")
    assert (tmp_path / "jac" / "jacobian_final_summary.csv").exists() and (tmp_path / "jac" / "jacobian_final_summary.tex").exists()
    assert any(Path(f).stem == "jacobian_spec_mean_vs_tokens" for f in out["figures"])


def test_grad_parity_report(tmp_path):
    rows = generate_grad_parity_report.generate_report(
        output_dir=tmp_path, case_names=["transformer_multi_region", "mamba2_multi_region", "transformer_multi_region_cuda_bf16"],
        preset="test", plot=True, interface_jacobian_mode="recompute", jacobian_basis_chunk=3)
    by_name = {r["case_name"]: r for r in rows}
    assert by_name["transformer_multi_region"]["status"] == "ok" and by_name["transformer_multi_region"]["num_trials_passed"] == 1
    for name in ("case_summary.csv", "case_summary.json", "case_summary.md", "trial_summary.csv", "per_parameter.csv",
                 "report_config.json", "summary.csv", "summary.json", "summary.md", "paper_table.csv", "paper_table.tex"):
        assert (tmp_path / name).exists(), name
    assert "Transformer" in (tmp_path / "paper_table.tex").read_text()
    assert generate_grad_parity_report.latex_number(1.5e-9) == r"$1.50\times 10^{-9}$"


def test_attention_benchmark_takes_the_sweep_flags_of_the_reference():
    import torch

    from lbi_b200.benchmarks import time_attention_pullback as bench

    default = bench.sweep_from_args(bench.build_parser().parse_args([]))
    assert default == {"batches": (8,), "heads": (16,), "seqs": (128, 512, 2048), "dims": (64, 128), "basis": (4, 16),
                       "dtypes": (torch.float16, torch.bfloat16)}
    args = bench.build_parser().parse_args(
        ["--batches", "1", "--heads", "8", "--seq-lens", "128,512", "--head-dims", "64", "--basis-sizes", "4", "--dtype", "float16",
         "--causal", "true", "--warmup", "5", "--iters", "20", "--include-autograd", "--include-simple", "--include-fa2-loop",
         "--include-fa2-mma-pblock4", "--skip-torch-formula", "--check", "--check-max-tokens", "131072", "--no-default-kernel"])
    assert bench.sweep_from_args(args) == {"batches": (1,), "heads": (8,), "seqs": (128, 512), "dims": (64,), "basis": (4,),
                                           "dtypes": (torch.float16,)}
    assert bench.modes_for_cell(args, torch.float16, 64, 8, 128, True) == ["fa2_loop", "reference_wmma_pblock4", "dense", "autograd"]
    assert bench.modes_for_cell(args, torch.float32, 64, 8, 128, False) == ["dense", "autograd"]
    row = dict(dtype="float16", seq_len=128, head_dim=64, basis=4, batch=8, heads=16)
    assert bench.cell_name(row) == "float16_T128_D64_P4" and bench.cell_name({**row, "batch": 1}) == "float16_T128_D64_P4_B1_H16"
    q, k, v, do = torch.randn(1, 2, 8, 4), torch.randn(1, 2, 8, 4), torch.randn(1, 2, 8, 4), torch.randn(1, 3, 2, 8, 4)
    from lbi_b200.ops.attention import attention_input_pullback_basis

    for got, want in zip(bench.autograd_mode(q, k, v, do, 0.5), attention_input_pullback_basis(q, k, v, do, scale=0.5, kernel_mode="dense")):
        assert torch.allclose(got, want, atol=1e-5)
