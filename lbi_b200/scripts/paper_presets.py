"""Architecture and optimiser presets of the paper runs, and the launcher that turns them into a training command.

The reference keeps these tables inside two bash wrappers (scripts/train_lbi_paper.sh:226-339,
scripts/train_dense_paper.sh) that read their settings from environment variables; here the tables are data, the
launcher is ``python -m lbi_b200.scripts.paper_presets {lbi,dense}``, and the same environment variables are honoured
(BACKBONE, MODEL_SCALE, TARGET_STEPS, SEED, MESSAGE_DIM, REGION_SIZE, VARIANT_NAME, RUN_NAME, OUTPUT_ROOT, LR_MODEL, ...),
so the two ``.sh`` files beside this module are one-line shims.
"""
from __future__ import annotations

import argparse
import os
import shlex
import sys
from dataclasses import dataclass, field


@dataclass(frozen=True)
class ArchPreset:
    layers: int
    dim: int
    flags: dict = field(default_factory=dict)


_HYBRID_UNIT = ("mamba3", "mamba3", "mamba3", "transformer")

# (scale, backbone) -> architecture (reference scripts/train_lbi_paper.sh:226-339)
ARCHITECTURES: dict[tuple[str, str], ArchPreset] = {
    ("canonical", "mamba2"): ArchPreset(14, 768, dict(d_state=64, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=128)),
    ("canonical", "mamba3"): ArchPreset(14, 768, dict(d_state=128, expand=2, headdim=64, chunk_size=64)),
    ("canonical", "transformer"): ArchPreset(12, 512, dict(n_heads=8, n_kv_heads=4, attn_head_dim=64, d_intermediate=2048)),
    ("canonical", "hybrid"): ArchPreset(12, 768, dict(d_state=128, expand=2, headdim=64, chunk_size=64, n_heads=12, n_kv_heads=6,
                                                      attn_head_dim=64, d_intermediate=3072,
                                                      layer_types=",".join(_HYBRID_UNIT * 3))),
    ("large", "mamba2"): ArchPreset(28, 768, dict(d_state=64, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=128)),
    ("large", "mamba3"): ArchPreset(28, 768, dict(d_state=128, expand=2, headdim=64, chunk_size=64)),
    ("large", "transformer"): ArchPreset(12, 768, dict(n_heads=12, n_kv_heads=6, attn_head_dim=64, d_intermediate=3072)),
    ("large", "hybrid"): ArchPreset(20, 768, dict(d_state=128, expand=2, headdim=64, chunk_size=64, n_heads=12, n_kv_heads=6,
                                                  attn_head_dim=64, d_intermediate=3072,
                                                  layer_types=",".join(_HYBRID_UNIT * 5))),
}

# backbone -> (dense lr, weight decay, warm-up)  (reference scripts/README.md:79-86)
DENSE_RECIPE = {"mamba2": (8e-4, 0.03, 1000), "mamba3": (6e-4, 0.03, 500), "transformer": (6e-4, 0.01, 1000),
                "hybrid": (6e-4, 0.03, 500)}


def lbi_learning_rate(backbone: str, message_dim: int) -> float:
    """Selected LBI learning rates (reference scripts/README.md:90-98)."""
    if backbone == "mamba2":
        return 8e-4
    if backbone == "mamba3":
        return 3e-4
    if backbone == "transformer":
        return 6e-4
    return 6e-4 if message_dim <= 16 else 3e-4


def family_name(*, backbone: str, scale: str, seq_len: int, steps: int, tokenizer_tag: str, tied: bool) -> str:
    """Directory name shared by the runs of one comparison family (training, evaluation and plotting agree on it)."""
    return f"{backbone}_{scale}_seq{seq_len}_{steps // 1000}k_{tokenizer_tag}_{'tied' if tied else 'untied'}"


def _env(name: str, default):
    raw = os.environ.get(name)
    if raw is None or raw == "":
        return default
    return type(default)(raw) if not isinstance(default, bool) else raw.lower() in {"1", "true", "yes"}


def build_command(kind: str, extra: list[str] | None = None) -> list[str]:
    backbone = _env("BACKBONE", "mamba3")
    scale = _env("MODEL_SCALE", "canonical")
    if (scale, backbone) not in ARCHITECTURES:
        raise SystemExit(f"unknown MODEL_SCALE:BACKBONE {scale}:{backbone}")
    arch = ARCHITECTURES[(scale, backbone)]
    steps = _env("TARGET_STEPS", 20000)
    seed = _env("SEED", 7)
    seq_len = _env("SEQ_LEN", 1024)
    batch = _env("BATCH_SIZE", 1)
    tied = _env("TIE_EMBEDDINGS", True)
    tokenizer_type = _env("TOKENIZER_TYPE", "llama")
    tokenizer_path = _env("TOKENIZER_PATH", "")
    vocab = _env("VOCAB_SIZE", 32000)
    message_dim = _env("MESSAGE_DIM", 32)
    dense_lr, wd, warmup = DENSE_RECIPE[backbone]
    lr = dense_lr if kind == "dense" else lbi_learning_rate(backbone, message_dim)
    lr = _env("LR_MODEL", lr)
    wd = _env("WEIGHT_DECAY", wd)
    warmup = _env("WARMUP_STEPS", warmup)
    tag = _env("TOKENIZER_TAG", "llama32k" if tokenizer_type == "llama" else f"{tokenizer_type}{vocab}")
    family = _env("FAMILY_NAME", family_name(backbone=backbone, scale=scale, seq_len=seq_len, steps=steps, tokenizer_tag=tag, tied=tied))
    default_variant = f"dense_seed{seed}" if kind == "dense" else f"lbi_r{message_dim}_seed{seed}"
    run_name = _env("RUN_NAME", _env("VARIANT_NAME", default_variant))
    out_root = _env("OUTPUT_ROOT", "out/region_interface")
    out_dir = _env("OUTPUT_DIR", os.path.join(out_root, family, run_name))

    args = [
        _env("PYTHON_BIN", sys.executable), "-m", "lbi_b200.train.lbi",
        "--variants", "dense" if kind == "dense" else "lbi", "--output-dir", out_dir, "--run-name", run_name,
        "--backbone", backbone, "--layers", str(arch.layers), "--dim", str(arch.dim),
        "--data-mode", _env("DATA_MODE", "text_bpe_sharded"), "--text-corpus", _env("TEXT_CORPUS", "fineweb_edu"),
        "--tokenizer-type", tokenizer_type, "--vocab-size", str(vocab), "--seq-len", str(seq_len), "--batch-size", str(batch),
        "--steps", str(steps), "--seed", str(seed), "--lr-model", str(lr), "--weight-decay", str(wd),
        "--warmup-steps", str(warmup), "--lr-schedule", _env("LR_SCHEDULE", "cosine"),
        "--min-lr-ratio", str(_env("MIN_LR_RATIO", 0.1)), "--grad-clip", str(_env("GRAD_CLIP", 1.0)),
        "--eval-every", str(_env("EVAL_EVERY", 200)), "--eval-batches", str(_env("EVAL_BATCHES", 4)),
        "--log-every", str(_env("LOG_EVERY", 50)), "--save-every", str(_env("SAVE_EVERY", 1000)),
    ]
    if tokenizer_path:
        args += ["--tokenizer-path", tokenizer_path]
    if tied:
        args += ["--tie-embeddings"]
    ckpt_root = _env("CHECKPOINT_ROOT", "")
    if ckpt_root:
        args += ["--checkpoint-root", ckpt_root]
    for key, value in arch.flags.items():
        args += ["--" + key.replace("_", "-"), str(value)]
    if backbone in {"mamba3", "hybrid"}:
        args += ["--dtype", "bfloat16", "--device", "cuda"]
    if kind == "lbi":
        args += [
            "--region-size", str(_env("REGION_SIZE", 2)), "--message-dim", str(message_dim),
            "--message-hidden-dim", str(_env("MESSAGE_HIDDEN_DIM", arch.dim)),
            "--message-scale-init", str(_env("MESSAGE_SCALE_INIT", 0.1)),
            "--interface-jacobian-mode", _env("INTERFACE_JACOBIAN_MODE", "recompute"),
            "--jacobian-basis-chunk", str(_env("JACOBIAN_BASIS_CHUNK", 32)),
        ]
    return args + list(extra or [])


def main(argv: list[str] | None = None) -> None:
    p = argparse.ArgumentParser(description="Launch one paper run (settings from environment variables).")
    p.add_argument("kind", choices=("lbi", "dense"))
    p.add_argument("--dry-run", action="store_true", help="print the training command instead of running it")
    ns, extra = p.parse_known_args(argv)
    cmd = build_command(ns.kind, extra)
    if ns.dry_run:
        print(" ".join(shlex.quote(c) for c in cmd))
        return
    os.execv(cmd[0], cmd)


if __name__ == "__main__":
    main()
