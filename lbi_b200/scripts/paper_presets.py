"""Architecture and optimiser presets of the paper runs, and the launcher that turns them into a training command.

The reference keeps these tables inside bash wrappers (scripts/train_lbi_paper.sh, scripts/train_dense_paper.sh,
scripts/evaluate_paper_checkpoints.sh, scripts/plot_paper_results.sh) that read their settings from environment variables;
here the tables are data, the launcher is ``python -m lbi_b200.scripts.paper_presets {lbi,dense}`` and the ``.sh`` files beside
this module are shims over it.  The same variables are honoured with the same defaults (OUTPUT_ROOT and BACKBONE also as leading
arguments, MODEL_SCALE, TARGET_STEPS, SEQ_LEN, BATCH_SIZE, SEED, MESSAGE_DIM, MESSAGE_HIDDEN_DIM, MESSAGE_SCALE_INIT, REGION_SIZE,
LR_MODEL, WARMUP_STEPS, WEIGHT_DECAY, TIE_EMBEDDINGS, TOKENIZER_TYPE / PATH, VOCAB_SIZE, FAMILY_NAME, VARIANT_NAME, RUN_NAME,
OUTPUT_DIR, CHECKPOINT_ROOT, ...), the learning rate / warm-up / weight decay follow the same scale-and-backbone rules, and runs land
in ``<OUTPUT_ROOT>/<family>/<run name>/<variant>`` with the same family name, so the evaluation and plotting launchers of either
code base find them.  Added: BACKWARD_ENGINE (e.g. ``fast``), NPROC_PER_NODE (with BACKWARD_ENGINE=fast: one process per GPU
through ``torch.distributed.run``), MASTER_PORT, REGION_AXIS / SEQUENCE_REGIONS, DATA_MODE, TEXT_CORPUS.
"""
from __future__ import annotations

import argparse
import os
import shlex
import sys
from dataclasses import dataclass, field


@dataclass(frozen=True)
class ArchPreset:
    """Layers, width and the remaining architecture flags of one (scale, backbone) pair."""

    layers: int
    dim: int
    flags: dict = field(default_factory=dict)


_HYBRID_UNIT = ("mamba3", "mamba3", "mamba3", "transformer")

# (scale, backbone) -> architecture (reference scripts/train_lbi_paper.sh:226-339)
ARCHITECTURES: dict[tuple[str, str], ArchPreset] = {
    ("canonical", "mamba2"): ArchPreset(14, 768, dict(d_state=64, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=128)),
    ("canonical", "mamba3"): ArchPreset(14, 768, dict(d_state=128, expand=2, headdim=64, ngroups=1, chunk_size=64)),
    ("canonical", "transformer"): ArchPreset(12, 512, dict(n_heads=8, n_kv_heads=4, attn_head_dim=64, d_intermediate=2048)),
    ("canonical", "hybrid"): ArchPreset(12, 768, dict(d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=64, n_heads=12, n_kv_heads=6,
                                                      attn_head_dim=64, d_intermediate=3072,
                                                      layer_types=",".join(_HYBRID_UNIT * 3))),
    ("large", "mamba2"): ArchPreset(28, 768, dict(d_state=64, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=128)),
    ("large", "mamba3"): ArchPreset(28, 768, dict(d_state=128, expand=2, headdim=64, ngroups=1, chunk_size=64)),
    ("large", "transformer"): ArchPreset(12, 768, dict(n_heads=12, n_kv_heads=6, attn_head_dim=64, d_intermediate=3072)),
    ("large", "hybrid"): ArchPreset(20, 768, dict(d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=64, n_heads=12, n_kv_heads=6,
                                                  attn_head_dim=64, d_intermediate=3072,
                                                  layer_types=",".join(_HYBRID_UNIT * 5))),
}


# ---- optimiser settings by scale and backbone, as the reference's launchers choose them when the environment does not
#      (scripts/train_lbi_paper.sh:44-92, scripts/train_dense_paper.sh:40-83)
def lbi_learning_rate(backbone: str, message_dim: int, scale: str = "canonical") -> float:
    if scale == "canonical" and backbone == "mamba2":
        return 8e-4
    if scale == "canonical" and backbone == "mamba3":
        return 3e-4
    if scale == "canonical" and backbone == "hybrid":
        return 3e-4 if message_dim in (32, 64) else 6e-4
    return 6e-4 if backbone in ("mamba2", "transformer") else 3e-4


def dense_learning_rate(backbone: str, scale: str = "canonical") -> float:
    if scale == "canonical" and backbone == "mamba2":
        return 8e-4
    if scale == "canonical" and backbone in ("mamba3", "hybrid"):
        return 6e-4
    return 6e-4 if backbone in ("mamba2", "transformer") else 3e-4


def warmup_steps(backbone: str, scale: str = "canonical") -> int:
    return 500 if (scale == "canonical" and backbone in ("mamba3", "hybrid")) else 1000


def weight_decay(backbone: str, scale: str = "canonical") -> float:
    if scale == "canonical" and backbone in ("mamba2", "mamba3", "hybrid"):
        return 0.03
    return 0.1 if backbone == "mamba3" else 0.01


# backbone -> (dense lr, weight decay, warm-up) at the canonical scale
DENSE_RECIPE = {b: (dense_learning_rate(b), weight_decay(b), warmup_steps(b)) for b in ("mamba2", "mamba3", "transformer", "hybrid")}


def step_tag(steps: int) -> str:
    if steps % 1_000_000 == 0:
        return f"{steps // 1_000_000}msteps"
    if steps % 1000 == 0:
        return f"{steps // 1000}ksteps"
    return f"{steps}steps"


def tokenizer_tag(tokenizer_type: str, vocab_size: int) -> str:
    if tokenizer_type == "llama" and int(vocab_size) == 32000:
        return "llama32k"
    if tokenizer_type == "llama31":
        return "llama31"
    return f"{tokenizer_type}{vocab_size}"


def arch_tag(backbone: str, scale: str) -> str:
    arch = ARCHITECTURES[(scale, backbone)]
    return f"{arch.layers}l_{arch.dim}d"


def family_name(*, backbone: str, scale: str, seq_len: int, steps: int, tokenizer_tag: str, tied: bool) -> str:
    """Directory shared by the runs of one comparison family; the training, evaluation and plotting launchers agree on it
    (``paper_<backbone>_<layers>l_<dim>d_<tokenizer>_<tied|untied>_seq<T>_<steps>``, reference scripts/train_lbi_paper.sh:171)."""
    return f"paper_{backbone}_{arch_tag(backbone, scale)}_{tokenizer_tag}_{'tied' if tied else 'untied'}_seq{seq_len}_{step_tag(steps)}"


_POSITIONAL: dict[str, str] = {}  # OUTPUT_ROOT / BACKBONE given as leading arguments of the current command


def _env(name: str, default):
    raw = os.environ.get(name, _POSITIONAL.get(name))
    if raw is None or raw == "":
        return default
    return type(default)(raw) if not isinstance(default, bool) else raw.lower() in {"1", "true", "yes"}


def _tied_from_env() -> bool:
    raw = os.environ.get("TIE_EMBEDDINGS", "true").lower()
    if raw in {"true", "1", "yes"}:
        return True
    if raw in {"false", "0", "no"}:
        return False
    raise SystemExit(f"TIE_EMBEDDINGS must be true/false, got '{raw}'")


def family_from_env(seq_len_var: str = "SEQ_LEN") -> tuple[str, str]:
    """(family name, family directory) from the environment the launchers share: FAMILY_NAME / FAMILY_DIR when set, else built
    from BACKBONE, MODEL_SCALE, TARGET_STEPS, TOKENIZER_TYPE, VOCAB_SIZE, TIE_EMBEDDINGS and the sequence length."""
    backbone, scale = _env("BACKBONE", "mamba3"), _env("MODEL_SCALE", "canonical")
    if scale not in ("canonical", "large"):
        raise SystemExit(f"MODEL_SCALE must be canonical or large, got '{scale}'")
    if (scale, backbone) not in ARCHITECTURES:
        raise SystemExit(f"Unsupported BACKBONE='{backbone}'. Expected one of: mamba2, mamba3, transformer, hybrid")
    name = _env("FAMILY_NAME", family_name(
        backbone=backbone, scale=scale, seq_len=_env(seq_len_var, 1024), steps=_env("TARGET_STEPS", 20000),
        tokenizer_tag=tokenizer_tag(_env("TOKENIZER_TYPE", "llama"), _env("VOCAB_SIZE", 32000)), tied=_tied_from_env()))
    return name, _env("FAMILY_DIR", os.path.join(_env("OUTPUT_ROOT", "out/region_interface").rstrip("/"), name))


def build_command(kind: str, extra: list[str] | None = None) -> list[str]:
    """The training command of one paper run.  Leading arguments that are not flags fill OUTPUT_ROOT and then BACKBONE when the
    environment does not set them, as in the reference's launchers (scripts/train_lbi_paper.sh:7-23)."""
    extra = list(extra or [])
    _POSITIONAL.clear()
    for var in ("OUTPUT_ROOT", "BACKBONE"):
        if var not in os.environ and extra and not extra[0].startswith("--"):
            _POSITIONAL[var] = extra.pop(0)
    backbone = _env("BACKBONE", "mamba3")
    scale = _env("MODEL_SCALE", "canonical")
    if scale not in ("canonical", "large"):
        raise SystemExit(f"MODEL_SCALE must be canonical or large, got '{scale}'")
    if (scale, backbone) not in ARCHITECTURES:
        raise SystemExit(f"Unsupported BACKBONE='{backbone}'. Expected one of: mamba2, mamba3, transformer, hybrid")
    arch = ARCHITECTURES[(scale, backbone)]
    steps = _env("TARGET_STEPS", 20000)
    seed = _env("SEED", 7)
    seq_len = _env("SEQ_LEN", 1024)
    batch = _env("BATCH_SIZE", 1)
    for label, value in (("BATCH_SIZE", batch), ("SEQ_LEN", seq_len), ("TARGET_STEPS", steps)):
        if value <= 0:
            raise SystemExit(f"{label} must be > 0")
    tied = _tied_from_env()
    tokenizer_type = _env("TOKENIZER_TYPE", "llama")
    tokenizer_path = _env("TOKENIZER_PATH", "")
    vocab = _env("VOCAB_SIZE", 32000)
    message_dim = _env("MESSAGE_DIM", 64)
    lr = dense_learning_rate(backbone, scale) if kind == "dense" else lbi_learning_rate(backbone, message_dim, scale)
    lr = _env("LR_MODEL", lr)
    wd = _env("WEIGHT_DECAY", weight_decay(backbone, scale))
    warmup = _env("WARMUP_STEPS", warmup_steps(backbone, scale))
    family, _ = family_from_env()
    default_variant = f"dense_seed{seed}" if kind == "dense" else f"lbi_r{message_dim}_seed{seed}"
    variant_name = _env("VARIANT_NAME", default_variant)
    run_name = _env("RUN_NAME", variant_name)
    out_root = _env("OUTPUT_ROOT", "out/region_interface")
    out_dir = _env("OUTPUT_DIR", os.path.join(out_root.rstrip("/"), family))  # runs land in <family>/<run name>/<variant>

    nproc = _env("NPROC_PER_NODE", 1)
    if nproc > 1 and (kind != "lbi" or _env("BACKWARD_ENGINE", "") != "fast"):
        raise SystemExit("NPROC_PER_NODE > 1 spreads the regions of an LBI run over GPUs: it needs kind lbi and BACKWARD_ENGINE=fast")
    launcher = [_env("PYTHON_BIN", sys.executable), "-m"]
    if nproc > 1:  # one process per GPU on this node; the rendezvous address is numeric on purpose
        launcher += ["torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
                     "--master-port", str(_env("MASTER_PORT", 29500)), "-m"]
    args = [
        *launcher, "lbi_b200.train.lbi",
        "--variants", "dense" if kind == "dense" else "lbi", "--backbone", backbone, "--output-dir", out_dir, "--run-name", run_name,
        "--seed", str(seed), "--data-mode", _env("DATA_MODE", "text_bpe_sharded"), "--text-corpus", _env("TEXT_CORPUS", "fineweb_edu"),
        "--tokenizer-type", tokenizer_type, "--vocab-size", str(vocab), "--seq-len", str(seq_len), "--batch-size", str(batch),
        "--steps", str(steps), "--eval-every", str(_env("EVAL_EVERY", 200)), "--eval-batches", str(_env("EVAL_BATCHES", 4)),
        "--log-every", str(_env("LOG_EVERY", 20)), "--save-every", str(_env("SAVE_EVERY", 5000)),
        "--lr-model", str(lr), "--lr-schedule", _env("LR_SCHEDULE", "cosine"), "--warmup-steps", str(warmup),
        "--min-lr-ratio", str(_env("MIN_LR_RATIO", 0.1)), "--weight-decay", str(wd), "--grad-clip", str(_env("GRAD_CLIP", 1.0)),
    ]
    if kind == "lbi":
        mode = _env("INTERFACE_JACOBIAN_MODE", "recompute")
        chunk = _env("JACOBIAN_BASIS_CHUNK", 32)
        if mode not in ("graph", "recompute", "structured", "forward"):
            raise SystemExit(f"INTERFACE_JACOBIAN_MODE must be graph, recompute, structured or forward, got '{mode}'")
        if chunk <= 0:
            raise SystemExit("JACOBIAN_BASIS_CHUNK must be > 0")
        args += [
            "--region-size", str(_env("REGION_SIZE", 2)), "--message-dim", str(message_dim),
            "--message-hidden-dim", str(_env("MESSAGE_HIDDEN_DIM", 0)),  # 0: the model width
            "--message-scale-init", str(_env("MESSAGE_SCALE_INIT", 0.5)),
            "--interface-jacobian-mode", mode, "--jacobian-basis-chunk", str(chunk),
        ]
        axis = _env("REGION_AXIS", "")
        if axis:  # REGION_AXIS=sequence SEQUENCE_REGIONS=8: cut the tokens instead of the layers (one span per GPU at 8 GPUs)
            args += ["--region-axis", axis, "--sequence-regions", str(_env("SEQUENCE_REGIONS", 8))]
    engine = _env("BACKWARD_ENGINE", "")
    if engine:  # BACKWARD_ENGINE=fast: the structured kernels without autograd (LBI: one process per GPU under NPROC_PER_NODE)
        args += ["--backward-engine", engine]
    args += ["--tie-embeddings" if tied else "--no-tie-embeddings"]
    ckpt_root = _env("CHECKPOINT_ROOT", "")
    if ckpt_root:
        args += ["--checkpoint-root", ckpt_root]
    if tokenizer_path:
        args += ["--tokenizer-path", tokenizer_path]
    if backbone in {"mamba3", "hybrid"}:
        args += ["--device", "cuda", "--dtype", "bfloat16"]
    args += ["--layers", str(arch.layers), "--dim", str(arch.dim)]
    for key, value in arch.flags.items():
        args += ["--" + key.replace("_", "-"), str(value)]
    if os.environ.get("LBI_LAUNCH_QUIET", "") == "":
        tokens_per_step = batch * seq_len
        print(f"Backbone: {backbone}\nModel scale: {scale}\nArchitecture tag: {arch_tag(backbone, scale)}\nFamily name: {family}\n"
              f"Variant name: {variant_name}\nOutput dir: {out_dir}\nRun name: {run_name}\nTarget steps: {steps}\n"
              f"Total tokens: {steps * tokens_per_step}\nTokens/step: {tokens_per_step}\nPeak LR: {lr}\nWarmup steps: {warmup}\n"
              f"Weight decay: {wd}\nTie embeddings: {tied}\nTokenizer type: {tokenizer_type}", file=sys.stderr, flush=True)
    return args + extra


def main(argv: list[str] | None = None) -> None:
    p = argparse.ArgumentParser(description="Launch one paper run (settings from environment variables).")
    p.add_argument("kind", choices=("lbi", "dense", "family-name", "family-dir"))
    p.add_argument("--dry-run", action="store_true", help="print the training command instead of running it")
    ns, extra = p.parse_known_args(argv)
    if ns.kind in ("family-name", "family-dir"):  # for the evaluation / plotting launchers (they read FAMILY_SEQ_LEN)
        name, path = family_from_env("FAMILY_SEQ_LEN")
        print(name if ns.kind == "family-name" else path)
        return
    cmd = build_command(ns.kind, extra)
    if ns.dry_run:
        print(" ".join(shlex.quote(c) for c in cmd))
        return
    os.execv(cmd[0], cmd)


if __name__ == "__main__":
    main()
