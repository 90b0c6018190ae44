"""``python -m lbi_b200 <command> [arguments]``: one front door for the package's commands."""
from __future__ import annotations

import importlib
import sys

COMMANDS = {
    "train": ("lbi_b200.train.lbi", "train dense and / or LBI language models"),
    "generate": ("lbi_b200.inference", "continue a prompt with a trained run"),
    "serve": ("lbi_b200.serve", "serve a trained run over HTTP"),
    "build": ("lbi_b200.build", "compile the sm_100a extension in place"),
    "pretokenize": ("lbi_b200.data.pretokenize_corpus", "tokenize a text corpus into int32 shards"),
    "export-fineweb-edu": ("lbi_b200.data.export_fineweb_edu", "stream a FineWeb-Edu subset into text files"),
    "evaluate": ("lbi_b200.scripts.evaluate_paper_checkpoints", "post-hoc evaluation of a run family"),
    "plot-curves": ("lbi_b200.scripts.plot_training_curves", "training-curve figures and group summaries"),
    "plot-ablations": ("lbi_b200.scripts.plot_message_ablations", "message-ablation figures"),
    "plot-jacobians": ("lbi_b200.scripts.plot_jacobian_diagnostics", "interface-Jacobian figure and table"),
    "grad-parity": ("lbi_b200.scripts.generate_grad_parity_report", "gradient-parity report"),
    "launch": ("lbi_b200.scripts.paper_presets", "paper launcher: launch {lbi,dense} [--dry-run]"),
}


def usage() -> str:
    width = max(len(name) for name in COMMANDS)
    lines = ["usage: python -m lbi_b200 <command> [arguments]", "", "commands:"]
    lines += [f"  {name.ljust(width)}  {text}" for name, (_, text) in COMMANDS.items()]
    return "\n".join(lines)


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(usage())
        return 0
    name, rest = argv[0], argv[1:]
    if name not in COMMANDS:
        print(f"unknown command {name!r}\n\n{usage()}", file=sys.stderr)
        return 2
    module = importlib.import_module(COMMANDS[name][0])
    saved = sys.argv
    sys.argv = [f"python -m lbi_b200 {name}", *rest]  # the commands read sys.argv through argparse
    try:
        module.main()
    finally:
        sys.argv = saved
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
