"""Run metadata and metric rows (reference train/metrics.py:97-215).

Artefacts per run directory: config.json, data_info.json, model_info.json, metrics.csv (fixed 15-column header),
metrics.jsonl (one JSON object per row), summary.json.
"""
from __future__ import annotations

import csv
import json
from pathlib import Path
from typing import Any

from torch import nn

from ..data.token_shards import corpus_numel
from ..models.dense_language_model import DenseLanguageModel
from ..models.lbi_language_model import LBILanguageModel

CSV_FIELDS = [
    "step", "tokens_seen", "split", "ce_loss", "message_norm", "scan_align", "jac_local_spec_mean", "jac_local_spec_max",
    "jac_local_frob_mean", "jac_local_frob_max", "jac_local_frob_normed_mean", "jac_suffix_spec_mean",
    "jac_suffix_spec_max", "tokens_per_s", "wall_time_s",
]


def count_parameters(module: nn.Module) -> int:
    return int(sum(p.numel() for p in module.parameters()))


def _readout_parts(model: nn.Module) -> tuple[int, int, bool]:
    readout = getattr(model, "readout", None)
    head = int(readout.output_head_parameter_count()) if readout is not None else 0
    norm = count_parameters(readout.norm) if readout is not None else 0
    tied = bool(getattr(readout, "tie_embeddings", False) and getattr(readout, "lm_head", None) is None)
    return head, norm, tied


# The per-component counts under the names the reference exports (train/metrics.py:20-43).
def canvas_component_params(model: nn.Module) -> int:
    canvas = getattr(model, "canvas", None)
    return count_parameters(canvas) if isinstance(canvas, nn.Module) else 0


def readout_lm_head_component_params(model: nn.Module) -> int:
    return _readout_parts(model)[0]


def readout_norm_component_params(model: nn.Module) -> int:
    return _readout_parts(model)[1]


def readout_uses_tied_output_weight(model: nn.Module) -> bool:
    return _readout_parts(model)[2]


def infer_data_info(cfg: Any, *, train_corpus: Any, val_corpus: Any, corpora_root: Any = None, resolve_text_paths_fn=None,
                    resolve_tokenizer_path_fn=None, resolve_token_shard_manifests_fn=None,
                    resolve_token_shards_dir_fn=None) -> dict[str, Any]:
    """Where the run's data came from.  The five optional arguments are the reference's injection points
    (train/metrics.py:46-56); left out, the resolvers of ``train.data`` are used."""
    from . import data as glue

    corpora_root = glue.CORPORA_ROOT if corpora_root is None else corpora_root
    text_paths = resolve_text_paths_fn or glue.resolve_text_paths
    tokenizer_path = resolve_tokenizer_path_fn or glue.resolve_tokenizer_path
    shard_manifests = resolve_token_shard_manifests_fn or glue.resolve_token_shard_manifests
    shards_dir = resolve_token_shards_dir_fn or glue.resolve_token_shards_dir
    info: dict[str, Any] = {
        "data_mode": cfg.data_mode, "text_corpus": cfg.text_corpus, "vocab_size": int(cfg.vocab_size),
        "seq_len": int(cfg.seq_len), "train_stream_length": corpus_numel(train_corpus),
        "val_stream_length": corpus_numel(val_corpus),
    }
    if cfg.data_mode == "synthetic":
        info.update(task=cfg.task, train_sequences=int(cfg.train_sequences), val_sequences=int(cfg.val_sequences))
        return info
    if cfg.data_mode == "text_bpe_sharded" and resolve_text_paths_fn is None:
        train_path, val_path = glue._shard_train_path(cfg), None
    else:
        train_path, val_path, _ = text_paths(cfg)
    info.update(
        corpora_root=str(corpora_root), train_path=str(train_path), val_path=str(val_path) if val_path else "",
        train_file_bytes=int(train_path.stat().st_size) if train_path.exists() else 0,
        val_file_bytes=int(val_path.stat().st_size) if (val_path and val_path.exists()) else 0,
    )
    if cfg.data_mode in {"text_bpe", "text_bpe_sharded"}:
        tok = tokenizer_path(cfg, train_path=train_path)
        vocab = tok.with_suffix(".vocab") if tok.suffix == ".model" else None
        info.update(tokenizer_path=str(tok), tokenizer_type=cfg.tokenizer_type, tokenizer_exists=tok.exists(),
                    tokenizer_vocab_path=str(vocab) if vocab else "", tokenizer_vocab_exists=bool(vocab and vocab.exists()))
    if cfg.data_mode == "text_bpe":
        info["tokenizer_train_bytes"] = int(cfg.tokenizer_train_bytes)
    if cfg.data_mode == "text_bpe_sharded":
        tm, vm = shard_manifests(cfg, train_path=train_path)
        info.update(token_shards_dir=str(shards_dir(cfg, train_path=train_path)), train_manifest=str(tm),
                    train_manifest_exists=tm.exists(), val_manifest=str(vm), val_manifest_exists=vm.exists())
    return info


def infer_model_info(cfg: Any, *, model: nn.Module) -> dict[str, Any]:
    """Parameter counts in total and per component, region layout and tying, as written to ``model_info.json``."""
    info: dict[str, Any] = {
        "model_class": type(model).__name__, "total_params": count_parameters(model), "layers": int(cfg.layers),
        "dim": int(cfg.dim), "d_state": int(cfg.d_state), "dt_rank": cfg.dt_rank if cfg.dt_rank is not None else "auto",
        "tie_embeddings": bool(cfg.tie_embeddings),
    }
    if isinstance(model, (LBILanguageModel, DenseLanguageModel)):
        canvas = count_parameters(model.canvas)
        head, norm, tied = _readout_parts(model)
        info["tokenizer_params"] = canvas + head
        info["lm_head_tied_to_embedding"] = tied
        parts = {"canvas": canvas, "canvas.embedding": canvas, "readout.norm": norm, "readout.lm_head": head}
    if isinstance(model, LBILanguageModel):
        iface = model.interface
        backbone = int(model.region_backend.count_parameters())
        info.update(n_regions=int(model.num_regions), region_ranges=[list(r) for r in model.region_ranges],
                    region_axis=model.region_axis, backbone_params=backbone, interface_params=count_parameters(iface),
                    owned_lbi_model=True)
        parts.update({
            "region_backend": backbone,
            "interface.initial_encoder": count_parameters(iface.initial_encoder),
            "interface.decoders": int(sum(count_parameters(m) for m in iface.decoders)),
            "interface.encoders": int(sum(count_parameters(m) for m in iface.encoders)),
            "interface.norms": int(sum(count_parameters(m) for m in iface.norms)),
            "interface.update_scale": int(iface.update_scale.numel()),
        })
        info["component_params"] = parts
    elif isinstance(model, DenseLanguageModel):
        backbone = int(sum(count_parameters(b) for b in model.blocks))
        info.update(backbone_params=backbone, interface_params=0)
        parts["blocks"] = backbone
        info["component_params"] = parts
    return info


def write_run_metadata(*, cfg: Any, run_dir: Path, model: nn.Module, train_corpus: Any, val_corpus: Any, corpora_root: Any = None,
                       resolve_text_paths_fn=None, resolve_tokenizer_path_fn=None, resolve_token_shard_manifests_fn=None,
                       resolve_token_shards_dir_fn=None) -> None:
    """Write ``config.json``, ``data_info.json`` and ``model_info.json`` of a run directory (the optional arguments are passed on
    to ``infer_data_info``)."""
    dump = lambda obj: json.dumps(obj, indent=2, sort_keys=True)
    (run_dir / "config.json").write_text(dump(cfg.to_dict()), encoding="utf-8")
    data_info = infer_data_info(cfg, train_corpus=train_corpus, val_corpus=val_corpus, corpora_root=corpora_root,
                                resolve_text_paths_fn=resolve_text_paths_fn, resolve_tokenizer_path_fn=resolve_tokenizer_path_fn,
                                resolve_token_shard_manifests_fn=resolve_token_shard_manifests_fn,
                                resolve_token_shards_dir_fn=resolve_token_shards_dir_fn)
    (run_dir / "data_info.json").write_text(dump(data_info), encoding="utf-8")
    (run_dir / "model_info.json").write_text(dump(infer_model_info(cfg, model=model)), encoding="utf-8")


def write_csv_row(path: Path, row: dict[str, Any]) -> None:
    is_new = not path.exists()
    with path.open("a", encoding="utf-8", newline="") as f:
        writer = csv.DictWriter(f, fieldnames=CSV_FIELDS)
        if is_new:
            writer.writeheader()
        writer.writerow({k: row.get(k, "") for k in CSV_FIELDS})


def log_row(run_dir: Path, row: dict[str, Any]) -> None:
    """One row to metrics.csv and the same object to metrics.jsonl."""
    write_csv_row(run_dir / "metrics.csv", row)
    with (run_dir / "metrics.jsonl").open("a", encoding="utf-8") as f:
        f.write(json.dumps(row, sort_keys=True) + "\n")
