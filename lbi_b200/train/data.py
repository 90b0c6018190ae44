"""Corpus and tokenizer resolution for the four data modes (reference train/data.py:14-196)."""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from ..data.bpe_tokenizer import build_token_stream, load_text_tokenizer
from ..data.data_paths import CORPORA_ROOT, LLAMA31_TOKENIZER_ROOT, LLAMA_TOKENIZER_ROOT, TOKENIZERS_ROOT
from ..data.lm_data import build_byte_stream, sample_batch_stream, split_stream_train_val
from ..data.token_shards import TokenShardCorpus, sample_batch_token_shards
from ..data.train_data import build_synthetic_corpus, sample_batch
from .config import BUNDLED_TEXT_CORPORA

__all__ = [
    "BUNDLED_TEXT_CORPORA", "CORPORA_ROOT", "resolve_text_paths", "resolve_tokenizer_path", "resolve_token_shards_dir",
    "resolve_token_shard_manifests", "resolve_runtime_vocab_size", "build_corpora", "sample_batch_any",
]


def resolve_text_paths(cfg: Any) -> tuple[Path, Path | None, Path]:
    """(train file, validation file or None, corpora root) from explicit paths or the bundled corpus name."""
    if cfg.train_text_path:
        return Path(cfg.train_text_path), (Path(cfg.val_text_path) if cfg.val_text_path else None), CORPORA_ROOT
    train_name, val_name = BUNDLED_TEXT_CORPORA[cfg.text_corpus]
    train_path = CORPORA_ROOT / train_name
    if not train_path.exists():
        raise FileNotFoundError(
            f"bundled corpus file missing: {train_path}. Prepare it with `python -m lbi_b200.data.export_fineweb_edu` "
            "or pass --train-text-path/--val-text-path."
        )
    return train_path, CORPORA_ROOT / val_name, CORPORA_ROOT


def resolve_tokenizer_path(cfg: Any, *, train_path: Path) -> Path:
    """The tokenizer file or directory of a run: explicit path, pretrained root for llama types, else the trained SentencePiece model."""
    if cfg.tokenizer_path:
        return Path(cfg.tokenizer_path)
    pretrained = {"llama": (LLAMA_TOKENIZER_ROOT, "llama"), "llama31": (LLAMA31_TOKENIZER_ROOT, "llama31")}
    if cfg.tokenizer_type in pretrained:
        root, legacy_name = pretrained[cfg.tokenizer_type]
        legacy = TOKENIZERS_ROOT / legacy_name
        return root if root.exists() or not legacy.exists() else legacy
    if not cfg.train_text_path:
        return TOKENIZERS_ROOT / f"{cfg.text_corpus}_sp_bpe_{cfg.vocab_size}.model"
    return train_path.parent / "tokenizers" / f"{train_path.stem}_sp_bpe_{cfg.vocab_size}.model"


def resolve_token_shards_dir(cfg: Any, *, train_path: Path) -> Path:
    """Where the token shards of a corpus / tokenizer pair live (explicit ``token_shards_dir`` wins)."""
    tag = cfg.tokenizer_type if cfg.tokenizer_type in {"llama", "llama31"} else f"sp_bpe_{cfg.vocab_size}"
    if cfg.token_shards_dir:
        return Path(cfg.token_shards_dir)
    if not cfg.train_text_path:
        return CORPORA_ROOT / cfg.text_corpus / "tokens" / f"{cfg.text_corpus}_{tag}"
    return train_path.parent / "tokens" / f"{train_path.stem}_{tag}"


def resolve_token_shard_manifests(cfg: Any, *, train_path: Path) -> tuple[Path, Path]:
    shard_dir = resolve_token_shards_dir(cfg, train_path=train_path)
    return shard_dir / "train_manifest.json", shard_dir / "val_manifest.json"


def _shard_train_path(cfg: Any) -> Path:
    """Sharded mode only needs the path for naming; the text file itself may be absent when shards exist."""
    if cfg.train_text_path:
        return Path(cfg.train_text_path)
    return CORPORA_ROOT / BUNDLED_TEXT_CORPORA[cfg.text_corpus][0]


def resolve_runtime_vocab_size(cfg: Any) -> int:
    """A pretrained HF tokenizer dictates the vocabulary; everything else keeps ``cfg.vocab_size``."""
    if cfg.data_mode not in {"text_bpe", "text_bpe_sharded"} or cfg.tokenizer_type not in {"llama", "llama31"}:
        return int(cfg.vocab_size)
    train_path = _shard_train_path(cfg)
    tokenizer_path = resolve_tokenizer_path(cfg, train_path=train_path)
    tok = load_text_tokenizer(tokenizer_type=cfg.tokenizer_type, tokenizer_path=tokenizer_path, train_path=train_path,
                              vocab_size=cfg.vocab_size, train_bytes=cfg.tokenizer_train_bytes, force_train=False)
    actual = int(tok.vocab_size)
    if actual != cfg.vocab_size:
        print(f"[tokenizer] overriding vocab_size from {cfg.vocab_size} to {cfg.tokenizer_type} tokenizer "
              f"vocab_size={actual} from {tokenizer_path}", flush=True)
    return actual


def build_corpora(cfg: Any, *, device: torch.device):
    """(train corpus, validation corpus) for the configured data mode: synthetic tensor, byte / token stream, or memory-mapped shards."""
    if cfg.data_mode == "synthetic":
        make = lambda n, seed: build_synthetic_corpus(num_sequences=n, seq_len=cfg.seq_len, vocab_size=cfg.vocab_size,
                                                      seed=seed, task=cfg.task, device=device)
        return make(cfg.train_sequences, cfg.seed + 11), make(cfg.val_sequences, cfg.seed + 29)
    if cfg.data_mode == "text_bpe_sharded":
        train_manifest, val_manifest = resolve_token_shard_manifests(cfg, train_path=_shard_train_path(cfg))
        for manifest in (train_manifest, val_manifest):
            if not manifest.exists():
                raise FileNotFoundError(
                    f"token shard manifest missing: {manifest}. Run: python -m lbi_b200.data.pretokenize_corpus "
                    f"--text-corpus {cfg.text_corpus} --vocab-size {cfg.vocab_size}"
                )
        return TokenShardCorpus(train_manifest), TokenShardCorpus(val_manifest)
    train_path, val_path, _ = resolve_text_paths(cfg)
    cpu = torch.device("cpu")
    if cfg.data_mode == "text_byte":
        load = lambda path: build_byte_stream(path, device=cpu)
    else:
        tokenizer = load_text_tokenizer(
            tokenizer_type=cfg.tokenizer_type, tokenizer_path=resolve_tokenizer_path(cfg, train_path=train_path),
            train_path=train_path, vocab_size=cfg.vocab_size, train_bytes=cfg.tokenizer_train_bytes,
            force_train=cfg.train_tokenizer,
        )
        load = lambda path: build_token_stream(path, tokenizer=tokenizer, device=cpu)
    train_stream = load(train_path)
    if cfg.val_text_path:
        return train_stream, load(cfg.val_text_path)
    if val_path is not None and val_path.exists():
        return train_stream, load(val_path)
    return split_stream_train_val(train_stream, val_fraction=cfg.val_split)


def sample_batch_any(*, cfg: Any, corpus, batch_size: int, generator: torch.Generator, device: torch.device):
    if cfg.data_mode == "synthetic":
        return sample_batch(corpus, batch_size=batch_size, generator=generator, device=device)
    if cfg.data_mode == "text_bpe_sharded":
        return sample_batch_token_shards(corpus, batch_size=batch_size, seq_len=cfg.seq_len, generator=generator, device=device)
    return sample_batch_stream(corpus, batch_size=batch_size, seq_len=cfg.seq_len, generator=generator, device=device)
