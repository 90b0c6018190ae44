"""Pre-tokenise a text corpus into int32 shards plus manifests:  python -m lbi_b200.data.pretokenize_corpus ...

Output format is the reference's (data/pretokenize_corpus.py:70-117): ``<split>_%04d.bin`` raw int32 files and
``<split>_manifest.json`` = {split, dtype, tokenizer_vocab_size, num_tokens_total, shards: [{path, num_tokens}]},
so shards written by either code base feed ``TokenShardCorpus``.  Lines are encoded one at a time and appended to
a preallocated int32 buffer, so memory stays at one shard regardless of corpus size.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np

from .bpe_tokenizer import TextTokenizerBackend, load_text_tokenizer
from .data_paths import CORPORA_ROOT, LLAMA31_TOKENIZER_ROOT, LLAMA_TOKENIZER_ROOT, TOKENIZERS_ROOT


def tokenizer_tag(tokenizer_type: str, vocab_size: int) -> str:
    return tokenizer_type if tokenizer_type in {"llama", "llama31"} else f"sp_bpe_{vocab_size}"


def default_output_dir(text_corpus: str, train_path: Path, vocab_size: int, tokenizer_type: str) -> Path:
    """Where shards go by default: below the corpus directory for bundled corpora, beside the text file otherwise."""
    tag = tokenizer_tag(tokenizer_type, vocab_size)
    try:
        inside = train_path.resolve().is_relative_to(CORPORA_ROOT.resolve())
    except OSError:
        inside = False
    if inside:
        base = train_path.parent if train_path.parent.name == text_corpus else CORPORA_ROOT / text_corpus
        return base / "tokens" / f"{text_corpus}_{tag}"
    return train_path.parent / "tokens" / f"{train_path.stem}_{tag}"


def resolve_tokenizer_path(tokenizer_type: str, tokenizer_path: str, text_corpus: str, train_path: Path, vocab_size: int) -> Path:
    """Explicit path, pretrained root for llama types, else the SentencePiece model named after the corpus or the text file."""
    if tokenizer_path:
        return Path(tokenizer_path)
    if tokenizer_type == "llama":
        return LLAMA_TOKENIZER_ROOT
    if tokenizer_type == "llama31":
        return LLAMA31_TOKENIZER_ROOT
    if text_corpus:
        return TOKENIZERS_ROOT / f"{text_corpus}_sp_bpe_{vocab_size}.model"
    return train_path.parent / "tokenizers" / f"{train_path.stem}_sp_bpe_{vocab_size}.model"


def write_shards(split_name: str, src_path: Path, tokenizer: TextTokenizerBackend, out_dir: Path, shard_tokens: int) -> Path:
    """Encode a text file line by line into ``<split>_%04d.bin`` int32 shards of about ``shard_tokens`` tokens plus ``<split>_manifest.json``."""
    out_dir.mkdir(parents=True, exist_ok=True)
    shards: list[dict] = []
    buf = np.empty(max(1, shard_tokens) + 65536, dtype=np.int32)
    fill = 0
    total = 0

    def flush() -> None:
        nonlocal fill, total
        if fill == 0:
            return
        name = f"{split_name}_{len(shards):04d}.bin"
        buf[:fill].tofile(out_dir / name)
        shards.append({"path": name, "num_tokens": int(fill)})
        total += fill
        fill = 0

    with src_path.open("rb") as f:
        for line in f:
            if not line:
                continue
            ids = tokenizer.encode_bytes(line if line.endswith(b"\n") else line + b"\n")
            if not ids:
                continue
            if fill + len(ids) > buf.size:
                grown = np.empty(max(buf.size * 2, fill + len(ids)), dtype=np.int32)
                grown[:fill] = buf[:fill]
                buf = grown
            buf[fill : fill + len(ids)] = ids
            fill += len(ids)
            if fill >= shard_tokens:
                flush()
    flush()
    if not shards:
        raise ValueError(f"no tokens were produced for split {split_name}: {src_path}")
    manifest_path = out_dir / f"{split_name}_manifest.json"
    manifest = {"split": split_name, "dtype": "int32", "tokenizer_vocab_size": int(tokenizer.vocab_size),
                "num_tokens_total": int(total), "shards": shards}
    manifest_path.write_text(json.dumps(manifest, indent=2, sort_keys=True), encoding="utf-8")
    print(f"[{split_name}] wrote {len(shards)} shards total_tokens={total} manifest={manifest_path}", flush=True)
    return manifest_path


def resolve_text_paths(text_corpus: str, train_text_path: str = "", val_text_path: str = "") -> tuple[Path, Path | None, str]:
    """(train file, validation file or None, corpus name for the default tokenizer / output names): explicit paths win over
    the bundled corpus of that name."""
    if train_text_path:
        return Path(train_text_path), (Path(val_text_path) if val_text_path else None), ""
    from ..train.config import BUNDLED_TEXT_CORPORA

    if text_corpus not in BUNDLED_TEXT_CORPORA:
        raise ValueError(f"unknown text corpus {text_corpus!r}; give train_text_path or one of {sorted(BUNDLED_TEXT_CORPORA)}")
    train_name, val_name = BUNDLED_TEXT_CORPORA[text_corpus]
    return CORPORA_ROOT / train_name, CORPORA_ROOT / val_name, text_corpus


def pretokenize_text_corpus(*, tokenizer_type: str, vocab_size: int, tokenizer_train_bytes: int, shard_tokens: int,
                            train_tokenizer: bool = False, tokenizer_path: Path | str = "", train_path: Path | None = None,
                            val_path: Path | None = None, out_dir: Path | None = None, text_corpus: str = "",
                            train_text_path: str = "", val_text_path: str = "",
                            output_dir: str = "") -> tuple[Path, Path | None]:
    """Two call forms.  With ``train_path`` (and optionally ``val_path``, ``out_dir``, a resolved ``tokenizer_path``) the files are
    taken as given and a missing validation split is skipped.  With the reference's keywords (``text_corpus``, ``train_text_path``,
    ``val_text_path``, ``output_dir``; data/pretokenize_corpus.py:146-182) the paths, the tokenizer file and the output directory
    are resolved from the corpus name, and both splits must exist."""
    if train_path is None:
        train_path, val_path, corpus_name = resolve_text_paths(text_corpus, train_text_path, val_text_path)
        if not train_path.exists():
            raise FileNotFoundError(f"train text not found: {train_path}")
        if val_path is None or not val_path.exists():
            raise FileNotFoundError(f"val text not found: {val_path}")
        tokenizer_path = resolve_tokenizer_path(tokenizer_type, str(tokenizer_path or ""), corpus_name, train_path, vocab_size)
        out_dir = Path(output_dir) if output_dir else default_output_dir(text_corpus, train_path, vocab_size, tokenizer_type)
    elif out_dir is None:
        out_dir = Path(output_dir) if output_dir else default_output_dir(text_corpus, train_path, vocab_size, tokenizer_type)
    tokenizer = load_text_tokenizer(tokenizer_type=tokenizer_type, tokenizer_path=Path(tokenizer_path), train_path=train_path,
                                    vocab_size=vocab_size, train_bytes=tokenizer_train_bytes, force_train=train_tokenizer)
    train_manifest = write_shards("train", train_path, tokenizer, out_dir, shard_tokens)
    val_manifest = write_shards("val", val_path, tokenizer, out_dir, shard_tokens) if val_path is not None else None
    return train_manifest, val_manifest


def pretokenize_sentencepiece_corpus(**kwargs) -> tuple[Path, Path | None]:
    """``pretokenize_text_corpus`` with the SentencePiece tokenizer (reference data/pretokenize_corpus.py:120-143)."""
    kwargs.pop("tokenizer_type", None)
    return pretokenize_text_corpus(tokenizer_type="sentencepiece", **kwargs)


def main() -> None:
    p = argparse.ArgumentParser(description="Tokenise a text corpus into int32 shards with manifests.")
    p.add_argument("--text-corpus", type=str, default="fineweb_edu")
    p.add_argument("--train-text-path", type=str, default="")
    p.add_argument("--val-text-path", type=str, default="")
    p.add_argument("--tokenizer-type", type=str, default="sentencepiece")
    p.add_argument("--tokenizer-path", type=str, default="")
    p.add_argument("--vocab-size", type=int, default=32000)
    p.add_argument("--tokenizer-train-bytes", type=int, default=8 * 1024 * 1024)
    p.add_argument("--train-tokenizer", action="store_true")
    p.add_argument("--output-dir", type=str, default="")
    p.add_argument("--shard-tokens", type=int, default=50_000_000)
    args = p.parse_args()
    train_path, val_path, corpus_name = resolve_text_paths(args.text_corpus, args.train_text_path, args.val_text_path)
    tok_path = resolve_tokenizer_path(args.tokenizer_type, args.tokenizer_path, corpus_name, train_path, args.vocab_size)
    out_dir = Path(args.output_dir) if args.output_dir else default_output_dir(args.text_corpus, train_path, args.vocab_size,
                                                                              args.tokenizer_type)
    pretokenize_text_corpus(train_path=train_path, val_path=val_path if (val_path and val_path.exists()) else None,
                            tokenizer_type=args.tokenizer_type, tokenizer_path=tok_path, vocab_size=args.vocab_size,
                            tokenizer_train_bytes=args.tokenizer_train_bytes, out_dir=out_dir, shard_tokens=args.shard_tokens,
                            train_tokenizer=args.train_tokenizer)


if __name__ == "__main__":
    main()
