"""Tokenizers: a self-contained byte-level BPE, a SentencePiece wrapper/trainer and a Hugging Face wrapper.

Public surface follows the reference's ``data/bpe_tokenizer.py`` (ByteBPETokenizer :76-136, trainers :139-199 and
:250-305, ``load_text_tokenizer`` :324-369, ``build_token_stream`` :372-385); the byte-BPE file format
(``{"merges": [[a, b, id]], "token_bytes": {id: [bytes]}}``) is the same, so tokenizer files are interchangeable.
The BPE trainer keeps pair counts incrementally instead of recounting the corpus for every merge.
"""
from __future__ import annotations

import json
import tempfile
from collections import Counter, defaultdict
from dataclasses import dataclass
from pathlib import Path
from typing import Protocol

import torch

try:  # optional
    import sentencepiece as spm
except ImportError:  # pragma: no cover
    spm = None

_PRETRAINED_HF_TOKENIZER_TYPES = {"llama", "llama31"}


class TextTokenizerBackend(Protocol):
    """What the data layer needs from a tokenizer: ``vocab_size`` and ``encode_bytes``."""

    @property
    def vocab_size(self) -> int: ...

    def encode_bytes(self, raw: bytes) -> list[int]: ...


def split_bytes_into_pieces(raw: bytes) -> list[bytes]:
    """Maximal runs of whitespace / non-whitespace bytes; merges never cross a piece boundary."""
    pieces, start, in_space = [], 0, None
    for idx, value in enumerate(raw):
        is_space = chr(value).isspace()
        if in_space is None:
            in_space = is_space
        elif is_space != in_space:
            pieces.append(raw[start:idx])
            start, in_space = idx, is_space
    if raw:
        pieces.append(raw[start:])
    return [p for p in pieces if p]


@dataclass
class ByteBPETokenizer:
    """Dependency-free byte-level BPE: 256 byte tokens plus learnt merges inside whitespace-delimited pieces; exact round trip."""

    merges: list[tuple[int, int, int]]
    token_bytes: dict[int, bytes]

    def __post_init__(self) -> None:
        self._ranks = {(a, b): (rank, new_id) for rank, (a, b, new_id) in enumerate(self.merges)}

    @property
    def vocab_size(self) -> int:
        return len(self.token_bytes)

    @property
    def pair_to_merge(self) -> dict[tuple[int, int], tuple[int, int]]:
        return self._ranks

    def encode_piece(self, piece: bytes) -> list[int]:
        word = list(piece)
        while len(word) >= 2:
            best = None
            for idx in range(len(word) - 1):
                hit = self._ranks.get((word[idx], word[idx + 1]))
                if hit is not None and (best is None or hit[0] < best[0]):
                    best = (hit[0], idx, hit[1])
            if best is None:
                break
            _, idx, new_id = best
            word[idx : idx + 2] = [new_id]
        return word

    def encode_bytes(self, raw: bytes) -> list[int]:
        cache: dict[bytes, list[int]] = {}
        ids: list[int] = []
        for piece in split_bytes_into_pieces(raw):
            hit = cache.get(piece)
            if hit is None:
                hit = cache[piece] = self.encode_piece(piece)
            ids.extend(hit)
        return ids

    def decode(self, ids) -> bytes:
        return b"".join(self.token_bytes[int(i)] for i in ids)

    def save(self, path: str | Path) -> None:
        out = Path(path)
        out.parent.mkdir(parents=True, exist_ok=True)
        payload = {"merges": [list(m) for m in self.merges], "token_bytes": {str(k): list(v) for k, v in self.token_bytes.items()}}
        out.write_text(json.dumps(payload), encoding="utf-8")

    @classmethod
    def load(cls, path: str | Path) -> "ByteBPETokenizer":
        payload = json.loads(Path(path).read_text(encoding="utf-8"))
        return cls(merges=[tuple(int(x) for x in row) for row in payload["merges"]],
                   token_bytes={int(k): bytes(v) for k, v in payload["token_bytes"].items()})


def train_byte_bpe_tokenizer(path: str | Path, *, vocab_size: int, max_bytes: int, min_pair_count: int = 2) -> ByteBPETokenizer:
    """Learn byte-pair merges on the first ``max_bytes`` of a file until the vocabulary reaches ``vocab_size``."""
    if vocab_size <= 256:
        raise ValueError("byte BPE vocab_size must be > 256")
    raw = Path(path).read_bytes()
    if not raw:
        raise ValueError(f"empty tokenizer training file: {path}")
    words = [(list(piece), freq) for piece, freq in Counter(split_bytes_into_pieces(raw[:max_bytes])).items()]
    pair_counts: Counter = Counter()
    where: dict[tuple[int, int], set[int]] = defaultdict(set)
    for w_idx, (word, freq) in enumerate(words):
        for a, b in zip(word, word[1:]):
            pair_counts[(a, b)] += freq
            where[(a, b)].add(w_idx)
    token_bytes = {i: bytes([i]) for i in range(256)}
    merges: list[tuple[int, int, int]] = []
    next_id = 256
    while next_id < vocab_size and pair_counts:
        # highest count wins; ties go to the pair that was counted first (Counter.most_common order)
        (left, right), count = max(pair_counts.items(), key=lambda kv: kv[1])
        if count < min_pair_count:
            break
        token_bytes[next_id] = token_bytes[left] + token_bytes[right]
        for w_idx in list(where[(left, right)]):
            word, freq = words[w_idx]
            for a, b in zip(word, word[1:]):
                pair_counts[(a, b)] -= freq
                if pair_counts[(a, b)] <= 0:
                    del pair_counts[(a, b)]
                where[(a, b)].discard(w_idx)
            merged, i = [], 0
            while i < len(word):
                if i + 1 < len(word) and word[i] == left and word[i + 1] == right:
                    merged.append(next_id)
                    i += 2
                else:
                    merged.append(word[i])
                    i += 1
            words[w_idx] = (merged, freq)
            for a, b in zip(merged, merged[1:]):
                pair_counts[(a, b)] += freq
                where[(a, b)].add(w_idx)
        where.pop((left, right), None)
        merges.append((left, right, next_id))
        next_id += 1
    return ByteBPETokenizer(merges=merges, token_bytes=token_bytes)


def load_or_train_byte_bpe_tokenizer(*, tokenizer_path, train_path, vocab_size: int, train_bytes: int,
                                     force_train: bool = False, min_pair_count: int = 2) -> ByteBPETokenizer:
    """Load the byte-BPE tokenizer file if present (and not ``force_train``), else train and save it."""
    path = Path(tokenizer_path)
    if path.exists() and not force_train:
        return ByteBPETokenizer.load(path)
    tok = train_byte_bpe_tokenizer(train_path, vocab_size=vocab_size, max_bytes=train_bytes, min_pair_count=min_pair_count)
    tok.save(path)
    return tok


class SentencePieceBPETokenizer:
    """A SentencePiece BPE model file."""

    def __init__(self, model_path: str | Path) -> None:
        if spm is None:
            raise ImportError("sentencepiece is required for text_bpe mode")
        self.model_path = Path(model_path)
        self.processor = spm.SentencePieceProcessor(model_file=str(self.model_path))

    @property
    def vocab_size(self) -> int:
        return int(self.processor.get_piece_size())

    def encode_bytes(self, raw: bytes) -> list[int]:
        return list(self.processor.encode(raw.decode("utf-8", errors="replace"), out_type=int))

    def decode(self, ids) -> bytes:
        return self.processor.decode([int(i) for i in ids]).encode("utf-8")


class HFAutoTextTokenizer:
    """A local Hugging Face tokenizer directory (the ``llama`` / ``llama31`` tokenizer types)."""

    def __init__(self, model_path: str | Path) -> None:
        from transformers import AutoTokenizer

        self.model_path = Path(model_path)
        self.tokenizer = AutoTokenizer.from_pretrained(str(self.model_path), local_files_only=True)

    @property
    def vocab_size(self) -> int:
        return int(len(self.tokenizer))

    def encode_bytes(self, raw: bytes) -> list[int]:
        return list(self.tokenizer.encode(raw.decode("utf-8", errors="replace"), add_special_tokens=False))

    def decode(self, ids) -> bytes:
        return self.tokenizer.decode([int(i) for i in ids], skip_special_tokens=True).encode("utf-8")


def train_sentencepiece_bpe_tokenizer(train_path, *, model_prefix, vocab_size: int, train_bytes: int) -> SentencePieceBPETokenizer:
    """Train a SentencePiece BPE model (byte fallback, identity normalisation, no bos / eos / pad) on the first ``train_bytes``."""
    if spm is None:
        raise ImportError("sentencepiece is required for text_bpe mode")
    raw = Path(train_path).read_bytes()
    if not raw:
        raise ValueError(f"empty tokenizer training file: {train_path}")
    prefix = Path(model_prefix)
    prefix.parent.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="spm_train_") as td:
        sample = Path(td) / "tokenizer_sample.txt"
        sample.write_text(raw[:train_bytes].decode("utf-8", errors="replace"), encoding="utf-8")
        # byte fallback, identity normalisation, no bos/eos/pad: ids cover exactly the requested vocabulary
        spm.SentencePieceTrainer.train(
            input=str(sample), model_prefix=str(prefix), vocab_size=vocab_size, model_type="bpe", character_coverage=1.0,
            bos_id=-1, eos_id=-1, pad_id=-1, unk_id=0, byte_fallback=True, normalization_rule_name="identity",
            max_sentence_length=1_000_000,
        )
    return SentencePieceBPETokenizer(f"{prefix}.model")


def load_or_train_sentencepiece_bpe_tokenizer(*, tokenizer_path, train_path, vocab_size: int, train_bytes: int,
                                              force_train: bool = False) -> SentencePieceBPETokenizer:
    """Load the ``.model`` file if present (and not ``force_train``), else train it."""
    model_path = Path(tokenizer_path)
    if model_path.suffix != ".model":
        model_path = model_path.with_suffix(".model")
    if model_path.exists() and not force_train:
        return SentencePieceBPETokenizer(model_path)
    return train_sentencepiece_bpe_tokenizer(train_path, model_prefix=model_path.with_suffix(""), vocab_size=vocab_size,
                                             train_bytes=train_bytes)


def load_text_tokenizer(*, tokenizer_type: str, tokenizer_path, train_path, vocab_size: int, train_bytes: int,
                        force_train: bool = False) -> TextTokenizerBackend:
    """The tokenizer backend for ``tokenizer_type`` (sentencepiece, llama, llama31, byte_bpe); pretrained types cannot be trained."""
    if tokenizer_type == "sentencepiece":
        tok = load_or_train_sentencepiece_bpe_tokenizer(tokenizer_path=tokenizer_path, train_path=train_path,
                                                        vocab_size=vocab_size, train_bytes=train_bytes, force_train=force_train)
        if tok.vocab_size != vocab_size:
            raise ValueError(f"sentencepiece tokenizer vocab mismatch: requested vocab_size={vocab_size}, "
                             f"but loaded tokenizer has vocab_size={tok.vocab_size}")
        return tok
    if tokenizer_type in _PRETRAINED_HF_TOKENIZER_TYPES:
        if force_train:
            raise ValueError(f"{tokenizer_type} tokenizer does not support --train-tokenizer; provide a local tokenizer path instead")
        model_path = Path(tokenizer_path)
        if not model_path.exists():
            raise FileNotFoundError(f"{tokenizer_type} tokenizer path not found: {model_path}. Provide a local HF-compatible "
                                    "tokenizer directory (tokenizer.json, tokenizer_config.json).")
        return HFAutoTextTokenizer(model_path)
    if tokenizer_type == "byte_bpe":
        return load_or_train_byte_bpe_tokenizer(tokenizer_path=tokenizer_path, train_path=train_path, vocab_size=vocab_size,
                                                train_bytes=train_bytes, force_train=force_train)
    raise ValueError(f"unsupported tokenizer_type: {tokenizer_type}")


def build_token_stream(path, *, tokenizer: TextTokenizerBackend, device: torch.device | None = None) -> torch.Tensor:
    """A text file encoded into one 1-D int64 token stream."""
    raw = Path(path).read_bytes()
    if not raw:
        raise ValueError(f"text file is empty: {path}")
    ids = tokenizer.encode_bytes(raw)
    if not ids:
        raise ValueError(f"tokenizer produced empty stream for: {path}")
    return torch.tensor(ids, dtype=torch.long, device=device if device is not None else torch.device("cpu"))


build_bpe_stream = build_token_stream
build_sentencepiece_bpe_stream = build_token_stream
