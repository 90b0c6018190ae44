"""Data roots, overridable through the same environment variables as the reference (data/data_paths.py:7-21)."""
from __future__ import annotations

import os
from pathlib import Path


def _root(var: str, default: Path) -> Path:
    return Path(os.environ.get(var, default)).expanduser()


DATA_ROOT = _root("LBI_DATA_ROOT", Path("data"))
U2_DATA_ROOT = DATA_ROOT
CORPORA_ROOT = _root("LBI_CORPORA_ROOT", DATA_ROOT / "corpora")
TOKENIZERS_ROOT = _root("LBI_TOKENIZERS_ROOT", CORPORA_ROOT / "tokenizers")
PRETRAINED_TOKENIZERS_ROOT = _root("LBI_PRETRAINED_TOKENIZERS_ROOT", DATA_ROOT / "tokenizers")
LLAMA_TOKENIZER_ROOT = _root("LBI_LLAMA_TOKENIZER_ROOT", PRETRAINED_TOKENIZERS_ROOT / "llama")
LLAMA31_TOKENIZER_ROOT = _root("LBI_LLAMA31_TOKENIZER_ROOT", PRETRAINED_TOKENIZERS_ROOT / "llama-3.1")
