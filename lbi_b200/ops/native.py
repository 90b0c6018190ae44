"""Loader of the in-tree CUDA extension ``lbi_b200/_C*.so`` (built by ``python -m lbi_b200.build``)."""
from __future__ import annotations

import importlib
import os

import torch

_EXT = None
_ERR: Exception | None = None


def _load():
    global _EXT, _ERR
    if _EXT is not None or _ERR is not None:
        return
    try:
        # LBI_B200_DEBUG_EXT=1: the bounds-checking debug build (python -m lbi_b200.build --bounds-check)
        _EXT = importlib.import_module("lbi_b200._Cdbg" if os.environ.get("LBI_B200_DEBUG_EXT", "0") == "1" else "lbi_b200._C")
    except Exception as exc:  # noqa: BLE001 - reported by require_native
        _ERR = exc


def native_available() -> bool:
    _load()
    return _EXT is not None


def ext():
    _load()
    return _EXT


def require_native():
    """Return the extension module or raise with the build instruction."""
    _load()
    if _EXT is None:
        raise RuntimeError(
            "lbi_b200._C (sm_100a CUDA extension) is not built or failed to load: "
            f"{_ERR!r}. Build it in-tree with `python -m lbi_b200.build`."
        )
    return _EXT


if torch.cuda.is_available() and os.environ.get("LBI_B200_ALLOW_NO_NATIVE", "0") != "1":
    require_native()
