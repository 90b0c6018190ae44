"""NVTX ranges for the phases of a training step (forward region k / pullback / scan / local VJP / optimizer).

The reference has no tracing hooks (only ``time.perf_counter`` per step, train/runners.py:159-176).  Ranges are emitted
only when ``LBI_B200_NVTX=1`` (or ``enable()``) and a CUDA build of torch is present, so the hot path pays one branch.
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("LBI_B200_NVTX", "0") == "1"


def enable(flag: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(flag)


def enabled() -> bool:
    return _ENABLED and torch.cuda.is_available()


@contextlib.contextmanager
def range(name: str):  # noqa: A001 - mirrors torch.cuda.nvtx.range
    if not enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
