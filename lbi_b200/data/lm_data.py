"""Byte-level text streams (reference data/lm_data.py:13-64)."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch


def build_byte_stream(path: str | Path, *, device: torch.device | None = None) -> torch.Tensor:
    """The file's bytes as a 1-D int64 token stream."""
    p = Path(path)
    if not p.exists():
        raise FileNotFoundError(f"text file not found: {p}")
    raw = p.read_bytes()
    if not raw:
        raise ValueError(f"text file is empty: {p}")
    stream = torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).astype(np.int64))
    return stream.to(device) if device is not None else stream


def split_stream_train_val(stream: torch.Tensor, *, val_fraction: float):
    """The last ``val_fraction`` of a stream as validation, the rest as training."""
    if stream.dim() != 1:
        raise ValueError("stream must be 1D")
    if not (0.0 < val_fraction < 1.0):
        raise ValueError("val_fraction must be in (0, 1)")
    n = int(stream.numel())
    n_val = max(1, int(n * val_fraction))
    if n - n_val < 2:
        raise ValueError("stream too small after split")
    return stream[:-n_val].contiguous(), stream[-n_val:].contiguous()


def sample_batch_stream(stream: torch.Tensor, *, batch_size: int, seq_len: int, generator: torch.Generator,
                        device: torch.device):
    """Random contiguous windows of seq_len + 1 tokens."""
    if batch_size <= 0:
        raise ValueError("batch_size must be > 0")
    if seq_len <= 0:
        raise ValueError("seq_len must be > 0")
    if stream.dim() != 1:
        raise ValueError("stream must be 1D")
    n, needed = int(stream.numel()), seq_len + 1
    if n <= needed:
        raise ValueError(f"stream length {n} must be > seq_len + 1 ({needed})")
    starts = torch.randint(0, n - needed + 1, (batch_size,), generator=generator, device=stream.device)
    seq = stream[starts.unsqueeze(1) + torch.arange(needed, device=stream.device).unsqueeze(0)]
    return seq[:, :-1].to(device=device, non_blocking=True), seq[:, 1:].to(device=device, non_blocking=True)
