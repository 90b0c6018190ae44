"""Deterministic synthetic token tasks (arith, copy, reverse, selective_copy, induction).

Same task definitions, marker-token convention (bos = V-1, sep = V-2, pad = V-3) and sampling contract as the
reference's ``data/train_data.py:20-180``: corpora are [N, seq_len + 1] int64 and ``sample_batch`` returns the
(x, y) shift pair.  The generators draw in the same order from the same ``torch.Generator`` seed, so corpora are
reproducible across the two code bases.
"""
from __future__ import annotations

import torch

SYNTHETIC_TASKS = ("arith", "copy", "reverse", "selective_copy", "induction")


def _markers(vocab_size: int) -> tuple[int, int, int]:
    if vocab_size < 8:
        raise ValueError("vocab_size must be >= 8 for long-range synthetic tasks.")
    return vocab_size - 1, vocab_size - 2, vocab_size - 3


def _arith(n: int, total_len: int, vocab: int, gen: torch.Generator, dev: torch.device) -> torch.Tensor:
    start = torch.randint(0, vocab, (n, 1), generator=gen, device=dev)
    stride = torch.randint(1, min(vocab, 8), (n, 1), generator=gen, device=dev)
    return ((start + stride * torch.arange(total_len, device=dev).unsqueeze(0)) % vocab).to(torch.long)


def _copy_family(n: int, total_len: int, vocab: int, gen: torch.Generator, dev: torch.device, mode: str) -> torch.Tensor:
    bos, sep, pad = _markers(vocab)
    payload_len = max(2, (total_len - 2) // 2)
    payload = torch.randint(0, vocab - 3, (n, payload_len), generator=gen, device=dev)
    answer = {"copy": payload, "reverse": payload.flip(dims=(1,)), "selective_copy": payload[:, ::2]}[mode]
    seq = torch.full((n, total_len), pad, device=dev, dtype=torch.long)
    seq[:, 0] = bos
    seq[:, 1 : 1 + payload_len] = payload
    seq[:, 1 + payload_len] = sep
    start = 2 + payload_len
    width = max(0, min(total_len, start + answer.size(1)) - start)
    if width > 0:
        seq[:, start : start + width] = answer[:, :width]
    return seq


def _induction(n: int, total_len: int, vocab: int, gen: torch.Generator, dev: torch.device) -> torch.Tensor:
    bos, sep, pad = _markers(vocab)
    pairs = max(1, (total_len - 6) // 2)
    keys = torch.randint(0, vocab - 3, (n, pairs), generator=gen, device=dev)
    vals = torch.randint(0, vocab - 3, (n, pairs), generator=gen, device=dev)
    kv = torch.stack((keys, vals), dim=-1).reshape(n, 2 * pairs)
    pick = torch.randint(0, pairs, (n,), generator=gen, device=dev)
    q_key = keys.gather(1, pick.unsqueeze(1)).squeeze(1)
    q_val = vals.gather(1, pick.unsqueeze(1)).squeeze(1)
    seq = torch.full((n, total_len), pad, device=dev, dtype=torch.long)
    seq[:, 0] = bos
    end_kv = min(total_len, 1 + kv.size(1))
    seq[:, 1:end_kv] = kv[:, : end_kv - 1]
    for offset, value in enumerate((sep, q_key, sep, q_val)):
        pos = end_kv + offset
        if pos < total_len:
            seq[:, pos] = value
    return seq


def build_synthetic_corpus(*, num_sequences: int, seq_len: int, vocab_size: int, seed: int, task: str = "arith",
                           device: torch.device | None = None) -> torch.Tensor:
    """Deterministic token sequences of shape [N, seq_len + 1]."""
    if num_sequences <= 0:
        raise ValueError("num_sequences must be > 0")
    if seq_len <= 1:
        raise ValueError("seq_len must be > 1")
    if vocab_size <= 1:
        raise ValueError("vocab_size must be > 1")
    dev = device if device is not None else torch.device("cpu")
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    total_len = seq_len + 1
    if task == "arith":
        return _arith(num_sequences, total_len, vocab_size, gen, dev)
    if task in ("copy", "reverse", "selective_copy"):
        return _copy_family(num_sequences, total_len, vocab_size, gen, dev, task)
    if task == "induction":
        return _induction(num_sequences, total_len, vocab_size, gen, dev)
    raise ValueError("task must be one of: " + ", ".join(SYNTHETIC_TASKS))


def sample_batch(corpus: torch.Tensor, *, batch_size: int, generator: torch.Generator, device: torch.device):
    """Random rows of the corpus as an (x, y) next-token pair."""
    if batch_size <= 0:
        raise ValueError("batch_size must be > 0")
    idx = torch.randint(0, corpus.size(0), (batch_size,), generator=generator, device=corpus.device)
    seq = corpus.index_select(0, idx)
    return seq[:, :-1].to(device=device, non_blocking=True), seq[:, 1:].to(device=device, non_blocking=True)
