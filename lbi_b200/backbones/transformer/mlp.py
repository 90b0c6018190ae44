"""SwiGLU feed-forward block (``fc1`` -> split -> ``up * silu(gate)`` -> ``fc2``).

Key names and the round-up of the hidden width to a multiple of 128 follow the
reference's ``backbones/transformer/mlp.py:10-29`` so checkpoints load unchanged;
``up`` is the first half of ``fc1``'s output and ``gate`` the second.
"""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F


def swiglu_hidden(dim: int, hidden_features: int | None, multiple_of: int = 128) -> int:
    hidden = hidden_features if hidden_features is not None else int(8 * dim / 3)
    return max(multiple_of, -(-hidden // multiple_of) * multiple_of)


class GatedMLP(nn.Module):
    """SwiGLU: ``fc2(up * silu(gate))`` with ``up | gate = fc1(x)``; the hidden width is rounded up to a multiple of ``multiple_of``."""

    def __init__(
        self,
        dim: int,
        *,
        hidden_features: int | None = None,
        out_features: int | None = None,
        bias: bool = False,
        multiple_of: int = 128,
    ) -> None:
        super().__init__()
        hidden = swiglu_hidden(dim, hidden_features, multiple_of)
        self.hidden_features = hidden
        self.fc1 = nn.Linear(dim, 2 * hidden, bias=bias)
        self.fc2 = nn.Linear(hidden, dim if out_features is None else out_features, bias=bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        up, gate = self.fc1(x).chunk(2, dim=-1)
        return self.fc2(up * F.silu(gate))


class SwiGLUMLP(GatedMLP):
    """``GatedMLP`` with the hidden width given as a ratio of the model width and no rounding."""

    def __init__(self, dim: int, mlp_ratio: float = 4.0, bias: bool = False) -> None:
        super().__init__(dim, hidden_features=max(1, int(dim * mlp_ratio)), out_features=dim, bias=bias, multiple_of=1)
