"""XGLU: a gated feed-forward layer whose multiplicative branch sees only a low-rank, normalised
summary of the input (reference: experiments/xglu/xglu.py:22-88).

``y = down(act(up(x)) * gate(norm(compress(x)) * rank / dim))`` with ``compress: dim -> rank``.
Against a GLU of the same hidden width it replaces one ``dim x hidden`` matrix by
``dim x rank + rank x hidden`` parameters."""

from __future__ import annotations

import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.modules.norm import RMSNorm

ACTIVATIONS = {"relu": F.relu, "silu": F.silu, "gelu": F.gelu, "tanh": F.tanh,
               "sigmoid": F.sigmoid, "relu2": lambda x: F.relu(x).square()}


def default_hidden(dim: int, multiple_of: int = 4) -> int:
    hidden = int(2 * 4 * dim / 3)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


class XGLU(nn.Module):
    def __init__(self, dim: int, hidden_dim: int | None = None, xglu_rank: int = 128,
                 activation_fn: str = "silu", dropout: float = 0.0, bias: bool = False,
                 multiple_of: int = 4) -> None:
        super().__init__()
        self.dim, self.rank = dim, xglu_rank
        self.hidden_dim = hidden_dim or default_hidden(dim, multiple_of)
        self.compress = nn.Linear(dim, xglu_rank, bias=bias)
        self.compress_norm = RMSNorm(xglu_rank)
        self.up = nn.Linear(dim, self.hidden_dim, bias=bias)
        self.gate = nn.Linear(xglu_rank, self.hidden_dim, bias=bias)
        self.down = nn.Linear(self.hidden_dim, dim, bias=bias)
        self.activation = ACTIVATIONS[activation_fn]
        self.dropout = nn.Dropout(dropout)
        self.reset_parameters()

    def forward(self, x: Tensor) -> Tensor:
        summary = self.compress_norm(self.compress(x)) * (self.rank / self.dim)
        return self.dropout(self.down(self.activation(self.up(x)) * self.gate(summary)))

    def reset_parameters(self, init_std: float | None = None, factor: float = 1.0) -> None:
        inner = init_std or self.dim**-0.5
        outer = (init_std or self.hidden_dim**-0.5) / factor
        for layer in (self.up, self.gate, self.compress):
            nn.init.trunc_normal_(layer.weight, std=inner, a=-3 * inner, b=3 * inner)
        nn.init.trunc_normal_(self.down.weight, std=outer, a=-3 * outer, b=3 * outer)

    def parameter_saving(self) -> int:
        """Parameters saved against a GLU of the same widths."""
        return self.dim * self.hidden_dim - (self.dim * self.rank + self.rank * self.hidden_dim
                                             + self.rank)
